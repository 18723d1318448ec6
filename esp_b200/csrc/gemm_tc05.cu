// Tensor-core matrix product for many rows (prefill) on the 5th-generation
// tensor cores: operands travel global -> shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), tcgen05.mma accumulates in tensor
// memory (TMEM), and the epilogue reads the accumulator back with tcgen05.ld.
//
//   PLAIN:  C[m, n]   = scale[m] * sum_k A[m, k] * W[g][n, k]                (float out)
//   SWIGLU: act[m, j] = silu(A W_gate[g][j]) * (A W_up[g][j])                (bfloat16 out)
//           W[g] = [gate rows; up rows]
//
// A is [rows, K] bfloat16, rows sorted by group; W is [G, Nw, K] bfloat16 (G = 1
// for a dense product).  The weights are the 128-row operand of the MMA and a
// run of up to 128 or 256 token rows is its N side, so the accumulator holds
// D[feature, token]: TMEM lane = output feature, TMEM column = token.  The width
// of a token tile is whatever its group has left, rounded up to 16, which keeps
// ragged groups (a handful of rows for one expert, hundreds for another) from
// wasting tensor work.  A token tile never mixes groups: the tile list (group,
// first row, rows) is made on the device by the routing kernels.
//
// One tile = 128 features x one token tile.  Warp 0 issues the TMA loads, warp 1
// owns TMEM and issues the MMAs, warps 2..5 are the epilogue (each reads the 32
// TMEM lanes that its position in the warpgroup may touch).  A ring of
// shared-memory stages is handed back and forth with mbarriers.  Every wait is
// bounded: if one runs out the kernel raises ESP_STATUS_WAIT_EXPIRED in the
// status word, stops issuing work, lets its own copies land, frees its TMEM and
// returns.
#include <cuda.h>

#include "common.cuh"

namespace {
constexpr int BF = 128;            // features (weight rows) per tile: the M side of the MMA
constexpr int TOK_BOX = 16;         // token rows per TMA box; a tile's width is a multiple of it
constexpr int BK = 64, THREADS = 192;
constexpr int W_BYTES = BF * BK * 2;
constexpr unsigned WAIT_LIMIT = 1u << 22;

struct Tc05Params {
    const int* tile_group;        // [tiles] or null (dense)
    const int* tile_row0;         // [tiles]
    const int* tile_rows;         // [tiles]
    const int* n_tiles;           // device scalar or null
    const float* row_scale;       // [rows] or null
    void* C;
    long long ldc;
    int M, N, K;                  // N: output columns (SWIGLU: the intermediate size)
    int* status;
};

// ---- PTX wrappers ----------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity) {
    const unsigned addr = smem_u32(bar);
    for (unsigned i = 0; i < WAIT_LIMIT; i++) {
        unsigned done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, void* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, void* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive float columns of this thread's TMEM lane
__device__ __forceinline__ void tc_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// Shared-memory operand descriptor: K-major tile whose rows are 128 bytes (64 bfloat16), written by TMA
// with the 128-byte swizzle; groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc(const void* p) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(p) & 0x3FFFFu) >> 4);       // start address, 16-byte units
    d |= (unsigned long long)1 << 16;                                // leading byte offset: unused for this layout
    d |= (unsigned long long)(1024 >> 4) << 32;                      // stride byte offset between 8-row groups
    d |= (unsigned long long)1 << 46;                                // descriptor version of this architecture
    d |= (unsigned long long)2 << 61;                                // 128-byte swizzle
    return d;
}
// Instruction descriptor: bfloat16 x bfloat16 -> float, both operands K-major, M = 128, N = n.
__device__ __forceinline__ unsigned instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(BF >> 4) << 24);
}

// Persistent form: a CTA per SM walks the list of (token tile, feature tile) pairs with stride gridDim.x.
// The producer runs ahead across tile boundaries, so the weight stream never pauses; the accumulator is
// double-buffered in TMEM, so the epilogue of one tile overlaps the MMAs of the next.
constexpr int MAX_TOK = 128;        // token rows per tile at most (the N side of the MMA)
constexpr int TOK_BYTES = MAX_TOK * BK * 2;
constexpr int RING_BYTES = 192 * 1024;

__device__ __forceinline__ void mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

struct TileInfo {
    int group, row0, n_rows, n_tok, f0;
};

template <bool SWIGLU>
__device__ __forceinline__ TileInfo tile_info(const Tc05Params& p, int tile, int feat_tiles) {
    TileInfo t;
    const int tt = tile / feat_tiles, ft = tile - tt * feat_tiles;     // feature tiles vary fastest: neighbours share tokens
    if (p.tile_group) {
        t.group = p.tile_group[tt];
        t.row0 = p.tile_row0[tt];
        t.n_rows = min(MAX_TOK, p.tile_rows[tt]);
    } else {
        t.group = 0;
        t.row0 = tt * MAX_TOK;
        t.n_rows = min(MAX_TOK, p.M - t.row0);
    }
    t.n_tok = min(MAX_TOK, (max(t.n_rows, 1) + TOK_BOX - 1) / TOK_BOX * TOK_BOX);
    t.f0 = ft * BF;
    return t;
}

template <bool SWIGLU>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a64,
                 const __grid_constant__ CUtensorMap map_a128, const __grid_constant__ CUtensorMap map_w, Tc05Params p) {
    constexpr int STAGE_BYTES = (SWIGLU ? 2 : 1) * W_BYTES + TOK_BYTES;
    constexpr int STAGES = RING_BYTES / STAGE_BYTES;
    constexpr int ACC_COLS = (SWIGLU ? 2 : 1) * MAX_TOK;       // TMEM columns of one accumulator buffer
    constexpr int TMEM_COLS = 2 * ACC_COLS;                      // two buffers
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + STAGES * STAGE_BYTES);
    unsigned long long* empty_bar = full_bar + STAGES;
    unsigned long long* acc_full_bar = empty_bar + STAGES;       // [2]
    unsigned long long* acc_empty_bar = acc_full_bar + 2;        // [2]
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int feat_tiles = (p.N + BF - 1) / BF;
    const int token_tiles = p.tile_group ? *p.n_tiles : (p.M + MAX_TOK - 1) / MAX_TOK;
    const int total_tiles = token_tiles * feat_tiles;
    if ((int)blockIdx.x >= total_tiles) return;                      // the whole CTA leaves before any barrier exists
    const int k_iters = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full_bar[b], 1);
            mbar_init(&acc_empty_bar[b], 4);                         // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                              // stage counter, runs on across tiles
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                const TileInfo t = tile_info<SWIGLU>(p, tile, feat_tiles);
                const unsigned stage_tx = (SWIGLU ? 2 : 1) * W_BYTES + t.n_tok * BK * 2;
                for (int k = 0; k < k_iters; k++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1)) {
                        atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
                        *abort_flag = 1;
                        break;
                    }
                    unsigned char* w_dst = smem + s * STAGE_BYTES;
                    unsigned char* t_dst = w_dst + (SWIGLU ? 2 : 1) * W_BYTES;
                    mbar_expect_tx(&full_bar[s], stage_tx);
                    tma_load_3d(w_dst, &map_w, k * BK, t.f0, t.group, &full_bar[s]);
                    if (SWIGLU) tma_load_3d(w_dst + W_BYTES, &map_w, k * BK, p.N + t.f0, t.group, &full_bar[s]);
                    int r = 0;
                    if (t.n_tok == MAX_TOK) {                          // a full tile: one box of 128 token rows
                        tma_load_2d(t_dst, &map_a128, k * BK, t.row0, &full_bar[s]);
                        r = MAX_TOK;
                    }
                    for (; r + 64 <= t.n_tok; r += 64)                 // boxes of 64 token rows while they fit,
                        tma_load_2d(t_dst + r * BK * 2, &map_a64, k * BK, t.row0 + r, &full_bar[s]);
                    for (; r < t.n_tok; r += TOK_BOX)                  // boxes of 16 for the ragged rest
                        tma_load_2d(t_dst + r * BK * 2, &map_a, k * BK, t.row0 + r, &full_bar[s]);
                }
            }
            if (*abort_flag) {
                // let this CTA's own copies land before its shared memory is given up
                for (int j = max(0, it - STAGES); j < it; j++) mbar_wait(&full_bar[j % STAGES], (j / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, local = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, local++) {
                const TileInfo t = tile_info<SWIGLU>(p, tile, feat_tiles);
                const unsigned idesc = instr_desc(t.n_tok);
                const int buf = local & 1;
                // the epilogue must have emptied this accumulator buffer (two tiles ago)
                if (!mbar_wait(&acc_empty_bar[buf], ((local >> 1) & 1) ^ 1)) {
                    atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const unsigned acc = tmem_base + buf * ACC_COLS;
                for (int k = 0; k < k_iters; k++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
                        atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
                        *abort_flag = 1;
                        break;
                    }
                    tc_fence_after();
                    const unsigned char* w_src = smem + s * STAGE_BYTES;
                    const unsigned char* t_src = w_src + (SWIGLU ? 2 : 1) * W_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; kk++) {
                        const unsigned accum = (k > 0 || kk > 0) ? 1u : 0u;
                        tc_mma(acc, smem_desc(w_src + kk * 32), smem_desc(t_src + kk * 32), idesc, accum);
                        if (SWIGLU) tc_mma(acc + MAX_TOK, smem_desc(w_src + W_BYTES + kk * 32), smem_desc(t_src + kk * 32), idesc, accum);
                    }
                    tc_commit(&empty_bar[s]);                         // the stage is free once these MMAs have read it
                }
                if (*abort_flag) break;
                tc_commit(&acc_full_bar[buf]);                        // the accumulator is complete once all MMAs are done
            }
        }
    } else {
        const int quad = warp & 3;                                   // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, local++) {
            const TileInfo t = tile_info<SWIGLU>(p, tile, feat_tiles);
            const int buf = local & 1;
            const bool ok = !*abort_flag && mbar_wait(&acc_full_bar[buf], (local >> 1) & 1);
            if (!ok) {
                if (lane == 0) {
                    atomicOr(p.status, ESP_STATUS_WAIT_EXPIRED);
                    *abort_flag = 1;
                }
                break;
            }
            tc_fence_after();
            const int f = t.f0 + quad * 32 + lane;                    // this thread's output feature
            const bool f_ok = f < p.N;
            const unsigned lane_addr = tmem_base + buf * ACC_COLS + ((unsigned)(quad * 32) << 16);
            for (int c0 = 0; c0 < t.n_tok; c0 += 32) {
                float acc[32];
                tc_ld32(lane_addr + c0, acc);
                if (SWIGLU) {
                    float up[32];
                    tc_ld32(lane_addr + MAX_TOK + c0, up);
                    bf16* out = reinterpret_cast<bf16*>(p.C);
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        if (f_ok && c0 + i < t.n_rows) {
                            const float v = acc[i] / (1.0f + expf(-acc[i])) * up[i];
                            out[(size_t)(t.row0 + c0 + i) * p.ldc + f] = __float2bfloat16_rn(v);
                        }
                    }
                } else {
                    float* out = reinterpret_cast<float*>(p.C);
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        if (f_ok && c0 + i < t.n_rows) {
                            const float scale = p.row_scale ? p.row_scale[t.row0 + c0 + i] : 1.0f;
                            out[(size_t)(t.row0 + c0 + i) * p.ldc + f] = acc[i] * scale;
                        }
                    }
                }
            }
            // this warp has read its part of the buffer: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// bfloat16 tensor [d2][d1][d0] (d0 innermost), box [1][box1][64], 128-byte swizzle, zero fill out of bounds
int make_map(CUtensorMap* map, const void* base, unsigned long long d0, unsigned long long d1, unsigned long long d2,
             unsigned box1, int rank) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[3] = {d0, d1, d2};
    const cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
    const cuuint32_t box[3] = {BK, box1, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}
}  // namespace

// A [rows_total, K] bfloat16 (row-major, contiguous), W [G, w_rows, K] bfloat16.  Dense: tile_group = null,
// M rows.  Grouped: the token-tile list on the device (tiles of at most 128 rows); ``max_tiles`` bounds
// their number.  swiglu: N is the intermediate size and w_rows = 2N.  K must be a multiple of 8, the
// bases 16-byte aligned.
ESP_API int esp_gemm_tc05(const void* A, long long rows_total, const void* W, int groups, int w_rows,
                          const float* row_scale, void* C, long long ldc, const int* tile_group, const int* tile_row0,
                          const int* tile_rows, const int* n_tiles, int max_tiles, int M, int N, int K, int swiglu,
                          int* status, cudaStream_t stream) {
    if (N <= 0 || K <= 0 || rows_total <= 0) return 0;
    if (K % 8 != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    CUtensorMap map_a, map_a64, map_a128, map_w;
    int rc = make_map(&map_a, A, (unsigned long long)K, (unsigned long long)rows_total, 1, TOK_BOX, 2);
    if (rc) return rc;
    rc = make_map(&map_a64, A, (unsigned long long)K, (unsigned long long)rows_total, 1, 64, 2);
    if (rc) return rc;
    rc = make_map(&map_a128, A, (unsigned long long)K, (unsigned long long)rows_total, 1, MAX_TOK, 2);
    if (rc) return rc;
    // the weights always use a 3-D map so that the kernel has one code path; a dense product is one group
    rc = make_map(&map_w, W, (unsigned long long)K, (unsigned long long)w_rows, (unsigned long long)groups, BF, 3);
    if (rc) return rc;
    Tc05Params p{tile_group, tile_row0, tile_rows, n_tiles, row_scale, C, ldc, M, N, K, status};
    const int token_tiles = tile_group ? max_tiles : (M + MAX_TOK - 1) / MAX_TOK;     // upper bound when grouped
    if (token_tiles <= 0) return 0;
    const long long tiles_bound = (long long)token_tiles * ((N + BF - 1) / BF);
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    const size_t smem = RING_BYTES + 1024 + 256;
    static bool raised[2] = {false, false};
    if (!raised[swiglu ? 1 : 0]) {
        cudaError_t e = swiglu ? cudaFuncSetAttribute(gemm_tc05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                               : cudaFuncSetAttribute(gemm_tc05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised[swiglu ? 1 : 0] = true;
    }
    const int grid = (int)(tiles_bound < sm_count ? tiles_bound : sm_count);
    if (swiglu) gemm_tc05_kernel<true><<<grid, THREADS, smem, stream>>>(map_a, map_a64, map_a128, map_w, p);
    else gemm_tc05_kernel<false><<<grid, THREADS, smem, stream>>>(map_a, map_a64, map_a128, map_w, p);
    return esp_launch_status();
}
