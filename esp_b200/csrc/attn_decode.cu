// Decode attention over the paged bfloat16 cache (pages of 64 positions), split over the keys.
//
// One block = one token row, one key/value head with the query heads that share
// it, and one split of ``split_keys`` consecutive key positions aligned to absolute
// multiples of that number.  The block streams its pages' keys and values once from
// HBM by TMA, keeps scores, softmax and sums in float, and writes an
// unnormalised partial result (running maximum, sum, weighted values) to
// scratch.  The last block of a row to finish combines the row's splits in
// ascending order.  Which splits a row has depends on its position (and window)
// alone, so the result does not depend on the batch around it.
//
// The query at position a sees key j iff j <= a and (window == 0 or a - j < window);
// score = dot(q, k) / sqrt(hd).
#include <cuda.h>

#include "common.cuh"

namespace {
constexpr int THREADS = 128;

// ---- mbarrier helpers (one thread issues the copies, an mbarrier counts their bytes) ---------------------
__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
constexpr unsigned WAIT_LIMIT = 1u << 22;
// Bounded wait for the phase with the given parity; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity) {
    const unsigned addr = smem_addr(bar);
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
constexpr int PAGE_KEYS = 64, RING = 2;

// One block = one token row, one key/value head with the (up to 16) query heads that share it, and one split
// of split_keys key positions, i.e. split_keys / 64 pages.  The pages' keys and values are fetched by TMA into a ring
// of RING shared-memory buffers while earlier pages are being used.  Both products run on the tensor cores
// (mma.sync m16n8k16) with the block's heads as the 16-row operand, so a page costs the same whether one
// head or sixteen read it.  Scores: warp w takes keys 16w..16w+15 of the page, key fragments by ldmatrix.
// Softmax: a running maximum and sum per head, updated page by page in float; warp w owns heads w, w+4, ...;
// probabilities go to shared memory in bfloat16.  Values: warp w takes a quarter of the head's columns,
// value fragments by ldmatrix.trans.  Pages are walked in ascending order, so a row's arithmetic depends on
// its position alone.
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int MMA_HEADS = 16;

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, void* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1) : "memory");
}
// A page's keys (or values) lie in shared memory as HD/64 sub-tiles of 64 rows x 64 columns (128 bytes a
// row), written by TMA with the 128-byte swizzle: the 16-byte piece c of row r sits at piece c ^ (r % 8).
// That makes the 8 rows of an ldmatrix fall into distinct banks.  d is a multiple of 8.
__device__ __forceinline__ const bf16* tile_at(const bf16* tile, int r, int d) {
    return tile + (d >> 6) * (PAGE_KEYS * 64) + r * 64 + ((((d & 63) >> 3) ^ (r & 7)) << 3);
}

template <int HD>
__global__ void __launch_bounds__(THREADS)
attn_split_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const bf16* __restrict__ q, bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                      int* __restrict__ counters, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                      const int* __restrict__ seq_past, const int* __restrict__ block_table, int table_stride, int n_pages,
                      int page, int nh, int nkv, int window, int split_keys, int n_splits, int* __restrict__ status) {
    pdl_trigger();
    constexpr int ITEM = PAGE_KEYS * HD;
    constexpr int NBW = HD / 32;                   // 8-column blocks of the head that one warp accumulates
    constexpr int PLD = PAGE_KEYS + 8;             // row stride of the probabilities (bfloat16)
    extern __shared__ unsigned char dyn_raw[];
    bf16* ring = reinterpret_cast<bf16*>((reinterpret_cast<uintptr_t>(dyn_raw) + 1023) & ~(uintptr_t)1023);   // [RING][ITEM]
    __shared__ __align__(8) unsigned long long full_bar[RING];
    __shared__ float s_s[MMA_HEADS][PAGE_KEYS];
    __shared__ __align__(16) bf16 p_s[MMA_HEADS][PLD];
    __shared__ float m_s[MMA_HEADS], l_s[MMA_HEADS], scale_s[MMA_HEADS];
    __shared__ int item_ok[RING];

    const int n = blockIdx.x, split = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g8 = lane >> 2, tg = lane & 3;
    const int group = nh / nkv, blocks_per_kv = (group + MMA_HEADS - 1) / MMA_HEADS;
    const int kvh = blockIdx.y / blocks_per_kv, h0 = kvh * group + (blockIdx.y % blocks_per_kv) * MMA_HEADS;
    const int heads = min(MMA_HEADS, (kvh + 1) * group - h0);
    const int pos = tok_pos[n], seq = tok_seq[n];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int j0 = max(lo, split * split_keys), j1 = min(pos, split * split_keys + split_keys - 1);
    if (j0 > j1) return;
    const int first_page = j0 / PAGE_KEYS, n_pg = j1 / PAGE_KEYS - first_page + 1, n_items = 2 * n_pg;

    if (tid < MMA_HEADS) {
        m_s[tid] = -INFINITY;
        l_s[tid] = 0.f;
    }
    if (tid == 0) {
        for (int r = 0; r < RING; r++) mbar_init(&full_bar[r], 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    auto issue = [&](int item) {
        const int slot = item % RING;
        int pg = block_table[(size_t)seq * table_stride + first_page + item / 2];
        const bool ok = pg >= 0 && pg < n_pages;
        if (!ok) atomicOr(status, ESP_STATUS_BAD_INDEX);
        item_ok[slot] = ok ? 1 : 0;
        if (ok) {
            const int row0 = (pg * nkv + kvh) * PAGE_KEYS;       // the page's first row in the cache seen as [rows, HD]
            mbar_expect_tx(&full_bar[slot], ITEM * 2);
#pragma unroll
            for (int sub = 0; sub < HD / 64; sub++)
                tma_load_2d(ring + (size_t)slot * ITEM + sub * (PAGE_KEYS * 64), (item & 1) ? &map_v : &map_k, sub * 64, row0,
                            &full_bar[slot]);
        } else {
            mbar_arrive(&full_bar[slot]);
        }
    };
    // Keys and values that were cached before this step do not depend on the kernel before this one (which
    // writes the step's new keys and values): a block all of whose positions are old asks for its first pages
    // at once and only then waits for that kernel, whose queries it needs.  ``seq_past`` (may be null): per
    // sequence, the positions cached before the step.
    const bool early = seq_past != nullptr && j1 < seq_past[seq];
    int issued = 0;
    if (early && tid == 0) {
        for (; issued < min(RING, n_items); issued++) issue(issued);
    }
    pdl_wait();
    // the query fragments of the block's heads (rows beyond ``heads`` are zero)
    unsigned qa[HD / 16][4];
    {
        const bf16* q0 = q + ((size_t)n * nh + h0 + g8) * HD;
        const bf16* q1 = q + ((size_t)n * nh + h0 + g8 + 8) * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) {
            const int c = kk * 16 + tg * 2;
            qa[kk][0] = g8 < heads ? *reinterpret_cast<const unsigned*>(q0 + c) : 0u;
            qa[kk][1] = g8 + 8 < heads ? *reinterpret_cast<const unsigned*>(q1 + c) : 0u;
            qa[kk][2] = g8 < heads ? *reinterpret_cast<const unsigned*>(q0 + c + 8) : 0u;
            qa[kk][3] = g8 + 8 < heads ? *reinterpret_cast<const unsigned*>(q1 + c + 8) : 0u;
        }
    }
    __syncthreads();
    if (!early && tid == 0) {
        for (; issued < min(RING, n_items); issued++) issue(issued);
    }

    const float root = sqrtf((float)HD);
    float o[NBW][4];
#pragma unroll
    for (int i = 0; i < NBW; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o[i][j] = 0.f;
    bool failed = false;

    for (int pi = 0; pi < n_pg; pi++) {
        const int key0 = (first_page + pi) * PAGE_KEYS;
        const int item_k = 2 * pi, slot_k = item_k % RING;
        if (__syncthreads_or(!mbar_wait(&full_bar[slot_k], (item_k / RING) & 1))) { failed = true; break; }
        const bf16* kp = ring + (size_t)slot_k * ITEM;
        const bool page_ok = item_ok[slot_k] != 0;
        // ---- scores of keys 16*warp .. 16*warp+15 for all heads
        float sc[2][4];
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) sc[i][j] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) {
            unsigned kf[4];
            ldsm_x4(kf, tile_at(kp, warp * 16 + (lane & 7) + (lane >> 4) * 8, kk * 16 + ((lane >> 3) & 1) * 8));
            mma_16816(sc[0], qa[kk], kf[0], kf[1]);
            mma_16816(sc[1], qa[kk], kf[2], kf[3]);
        }
#pragma unroll
        for (int nb = 0; nb < 2; nb++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int t = warp * 16 + nb * 8 + tg * 2 + (j & 1), key = key0 + t;
                const bool live = page_ok && key >= j0 && key <= j1;
                if (g8 + (j >> 1) * 8 < heads) s_s[g8 + (j >> 1) * 8][t] = live ? sc[nb][j] / root : -INFINITY;
            }
        __syncthreads();                           // scores are written; the key buffer is free
        if (tid == 0 && issued < n_items) issue(issued++);
        // ---- running maximum and sum: warp w owns heads w, w+4, w+8, w+12
        for (int h = warp; h < heads; h += 4) {   // rows beyond ``heads`` feed accumulator rows that are never stored
            const float a = s_s[h][lane], b = s_s[h][lane + 32];
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, warp_max(fmaxf(a, b)));
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float pa = a == -INFINITY ? 0.f : expf(a - m_use), pb = b == -INFINITY ? 0.f : expf(b - m_use);
            const float sum = warp_sum(pa + pb);
            p_s[h][lane] = __float2bfloat16_rn(pa);
            p_s[h][lane + 32] = __float2bfloat16_rn(pb);
            if (lane == 0) {
                const float scale = expf(m_old - m_use);
                scale_s[h] = scale;
                l_s[h] = l_s[h] * scale + sum;
                m_s[h] = m_new;
            }
        }
        // ---- weighted values: this warp's quarter of the columns
        const int item_v = 2 * pi + 1, slot_v = item_v % RING;
        if (__syncthreads_or(!mbar_wait(&full_bar[slot_v], (item_v / RING) & 1))) { failed = true; break; }
        const bf16* vp = ring + (size_t)slot_v * ITEM;
        const float sc_lo = scale_s[g8], sc_hi = scale_s[g8 + 8];
#pragma unroll
        for (int i = 0; i < NBW; i++) {
            o[i][0] *= sc_lo;
            o[i][1] *= sc_lo;
            o[i][2] *= sc_hi;
            o[i][3] *= sc_hi;
        }
        if (item_ok[slot_v]) {
#pragma unroll
            for (int kt = 0; kt < PAGE_KEYS / 16; kt++) {
                unsigned pf[4];
                ldsm_x4(pf, &p_s[lane & 15][kt * 16 + (lane >> 4) * 8]);
#pragma unroll
                for (int nb2 = 0; nb2 < NBW / 2; nb2++) {
                    unsigned vf[4];
                    ldsm_x4_trans(vf, tile_at(vp, kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                              warp * (HD / 4) + nb2 * 16 + (lane >> 4) * 8));
                    mma_16816(o[2 * nb2], pf, vf[0], vf[1]);
                    mma_16816(o[2 * nb2 + 1], pf, vf[2], vf[3]);
                }
            }
        }
        __syncthreads();                           // the value buffer, the scores and the probabilities are free
        if (tid == 0 && issued < n_items) issue(issued++);
    }
    if (failed) {
        // A wait ran out: flag it, let the copies in flight land, and still take part in the row's count below
        // with an empty partial (maximum -inf, sum 0), so that the counter returns to zero and the row's last
        // block finishes.  The row's output is then incomplete, which the status word tells the host.
        if (tid == 0) {
            atomicOr(status, ESP_STATUS_WAIT_EXPIRED);
            for (int it = max(0, issued - RING); it < issued; it++) mbar_wait(&full_bar[it % RING], (it / RING) & 1);
        }
        if (tid < heads) {
            m_s[tid] = -INFINITY;
            l_s[tid] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < NBW; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) o[i][j] = 0.f;
        __syncthreads();
    }
    // ---- partial results: rows g8 and g8+8, this warp's columns
#pragma unroll
    for (int i = 0; i < NBW; i++) {
        const int d = warp * (HD / 4) + i * 8 + tg * 2;
        if (g8 < heads) {
            float* po = part_o + (((size_t)n * nh + h0 + g8) * n_splits + split) * HD + d;
            po[0] = o[i][0];
            po[1] = o[i][1];
        }
        if (g8 + 8 < heads) {
            float* po = part_o + (((size_t)n * nh + h0 + g8 + 8) * n_splits + split) * HD + d;
            po[0] = o[i][2];
            po[1] = o[i][3];
        }
    }
    if (tid < heads) {
        float* ml = part_ml + (((size_t)n * nh + h0 + tid) * n_splits + split) * 2;
        ml[0] = m_s[tid];
        ml[1] = l_s[tid];
    }
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    const int s0 = lo / split_keys, s1 = pos / split_keys;
    if (tid == 0) {
        int* c = counters + (size_t)n * gridDim.y + blockIdx.y;
        const int done = atomicAdd(c, 1);
        is_last = done == s1 - s0;
        if (is_last) *c = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // The row's splits: a warp takes a head at a time.  The weight exp(m - max) and the sum of every split are worked
    // out once, a lane each, into the page buffers (free by now); then each lane adds up its columns over the splits
    // in ascending order, several loads in flight, so a result does not depend on how the work is shared out.
    constexpr int WCH = RING * ITEM * (int)sizeof(bf16) / ((THREADS / 32) * 2 * (int)sizeof(float));   // splits a pass
    constexpr int NV = HD / 64;                             // pairs of columns per lane: 64 j + 2 lane, + 1
    float* w_w = reinterpret_cast<float*>(ring) + (size_t)warp * 2 * WCH;
    float* l_w = w_w + WCH;
    for (int g = warp; g < heads; g += THREADS / 32) {
        const float* ml = part_ml + ((size_t)n * nh + h0 + g) * n_splits * 2;
        const float* po = part_o + ((size_t)n * nh + h0 + g) * n_splits * HD;
        float mx = -INFINITY;
        for (int sp = s0 + lane; sp <= s1; sp += 32) mx = fmaxf(mx, __ldcg(ml + 2 * sp));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        float denom = 0.f, num[NV][2];
#pragma unroll
        for (int j = 0; j < NV; j++) num[j][0] = num[j][1] = 0.f;
        for (int c0 = s0; c0 <= s1; c0 += WCH) {
            const int cn = min(WCH, s1 + 1 - c0);
            __syncwarp();                                  // the pass (or head) before this one has been read
            for (int i = lane; i < cn; i += 32) {
                const float m_sp = __ldcg(ml + 2 * (c0 + i));
                w_w[i] = m_sp == -INFINITY ? 0.f : expf(m_sp - mx);
                l_w[i] = __ldcg(ml + 2 * (c0 + i) + 1);
            }
            __syncwarp();
            const float* pc = po + (size_t)c0 * HD + lane * 2;
#pragma unroll 8
            for (int i = 0; i < cn; i++) {
                const float w = w_w[i];
                denom += l_w[i] * w;
#pragma unroll
                for (int j = 0; j < NV; j++) {
                    const float2 v = __ldcg(reinterpret_cast<const float2*>(pc + (size_t)i * HD + j * 64));
                    num[j][0] += v.x * w;
                    num[j][1] += v.y * w;
                }
            }
        }
        bf16* orow = out + ((size_t)n * nh + h0 + g) * HD + lane * 2;
#pragma unroll
        for (int j = 0; j < NV; j++)
            *reinterpret_cast<__nv_bfloat162*>(orow + j * 64) =
                __nv_bfloat162(__float2bfloat16_rn(denom > 0.f ? num[j][0] / denom : 0.f),
                               __float2bfloat16_rn(denom > 0.f ? num[j][1] / denom : 0.f));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The cache of one layer seen as a matrix [pages * kv heads * 64 rows, hd]; boxes of 64 rows x 64 columns.
int make_cache_map(CUtensorMap* map, const void* base, unsigned long long rows, int hd) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return (int)cudaErrorNotSupported;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    const cuuint64_t dims[2] = {(cuuint64_t)hd, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    const cuuint32_t box[2] = {64, PAGE_KEYS};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int HD>
int launch_split_mma(int split, const bf16* q, const bf16* k, const bf16* v, bf16* out, float* po, float* pml, int* counters,
                     const int* tok_seq, const int* tok_pos, const int* seq_past, const int* table, int stride, int n_pages, int page,
                     int n_tokens, int nh, int nkv, int window, int n_splits, int* status, cudaStream_t stream) {
    CUtensorMap map_k, map_v;
    const unsigned long long rows = (unsigned long long)n_pages * nkv * PAGE_KEYS;
    int rc = make_cache_map(&map_k, k, rows, HD);
    if (rc) return rc;
    rc = make_cache_map(&map_v, v, rows, HD);
    if (rc) return rc;
    const size_t dyn = (size_t)RING * PAGE_KEYS * HD * sizeof(bf16) + 1024;
    static bool raised[64] = {false};              // per device: the attribute belongs to the device's context
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
    if (!raised[device]) {
        cudaError_t e = cudaFuncSetAttribute(attn_split_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
        if (e != cudaSuccess) return (int)e;
        raised[device] = true;
    }
    const int group = nh / nkv;
    dim3 grid(n_tokens, nkv * ((group + MMA_HEADS - 1) / MMA_HEADS), n_splits);
    esp_launch_pdl(ESP_PDL_ATTENTION, attn_split_mma_kernel<HD>, dim3(grid), dim3(THREADS), dyn, stream, map_k, map_v, q, out, po, pml,
                   counters, tok_seq, tok_pos, seq_past, table, stride, n_pages, page, nh, nkv, window, split, n_splits, status);
    return esp_launch_status();
}
}  // namespace

// Scratch: part_o float [n_tokens, nh, n_splits, hd], part_ml float [n_tokens, nh, n_splits, 2];
// counters int [n_tokens * head groups], all zero when the call starts (the kernel leaves them zero);
// split: key positions per block, a multiple of 64 (the caller picks: short splits when there are few rows, so
// that every SM still gets blocks); n_splits >= ceil(longest sequence / split).  Head sizes 64, 128, 192, 256; pages of 64 positions or any
// size; any head counts with nh % nkv == 0.  ``seq_past`` (may be null): per sequence of the step, the positions
// that were cached before it; with it, blocks whose keys are all older start their loads without waiting for the
// kernel before this one.
ESP_API int esp_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o,
                            float* part_ml, int* counters, const int* tok_seq, const int* tok_pos, const int* seq_past,
                            const int* block_table, int table_stride, int n_pages, int page, int n_tokens, int nh, int nkv,
                            int hd, int window, int split, int n_splits, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || n_splits <= 0 || n_splits > 65535 || nh > 65535 || split < PAGE_KEYS || split % PAGE_KEYS != 0 ||
        page != PAGE_KEYS)
        return (int)cudaErrorInvalidValue;
#define ESP_HD(HD) return launch_split_mma<HD>(split, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, part_o, \
                                               part_ml, counters, tok_seq, tok_pos, seq_past, block_table, table_stride, n_pages, \
                                               page, n_tokens, nh, nkv, window, n_splits, status, stream)
    switch (hd) {
        case 64: ESP_HD(64);
        case 128: ESP_HD(128);
        case 192: ESP_HD(192);
        case 256: ESP_HD(256);
    }
#undef ESP_HD
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------------------------------
// The same attention for callers that must not allocate (see attn_decode_noalloc.h).
// ---------------------------------------------------------------------------------------------------
#include "attn_decode_noalloc.h"

// Scratch of the no-allocation entry point.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer that a kernel may be given.
static __device__ __align__(256) float esp_noalloc_scratch[ESP_ATTN_DECODE_NOALLOC_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* noalloc_scratch_of_device[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace

// The last ESP_NOALLOC_COUNTERS words of the array are the kernel's (row, head group) counters.  They sit at a
// fixed place so that no call's partial results are ever written over them: they must read zero when a
// call starts, and every call leaves them zero.
extern "C" long long esp_attn_decode_noalloc_capacity(void) {
    return (long long)ESP_ATTN_DECODE_NOALLOC_FLOATS - ESP_NOALLOC_COUNTERS;
}

extern "C" int esp_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                       const int* tok_seq, const int* tok_pos, const int* block_table, int table_stride,
                                       int n_pages, int page, int n_tokens, int nh, int nkv, int hd, int window,
                                       int split, int n_splits, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || hd <= 0 || n_splits <= 0 || nkv <= 0) return (int)cudaErrorInvalidValue;
    const unsigned long long need = (unsigned long long)n_tokens * nh * n_splits * (hd + 2);
    if (need > (unsigned long long)esp_attn_decode_noalloc_capacity() ||
        (unsigned long long)n_tokens * nh > ESP_NOALLOC_COUNTERS)
        return ESP_NOALLOC_TOO_LARGE;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= NOALLOC_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    if (!noalloc_scratch_of_device[device]) {
        // first call on this device: turn the symbol into the address that kernels can use
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, esp_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        noalloc_scratch_of_device[device] = ptr;
    }
    float* part_o = noalloc_scratch_of_device[device];
    float* part_ml = part_o + (size_t)n_tokens * nh * n_splits * hd;
    int* counters = reinterpret_cast<int*>(noalloc_scratch_of_device[device] + esp_attn_decode_noalloc_capacity());
    return esp_attn_decode(q, k_cache, v_cache, out, part_o, part_ml, counters, tok_seq, tok_pos, nullptr, block_table, table_stride,
                           n_pages, page, n_tokens, nh, nkv, hd, window, split, n_splits, status, stream);
}
