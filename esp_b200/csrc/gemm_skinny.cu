// Weight-streaming matrix product for a handful of rows (decode):
//   C[m, n] = scale[m] * sum_k A[row(m), k] * W[g][n, k]          (PLAIN)
//   act[m, j] = silu(A W_gate[j]) * (A W_up[j])                   (SWIGLU; W = [gate rows; up rows])
//   q / k / v of a decode step: the packed q/k/v projection whose epilogue adds the bias, rotates queries and
//   keys by the token's position (split-half pairs (i, i + hd/2)) and writes the keys and values into the
//   paged cache                                                  (ROPE; a tile holds 8 pairs)
// bfloat16 operands, float accumulation on the tensor cores (mma.sync
// m16n8k16 with the weight rows as the 16-row operand and up to 8 tokens as the
// 8-column operand, so a step with few rows wastes no tensor work and every
// weight byte is read from HBM exactly once).  The kernel is bound by the
// weight stream: each lane loads 16 contiguous bytes of a weight row straight
// into its fragment registers (no shared-memory staging), with a permutation
// of k inside each group of 32 that the activation fragment mirrors.
//
// One block = one tile of 16 weight rows (PLAIN) or 8 gate + 8 up rows
// (SWIGLU) and, in the grouped form, one group (expert).  Its 8 warps split K
// into 8 slices and their partial sums are added in warp order, so a result
// does not depend on anything but its own row and weights.  Activation rows of
// the block's group are staged in shared memory (gathered through ``a_rows``),
// 8 * NBLK rows at a time.
#include "common.cuh"
#include <cmath>

namespace {
constexpr int WARPS = 8;
// 16-byte pieces of each of its two weight rows that a lane has in flight, and blocks per SM.  Measured on the
// 24-layer decode step: 4 pieces and 3 blocks beat 8 and 2, 6 and 2, 2 and 4 at batch 1 and at batch 8.
constexpr int UNROLL = 4;
#define ESP_SKINNY_BLOCKS 3

struct SkinnyParams {
    const bf16* W;
    long long w_group_stride;       // elements between groups
    const bf16* A;
    long long lda;
    const int* a_rows;
    const int* group_offsets;
    const float* row_scale;
    void* C;
    long long ldc;
    int M, N, K;
    int groups;                     // grouped form: how many groups there are (the grid's y may be smaller)
    int offsets_ready;              // grouped form: the offsets were complete before the kernel before this one started
    // ROPE form only: N counts pairs (i, i + hd/2) over the nh + 2 nkv heads of the packed projection
    const float* bias;              // [(nh + 2 nkv) * hd] or null
    const int* tok_seq;
    const int* tok_pos;
    const float* cos_t;             // [max_pos, hd / 2]
    const float* sin_t;
    void* q_out;                    // [M, nh * hd] bfloat16
    void* k_cache;                  // [pages, nkv, page, hd] bfloat16
    void* v_cache;
    const int* block_table;
    int table_stride, n_pages, page, nh, nkv, hd, max_pos, write_kv;
    int* status;
};

enum : int { MODE_PLAIN = 0, MODE_SWIGLU = 1, MODE_ROPE = 2 };

// One pair (x[i], x[i + hd/2]) of head ``head`` of token row m: bias, rotation in float with the same
// operations in the same order as the separate kernel (rope_kv.cu), then the query row or the cache.
__device__ __forceinline__ void emit_rope_pair(const SkinnyParams& p, int m, int pair, float lo, float hi) {
    const int half = p.hd / 2, head = pair / half, i = pair - head * half;
    if (p.bias) {
        lo += p.bias[(size_t)head * p.hd + i];
        hi += p.bias[(size_t)head * p.hd + i + half];
    }
    const int pos = p.tok_pos[m];
    if (pos < 0 || pos >= p.max_pos) {
        atomicOr(p.status, ESP_STATUS_BAD_INDEX);
        return;
    }
    float ol = lo, oh = hi;
    if (head < p.nh + p.nkv) {                       // queries and keys rotate, values do not
        const float c = p.cos_t[(size_t)pos * half + i], sn = p.sin_t[(size_t)pos * half + i];
        ol = lo * c - hi * sn;
        oh = hi * c + lo * sn;
    }
    bf16* dst = nullptr;
    if (head < p.nh) {
        dst = reinterpret_cast<bf16*>(p.q_out) + ((size_t)m * p.nh + head) * p.hd;
    } else if (p.write_kv) {
        const int page_id = p.block_table[(size_t)p.tok_seq[m] * p.table_stride + pos / p.page];
        if (page_id < 0 || page_id >= p.n_pages) {
            atomicOr(p.status, ESP_STATUS_BAD_INDEX);
            return;
        }
        const bool is_k = head < p.nh + p.nkv;
        const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
        dst = reinterpret_cast<bf16*>(is_k ? p.k_cache : p.v_cache) +
              (((size_t)page_id * p.nkv + kvh) * p.page + pos % p.page) * p.hd;
    }
    if (dst) {
        dst[i] = __float2bfloat16_rn(ol);
        dst[i + half] = __float2bfloat16_rn(oh);
    }
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream(const bf16* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}

// KS: how many of the block's 8 warps share one tile of weight rows, each with its own slice of K (8 / KS
// tiles per block).  Few tiles: KS = 8, so that every SM still gets work; many tiles: KS = 1, each warp
// walks all of K of its own tile (longer streams per warp, no reduction between warps); 2 and 4 lie between.
template <int NBLK, int MODE, typename TC, int KS>
__global__ void __launch_bounds__(WARPS * 32, ESP_SKINNY_BLOCKS)
gemm_skinny_kernel(SkinnyParams p) {
    constexpr bool SWIGLU = MODE == MODE_SWIGLU, ROPE = MODE == MODE_ROPE, PAIRS = SWIGLU || ROPE;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = p.K;
    const int a_stride = K + 32;                                    // elements; 64 bytes of padding per row
    bf16* a_s = reinterpret_cast<bf16*>(smem_raw);                   // [8*NBLK][a_stride]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)8 * NBLK * a_stride * sizeof(bf16));   // [WARPS][NBLK][32][4]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
    int m_begin = 0, m_end = p.M;
    const bf16* W = p.W;
    // The next kernel may be set up as soon as every block has said so.  A dense product says so at once; a grouped
    // one only when its weights have been streamed, so that a dependent launch takes SM room from its last blocks,
    // not from the waves that have yet to start.
    if (!p.group_offsets) pdl_trigger();
    if (p.group_offsets) {
        if (!p.offsets_ready) pdl_wait();                             // which group a block takes was written by the kernel before
        int group = blockIdx.y;
        if ((int)gridDim.y < p.groups) {
            // fewer rows than groups (a decode step of one sequence names a few experts of many): the grid has
            // one y per row, and y takes the group whose first row is row y; the other blocks leave at once
            int* found = reinterpret_cast<int*>(smem_raw);            // read by all before the first rows are staged there
            if (tid == 0) *found = -1;
            __syncthreads();
            for (int e = tid; e < p.groups; e += WARPS * 32)
                if (p.group_offsets[e] == (int)blockIdx.y && p.group_offsets[e + 1] > (int)blockIdx.y) *found = e;
            __syncthreads();
            group = *found;
            if (group < 0) return;
        }
        m_begin = p.group_offsets[group];
        m_end = p.group_offsets[group + 1];
        W += (size_t)group * p.w_group_stride;
    }
    if (m_begin >= m_end) return;

    // the two weight rows this lane streams
    int row_a, row_b;
    bool ok_a, ok_b;
    constexpr int TILES = WARPS / KS;              // tiles of weight rows per block
    const int tile = blockIdx.x * TILES + warp / KS, kslice = warp % KS;
    if (ROPE) {
        // pair j of the packed projection: feature i of head ``head`` and its partner half a head further
        const int j = tile * 8 + g, half = p.hd / 2, head = j / half;
        ok_a = ok_b = j < p.N;
        row_a = head * p.hd + (j - head * half);
        row_b = row_a + half;
    } else if (SWIGLU) {
        const int j = tile * 8 + g;
        ok_a = ok_b = j < p.N;
        row_a = j;
        row_b = p.N + j;
    } else {
        row_a = tile * 16 + g;
        row_b = row_a + 8;
        ok_a = row_a < p.N;
        ok_b = row_b < p.N;
    }
    const bf16* wa_ptr = W + (size_t)(ok_a ? row_a : 0) * K;
    const bf16* wb_ptr = W + (size_t)(ok_b ? row_b : 0) * K;
    // K slice of this warp, in whole groups of 32
    const int groups32 = (K + 31) / 32;
    const int per_warp = (groups32 + KS - 1) / KS;
    const int k_lo = min(K, kslice * per_warp * 32);
    const int k_hi = min(K, (kslice + 1) * per_warp * 32);

    // The first pieces of the weight rows are asked for before the activation rows are staged: the two trips to
    // memory (rows from L2, weights from DRAM) then run side by side, which is most of what a short product
    // (K / KS of a few hundred) takes.
    uint4 wa[UNROLL], wb[UNROLL];
    auto load_weights = [&](int k0) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int k = k0 + u * 32 + tg * 8;
            const bool in = k < k_hi;                                 // K is a multiple of 8: a piece is whole or absent
            wa[u] = (in && ok_a) ? load_stream(wa_ptr + k) : make_uint4(0, 0, 0, 0);
            wb[u] = (in && ok_b) ? load_stream(wb_ptr + k) : make_uint4(0, 0, 0, 0);
        }
    };
    load_weights(k_lo);
    if (!p.group_offsets) {
        // The dense form knows its weights without the kernel before it: besides the first pieces, the lines
        // that follow them (up to 1 KB of each row) are asked into L2, so that the weight stream is under way
        // while the predecessor finishes; then wait for the predecessor, whose output the rows below are.
        const int pre_hi = min(k_hi, k_lo + 32 * UNROLL + 512);
        for (int k = k_lo + 32 * UNROLL + tg * 64; k < pre_hi; k += 256) {
            if (ok_a) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wa_ptr + k));
            if (ok_b) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wb_ptr + k));
        }
        pdl_wait();
    } else if (p.offsets_ready) {
        // a grouped product whose groups were known before its predecessor started (the experts' second product):
        // group, weights' first pieces and all, before the wait; only the rows below are the predecessor's
        pdl_wait();
    }

    for (int m0 = m_begin; m0 < m_end; m0 += 8 * NBLK) {
        const int cnt = min(8 * NBLK, m_end - m0);
        __syncthreads();                                              // the previous chunk's readers are done
        // stage the activation rows (16-byte pieces), zero rows beyond cnt
        const int pieces = K / 8;
        for (int idx = tid; idx < 8 * NBLK * pieces; idx += WARPS * 32) {
            const int r = idx / pieces, q = idx - r * pieces;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < cnt) {
                const int src = p.a_rows ? p.a_rows[m0 + r] : (m0 + r);
                v = *reinterpret_cast<const uint4*>(p.A + (size_t)src * p.lda + q * 8);
            }
            *reinterpret_cast<uint4*>(a_s + (size_t)r * a_stride + q * 8) = v;
        }
        __syncthreads();

        float acc[NBLK][4];
#pragma unroll
        for (int nb = 0; nb < NBLK; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[nb][i] = 0.f;

        for (int k0 = k_lo; k0 < k_hi; k0 += 32 * UNROLL) {
            if (k0 != k_lo || m0 != m_begin) load_weights(k0);        // the very first pieces are on their way already
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const int k = k0 + u * 32 + tg * 8;
                if (k0 + u * 32 >= k_hi) break;
#pragma unroll
                for (int nb = 0; nb < NBLK; nb++) {
                    if (nb * 8 >= cnt) break;
                    uint4 av = make_uint4(0, 0, 0, 0);
                    if (k < k_hi) av = *reinterpret_cast<const uint4*>(a_s + (size_t)(nb * 8 + g) * a_stride + k);
                    mma_bf16(acc[nb], wa[u].x, wb[u].x, wa[u].y, wb[u].y, av.x, av.y);
                    mma_bf16(acc[nb], wa[u].z, wb[u].z, wa[u].w, wb[u].w, av.z, av.w);
                }
            }
        }
        if (p.group_offsets && m0 + 8 * NBLK >= m_end) pdl_trigger();   // the weights are in: see the top
        if constexpr (KS == 1) {
            // this warp owns its tile: results go out straight from the accumulators
#pragma unroll
            for (int nb = 0; nb < NBLK; nb++) {
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int tok = nb * 8 + tg * 2 + i;
                    if (tok >= cnt) continue;
                    if (ROPE) {
                        const int j = tile * 8 + g;
                        if (j < p.N) emit_rope_pair(p, m0 + tok, j, acc[nb][i], acc[nb][2 + i]);
                    } else if (SWIGLU) {
                        const int j = tile * 8 + g;
                        if (j < p.N) {
                            const float gate = acc[nb][i], up = acc[nb][2 + i];
                            reinterpret_cast<TC*>(p.C)[(size_t)(m0 + tok) * p.ldc + j] =
                                from_f32<TC>(gate / (1.0f + expf(-gate)) * up);
                        }
                    } else {
                        const float scale = p.row_scale ? p.row_scale[m0 + tok] : 1.0f;
                        const int n_lo = tile * 16 + g, n_hi = n_lo + 8;
                        if (n_lo < p.N) reinterpret_cast<TC*>(p.C)[(size_t)(m0 + tok) * p.ldc + n_lo] = from_f32<TC>(acc[nb][i] * scale);
                        if (n_hi < p.N) reinterpret_cast<TC*>(p.C)[(size_t)(m0 + tok) * p.ldc + n_hi] = from_f32<TC>(acc[nb][2 + i] * scale);
                    }
                }
            }
        } else {
        // partial sums of the KS warps of a tile, added in warp order
#pragma unroll
        for (int nb = 0; nb < NBLK; nb++)
            *reinterpret_cast<float4*>(red + (((size_t)warp * NBLK + nb) * 32 + lane) * 4) =
                make_float4(acc[nb][0], acc[nb][1], acc[nb][2], acc[nb][3]);
        __syncthreads();
        if (PAIRS) {
            for (int e = tid; e < TILES * NBLK * 64; e += WARPS * 32) {
                const int tl = e / (NBLK * 64), rem = e % (NBLK * 64);
                const int nb = rem / 64, ln = (rem % 64) / 2, i = rem & 1;
                float gate = 0.f, up = 0.f;
#pragma unroll
                for (int w = 0; w < KS; w++) {
                    gate += red[(((size_t)(tl * KS + w) * NBLK + nb) * 32 + ln) * 4 + i];
                    up += red[(((size_t)(tl * KS + w) * NBLK + nb) * 32 + ln) * 4 + 2 + i];
                }
                const int tok = nb * 8 + (ln & 3) * 2 + i, j = (blockIdx.x * TILES + tl) * 8 + (ln >> 2);
                if (tok < cnt && j < p.N) {
                    if (ROPE) {
                        emit_rope_pair(p, m0 + tok, j, gate, up);
                    } else {
                        const float v = gate / (1.0f + expf(-gate)) * up;
                        reinterpret_cast<TC*>(p.C)[(size_t)(m0 + tok) * p.ldc + j] = from_f32<TC>(v);
                    }
                }
            }
        } else {
            for (int e = tid; e < TILES * NBLK * 128; e += WARPS * 32) {
                const int tl = e / (NBLK * 128), rem = e % (NBLK * 128);
                const int nb = rem / 128, ln = (rem % 128) / 4, i = rem & 3;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < KS; w++) v += red[(((size_t)(tl * KS + w) * NBLK + nb) * 32 + ln) * 4 + i];
                const int tok = nb * 8 + (ln & 3) * 2 + (i & 1);
                const int n = (blockIdx.x * TILES + tl) * 16 + (ln >> 2) + (i >= 2 ? 8 : 0);
                if (tok < cnt && n < p.N) {
                    if (p.row_scale) v *= p.row_scale[m0 + tok];
                    reinterpret_cast<TC*>(p.C)[(size_t)(m0 + tok) * p.ldc + n] = from_f32<TC>(v);
                }
            }
        }
        }
    }
}

template <int NBLK, int MODE, typename TC, int KS>
int launch_variant(const SkinnyParams& p, int groups, int tiles, cudaStream_t stream) {
    const size_t smem = (size_t)8 * NBLK * (p.K + 32) * sizeof(bf16) + (size_t)WARPS * NBLK * 32 * 4 * sizeof(float);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    static bool raised = false;        // per instantiation
    if (smem > 48 * 1024 && !raised) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<NBLK, MODE, TC, KS>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    constexpr int TILES = WARPS / KS;
    dim3 grid((tiles + TILES - 1) / TILES, p.group_offsets && p.M < groups ? p.M : groups);   // every group that has rows starts below M
    // A grouped product set up early holds SM room while it waits for the routing, room that the shared expert's
    // products on the second stream want: measured, it costs 1 to 5 % of a step of 3 to 8 tokens.  A short one (a few
    // rows, a grid that fits the device at once, at most 128 MB of weights) gains by it: 3 % of the step at one and
    // two tokens with 46 MB an expert set; with 293 MB (eight experts of 2560 x 3584) it lost 1.5 %.
    const long long weight_bytes = (long long)p.M * (MODE == MODE_SWIGLU ? 2 : 1) * p.N * p.K * (long long)sizeof(bf16);
    const bool fits = p.M <= 8 && (long long)grid.x * grid.y <= 148 * ESP_SKINNY_BLOCKS && weight_bytes <= (128ll << 20);
    const int kind = !p.group_offsets ? ESP_PDL_DENSE : p.offsets_ready ? ESP_PDL_GROUPED_AFTER
                     : fits && esp_pdl_enabled(ESP_PDL_GROUPED_FITS) ? ESP_PDL_GROUPED_FITS : ESP_PDL_GROUPED;
    esp_launch_pdl(kind, gemm_skinny_kernel<NBLK, MODE, TC, KS>, grid, dim3(WARPS * 32), smem, stream, p);
    return esp_launch_status();
}

template <int NBLK, int MODE, typename TC>
int launch(const SkinnyParams& p, int groups, cudaStream_t stream) {
    const int tiles = MODE != MODE_PLAIN ? (p.N + 7) / 8 : (p.N + 15) / 16;
    // warps wanted: about a dozen per SM.  The fewer tiles there are, the more warps share one.
    const long long spread = (long long)tiles * (p.group_offsets ? (groups < p.M ? groups : p.M) : 1);
    constexpr int SLOTS = 12;      // measured: 8 and 16 were slower at batch 8, 24 slower at batch 1
    // a warp takes a tile all by itself only with several waves of tiles (measured: batch 1 gains 4 % over a
    // limit of 12, batch 8 and 64 are the same)
    // one wave: with a warp per tile the launch has about as many blocks as the device holds at once (three per
    // SM), so no second, partly filled wave follows (the down-projection of 32 (token, expert) rows: 512 blocks
    // of which three quarters have an expert; batch 8 4.11 -> 4.03 ms a step)
    // Blocks of a grid row without a group end at once, so what counts against the device's room is the
    // number of groups with rows: unknown here, expected groups * (1 - (1 - 1/groups)^rows) for rows drawn
    // evenly (24 rows over 60 groups: 19.9 expected, 19.1 measured with random weights).  Measured: 24 rows of the
    // gate/up product (438 expected blocks) gain 2 % of the step this way, 28 rows (495) lose 1 %.
    const long long blocks_x = (tiles + WARPS - 1) / WARPS;
    const long long blocks1 = blocks_x * (p.group_offsets ? (groups < p.M ? groups : p.M) : 1);
    const double with_rows = p.group_offsets ? groups * (1.0 - pow(1.0 - 1.0 / groups, (double)p.M)) : 1.0;
    if (p.group_offsets && blocks1 >= 148 * 2 && blocks_x * with_rows <= 148 * ESP_SKINNY_BLOCKS + 148 / 8)
        return launch_variant<NBLK, MODE, TC, 1>(p, groups, tiles, stream);
    if (spread >= 148 * 48) return launch_variant<NBLK, MODE, TC, 1>(p, groups, tiles, stream);
    if (spread * 2 >= 148 * SLOTS) return launch_variant<NBLK, MODE, TC, 2>(p, groups, tiles, stream);
    if (spread * 4 >= 148 * SLOTS) return launch_variant<NBLK, MODE, TC, 4>(p, groups, tiles, stream);
    return launch_variant<NBLK, MODE, TC, 8>(p, groups, tiles, stream);
}
}  // namespace

// ``max_rows``: an upper bound of the rows of any one group (of M when dense); it
// selects how many rows are staged at a time.  swiglu: N is the intermediate
// size and W holds 2N rows per group.  c_dtype: 0 float, 1 bfloat16.
ESP_API int esp_gemm_skinny(const void* A, long long lda, const int* a_rows, const void* W, long long w_group_stride,
                            const float* row_scale, void* C, int c_dtype, long long ldc, const int* group_offsets,
                            int groups, int M, int N, int K, int max_rows, int swiglu, int offsets_ready, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K % 8 != 0 || lda % 8 != 0 || groups > 65535) return (int)cudaErrorInvalidValue;
    SkinnyParams p{};
    p.offsets_ready = group_offsets && offsets_ready ? 1 : 0;
    p.W = (const bf16*)W; p.w_group_stride = w_group_stride; p.A = (const bf16*)A; p.lda = lda; p.a_rows = a_rows;
    p.group_offsets = group_offsets; p.row_scale = row_scale; p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K;
    p.groups = groups;
    const int g = group_offsets ? groups : 1;
    const bool two = max_rows > 8 && (size_t)16 * (K + 32) * 2 + WARPS * 2 * 512 <= 227 * 1024;
#define ESP_GO(NB, SW, TC) return launch<NB, SW, TC>(p, g, stream)
    if (swiglu) {
        if (c_dtype == 1) { if (two) ESP_GO(2, MODE_SWIGLU, bf16); else ESP_GO(1, MODE_SWIGLU, bf16); }
        else { if (two) ESP_GO(2, MODE_SWIGLU, float); else ESP_GO(1, MODE_SWIGLU, float); }
    } else {
        if (c_dtype == 1) { if (two) ESP_GO(2, MODE_PLAIN, bf16); else ESP_GO(1, MODE_PLAIN, bf16); }
        else { if (two) ESP_GO(2, MODE_PLAIN, float); else ESP_GO(1, MODE_PLAIN, float); }
    }
    return (int)cudaErrorInvalidValue;
}

// The packed q/k/v projection of a step of few rows with the position encoding and the cache write in its
// epilogue: out = A W^T (+ bias), heads [nh queries | nkv keys | nkv values] of width hd; queries and keys
// are rotated by their token's position (full split-half rotation, cos/sin tables [max_pos, hd / 2]), queries
// go to q_out [M, nh * hd], keys and values into the paged cache (all bfloat16).  Same arithmetic as
// esp_gemm_skinny followed by esp_rope_kvwrite, without the float intermediate.  hd a multiple of 16.
ESP_API int esp_qkv_rope_skinny(const void* A, long long lda, const void* W, const float* bias, const int* tok_seq,
                                const int* tok_pos, const float* cos_t, const float* sin_t, int max_pos, void* q_out,
                                void* k_cache, void* v_cache, const int* block_table, int table_stride, int n_pages, int page,
                                int M, int K, int nh, int nkv, int hd, int write_kv, int* status, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (K % 8 != 0 || lda % 8 != 0 || hd % 16 != 0 || hd <= 0 || nh <= 0 || nkv <= 0 || page <= 0 || M > 16)
        return (int)cudaErrorInvalidValue;
    SkinnyParams p{};
    p.W = (const bf16*)W; p.A = (const bf16*)A; p.lda = lda; p.M = M; p.N = (nh + 2 * nkv) * (hd / 2); p.K = K; p.groups = 1;
    p.bias = bias; p.tok_seq = tok_seq; p.tok_pos = tok_pos; p.cos_t = cos_t; p.sin_t = sin_t; p.q_out = q_out;
    p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table; p.table_stride = table_stride;
    p.n_pages = n_pages; p.page = page; p.nh = nh; p.nkv = nkv; p.hd = hd; p.max_pos = max_pos; p.write_kv = write_kv;
    p.status = status;
    const int g = 1;
    const bool two = M > 8 && (size_t)16 * (K + 32) * 2 + WARPS * 2 * 512 <= 227 * 1024;
    if (two) ESP_GO(2, MODE_ROPE, bf16); else ESP_GO(1, MODE_ROPE, bf16);
#undef ESP_GO
    return (int)cudaErrorInvalidValue;
}
