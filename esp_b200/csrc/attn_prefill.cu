// Prefill attention over the paged bfloat16 cache: causal, optionally
// windowed, grouped query heads, sequences of unequal length packed back to
// back.  Flash style: a block owns 64 consecutive query tokens of one sequence
// and one query head, walks the sequence's key pages in ascending order, keeps
// the running maximum, the running sum and the weighted values in float
// registers and never writes scores to memory.  Q K^T and P V run on the tensor
// cores (mma.sync m16n8k16, bfloat16 in, float out); P is rounded to bfloat16
// for the second product.  Keys and values of a page are fetched with
// cp.async into shared memory, the next page while the current one is used.
//
// The new keys and values are already in the cache when this runs, so a step
// that continues a sequence (past > 0) and a first step are the same case.
// Head sizes up to HDB (64 or 128) are padded with zeros to HDB in shared
// memory; they must be multiples of 8.  The page size is 64.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, THREADS = 128;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;          // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <int HDB>
__global__ void __launch_bounds__(THREADS, 3)
attn_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                    bf16* __restrict__ out, const int* __restrict__ tile_seq, const int* __restrict__ tile_first,
                    const int* __restrict__ seq_start, const int* __restrict__ seq_past,
                    const int* __restrict__ block_table, int table_stride, int n_pages, int nh, int nkv, int hd,
                    int window, int* __restrict__ status) {
    constexpr int LDS = HDB + 8;                     // row stride in elements: 16 bytes of padding against bank conflicts
    constexpr int PIECES = HDB / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* k_s = reinterpret_cast<bf16*>(smem_raw);                    // [2][BN][LDS]
    bf16* v_s = k_s + 2 * BN * LDS;                                    // [2][BN][LDS]
    bf16* q_s = k_s + BN * LDS;                                        // [BM][LDS]: the tile's queries borrow the second
                                                                       // key buffer until their fragments are in registers

    // tiles are listed in order of position; the last ones see the most keys, so they start first
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;
    const int seq = tile_seq[tile], first = tile_first[tile];          // first: index of the tile's first token in its sequence's new tokens
    const int row0 = seq_start[seq] + first;                           // its row among the packed tokens
    const int n_new = seq_start[seq + 1] - seq_start[seq];
    const int rows = min(BM, n_new - first);                           // live query rows of the tile
    const int past = seq_past[seq];
    const int pos0 = past + first;                                     // absolute position of the tile's first query
    const int pos_last = pos0 + rows - 1;
    const int kvh = h / (nh / nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
    const int hd_pieces = hd / 8;

    // ---- the tile's queries -> shared memory (rows beyond the tile and columns beyond hd are zero)
    for (int idx = tid; idx < BM * PIECES; idx += THREADS) {
        const int r = idx / PIECES, p = idx - r * PIECES;
        const bool ok = r < rows && p < hd_pieces;
        cp_async16(q_s + r * LDS + p * 8, q + ((size_t)(row0 + (ok ? r : 0)) * nh + h) * hd + (ok ? p : 0) * 8, ok);
    }
    cp_async_commit();

    const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;     // first key any row of the tile sees
    const int blk_lo = key_lo / BN, blk_hi = pos_last / BN;

    auto load_kv = [&](int blk, int buf) {
        int pg = block_table[(size_t)seq * table_stride + blk];
        const bool pg_ok = pg >= 0 && pg < n_pages;
        if (!pg_ok) {
            if (tid == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            pg = 0;
        }
        const bf16* kp = k_cache + ((size_t)pg * nkv + kvh) * BN * hd;
        const bf16* vp = v_cache + ((size_t)pg * nkv + kvh) * BN * hd;
        for (int idx = tid; idx < BN * PIECES; idx += THREADS) {
            const int r = idx / PIECES, p = idx - r * PIECES;
            const bool ok = pg_ok && p < hd_pieces;
            const size_t off = (size_t)r * hd + (ok ? p : 0) * 8;
            cp_async16(k_s + (buf * BN + r) * LDS + p * 8, kp + off, ok);
            cp_async16(v_s + (buf * BN + r) * LDS + p * 8, vp + off, ok);
        }
        cp_async_commit();
    };
    load_kv(blk_lo, 0);

    // ---- query fragments of this warp's 16 rows stay in registers
    cp_async_wait<1>();
    __syncthreads();
    unsigned qf[HDB / 16][4];
#pragma unroll
    for (int kk = 0; kk < HDB / 16; kk++)
        ldmatrix_x4(qf[kk], q_s + (warp * 16 + (lane & 15)) * LDS + kk * 16 + (lane >> 4) * 8);
    __syncthreads();                                                   // the borrowed buffer may now be refilled with keys

    float o[HDB / 8][4];
#pragma unroll
    for (int i = 0; i < HDB / 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o[i][j] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float root = sqrtf((float)hd);
    const float log2e = 1.4426950408889634f;
    const int my_pos[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};   // absolute positions of this lane's two rows

    for (int blk = blk_lo; blk <= blk_hi; blk++) {
        const int buf = (blk - blk_lo) & 1;
        if (blk < blk_hi) load_kv(blk + 1, buf ^ 1);
        if (blk < blk_hi) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();
        const bf16* kb = k_s + buf * BN * LDS;
        const bf16* vb = v_s + buf * BN * LDS;

        // S = Q K^T for 16 rows x 64 keys
        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) s[i][j] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HDB / 16; kk++) {
#pragma unroll
            for (int nb = 0; nb < BN / 16; nb++) {
                unsigned kf[4];
                ldmatrix_x4(kf, kb + (nb * 16 + (lane & 7) + (lane >> 4) * 8) * LDS + kk * 16 + ((lane >> 3) & 1) * 8);
                mma16816(s[2 * nb], qf[kk], kf[0], kf[1]);
                mma16816(s[2 * nb + 1], qf[kk], kf[2], kf[3]);
            }
        }
        // scale, mask, running maximum
        const int key0 = blk * BN;
        // does any (row of this warp, key of this block) pair need the mask?
        const bool edge = key0 + BN - 1 > pos0 + warp * 16 || (window > 0 && key0 < pos0 + warp * 16 + 15 - window + 1);
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nb = 0; nb < BN / 8; nb++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int r = j >> 1;
                const int key = key0 + nb * 8 + tg * 2 + (j & 1);
                float v = s[nb][j] / root;
                if (edge) {
                    const bool seen = key <= my_pos[r] && (window <= 0 || my_pos[r] - key < window);
                    if (!seen) v = -INFINITY;
                }
                s[nb][j] = v;
                m_new[r] = fmaxf(m_new[r], v);
            }
        }
        float scale_old[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            m_use[r] = m_new[r] == -INFINITY ? 0.f : m_new[r];
            scale_old[r] = exp2f((m_run[r] - m_use[r]) * log2e);       // m_run = -inf gives 0
            m_run[r] = m_new[r];
        }
        float l_add[2] = {0.f, 0.f};
#pragma unroll
        for (int nb = 0; nb < BN / 8; nb++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int r = j >> 1;
                const float p = exp2f((s[nb][j] - m_use[r]) * log2e);
                s[nb][j] = p;
                l_add[r] += p;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; r++) l_run[r] = l_run[r] * scale_old[r] + l_add[r];
#pragma unroll
        for (int i = 0; i < HDB / 8; i++) {
            o[i][0] *= scale_old[0];
            o[i][1] *= scale_old[0];
            o[i][2] *= scale_old[1];
            o[i][3] *= scale_old[1];
        }
        // O += P V
#pragma unroll
        for (int kt = 0; kt < BN / 16; kt++) {
            unsigned pf[4];
            pf[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
            pf[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
            pf[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            pf[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
            for (int nb = 0; nb < HDB / 16; nb++) {
                unsigned vf[4];
                ldmatrix_x4_trans(vf, vb + (kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + nb * 16 + (lane >> 4) * 8);
                mma16816(o[2 * nb], pf, vf[0], vf[1]);
                mma16816(o[2 * nb + 1], pf, vf[2], vf[3]);
            }
        }
        __syncthreads();                                 // every warp is done with this buffer before it is refilled
    }
    // ---- normalise and store
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = warp * 16 + g + r * 8;
        if (row >= rows) continue;
        const float inv = l_run[r] > 0.f ? 1.0f / l_run[r] : 0.f;
        bf16* orow = out + ((size_t)(row0 + row) * nh + h) * hd;
#pragma unroll
        for (int i = 0; i < HDB / 8; i++) {
            const int d = i * 8 + tg * 2;
            if (d < hd) {
                __nv_bfloat162 v = __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
                *reinterpret_cast<__nv_bfloat162*>(orow + d) = v;
            }
        }
    }
}

template <int HDB>
int launch(const bf16* q, const bf16* k, const bf16* v, bf16* out, const int* tile_seq, const int* tile_first,
           const int* seq_start, const int* seq_past, const int* table, int stride, int n_pages, int n_tiles, int nh,
           int nkv, int hd, int window, int* status, cudaStream_t stream) {
    static_assert(BM <= BN, "the queries borrow a key buffer");
    const size_t smem = (size_t)(4 * BN) * (HDB + 8) * sizeof(bf16);
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HDB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    dim3 grid(n_tiles, nh);
    attn_prefill_kernel<HDB><<<grid, THREADS, smem, stream>>>(q, k, v, out, tile_seq, tile_first, seq_start, seq_past,
                                                              table, stride, n_pages, nh, nkv, hd, window, status);
    return esp_launch_status();
}
}  // namespace

// tile_seq / tile_first: for every tile of 64 new tokens, its sequence and the index of its first token
// among that sequence's new tokens.  hd: a multiple of 8, at most 128.  The cache page holds 64 positions.
ESP_API int esp_attn_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tile_seq,
                             const int* tile_first, const int* seq_start, const int* seq_past, const int* block_table,
                             int table_stride, int n_pages, int page, int n_tiles, int nh, int nkv, int hd, int window,
                             int* status, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (page != BN || hd % 8 != 0 || hd > 128 || hd <= 0 || nkv <= 0 || nh % nkv != 0 || nh > 65535)
        return (int)cudaErrorInvalidValue;
    if (hd <= 64)
        return launch<64>((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, tile_seq, tile_first,
                          seq_start, seq_past, block_table, table_stride, n_pages, n_tiles, nh, nkv, hd, window, status, stream);
    return launch<128>((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, tile_seq, tile_first,
                       seq_start, seq_past, block_table, table_stride, n_pages, n_tiles, nh, nkv, hd, window, status, stream);
}
