// Decode attention over the paged bfloat16 cache, split over the keys.
//
// One block = one token row, one key/value head (with up to GT of the query
// heads that share it) and one split of SPLIT consecutive key positions
// aligned to absolute multiples of SPLIT.  The block reads its keys and values
// once from HBM in 16-byte pieces, keeps scores, softmax and sums in float, and
// writes an unnormalised partial result (running maximum, sum, weighted
// values) to scratch.  A second kernel combines a row's splits in ascending
// order.  Which splits a row has depends on its position (and window) alone,
// so the result does not depend on the batch around it.
//
// The query at position a sees key j iff j <= a and (window == 0 or a - j < window);
// score = dot(q, k) / sqrt(hd).
#include "common.cuh"

namespace {
constexpr int THREADS = 128;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <int HD, int GT, int SPLIT>
__global__ void __launch_bounds__(THREADS, 6)
attn_split_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                  float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ tok_seq,
                  const int* __restrict__ tok_pos, const int* __restrict__ block_table, int table_stride, int n_pages,
                  int page, int nh, int nkv, int window, int n_splits, int* __restrict__ status) {
    constexpr int PIECES = HD / 8;                 // 16-byte pieces of a key or value row
    constexpr int PER_LANE = HD / 64;              // pieces each of the 8 lanes of a key group loads
    constexpr int KG = THREADS / PIECES;           // key groups of the value pass
    __shared__ float q_s[GT][HD];
    __shared__ float s_s[GT][SPLIT];
    __shared__ int pg_s[SPLIT];
    __shared__ float red[4][GT][2];
    extern __shared__ float o_red[];               // [KG][GT][HD]

    const int n = blockIdx.x, split = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = nh / nkv, blocks_per_kv = (group + GT - 1) / GT;
    const int kvh = blockIdx.y / blocks_per_kv, h0 = kvh * group + (blockIdx.y % blocks_per_kv) * GT;
    const int heads = min(GT, (kvh + 1) * group - h0);
    const int pos = tok_pos[n], seq = tok_seq[n];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int j0 = max(lo, split * SPLIT), j1 = min(pos, split * SPLIT + SPLIT - 1);
    if (j0 > j1) return;                           // this row has no keys in this split
    const int count = j1 - j0 + 1;

    for (int i = tid; i < GT * HD; i += THREADS) {
        const int g = i / HD, d = i - g * HD;
        q_s[g][d] = g < heads ? __bfloat162float(q[((size_t)n * nh + h0 + g) * HD + d]) : 0.f;
    }
    for (int t = tid; t < count; t += THREADS) {
        int pg = block_table[(size_t)seq * table_stride + (j0 + t) / page];
        if (pg < 0 || pg >= n_pages) {
            atomicOr(status, ESP_STATUS_BAD_INDEX);
            pg = -1;
        }
        pg_s[t] = pg;
    }
    __syncthreads();

    // ---- scores: 8 lanes per key, 16 keys in flight per pass --------------------
    const float root = sqrtf((float)HD);
    const int sub = tid & 7, slot = tid >> 3;      // lane within the key group, key slot 0..15
    constexpr int KB = 4;                          // keys whose loads are in flight together, per thread
    for (int t0 = slot; t0 < SPLIT; t0 += KB * (THREADS / 8)) {
        uint4 kraw[KB][PER_LANE];
        bool live[KB];
#pragma unroll
        for (int b = 0; b < KB; b++) {
            const int t = t0 + b * (THREADS / 8);
            live[b] = t < count && pg_s[t] >= 0;
            if (live[b]) {
                const int j = j0 + t;
                const bf16* krow = k_cache + (((size_t)pg_s[t] * nkv + kvh) * page + j % page) * HD;
#pragma unroll
                for (int i = 0; i < PER_LANE; i++) kraw[b][i] = *reinterpret_cast<const uint4*>(krow + (sub + 8 * i) * 8);
            }
        }
#pragma unroll
        for (int b = 0; b < KB; b++) {
            const int t = t0 + b * (THREADS / 8);
            float dot[GT];
#pragma unroll
            for (int g = 0; g < GT; g++) dot[g] = 0.f;
            if (live[b]) {
#pragma unroll
                for (int i = 0; i < PER_LANE; i++) {
                    const int piece = sub + 8 * i;
                    float kf[8];
                    unpack8(kraw[b][i], kf);
#pragma unroll
                    for (int g = 0; g < GT; g++)
#pragma unroll
                        for (int e = 0; e < 8; e++) dot[g] = fmaf(q_s[g][piece * 8 + e], kf[e], dot[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < GT; g++) {
                float v = dot[g];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if (sub == 0 && t < SPLIT) s_s[g][t] = live[b] ? v / root : -INFINITY;
            }
        }
    }
    __syncthreads();

    // ---- softmax pieces of this split ----------------------------------------------
    float m_loc[GT], l_loc[GT];
#pragma unroll
    for (int g = 0; g < GT; g++) {
        float mx = -INFINITY;
        for (int t = tid; t < count; t += THREADS) mx = fmaxf(mx, s_s[g][t]);
        mx = warp_max(mx);
        if (lane == 0) red[warp][g][0] = mx;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GT; g++) {
        m_loc[g] = fmaxf(fmaxf(red[0][g][0], red[1][g][0]), fmaxf(red[2][g][0], red[3][g][0]));
        float sum = 0.f;
        for (int t = tid; t < count; t += THREADS) {
            const float pv = m_loc[g] == -INFINITY ? 0.f : expf(s_s[g][t] - m_loc[g]);
            s_s[g][t] = pv;
            sum += pv;
        }
        sum = warp_sum(sum);
        if (lane == 0) red[warp][g][1] = sum;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GT; g++) l_loc[g] = ((red[0][g][1] + red[1][g][1]) + red[2][g][1]) + red[3][g][1];

    // ---- weighted values: a thread owns one 16-byte piece of the head and every KG-th key ----
    const int piece = tid % PIECES, kg = tid / PIECES;
    float acc[GT][8];
#pragma unroll
    for (int g = 0; g < GT; g++)
#pragma unroll
        for (int e = 0; e < 8; e++) acc[g][e] = 0.f;
    for (int t0 = kg; t0 < count && kg < KG; t0 += KB * KG) {
        uint4 vraw[KB];
        bool live[KB];
#pragma unroll
        for (int b = 0; b < KB; b++) {
            const int t = t0 + b * KG;
            live[b] = t < count && pg_s[t] >= 0;
            if (live[b]) {
                const int j = j0 + t;
                vraw[b] = *reinterpret_cast<const uint4*>(v_cache + (((size_t)pg_s[t] * nkv + kvh) * page + j % page) * HD + piece * 8);
            }
        }
#pragma unroll
        for (int b = 0; b < KB; b++) {
            if (!live[b]) continue;
            const int t = t0 + b * KG;
            float vf[8];
            unpack8(vraw[b], vf);
#pragma unroll
            for (int g = 0; g < GT; g++) {
                const float pw = s_s[g][t];
#pragma unroll
                for (int e = 0; e < 8; e++) acc[g][e] = fmaf(pw, vf[e], acc[g][e]);
            }
        }
    }
    if (kg < KG) {
#pragma unroll
        for (int g = 0; g < GT; g++)
#pragma unroll
            for (int e = 0; e < 8; e++) o_red[((size_t)kg * GT + g) * HD + piece * 8 + e] = acc[g][e];
    }
    __syncthreads();
    for (int i = tid; i < heads * HD; i += THREADS) {
        const int g = i / HD, d = i - g * HD;
        float v = 0.f;
#pragma unroll
        for (int c = 0; c < KG; c++) v += o_red[((size_t)c * GT + g) * HD + d];
        part_o[(((size_t)n * nh + h0 + g) * n_splits + split) * HD + d] = v;
    }
    if (tid < heads) {
        float* ml = part_ml + (((size_t)n * nh + h0 + tid) * n_splits + split) * 2;
        ml[0] = m_loc[tid];
        ml[1] = l_loc[tid];
    }
}

template <int HD>
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, const int* __restrict__ tok_pos, int nh, int window,
                                    int n_splits, int SPLIT) {
    const int n = blockIdx.x, h = blockIdx.y;
    const int pos = tok_pos[n];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int s0 = lo / SPLIT, s1 = pos / SPLIT;
    const float* ml = part_ml + ((size_t)n * nh + h) * n_splits * 2;
    const float* po = part_o + ((size_t)n * nh + h) * n_splits * HD;
    float mx = -INFINITY;
    for (int s = s0; s <= s1; s++) mx = fmaxf(mx, ml[2 * s]);
    float denom = 0.f;
    for (int s = s0; s <= s1; s++) denom += ml[2 * s + 1] * (ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - mx));
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.f;
        for (int s = s0; s <= s1; s++) {
            const float w = ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - mx);
            acc += po[(size_t)s * HD + d] * w;
        }
        out[((size_t)n * nh + h) * HD + d] = __float2bfloat16_rn(denom > 0.f ? acc / denom : 0.f);
    }
}

template <int HD, int GT, int SPLIT>
int launch_split(const bf16* q, const bf16* k, const bf16* v, float* po, float* pml, const int* tok_seq,
                 const int* tok_pos, const int* table, int stride, int n_pages, int page, int n_tokens, int nh, int nkv,
                 int window, int n_splits, int* status, cudaStream_t stream) {
    constexpr int KG = THREADS / (HD / 8);
    const size_t dyn = (size_t)KG * GT * HD * sizeof(float);
    static bool raised = false;        // static + dynamic shared memory can pass 48 KB: always opt in
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(attn_split_kernel<HD, GT, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)dyn);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    const int group = nh / nkv;
    dim3 grid(n_tokens, nkv * ((group + GT - 1) / GT), n_splits);
    attn_split_kernel<HD, GT, SPLIT><<<grid, THREADS, dyn, stream>>>(q, k, v, po, pml, tok_seq, tok_pos, table, stride, n_pages,
                                                              page, nh, nkv, window, n_splits, status);
    return esp_launch_status();
}

template <int HD>
int dispatch(int gt, int split, const bf16* q, const bf16* k, const bf16* v, bf16* out, float* po, float* pml, const int* tok_seq,
             const int* tok_pos, const int* table, int stride, int n_pages, int page, int n_tokens, int nh, int nkv,
             int window, int n_splits, int* status, cudaStream_t stream) {
    int rc;
#define ESP_SPLIT(GT)                                                                                                  \
    (split == 256 ? launch_split<HD, GT, 256>(q, k, v, po, pml, tok_seq, tok_pos, table, stride, n_pages, page, n_tokens, \
                                              nh, nkv, window, n_splits, status, stream)                                 \
                  : launch_split<HD, GT, 512>(q, k, v, po, pml, tok_seq, tok_pos, table, stride, n_pages, page, n_tokens, \
                                              nh, nkv, window, n_splits, status, stream))
    if (gt == 1) rc = ESP_SPLIT(1);
    else if (gt == 2) rc = ESP_SPLIT(2);
    else if (gt == 4) rc = ESP_SPLIT(4);
    else rc = ESP_SPLIT(8);
#undef ESP_SPLIT
    if (rc != 0) return rc;
    dim3 grid(n_tokens, nh);
    attn_combine_kernel<HD><<<grid, HD / 2 < 32 ? 32 : HD / 2, 0, stream>>>(po, pml, out, tok_pos, nh, window, n_splits, split);
    return esp_launch_status();
}
}  // namespace

// Scratch: part_o float [n_tokens, nh, n_splits, hd], part_ml float [n_tokens, nh, n_splits, 2];
// split: key positions per block, 256 or 512 (the caller picks: short splits when there are few rows, so
// that every SM still gets blocks); n_splits >= ceil(longest sequence / split).  Head sizes 64, 128, 192, 256; pages of 64 positions or any
// size; any head counts with nh % nkv == 0.
ESP_API int esp_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o,
                            float* part_ml, const int* tok_seq, const int* tok_pos, const int* block_table,
                            int table_stride, int n_pages, int page, int n_tokens, int nh, int nkv, int hd, int window,
                            int split, int n_splits, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || n_splits <= 0 || n_splits > 65535 || nh > 65535 || (split != 256 && split != 512))
        return (int)cudaErrorInvalidValue;
    const int group = nh / nkv;
    const int gt = group >= 8 ? 8 : group >= 3 ? 4 : group;      // 1, 2, 4 or 8 heads per block
#define ESP_HD(HD) return dispatch<HD>(gt, split, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, part_o, \
                                       part_ml, tok_seq, tok_pos, block_table, table_stride, n_pages, page, n_tokens, nh,   \
                                       nkv, window, n_splits, status, stream)
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

extern "C" long long esp_attn_decode_noalloc_capacity(void) { return (long long)ESP_ATTN_DECODE_NOALLOC_FLOATS; }

extern "C" int esp_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                       const int* tok_seq, const int* tok_pos, const int* block_table, int table_stride,
                                       int n_pages, int page, int n_tokens, int nh, int nkv, int hd, int window,
                                       int split, int n_splits, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || hd <= 0 || n_splits <= 0) return (int)cudaErrorInvalidValue;
    const unsigned long long need = (unsigned long long)n_tokens * nh * n_splits * (hd + 2);
    if (need > ESP_ATTN_DECODE_NOALLOC_FLOATS) return ESP_NOALLOC_TOO_LARGE;
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
    return esp_attn_decode(q, k_cache, v_cache, out, part_o, part_ml, tok_seq, tok_pos, block_table, table_stride, n_pages,
                           page, n_tokens, nh, nkv, hd, window, split, n_splits, status, stream);
}
