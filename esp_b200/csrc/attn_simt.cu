// Plain attention over the paged cache, one block per (token, query head),
// every step of the arithmetic in 32-bit.  It serves the 32-bit path for
// prefill and decode alike and any head size up to 256.
//
// The query at absolute position a sees key j iff j <= a and (window == 0 or
// a - j < window).  score = dot(q, k_j) / sqrt(hd) (divided after the product).
// Keys are walked in chunks of CHUNK positions aligned to absolute multiples of
// CHUNK with a running maximum and sum, so the order of every addition depends
// on the query's position alone: not on how the sequence was cut into steps,
// nor on what else is in the batch.
#include "common.cuh"

namespace {
constexpr int CHUNK = 256;
constexpr int THREADS = 128;
constexpr int MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                 T* __restrict__ out, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                 const int* __restrict__ block_table, int table_stride, int n_pages, int page, int nh, int nkv, int hd,
                 int window, int* __restrict__ status) {
    __shared__ float qs[MAX_HD];
    __shared__ float ps[CHUNK];
    __shared__ int pages[CHUNK];      // page id of each key of the chunk (or -1)
    __shared__ float scratch[33];
    const int n = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int seq = tok_seq[n], pos = tok_pos[n];
    const int kvh = h / (nh / nkv);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const T* qrow = q + ((size_t)n * nh + h) * hd;
    for (int d = tid; d < hd; d += THREADS) qs[d] = to_f32(qrow[d]);
    const float root = sqrtf((float)hd);
    float m_run = -INFINITY, l_run = 0.f;
    float acc[MAX_HD / THREADS];
#pragma unroll
    for (int i = 0; i < MAX_HD / THREADS; i++) acc[i] = 0.f;
    __syncthreads();

    for (int c = lo / CHUNK; c <= pos / CHUNK; c++) {
        const int j0 = max(lo, c * CHUNK), j1 = min(pos, c * CHUNK + CHUNK - 1);
        const int count = j1 - j0 + 1;
        // scores
        float local_max = -INFINITY;
        for (int t = tid; t < count; t += THREADS) {
            const int j = j0 + t;
            int pg = block_table[(size_t)seq * table_stride + j / page];
            if (pg < 0 || pg >= n_pages) {
                atomicOr(status, ESP_STATUS_BAD_INDEX);
                pg = -1;
            }
            pages[t] = pg;
            float s = -INFINITY;
            if (pg >= 0) {
                const T* krow = k_cache + (((size_t)pg * nkv + kvh) * page + j % page) * hd;
                float dot = 0.f;
                for (int d = 0; d < hd; d++) dot = fmaf(qs[d], to_f32(krow[d]), dot);
                s = dot / root;
            }
            ps[t] = s;
            local_max = fmaxf(local_max, s);
        }
        const float m_chunk = block_max(local_max, scratch);
        const float m_new = fmaxf(m_run, m_chunk);
        if (m_new == -INFINITY) continue;          // every key of the chunk was skipped as a bad index
        float local_sum = 0.f;
        for (int t = tid; t < count; t += THREADS) {
            const float p = expf(ps[t] - m_new);
            ps[t] = p;
            local_sum += p;
        }
        const float l_chunk = block_sum(local_sum, scratch);   // also orders the writes of ps before the reads below
        const float rescale = expf(m_run - m_new);
        l_run = l_run * rescale + l_chunk;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < MAX_HD / THREADS; i++) {
            const int d = tid + i * THREADS;
            if (d < hd) {
                float a = acc[i] * rescale;
                for (int t = 0; t < count; t++) {
                    const int pg = pages[t];
                    if (pg < 0) continue;
                    const int j = j0 + t;
                    a = fmaf(ps[t], to_f32(v_cache[(((size_t)pg * nkv + kvh) * page + j % page) * hd + d]), a);
                }
                acc[i] = a;
            }
        }
        __syncthreads();
    }
    T* orow = out + ((size_t)n * nh + h) * hd;
#pragma unroll
    for (int i = 0; i < MAX_HD / THREADS; i++) {
        const int d = tid + i * THREADS;
        if (d < hd) orow[d] = from_f32<T>(l_run > 0.f ? acc[i] / l_run : 0.f);
    }
}
}  // namespace

ESP_API int esp_attn_simt(const void* q, const void* k_cache, const void* v_cache, void* out, int is_bf16,
                          const int* tok_seq, const int* tok_pos, const int* block_table, int table_stride, int n_pages,
                          int page, int n_tokens, int nh, int nkv, int hd, int window, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd > MAX_HD || hd <= 0 || nkv <= 0 || nh % nkv != 0 || nh > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid(n_tokens, nh);
    if (is_bf16)
        attn_simt_kernel<bf16><<<grid, THREADS, 0, stream>>>((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                                                            (bf16*)out, tok_seq, tok_pos, block_table, table_stride,
                                                            n_pages, page, nh, nkv, hd, window, status);
    else
        attn_simt_kernel<float><<<grid, THREADS, 0, stream>>>((const float*)q, (const float*)k_cache,
                                                             (const float*)v_cache, (float*)out, tok_seq, tok_pos,
                                                             block_table, table_stride, n_pages, page, nh, nkv, hd,
                                                             window, status);
    return esp_launch_status();
}
