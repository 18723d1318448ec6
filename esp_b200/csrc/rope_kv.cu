// Rotary position encoding (split-half) of the new queries and keys in 32-bit,
// and the write of the new keys and values into the paged cache.
//
// qkv: [n_tokens, (nh + 2*nkv) * hd] float; ``bias`` (same width, may be null) is
// added first.  Head h of the
// query block is columns [h*hd, (h+1)*hd); keys follow the queries, values the
// keys.  For i < rot/2 and the token's absolute position p:
//   o[i]         = x[i] * cos[p][i] - x[i + rot/2] * sin[p][i]
//   o[i + rot/2] = x[i + rot/2] * cos[p][i] + x[i] * sin[p][i]
// Columns at or beyond ``rot`` pass through (rot = 0: no rotation at all).
// Keys are cached after rotation.  A page holds PAGE consecutive positions of
// one sequence: K/V are [pages, nkv, PAGE, hd]; the page of position p is
// block_table[seq * table_stride + p / PAGE].
#include "common.cuh"

template <typename T>
__global__ void rope_kvwrite_kernel(const float* __restrict__ qkv, const float* __restrict__ bias,
                                    const int* __restrict__ tok_seq,
                                    const int* __restrict__ tok_pos, const float* __restrict__ cos_t,
                                    const float* __restrict__ sin_t, int rot, int max_pos, T* __restrict__ q_out,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ block_table,
                                    int table_stride, int n_pages, int page, int nh, int nkv, int hd, int write_kv,
                                    int heads_per_block, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int pos = tok_pos[n];
    const int seq = tok_seq[n];
    const int half = rot / 2;
    const int width = (nh + 2 * nkv) * hd;
    const float* src = qkv + (size_t)n * width;
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
        return;
    }
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    int page_id = -1;
    if (write_kv) {
        page_id = block_table[(size_t)seq * table_stride + pos / page];
        if (page_id < 0 || page_id >= n_pages) {
            if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            page_id = -1;
        }
    }
    const int in_page = pos % page;
    const int heads = nh + 2 * nkv;
    const int head_lo = blockIdx.y * heads_per_block, head_hi = min(heads, head_lo + heads_per_block);
    for (int idx = threadIdx.x; idx < (head_hi - head_lo) * hd; idx += blockDim.x) {
        const int head = head_lo + idx / hd, i = idx % hd;
        const float* x = src + (size_t)head * hd;
        const float* b = bias ? bias + (size_t)head * hd : nullptr;
        float v = x[i] + (b ? b[i] : 0.f);
        if (head < nh + nkv && i < rot) {          // queries and keys rotate, values do not
            if (i < half) {
                const float other = x[i + half] + (b ? b[i + half] : 0.f);
                v = v * cs[i] - other * sn[i];
            } else {
                const float other = x[i - half] + (b ? b[i - half] : 0.f);
                v = v * cs[i - half] + other * sn[i - half];
            }
        }
        if (head < nh) {
            q_out[((size_t)n * nh + head) * hd + i] = from_f32<T>(v);
        } else if (page_id >= 0) {
            const bool is_k = head < nh + nkv;
            const int kvh = is_k ? head - nh : head - nh - nkv;
            T* dst = (is_k ? k_cache : v_cache) + (((size_t)page_id * nkv + kvh) * page + in_page) * hd + i;
            *dst = from_f32<T>(v);
        }
    }
}

// The same for full rotation (rot == hd, hd a multiple of 8) with 16-byte accesses: a thread owns four
// consecutive pairs (i, i + hd/2) of one head of one token.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kvwrite_vec_kernel(const float* __restrict__ qkv, const float* __restrict__ bias, const int* __restrict__ tok_seq,
                        const int* __restrict__ tok_pos, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                        int max_pos, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                        const int* __restrict__ block_table, int table_stride, int n_pages, int page, int nh, int nkv,
                        int hd, int write_kv, int heads_per_block, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int pos = tok_pos[n], seq = tok_seq[n];
    const int half = hd / 2, quads = half / 4, heads = nh + 2 * nkv;
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
        return;
    }
    int page_id = -1;
    if (write_kv) {
        page_id = block_table[(size_t)seq * table_stride + pos / page];
        if (page_id < 0 || page_id >= n_pages) {
            if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            page_id = -1;
        }
    }
    const int in_page = pos % page;
    const float* src = qkv + (size_t)n * heads * hd;
    const float4* cs = reinterpret_cast<const float4*>(cos_t + (size_t)pos * half);
    const float4* sn = reinterpret_cast<const float4*>(sin_t + (size_t)pos * half);
    const int head_lo = blockIdx.y * heads_per_block, head_hi = min(heads, head_lo + heads_per_block);
    for (int idx = threadIdx.x; idx < (head_hi - head_lo) * quads; idx += blockDim.x) {
        const int head = head_lo + idx / quads, qd = idx % quads, i0 = qd * 4;
        const float* x = src + (size_t)head * hd;
        float4 lo = *reinterpret_cast<const float4*>(x + i0), hi = *reinterpret_cast<const float4*>(x + i0 + half);
        if (bias) {
            const float4 bl = *reinterpret_cast<const float4*>(bias + (size_t)head * hd + i0);
            const float4 bh = *reinterpret_cast<const float4*>(bias + (size_t)head * hd + i0 + half);
            lo.x += bl.x; lo.y += bl.y; lo.z += bl.z; lo.w += bl.w;
            hi.x += bh.x; hi.y += bh.y; hi.z += bh.z; hi.w += bh.w;
        }
        float4 ol = lo, oh = hi;
        if (head < nh + nkv) {                       // queries and keys rotate, values do not
            const float4 c = cs[qd], s = sn[qd];
            ol.x = lo.x * c.x - hi.x * s.x; oh.x = hi.x * c.x + lo.x * s.x;
            ol.y = lo.y * c.y - hi.y * s.y; oh.y = hi.y * c.y + lo.y * s.y;
            ol.z = lo.z * c.z - hi.z * s.z; oh.z = hi.z * c.z + lo.z * s.z;
            ol.w = lo.w * c.w - hi.w * s.w; oh.w = hi.w * c.w + lo.w * s.w;
        }
        T* dst = nullptr;
        if (head < nh) {
            dst = q_out + ((size_t)n * nh + head) * hd;
        } else if (page_id >= 0) {
            const bool is_k = head < nh + nkv;
            const int kvh = is_k ? head - nh : head - nh - nkv;
            dst = (is_k ? k_cache : v_cache) + (((size_t)page_id * nkv + kvh) * page + in_page) * hd;
        }
        if (dst) {
            Vec4<T>::store(dst + i0, ol.x, ol.y, ol.z, ol.w);
            Vec4<T>::store(dst + i0 + half, oh.x, oh.y, oh.z, oh.w);
        }
    }
}

ESP_API int esp_rope_kvwrite(const float* qkv, const float* bias, const int* tok_seq, const int* tok_pos, const float* cos_t,
                             const float* sin_t, int rot, int max_pos, void* q_out, void* k_cache, void* v_cache,
                             int is_bf16, const int* block_table, int table_stride, int n_pages, int page, int n_tokens,
                             int nh, int nkv, int hd, int write_kv, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot < 0 || rot > hd || (rot & 1) || nh + 2 * nkv > 65535) return (int)cudaErrorInvalidValue;
    // few tokens (decode): one head per block keeps every load in flight at once; many tokens: eight heads
    // per block keep the number of blocks down
    if (rot == hd && hd % 8 == 0 && cos_t && n_tokens > 64) {
        // many tokens, full rotation: the 16-byte version, 64 heads per block (several pieces in flight per thread)
        const int hpb = 64;
        const dim3 vgrid(n_tokens, (nh + 2 * nkv + hpb - 1) / hpb);
        if (is_bf16)
            esp_launch_pdl(ESP_PDL_SMALL, rope_kvwrite_vec_kernel<bf16>, dim3(vgrid), dim3(256), 0, stream, qkv, bias, tok_seq, tok_pos, cos_t, sin_t, max_pos,
                                                                    (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache,
                                                                    block_table, table_stride, n_pages, page, nh, nkv, hd,
                                                                    write_kv, hpb, status);
        else
            esp_launch_pdl(ESP_PDL_SMALL, rope_kvwrite_vec_kernel<float>, dim3(vgrid), dim3(256), 0, stream, qkv, bias, tok_seq, tok_pos, cos_t, sin_t, max_pos,
                                                                     (float*)q_out, (float*)k_cache, (float*)v_cache,
                                                                     block_table, table_stride, n_pages, page, nh, nkv,
                                                                     hd, write_kv, hpb, status);
        return esp_launch_status();
    }
    const int heads_per_block = n_tokens <= 64 ? 1 : 8;
    const dim3 grid(n_tokens, (nh + 2 * nkv + heads_per_block - 1) / heads_per_block);
    const int threads = heads_per_block == 1 ? (hd >= 128 ? 128 : (hd + 31) / 32 * 32) : 256;
    if (is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, rope_kvwrite_kernel<bf16>, dim3(grid), dim3(threads), 0, stream, qkv, bias, tok_seq, tok_pos, cos_t, sin_t, rot, max_pos,
                                                               (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, block_table,
                                                               table_stride, n_pages, page, nh, nkv, hd, write_kv, heads_per_block, status);
    else
        esp_launch_pdl(ESP_PDL_SMALL, rope_kvwrite_kernel<float>, dim3(grid), dim3(threads), 0, stream, qkv, bias, tok_seq, tok_pos, cos_t, sin_t, rot, max_pos,
                                                                (float*)q_out, (float*)k_cache, (float*)v_cache,
                                                                block_table, table_stride, n_pages, page, nh, nkv, hd,
                                                                write_kv, heads_per_block, status);
    return esp_launch_status();
}
