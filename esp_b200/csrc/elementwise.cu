// Embedding lookup, residual add + RMSNorm, SwiGLU product, finite check and
// the counter-based normal fill used for random weights.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// x[n, :] = scale * float(table[ids[n], :]); the residual stream is 32-bit in every mode.  ``scale`` is 1 for
// models that feed the table rows as they are (multiplying by 1 changes no bit).
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids, float* __restrict__ x,
                                    int n_tokens, int width, int vocab, float scale, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    if (n >= n_tokens) return;
    int id = ids[n];
    if (id < 0 || id >= vocab) {       // never read outside the table
        if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
        id = 0;
    }
    const TW* row = table + (size_t)id * width;
    float* out = x + (size_t)n * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = scale * to_f32(row[i]);
}

ESP_API int esp_embed_gather(const void* table, int table_is_bf16, const int* ids, float* x, int n_tokens, int width,
                             int vocab, float scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (table_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, embed_gather_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream, (const bf16*)table, ids, x, n_tokens, width, vocab, scale,
                                                                status);
    else
        esp_launch_pdl(ESP_PDL_SMALL, embed_gather_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (const float*)table, ids, x, n_tokens, width, vocab, scale,
                                                                 status);
    return esp_launch_status();
}

// ---------------------------------------------------------------- token ids from the last step's choices
// ids[j] = picks[src[j]] where src[j] >= 0: a step that follows a step can take its tokens from the device,
// before the host has seen them.
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ picks, const int* __restrict__ src, int n) {
    pdl_trigger();
    pdl_wait();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n && src[j] >= 0) ids[j] = picks[src[j]];
}

ESP_API int esp_feed_tokens(int* ids, const int* picks, const int* src, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    esp_launch_pdl(ESP_PDL_SMALL, feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, ids, picks, src, n);
    return esp_launch_status();
}

// ---------------------------------------------------------------- add + RMSNorm
// Row r works on source row s = rows ? rows[r] : r.
//   v = x[s] + (y ? y[s] : 0);  if (write_x) x[s] = v;
//   h[r] = v * (1 / sqrt(mean(v^2) + eps)) * gamma       (all in 32-bit)
// ``h32`` (may be null) receives the same rows unrounded, for consumers that
// must work from 32-bit values whatever the activation dtype (the router).
// The sum of squares is taken per thread in index order and combined by a
// fixed tree, so a row's result does not depend on the rest of the batch.
template <typename TH>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gamma,
                                   const int* __restrict__ rows, TH* __restrict__ h, float* __restrict__ h32, int width,
                                   float eps, int write_x) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + s * width;
    const float* yr = y ? y + s * width : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = xr[i];
        if (yr) {
            v += yr[i];
            if (write_x) xr[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    TH* hr = h + (size_t)r * width;
    float* h32r = h32 ? h32 + (size_t)r * width : nullptr;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = xr[i];
        if (yr && !write_x) v += yr[i];
        const float o = v * inv * gamma[i];
        hr[i] = from_f32<TH>(o);
        if (h32r) h32r[i] = o;
    }
}

// Same operation for rows whose width is a multiple of 4 and at most 4 * 4 * 1024: each thread keeps up
// to four float4 pieces of the row in registers, so x and y are read once and nothing is read back.
// The sum of squares is taken per thread in piece order and combined by the same fixed tree.
template <typename TH>
__global__ void __launch_bounds__(1024)
add_rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gamma,
                        const int* __restrict__ rows, TH* __restrict__ h, float* __restrict__ h32, int width, float eps,
                        int write_x) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    const int pieces = width / 4;
    float4* xr = reinterpret_cast<float4*>(x + s * width);
    const float4* yr = y ? reinterpret_cast<const float4*>(y + s * width) : nullptr;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) {
            v[i] = xr[q];
            if (yr) {
                const float4 a = yr[q];
                v[i].x += a.x; v[i].y += a.y; v[i].z += a.z; v[i].w += a.w;
                if (write_x) xr[q] = v[i];
            }
            ss = fmaf(v[i].x, v[i].x, ss);
            ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss);
            ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) {
            const float4 gm = reinterpret_cast<const float4*>(gamma)[q];
            const float o0 = v[i].x * inv * gm.x, o1 = v[i].y * inv * gm.y, o2 = v[i].z * inv * gm.z, o3 = v[i].w * inv * gm.w;
            TH* hr = h + (size_t)r * width + 4 * q;
            Vec4<TH>::store(hr, o0, o1, o2, o3);
            if (h32) reinterpret_cast<float4*>(h32 + (size_t)r * width)[q] = make_float4(o0, o1, o2, o3);
        }
    }
}

ESP_API int esp_add_rmsnorm(float* x, const float* y, const float* gamma, const int* rows, void* h, int h_is_bf16,
                            float* h32, int n_rows, int width, float eps, int write_x, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width % 4 == 0 && width <= 16384) {
        int threads = ((width / 4 + 3) / 4 + 31) / 32 * 32;       // up to four pieces per thread
        // one piece per thread while a block can hold them: a row's sum then has the same order whatever else is in
        // the step (the 32-bit path relies on it).  Many rows rounded to bfloat16: four pieces per thread, smaller
        // blocks, more rows in flight per SM.
        if (width / 4 <= 1024 && !(h_is_bf16 && n_rows >= 256)) threads = (width / 4 + 31) / 32 * 32;
        if (h_is_bf16)
            esp_launch_pdl(ESP_PDL_SMALL, add_rmsnorm_rows_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, y, gamma, rows, (bf16*)h, h32, width, eps, write_x);
        else
            esp_launch_pdl(ESP_PDL_SMALL, add_rmsnorm_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, y, gamma, rows, (float*)h, h32, width, eps, write_x);
        return esp_launch_status();
    }
    const int threads = width >= 1024 ? 256 : 128;
    if (h_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, add_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, y, gamma, rows, (bf16*)h, h32, width, eps, write_x);
    else
        esp_launch_pdl(ESP_PDL_SMALL, add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, y, gamma, rows, (float*)h, h32, width, eps, write_x);
    return esp_launch_status();
}

// ---------------------------------------------------------------- SwiGLU product
// act[m, i] = silu(gu[m, i]) * gu[m, inter + i], gu being [rows, 2*inter] in 32-bit.
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gu, TO* __restrict__ act, long long rows, int inter) {
    const long long total = rows * inter;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long m = idx / inter;
        const int i = (int)(idx - m * inter);
        const float g = gu[m * 2 * inter + i];
        const float u = gu[m * 2 * inter + inter + i];
        act[idx] = from_f32<TO>(g / (1.0f + expf(-g)) * u);
    }
}

ESP_API int esp_swiglu(const float* gu, void* act, int act_is_bf16, long long rows, int inter, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const long long total = rows * inter;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    if (act_is_bf16)
        swiglu_kernel<bf16><<<blocks, 256, 0, stream>>>(gu, (bf16*)act, rows, inter);
    else
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>(gu, (float*)act, rows, inter);
    return esp_launch_status();
}

// ---------------------------------------------------------------- row gather
// out[r, :] = src[rows[r], :] for bfloat16 rows whose width is a multiple of 8 (16-byte pieces).
__global__ void gather_rows_kernel(const bf16* __restrict__ src, const int* __restrict__ rows, bf16* __restrict__ out,
                                   int n_rows, int pieces) {
    const long long total = (long long)n_rows * pieces;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(idx / pieces), q = (int)(idx - (long long)r * pieces);
        reinterpret_cast<uint4*>(out)[idx] = reinterpret_cast<const uint4*>(src)[(size_t)rows[r] * pieces + q];
    }
}

ESP_API int esp_gather_rows(const void* src, const int* rows, void* out, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width % 8 != 0) return (int)cudaErrorInvalidValue;
    const long long total = (long long)n_rows * (width / 8);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    gather_rows_kernel<<<(int)blocks, 256, 0, stream>>>((const bf16*)src, rows, (bf16*)out, n_rows, width / 8);
    return esp_launch_status();
}

// ---------------------------------------------------------------- finite check
// ORs ``bit`` into *status if any value is a NaN or an infinity.  bfloat16 values are tested on their bits
// (an exponent of all ones), 16 bytes at a time where the count allows.
template <typename T>
__global__ void finite_check_kernel(const T* __restrict__ v, long long count, int* __restrict__ status, int bit) {
    pdl_trigger();
    pdl_wait();
    bool bad = false;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        bad |= !isfinite(to_f32(v[i]));
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(status, bit);
}

__global__ void finite_check_bf16x8_kernel(const uint4* __restrict__ v, long long pieces, int* __restrict__ status, int bit) {
    bool bad = false;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < pieces; i += (long long)gridDim.x * blockDim.x) {
        const uint4 q = v[i];
        const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; j++)
            bad |= ((w[j] & 0x7F80u) == 0x7F80u) || ((w[j] & 0x7F800000u) == 0x7F800000u);
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(status, bit);
}

ESP_API int esp_finite_check(const void* v, int is_bf16, long long count, int* status, int bit, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (is_bf16) {
        const long long pieces = ((uintptr_t)v & 15) ? 0 : count / 8;
        if (pieces > 0) {
            long long blocks = (pieces + 255) / 256;
            if (blocks > 148 * 16) blocks = 148 * 16;
            finite_check_bf16x8_kernel<<<(int)blocks, 256, 0, stream>>>((const uint4*)v, pieces, status, bit);
        }
        const long long rest = count - pieces * 8;
        if (rest > 0)
            finite_check_kernel<bf16><<<(int)((rest + 255) / 256 > 1184 ? 1184 : (rest + 255) / 256), 256, 0, stream>>>(
                (const bf16*)v + pieces * 8, rest, status, bit);
        return esp_launch_status();
    }
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    esp_launch_pdl(ESP_PDL_SMALL, finite_check_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (const float*)v, count, status,
                   bit);
    return esp_launch_status();
}

// ---------------------------------------------------------------- logit soft-cap
// v = cap * tanh(v / cap), in place, for heads that bound their logits this way.
__global__ void softcap_kernel(float* __restrict__ v, long long count, float cap) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        v[i] = cap * tanhf(v[i] / cap);
}

ESP_API int esp_softcap(float* v, long long count, float cap, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    softcap_kernel<<<(int)blocks, 256, 0, stream>>>(v, count, cap);
    return esp_launch_status();
}

// ---------------------------------------------------------------- random normal fill
// value(i) = mean + std * z(i), z from a counter-based generator: two 64-bit
// mixes of (key + i) give two uniforms, Box-Muller gives the normal.  The value
// of an element depends on (key, i) only, not on the launch shape.
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void normal_fill_kernel(T* __restrict__ out, long long count, unsigned long long key, float mean, float stddev) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long a = mix64(key + 2ull * (unsigned long long)i);
        const unsigned long long b = mix64(key + 2ull * (unsigned long long)i + 1ull);
        const float u1 = ((float)(a >> 40) + 1.0f) * (1.0f / 16777216.0f);   // (0, 1]
        const float u2 = (float)(b >> 40) * (1.0f / 16777216.0f);            // [0, 1)
        const float z = sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
        out[i] = from_f32<T>(mean + stddev * z);
    }
}

ESP_API int esp_normal_fill(void* out, int out_is_bf16, long long count, unsigned long long key, float mean, float stddev,
                            cudaStream_t stream) {
    if (count <= 0) return 0;
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (out_is_bf16)
        normal_fill_kernel<bf16><<<(int)blocks, 256, 0, stream>>>((bf16*)out, count, key, mean, stddev);
    else
        normal_fill_kernel<float><<<(int)blocks, 256, 0, stream>>>((float*)out, count, key, mean, stddev);
    return esp_launch_status();
}
