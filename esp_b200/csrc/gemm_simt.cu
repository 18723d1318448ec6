// Plain tiled matrix product on the CUDA cores with true 32-bit multiply-adds:
//   C[m, n] = (sum_k A[row(m), k] * W[g][n, k] + bias[n]) * row_scale[m]
// A and W may be float or bfloat16 (widened exactly), the sum is float, C is
// float or bfloat16.  Each output element adds its products in the order
// k = 0, 1, 2, ... whatever the tile it falls in, so a row's result does not
// depend on how many other rows are in the call.  This is the 32-bit path of
// every projection and the fallback for weight dtypes that the fast kernels
// do not take.
//
// Grouped form: rows are sorted by group, group g owns rows
// [group_offsets[g], group_offsets[g+1]) and its own [N, K] slice of W.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const int* __restrict__ a_rows, const TW* __restrict__ W,
                 const float* __restrict__ bias, const float* __restrict__ row_scale, TC* __restrict__ C,
                 const int* __restrict__ group_offsets, int M, int N, int K, long long lda, long long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    int m_begin = 0, m_end = M;
    const TW* Wg = W;
    if (group_offsets) {
        m_begin = group_offsets[blockIdx.z];
        m_end = group_offsets[blockIdx.z + 1];
        Wg = W + (size_t)blockIdx.z * N * K;
    }
    const int m0 = m_begin + blockIdx.y * BM;
    if (m0 >= m_end) return;
    const int n0 = blockIdx.x * BN;
    const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
    const int lrow = tid / 4, lk = (tid % 4) * 4;

    const int am = m0 + lrow;
    const TA* a_src = nullptr;
    if (am < m_end) a_src = A + (size_t)(a_rows ? a_rows[am] : am) * lda;
    const int wn = n0 + lrow;
    const TW* w_src = wn < N ? Wg + (size_t)wn * K : nullptr;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + lk + j;
            As[lk + j][lrow] = (a_src && k < K) ? to_f32(a_src[k]) : 0.f;
            Ws[lk + j][lrow] = (w_src && k < K) ? to_f32(w_src[k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; j++) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + ty * TM + i;
        if (m >= m_end) continue;
        const float scale = row_scale ? row_scale[m] : 1.0f;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            if (row_scale) v *= scale;
            C[(size_t)m * ldc + n] = from_f32<TC>(v);
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch(const void* A, const int* a_rows, const void* W, const float* bias, const float* row_scale, void* C,
           const int* group_offsets, int groups, int M, int N, int K, long long lda, long long ldc, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, group_offsets ? groups : 1);
    gemm_simt_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>((const TA*)A, a_rows, (const TW*)W, bias, row_scale, (TC*)C,
                                                           group_offsets, M, N, K, lda, ldc);
    return esp_launch_status();
}
}  // namespace

// dtype codes: 0 = float, 1 = bfloat16.  M is the total number of rows (for the
// grouped form: the upper bound of any group's row count as well).
ESP_API int esp_gemm_simt(const void* A, int a_dtype, const int* a_rows, const void* W, int w_dtype, const float* bias,
                          const float* row_scale, void* C, int c_dtype, const int* group_offsets, int groups, int M,
                          int N, int K, long long lda, long long ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if ((long long)((M + BM - 1) / BM) > 65535 || groups > 65535) return (int)cudaErrorInvalidValue;
    const int code = a_dtype * 4 + w_dtype * 2 + c_dtype;
#define ESP_CASE(code_, TA, TW, TC) \
    case code_: return launch<TA, TW, TC>(A, a_rows, W, bias, row_scale, C, group_offsets, groups, M, N, K, lda, ldc, stream);
    switch (code) {
        ESP_CASE(0, float, float, float)
        ESP_CASE(1, float, float, bf16)
        ESP_CASE(2, float, bf16, float)
        ESP_CASE(3, float, bf16, bf16)
        ESP_CASE(4, bf16, float, float)
        ESP_CASE(5, bf16, float, bf16)
        ESP_CASE(6, bf16, bf16, float)
        ESP_CASE(7, bf16, bf16, bf16)
    }
#undef ESP_CASE
    return (int)cudaErrorInvalidValue;
}
