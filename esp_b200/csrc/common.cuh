// Shared device helpers for every kernel file of this library (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ESP_API extern "C" __attribute__((visibility("default")))

// Status bits that kernels OR into the engine's device status word.
enum : int {
    ESP_STATUS_ROUTER_NONFINITE = 1,   // a router probability was not finite or the top-k mass was <= 0
    ESP_STATUS_LOGITS_NONFINITE = 2,   // a logits row holds a NaN or an infinity
    ESP_STATUS_WAIT_EXPIRED = 4,       // a bounded wait inside a kernel ran out
    ESP_STATUS_BAD_INDEX = 8,          // an index read from device memory was out of range and was skipped
    ESP_STATUS_SMEM_LAYOUT = 16,       // a block's shared memory did not start where its layout needs it: it did not run
};

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Warp sum with a fixed butterfly order: the result does not depend on which
// other warps or blocks run beside this one.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max over blockDim.x threads (a multiple of 32, at most 1024).
// ``scratch`` holds at least 33 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Launch-error helper: the C entry points return cudaGetLastError() as an int.
static inline int esp_launch_status() { return (int)cudaGetLastError(); }
