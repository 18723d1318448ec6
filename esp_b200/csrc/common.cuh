// Shared device helpers for every kernel file of this library (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

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

// four consecutive values stored as one piece (16 bytes of float, 8 of bfloat16); p is aligned to the piece
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void store(bf16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<unsigned*>(&lo);
        v.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(p) = v;
    }
};

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

// ---- programmatic dependent launch ---------------------------------------------------------------------
// A decode step is a chain of short kernels.  A kernel launched with esp_launch_pdl may be set up on the SMs
// while the kernel before it in the stream is still running: its blocks start, do what needs nothing of the
// predecessor (index arithmetic, the first loads of weights, which no kernel ever writes), and call pdl_wait()
// before they read anything the predecessor wrote and before they write anything at all (the predecessor, or
// the kernels before it, may still read what this kernel would overwrite).  pdl_wait() returns once the
// predecessor has finished and its writes are visible; as the predecessor itself has waited for its own
// predecessor, everything earlier in the stream is finished as well.  pdl_trigger() tells the scheduler that the
// next kernel may be set up; it is called at the top, so that the next kernel's set-up overlaps as much as it can.
// In a kernel launched the ordinary way both calls do nothing.  ESP_B200_PDL=0 turns the attribute off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

#define ESP_PDL_DEFAULT_MASK 61
// classes of kernels, so that the attribute can be tried class by class: ESP_B200_PDL is a bit mask.  GROUPED: every
// grouped product (off: it holds SM room while it waits for the routing); GROUPED_AFTER: a second grouped product
// whose offsets were complete before the first one started; GROUPED_FITS: a short grouped product (gemm_skinny.cu).
enum : int { ESP_PDL_DENSE = 1, ESP_PDL_GROUPED = 2, ESP_PDL_ATTENTION = 4, ESP_PDL_SMALL = 8, ESP_PDL_GROUPED_AFTER = 16,
              ESP_PDL_GROUPED_FITS = 32 };
static inline bool esp_pdl_enabled(int kind) {
    static int mask = -1;
    if (mask < 0) {
        const char* e = getenv("ESP_B200_PDL");
        mask = e ? atoi(e) : ESP_PDL_DEFAULT_MASK;
    }
    return (mask & kind) != 0;
}

// kernel<<<grid, block, smem, stream>>>(args...) with the attribute that lets the kernel be set up before its
// predecessor in the stream has finished.  Only for kernels that call pdl_wait() as described above.
template <typename... KArgs, typename... Args>
static inline void esp_launch_pdl(int kind, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = esp_pdl_enabled(kind) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
