// Shared helpers of the sm_100a kernels: element types, warp and block reductions, and the C ABI
// conventions of the launchers (every launcher takes raw device pointers and a stream, launches on
// that stream and returns the CUDA error code of the launch, 0 for success).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define ZAI_API extern "C" __attribute__((visibility("default")))

enum ZaiDtype { ZAI_F32 = 0, ZAI_BF16 = 1 };
enum ZaiError { ZAI_OK = 0, ZAI_BAD_DTYPE = -1, ZAI_BAD_SIZE = -2 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // `red` may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// Calls `expr` with T bound to the element type that `dtype` names.
#define ZAI_DISPATCH(dtype, ...)                                   \
    do {                                                           \
        if ((dtype) == ZAI_F32) { typedef float T; __VA_ARGS__; }  \
        else if ((dtype) == ZAI_BF16) { typedef bf16 T; __VA_ARGS__; } \
        else return ZAI_BAD_DTYPE;                                 \
    } while (0)
