// SwiGLU activation on the stacked gate|up product:  a[t, f] = silu(gu[t, f]) * gu[t, F + f],
// silu(g) = g * sigmoid(g), in 32-bit (src/transformer/ffn.zig:23-30, src/cuda/layer_kernels.cu:62-70).
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int F, size_t total) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / F, f = i % F;
    const float g = to_float(gu[t * 2 * F + f]);
    const float u = to_float(gu[t * 2 * F + F + f]);
    out[i] = from_float<T>(g / (1.f + expf(-g)) * u);
}

// bfloat16 rows with F a multiple of 8: one thread per 8 outputs, 16-byte loads and stores
__global__ void silu_mul_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gu, int F8, size_t total8) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const size_t t = i / F8, f = (i % F8) * 8;
    const size_t F = (size_t)F8 * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * F + f);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * F + F + f);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 g = __bfloat1622float2(gp[j]), u = __bfloat1622float2(up[j]);
        // the fast exponential and division: their error (a few 2^-22) is far below the result's rounding to bfloat16
        op[j] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * F + f) = o4;
}

ZAI_API int zai_silu_mul(void* out, const void* gu, int dtype, int N, int F, cudaStream_t stream) {
    const size_t total = (size_t)N * F;
    if (total == 0) return ZAI_OK;
    const int threads = 256;
    if (dtype == ZAI_BF16 && (F & 7) == 0) {
        const size_t total8 = total / 8;
        return launch_pdl(silu_mul_bf16x8_kernel, dim3((unsigned)((total8 + threads - 1) / threads)), dim3(threads), 0,
                          stream, (bf16*)out, (const bf16*)gu, F / 8, total8);
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    ZAI_DISPATCH(dtype, return launch_pdl(silu_mul_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (T*)out, (const T*)gu, F, total));
}
