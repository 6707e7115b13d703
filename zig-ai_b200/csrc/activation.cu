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

ZAI_API int zai_silu_mul(void* out, const void* gu, int dtype, int N, int F, cudaStream_t stream) {
    const size_t total = (size_t)N * F;
    if (total == 0) return ZAI_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    ZAI_DISPATCH(dtype, return launch_pdl(silu_mul_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (T*)out, (const T*)gu, F, total));
}
