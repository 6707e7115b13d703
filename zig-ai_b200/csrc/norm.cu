// RMSNorm fused with the residual addition before it:  h += delta;  out = h * rsqrt(mean(h^2) + eps) * gamma.
// The residual stream h is 32-bit and the sum, the mean of squares and the scaling are 32-bit; only
// `out` is rounded to the model's dtype.  Formula: src/transformer/norm.zig:14-32; the reference's
// device kernel (src/cuda/layer_kernels.cu:17-43) and its separate residual kernels (:46-59) are
// one kernel here.  The order of the reduction depends only on the row width, so a row's result
// does not depend on what else is in the batch.
#include "common.cuh"

template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                   const float* __restrict__ gamma, T* __restrict__ out, float eps, int H) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = h[base + c];
        if (delta) {
            v += to_float(delta[base + c]);
            h[base + c] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        out[base + c] = from_float<T>(h[base + c] * inv * gamma[c]);
}

ZAI_API int zai_add_rmsnorm(float* h, const void* delta, const float* gamma, void* out, int dtype, float eps,
                            int N, int H, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    const int threads = H >= 2048 ? 512 : 256;
    ZAI_DISPATCH(dtype, return launch_pdl(add_rmsnorm_kernel<T>, dim3(N), dim3(threads), 0, stream, h, (const T*)delta, gamma, (T*)out, eps, H));
}
