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

// Rows with H a multiple of 4 and at most 4 * 256 * VEC: each thread keeps its 4 * VEC values in
// registers, so the row is read once.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) add_rmsnorm_vec_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                                              const float* __restrict__ gamma, T* __restrict__ out,
                                                              float eps, int H) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float4 v[VEC];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int c = (threadIdx.x + i * 256) * 4;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < H) {
            v[i] = *reinterpret_cast<const float4*>(h + base + c);
            if (delta) {
                v[i].x += to_float(delta[base + c]);
                v[i].y += to_float(delta[base + c + 1]);
                v[i].z += to_float(delta[base + c + 2]);
                v[i].w += to_float(delta[base + c + 3]);
                *reinterpret_cast<float4*>(h + base + c) = v[i];
            }
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int c = (threadIdx.x + i * 256) * 4;
        if (c < H) {
            const float4 g = *reinterpret_cast<const float4*>(gamma + c);
            out[base + c] = from_float<T>(v[i].x * inv * g.x);
            out[base + c + 1] = from_float<T>(v[i].y * inv * g.y);
            out[base + c + 2] = from_float<T>(v[i].z * inv * g.z);
            out[base + c + 3] = from_float<T>(v[i].w * inv * g.w);
        }
    }
}

ZAI_API int zai_add_rmsnorm(float* h, const void* delta, const float* gamma, void* out, int dtype, float eps,
                            int N, int H, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if ((H & 3) == 0 && H <= 8192) {
        if (H <= 1024) { ZAI_DISPATCH(dtype, return launch_pdl(add_rmsnorm_vec_kernel<T, 1>, dim3(N), dim3(256), 0, stream, h, (const T*)delta, gamma, (T*)out, eps, H)); }
        if (H <= 2048) { ZAI_DISPATCH(dtype, return launch_pdl(add_rmsnorm_vec_kernel<T, 2>, dim3(N), dim3(256), 0, stream, h, (const T*)delta, gamma, (T*)out, eps, H)); }
        if (H <= 4096) { ZAI_DISPATCH(dtype, return launch_pdl(add_rmsnorm_vec_kernel<T, 4>, dim3(N), dim3(256), 0, stream, h, (const T*)delta, gamma, (T*)out, eps, H)); }
        ZAI_DISPATCH(dtype, return launch_pdl(add_rmsnorm_vec_kernel<T, 8>, dim3(N), dim3(256), 0, stream, h, (const T*)delta, gamma, (T*)out, eps, H));
    }
    const int threads = H >= 2048 ? 512 : 256;
    ZAI_DISPATCH(dtype, return launch_pdl(add_rmsnorm_kernel<T>, dim3(N), dim3(threads), 0, stream, h, (const T*)delta, gamma, (T*)out, eps, H));
}
