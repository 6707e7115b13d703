// Between the qkv projection and attention: per-head RMSNorm of q and k over the head size, the
// rotary position encoding of q and k, and the write of k and v into the request's pages.
//
//   q, k <- x * rsqrt(mean(x^2) + eps) * gamma            (src/transformer/hybrid_attn.zig:371-382; device :719,723)
//   for i < n/2: (x[i], x[i+n/2]) <- (a cos - b sin, a sin + b cos), angle = pos * inv_freq[i]
//                                                         (half-split pairing, src/cuda/layer_kernels.cu:353-365)
//   pages[page(pos), 0|1, kv_head, pos % page_size, :] <- k | v      (the reference's kvAppendF16Kernel,
//                                                         src/cuda/layer_kernels.cu:372-398, with its own layout)
//
// The position is the token's own absolute position (the reference's kernel takes `row % N`,
// layer_kernels.cu:351).  v is neither normed nor rotated.  The norm is 32-bit; the angle is the
// product of the position and a frequency table computed on the host in 64-bit, and its sine and
// cosine are taken in 64-bit and rounded to 32-bit once per token and step (rope_table_kernel),
// then shared by all heads and all layers with the same rotation.
// One block per token; each warp takes heads in turn.
#include "common.cuh"

// table[t][i] = (cos, sin) of positions[t] * inv_freq[i]
__global__ void rope_table_kernel(float2* __restrict__ table, const int* __restrict__ positions,
                                  const double* __restrict__ inv_freq, int N, int half) {
    pdl_trigger();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * half) return;
    const int t = idx / half, i = idx % half;
    double s, c;
    sincos((double)positions[t] * inv_freq[i], &s, &c);
    table[idx] = make_float2((float)c, (float)s);
}

template <typename T>
__global__ void qk_norm_rope_kernel(const T* __restrict__ qkv, int qkv_cols, const float* __restrict__ q_gamma,
                                    const float* __restrict__ k_gamma, float eps, const float2* __restrict__ cs_table,
                                    int rot, const int* __restrict__ positions, const int* __restrict__ seq_idx,
                                    const int* __restrict__ block_table, int table_width, T* __restrict__ pages,
                                    int page_size, T* __restrict__ q_out, T* __restrict__ k_out, int Hq, int Hkv,
                                    int D, int has_kv, int write) {
    extern __shared__ float smem[];
    const int half = rot / 2;
    float* cs = smem;                       // [half] cos
    float* sn = smem + half;                // [half] sin
    const int nwarp = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = smem + 2 * half + (size_t)warp * D;
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float2 v = cs_table[(size_t)t * half + i];
        cs[i] = v.x;
        sn[i] = v.y;
    }
    __syncthreads();
    size_t page_base = 0;
    int off = 0;
    if (has_kv && write) {
        const int page = block_table[(size_t)seq_idx[t] * table_width + pos / page_size];
        off = pos % page_size;
        page_base = (size_t)page * 2 * Hkv * page_size * D;
    }
    const int n_heads = Hq + (has_kv ? 2 * Hkv : 0);
    const T* row = qkv + (size_t)t * qkv_cols;
    for (int h = warp; h < n_heads; h += nwarp) {
        const T* x = row + (size_t)h * D;
        if (h >= Hq + Hkv) {                                  // a value head: copy into its page
            if (write) {
                T* dst = pages + page_base + (((size_t)1 * Hkv + (h - Hq - Hkv)) * page_size + off) * D;
                for (int d = lane; d < D; d += 32) dst[d] = x[d];
            }
            continue;
        }
        const bool is_q = h < Hq;
        const float* gamma = is_q ? q_gamma : k_gamma;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float v = to_float(x[d]);
            buf[d] = v;
            ss += v * v;
        }
        if (gamma) {
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)D + eps);
            for (int d = lane; d < D; d += 32) buf[d] = buf[d] * inv * gamma[d];
        }
        __syncwarp();
        T* dst = nullptr;
        T* dst2 = nullptr;
        if (is_q) {
            dst = q_out + ((size_t)t * Hq + h) * D;
        } else {
            if (write) dst = pages + page_base + (((size_t)0 * Hkv + (h - Hq)) * page_size + off) * D;
            if (k_out) dst2 = k_out + ((size_t)t * Hkv + (h - Hq)) * D;
        }
        for (int d = lane; d < D; d += 32) {
            float v;
            if (d < half) v = buf[d] * cs[d] - buf[d + half] * sn[d];
            else if (d < rot) v = buf[d - half] * sn[d - half] + buf[d] * cs[d - half];
            else v = buf[d];
            const T o = from_float<T>(v);
            if (dst) dst[d] = o;
            if (dst2) dst2[d] = o;
        }
        __syncwarp();
    }
}

// Writes already prepared k and v rows ([N, Hkv*D], row strides given) into the pages.
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k, int k_stride, const T* __restrict__ v, int v_stride,
                                const int* __restrict__ positions, const int* __restrict__ seq_idx,
                                const int* __restrict__ block_table, int table_width, T* __restrict__ pages,
                                int page_size, int Hkv, int D) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_idx[t] * table_width + pos / page_size];
    const int off = pos % page_size;
    const size_t base = (size_t)page * 2 * Hkv * page_size * D;
    for (int i = threadIdx.x; i < Hkv * D; i += blockDim.x) {
        const int h = i / D, d = i % D;
        pages[base + (((size_t)0 * Hkv + h) * page_size + off) * D + d] = k[(size_t)t * k_stride + i];
        pages[base + (((size_t)1 * Hkv + h) * page_size + off) * D + d] = v[(size_t)t * v_stride + i];
    }
}

ZAI_API int zai_rope_table(float2* table, const int* positions, const double* inv_freq, int N, int half,
                           cudaStream_t stream) {
    if (N <= 0 || half <= 0) return ZAI_OK;
    const int total = N * half;
    return launch_pdl(rope_table_kernel, dim3((total + 127) / 128), dim3(128), 0, stream, table, positions, inv_freq, N, half);
}

ZAI_API int zai_qk_norm_rope(const void* qkv, int qkv_cols, int dtype, const float* q_gamma, const float* k_gamma,
                             float eps, const float2* cs_table, int rot, const int* positions, const int* seq_idx,
                             const int* block_table, int table_width, void* pages, int page_size, void* q_out,
                             void* k_out, int N, int Hq, int Hkv, int D, int has_kv, int write,
                             cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (rot < 0 || rot > D || (rot & 1) || D < 1) return ZAI_BAD_SIZE;
    const int threads = 128;
    const size_t smem = (size_t)(rot + (threads / 32) * D) * sizeof(float);
    if (smem > 48 * 1024) return ZAI_BAD_SIZE;
    ZAI_DISPATCH(dtype, return launch_pdl(qk_norm_rope_kernel<T>, dim3(N), dim3(threads), smem, stream,
        (const T*)qkv, qkv_cols, q_gamma, k_gamma, eps, cs_table, rot, positions, seq_idx, block_table,
        table_width, (T*)pages, page_size, (T*)q_out, (T*)k_out, Hq, Hkv, D, has_kv, write));
}

ZAI_API int zai_kv_write(const void* k, int k_stride, const void* v, int v_stride, int dtype, const int* positions,
                         const int* seq_idx, const int* block_table, int table_width, void* pages, int page_size,
                         int N, int Hkv, int D, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    ZAI_DISPATCH(dtype, return launch_pdl(kv_write_kernel<T>, dim3(N), dim3(128), 0, stream,
        (const T*)k, k_stride, (const T*)v, v_stride, positions, seq_idx, block_table, table_width, (T*)pages,
        page_size, Hkv, D));
}
