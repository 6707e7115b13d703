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
                                    int D, int has_kv, int write, int num_pages, int* __restrict__ status) {
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
        const int page = zai_checked_page(block_table + (size_t)seq_idx[t] * table_width, table_width,
                                          pos < 0 ? -1 : pos / page_size, num_pages, status);
        off = pos < 0 ? 0 : pos % page_size;
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

// bfloat16, the whole head rotated (rot == D), D = 8 * TPH with TPH a power of two up to 32: TPH threads
// share a head, each with four values of the lower half and their four partners of the upper half,
// and ask for everything they need (the row, the norm's weight, cosines and sines) at once.
template <int TPH>
__global__ void __launch_bounds__(256) qk_norm_rope_vec_kernel(
    const bf16* __restrict__ qkv, int qkv_cols, const float* __restrict__ q_gamma, const float* __restrict__ k_gamma,
    float eps, const float2* __restrict__ cs_table, const int* __restrict__ positions, const int* __restrict__ seq_idx,
    const int* __restrict__ block_table, int table_width, bf16* __restrict__ pages, int page_size,
    bf16* __restrict__ q_out, bf16* __restrict__ k_out, int N, int Hq, int Hkv, int has_kv, int write, int num_pages,
    int* __restrict__ status) {
    constexpr int D = 8 * TPH, half = 4 * TPH;
    pdl_trigger();
    pdl_wait();
    const int n_heads = Hq + (has_kv ? 2 * Hkv : 0);
    const long long item = (long long)blockIdx.x * (256 / TPH) + threadIdx.x / TPH;
    if (item >= (long long)N * n_heads) return;                    // (a whole group of TPH lanes leaves together)
    const int t = (int)(item / n_heads), h = (int)(item % n_heads), d0 = (threadIdx.x % TPH) * 4;
    const bf16* x = qkv + (size_t)t * qkv_cols + (size_t)h * D;
    const uint2 lo2 = *reinterpret_cast<const uint2*>(x + d0), hi2 = *reinterpret_cast<const uint2*>(x + half + d0);
    const bool is_q = h < Hq, is_v = h >= Hq + Hkv;
    size_t page_base = 0;
    int off = 0;
    if (!is_q && write) {
        const int pos = positions[t];
        const int page = zai_checked_page(block_table + (size_t)seq_idx[t] * table_width, table_width,
                                          pos < 0 ? -1 : pos / page_size, num_pages, status);
        off = pos < 0 ? 0 : pos % page_size;
        page_base = (size_t)page * 2 * Hkv * page_size * D;
    }
    if (is_v) {
        if (write) {
            bf16* dst = pages + page_base + (((size_t)Hkv + (h - Hq - Hkv)) * page_size + off) * D;
            *reinterpret_cast<uint2*>(dst + d0) = lo2;
            *reinterpret_cast<uint2*>(dst + half + d0) = hi2;
        }
        return;
    }
    const float* gamma = is_q ? q_gamma : k_gamma;
    float4 glo = make_float4(1.f, 1.f, 1.f, 1.f), ghi = glo;
    if (gamma) {
        glo = *reinterpret_cast<const float4*>(gamma + d0);
        ghi = *reinterpret_cast<const float4*>(gamma + half + d0);
    }
    const float4 cs01 = *reinterpret_cast<const float4*>(cs_table + (size_t)t * half + d0);        // (cos, sin) of d0, d0+1
    const float4 cs23 = *reinterpret_cast<const float4*>(cs_table + (size_t)t * half + d0 + 2);
    float lo[4], hi[4];
    {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lo2.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lo2.y));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hi2.x));
        const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hi2.y));
        lo[0] = a.x; lo[1] = a.y; lo[2] = b.x; lo[3] = b.y;
        hi[0] = c.x; hi[1] = c.y; hi[2] = d.x; hi[3] = d.y;
    }
    if (gamma) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
#pragma unroll
        for (int o = TPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss / (float)D + eps);
        const float gl[4] = {glo.x, glo.y, glo.z, glo.w}, gh[4] = {ghi.x, ghi.y, ghi.z, ghi.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            lo[e] = lo[e] * inv * gl[e];
            hi[e] = hi[e] * inv * gh[e];
        }
    }
    const float cs[4] = {cs01.x, cs01.z, cs23.x, cs23.z}, sn[4] = {cs01.y, cs01.w, cs23.y, cs23.w};
    float rl[4], rh[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        rl[e] = lo[e] * cs[e] - hi[e] * sn[e];
        rh[e] = lo[e] * sn[e] + hi[e] * cs[e];
    }
    uint2 ol, oh;
    {
        __nv_bfloat162 a = __floats2bfloat162_rn(rl[0], rl[1]), b = __floats2bfloat162_rn(rl[2], rl[3]);
        __nv_bfloat162 c = __floats2bfloat162_rn(rh[0], rh[1]), d = __floats2bfloat162_rn(rh[2], rh[3]);
        ol.x = *reinterpret_cast<uint32_t*>(&a); ol.y = *reinterpret_cast<uint32_t*>(&b);
        oh.x = *reinterpret_cast<uint32_t*>(&c); oh.y = *reinterpret_cast<uint32_t*>(&d);
    }
    if (is_q) {
        bf16* dst = q_out + ((size_t)t * Hq + h) * D;
        *reinterpret_cast<uint2*>(dst + d0) = ol;
        *reinterpret_cast<uint2*>(dst + half + d0) = oh;
    } else {
        if (write) {
            bf16* dst = pages + page_base + ((size_t)(h - Hq) * page_size + off) * D;
            *reinterpret_cast<uint2*>(dst + d0) = ol;
            *reinterpret_cast<uint2*>(dst + half + d0) = oh;
        }
        if (k_out) {
            bf16* dst = k_out + ((size_t)t * Hkv + (h - Hq)) * D;
            *reinterpret_cast<uint2*>(dst + d0) = ol;
            *reinterpret_cast<uint2*>(dst + half + d0) = oh;
        }
    }
}

// The same with 16-byte accesses: D = 16 * TPH, TPH threads share a head, each with eight values of the lower
// half and their eight partners of the upper half.
template <int TPH>
__global__ void __launch_bounds__(256) qk_norm_rope_vec8_kernel(
    const bf16* __restrict__ qkv, int qkv_cols, const float* __restrict__ q_gamma, const float* __restrict__ k_gamma,
    float eps, const float2* __restrict__ cs_table, const int* __restrict__ positions, const int* __restrict__ seq_idx,
    const int* __restrict__ block_table, int table_width, bf16* __restrict__ pages, int page_size,
    bf16* __restrict__ q_out, bf16* __restrict__ k_out, int N, int Hq, int Hkv, int has_kv, int write, int num_pages,
    int* __restrict__ status) {
    constexpr int D = 16 * TPH, half = 8 * TPH;
    pdl_trigger();
    pdl_wait();
    const int n_heads = Hq + (has_kv ? 2 * Hkv : 0);
    const long long item = (long long)blockIdx.x * (256 / TPH) + threadIdx.x / TPH;
    if (item >= (long long)N * n_heads) return;                    // (a whole group of TPH lanes leaves together)
    const int t = (int)(item / n_heads), h = (int)(item % n_heads), d0 = (threadIdx.x % TPH) * 8;
    const bf16* x = qkv + (size_t)t * qkv_cols + (size_t)h * D;
    const uint4 lo4 = *reinterpret_cast<const uint4*>(x + d0), hi4 = *reinterpret_cast<const uint4*>(x + half + d0);
    const bool is_q = h < Hq, is_v = h >= Hq + Hkv;
    size_t page_base = 0;
    int off = 0;
    if (!is_q && write) {
        const int pos = positions[t];
        const int page = zai_checked_page(block_table + (size_t)seq_idx[t] * table_width, table_width,
                                          pos < 0 ? -1 : pos / page_size, num_pages, status);
        off = pos < 0 ? 0 : pos % page_size;
        page_base = (size_t)page * 2 * Hkv * page_size * D;
    }
    if (is_v) {
        if (write) {
            bf16* dst = pages + page_base + (((size_t)Hkv + (h - Hq - Hkv)) * page_size + off) * D;
            *reinterpret_cast<uint4*>(dst + d0) = lo4;
            *reinterpret_cast<uint4*>(dst + half + d0) = hi4;
        }
        return;
    }
    const float* gamma = is_q ? q_gamma : k_gamma;
    float lo[8], hi[8];
    {
        const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&lo4);
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&hi4);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 u = __bfloat1622float2(a[e]), v = __bfloat1622float2(b[e]);
            lo[2 * e] = u.x; lo[2 * e + 1] = u.y;
            hi[2 * e] = v.x; hi[2 * e + 1] = v.y;
        }
    }
    // (cos, sin) of d0 .. d0 + 7: four 16-byte loads
    float cs[8], sn[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float4 v = *reinterpret_cast<const float4*>(cs_table + (size_t)t * half + d0 + 2 * e);
        cs[2 * e] = v.x; sn[2 * e] = v.y; cs[2 * e + 1] = v.z; sn[2 * e + 1] = v.w;
    }
    if (gamma) {
        float gl[8], gh[8];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float4 u = *reinterpret_cast<const float4*>(gamma + d0 + 4 * e), v = *reinterpret_cast<const float4*>(gamma + half + d0 + 4 * e);
            gl[4 * e] = u.x; gl[4 * e + 1] = u.y; gl[4 * e + 2] = u.z; gl[4 * e + 3] = u.w;
            gh[4 * e] = v.x; gh[4 * e + 1] = v.y; gh[4 * e + 2] = v.z; gh[4 * e + 3] = v.w;
        }
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
#pragma unroll
        for (int o = TPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            lo[e] = lo[e] * inv * gl[e];
            hi[e] = hi[e] * inv * gh[e];
        }
    }
    uint4 ol, oh;
    {
        __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&ol);
        __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&oh);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 2 * e, j = 2 * e + 1;
            a[e] = __floats2bfloat162_rn(lo[i] * cs[i] - hi[i] * sn[i], lo[j] * cs[j] - hi[j] * sn[j]);
            b[e] = __floats2bfloat162_rn(lo[i] * sn[i] + hi[i] * cs[i], lo[j] * sn[j] + hi[j] * cs[j]);
        }
    }
    if (is_q) {
        bf16* dst = q_out + ((size_t)t * Hq + h) * D;
        *reinterpret_cast<uint4*>(dst + d0) = ol;
        *reinterpret_cast<uint4*>(dst + half + d0) = oh;
    } else {
        if (write) {
            bf16* dst = pages + page_base + ((size_t)(h - Hq) * page_size + off) * D;
            *reinterpret_cast<uint4*>(dst + d0) = ol;
            *reinterpret_cast<uint4*>(dst + half + d0) = oh;
        }
        if (k_out) {
            bf16* dst = k_out + ((size_t)t * Hkv + (h - Hq)) * D;
            *reinterpret_cast<uint4*>(dst + d0) = ol;
            *reinterpret_cast<uint4*>(dst + half + d0) = oh;
        }
    }
}

template <int TPH>
static int launch_qk_vec8(const void* qkv, int qkv_cols, const float* q_gamma, const float* k_gamma, float eps,
                          const float2* cs_table, const int* positions, const int* seq_idx, const int* block_table,
                          int table_width, void* pages, int page_size, void* q_out, void* k_out, int N, int Hq, int Hkv,
                          int has_kv, int write, int num_pages, int* status, cudaStream_t stream) {
    const long long items = (long long)N * (Hq + (has_kv ? 2 * Hkv : 0));
    const long long blocks = (items + 256 / TPH - 1) / (256 / TPH);
    if (blocks > 0x7fffffffLL) return ZAI_BAD_SIZE;
    return launch_pdl(qk_norm_rope_vec8_kernel<TPH>, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)qkv, qkv_cols,
                      q_gamma, k_gamma, eps, cs_table, positions, seq_idx, block_table, table_width, (bf16*)pages, page_size,
                      (bf16*)q_out, (bf16*)k_out, N, Hq, Hkv, has_kv, write, num_pages, status);
}

template <int TPH>
static int launch_qk_vec(const void* qkv, int qkv_cols, const float* q_gamma, const float* k_gamma, float eps,
                         const float2* cs_table, const int* positions, const int* seq_idx, const int* block_table,
                         int table_width, void* pages, int page_size, void* q_out, void* k_out, int N, int Hq, int Hkv,
                         int has_kv, int write, int num_pages, int* status, cudaStream_t stream) {
    const long long items = (long long)N * (Hq + (has_kv ? 2 * Hkv : 0));
    const long long blocks = (items + 256 / TPH - 1) / (256 / TPH);
    if (blocks > 0x7fffffffLL) return ZAI_BAD_SIZE;
    return launch_pdl(qk_norm_rope_vec_kernel<TPH>, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)qkv, qkv_cols,
                      q_gamma, k_gamma, eps, cs_table, positions, seq_idx, block_table, table_width, (bf16*)pages, page_size,
                      (bf16*)q_out, (bf16*)k_out, N, Hq, Hkv, has_kv, write, num_pages, status);
}

// Writes already prepared k and v rows ([N, Hkv*D], row strides given) into the pages.
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k, int k_stride, const T* __restrict__ v, int v_stride,
                                const int* __restrict__ positions, const int* __restrict__ seq_idx,
                                const int* __restrict__ block_table, int table_width, T* __restrict__ pages,
                                int page_size, int Hkv, int D, int num_pages, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int page = zai_checked_page(block_table + (size_t)seq_idx[t] * table_width, table_width,
                                      pos < 0 ? -1 : pos / page_size, num_pages, threadIdx.x == 0 ? status : nullptr);
    const int off = pos < 0 ? 0 : pos % page_size;
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
                             void* k_out, int N, int Hq, int Hkv, int D, int has_kv, int write, int num_pages,
                             int* status, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (rot < 0 || rot > D || (rot & 1) || D < 1) return ZAI_BAD_SIZE;
    // the vector kernel: bfloat16, the whole head rotated, 16-byte aligned rows and tables
    const uintptr_t all = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_gamma) | reinterpret_cast<uintptr_t>(k_gamma) |
                          reinterpret_cast<uintptr_t>(cs_table) | reinterpret_cast<uintptr_t>(pages) |
                          reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_out);
    if (dtype == ZAI_BF16 && rot == D && (D & 7) == 0 && (qkv_cols & 7) == 0 && (all & 15) == 0) {
        // many rows: 16 bytes a load (head sizes that are 16 times a power of two)
#define ZAI_QK_VEC8(tph) if (N >= 256 && D == 16 * tph) return launch_qk_vec8<tph>(qkv, qkv_cols, q_gamma, k_gamma, eps, cs_table, positions, \
        seq_idx, block_table, table_width, pages, page_size, q_out, k_out, N, Hq, Hkv, has_kv, write, num_pages, status, stream);
        ZAI_QK_VEC8(1) ZAI_QK_VEC8(2) ZAI_QK_VEC8(4) ZAI_QK_VEC8(8) ZAI_QK_VEC8(16)
#undef ZAI_QK_VEC8
#define ZAI_QK_VEC(tph) if (D == 8 * tph) return launch_qk_vec<tph>(qkv, qkv_cols, q_gamma, k_gamma, eps, cs_table, positions, \
        seq_idx, block_table, table_width, pages, page_size, q_out, k_out, N, Hq, Hkv, has_kv, write, num_pages, status, stream);
        ZAI_QK_VEC(2) ZAI_QK_VEC(4) ZAI_QK_VEC(8) ZAI_QK_VEC(16) ZAI_QK_VEC(32)
#undef ZAI_QK_VEC
    }
    const int threads = 128;
    const size_t smem = (size_t)(rot + (threads / 32) * D) * sizeof(float);
    if (smem > 48 * 1024) return ZAI_BAD_SIZE;
    ZAI_DISPATCH(dtype, return launch_pdl(qk_norm_rope_kernel<T>, dim3(N), dim3(threads), smem, stream,
        (const T*)qkv, qkv_cols, q_gamma, k_gamma, eps, cs_table, rot, positions, seq_idx, block_table,
        table_width, (T*)pages, page_size, (T*)q_out, (T*)k_out, Hq, Hkv, D, has_kv, write, num_pages, status));
}

ZAI_API int zai_kv_write(const void* k, int k_stride, const void* v, int v_stride, int dtype, const int* positions,
                         const int* seq_idx, const int* block_table, int table_width, void* pages, int page_size,
                         int N, int Hkv, int D, int num_pages, int* status, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    ZAI_DISPATCH(dtype, return launch_pdl(kv_write_kernel<T>, dim3(N), dim3(128), 0, stream,
        (const T*)k, k_stride, (const T*)v, v_stride, positions, seq_idx, block_table, table_width, (T*)pages,
        page_size, Hkv, D, num_pages, status));
}
