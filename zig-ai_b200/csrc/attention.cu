// Causal grouped-query attention over the paged cache, general kernel (any element type, head size,
// page size, window): one warp per (row, query head).
//
//   s_j = q . k_j * scale  for cached positions j <= pos (and j > pos - window), same request
//   o   = sum_j softmax(s)_j v_j
//
// Scale 1/sqrt(D) by default (src/transformer/hybrid_attn.zig:571), causal bound on the token's
// absolute position (:587; src/cuda/paged_attention.cu:245-248), max-subtracted softmax in 32-bit
// (:578-600), query head h reads kv head h / (Hq/Hkv) (src/cuda/paged_attention.cu:142).  Like the
// reference's kernels (paged_attention.cu:121-225, 230-337) a warp walks the keys with an online
// softmax; unlike them the lanes take 32 keys at a time for the scores and share each value row
// for the weighted sum.  Keys are always visited from the first visible position in steps of 32,
// so a row's result does not depend on how the request was cut into steps or on its batch.
// Pages: [num_pages, 2, Hkv, page_size, D].
#include "common.cuh"

template <typename T, int MAXR>
__global__ void paged_attention_warp_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ pages,
                                            const int* __restrict__ block_table, int table_width,
                                            const int* __restrict__ positions, const int* __restrict__ seq_idx,
                                            int page_size, int Hq, int Hkv, int D, float scale, int window,
                                            int num_pages, int* __restrict__ status) {
    extern __shared__ float qs[];                 // [D]
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const int kvh = h / (Hq / Hkv);
    const int pos = positions[t];
    const ZaiTableRow table{block_table + (size_t)seq_idx[t] * table_width, table_width, num_pages, status};
    const T* qrow = q + ((size_t)t * Hq + h) * D;
    for (int d = lane; d < D; d += 32) qs[d] = to_float(qrow[d]) * scale;
    __syncwarp();
    const int kend = pos + 1;
    const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const size_t page_stride = (size_t)2 * Hkv * page_size * D;
    const size_t v_off = (size_t)Hkv * page_size * D;
    float m = -INFINITY, l = 0.f;
    float acc[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;
    for (int base = kstart; base < kend; base += 32) {
        const int j = base + lane;
        const bool valid = j < kend;
        float s = -INFINITY;
        size_t krow = 0;
        if (valid) {
            const int page = table.page(j / page_size);
            krow = (size_t)page * page_stride + ((size_t)kvh * page_size + (j % page_size)) * D;
            const T* kp = pages + krow;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot += qs[d] * to_float(kp[d]);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);                 // m = -inf at first: 0
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int r = 0; r < MAXR; ++r) acc[r] *= corr;
        const int n = min(32, kend - base);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)krow, jj);
            const T* vp = pages + rj + v_off;
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                const int d = lane + 32 * r;
                if (d < D) acc[r] += pj * to_float(vp[d]);
            }
        }
        m = m_new;
    }
    const float inv = 1.f / l;
    T* orow = out + ((size_t)t * Hq + h) * D;
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        const int d = lane + 32 * r;
        if (d < D) orow[d] = from_float<T>(acc[r] * inv);
    }
}

ZAI_API int zai_paged_attention_general(void* out, const void* q, const void* pages, int dtype, const int* block_table,
                                        int table_width, const int* positions, const int* seq_idx, int page_size,
                                        int N, int Hq, int Hkv, int D, float scale, int window, int num_pages, int* status,
                                        cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (D < 1 || D > 256 || Hkv < 1 || Hq % Hkv != 0 || Hq > 65535) return ZAI_BAD_SIZE;
    const dim3 grid(N, Hq);
    const size_t smem = (size_t)D * sizeof(float);
    if (D <= 64) {
        ZAI_DISPATCH(dtype, return launch_pdl(paged_attention_warp_kernel<T, 2>, grid, dim3(32), smem, stream,
            (T*)out, (const T*)q, (const T*)pages, block_table, table_width, positions, seq_idx, page_size, Hq, Hkv,
            D, scale, window, num_pages, status));
    } else {
        ZAI_DISPATCH(dtype, return launch_pdl(paged_attention_warp_kernel<T, 8>, grid, dim3(32), smem, stream,
            (T*)out, (const T*)q, (const T*)pages, block_table, table_width, positions, seq_idx, page_size, Hq, Hkv,
            D, scale, window, num_pages, status));
    }
    return launch_status();
}
