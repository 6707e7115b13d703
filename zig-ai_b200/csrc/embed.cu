// Embedding row gather into the 32-bit residual stream, and the gather of the rows whose logits
// are wanted.  The reference gathers on the host and clamps ids (src/transformer/embedding.zig:6-31,
// clamp at :24; its device kernel embeddingGatherKernel, src/cuda/layer_kernels.cu:411, is unused);
// here ids are checked on the host before the step and the gather runs on the device; an id that is
// outside the vocabulary all the same reads row 0 and raises the step's status word.
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int H, int V, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if ((unsigned)id >= (unsigned)V) {               // never read outside the table
        if (threadIdx.x == 0) zai_raise(status, ZAI_ST_TOKEN);
        id = 0;
    }
    const T* row = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = to_float(row[c]);
}

// out[r] = h[rows[r]] (+ pending[rows[r]])
template <typename T>
__global__ void gather_add_kernel(float* __restrict__ out, const float* __restrict__ h,
                                  const T* __restrict__ pending, const int* __restrict__ rows, int H) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const size_t src = (size_t)rows[r] * H;
    float* o = out + (size_t)r * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = h[src + c];
        if (pending) v += to_float(pending[src + c]);
        o[c] = v;
    }
}

ZAI_API int zai_embed(float* out, const void* table, int table_dtype, const int* ids, int N, int H, int V,
                      int* status, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    ZAI_DISPATCH(table_dtype, return launch_pdl(embed_kernel<T>, dim3(N), dim3(256), 0, stream, out, (const T*)table, ids, H, V, status));
}

ZAI_API int zai_gather_add(float* out, const float* h, const void* pending, int pending_dtype, const int* rows,
                           int R, int H, cudaStream_t stream) {
    if (R <= 0) return ZAI_OK;
    ZAI_DISPATCH(pending_dtype,
                 return launch_pdl(gather_add_kernel<T>, dim3(R), dim3(256), 0, stream, out, h, (const T*)pending, rows, H));
}
