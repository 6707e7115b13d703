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

// bfloat16 table, H a multiple of 8, 16-byte aligned rows: a thread converts 8 values with one 16-byte load
// and two 16-byte stores
__global__ void embed_bf16x8_kernel(float* __restrict__ out, const bf16* __restrict__ table, const int* __restrict__ ids,
                                    int H, int V, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if ((unsigned)id >= (unsigned)V) {               // never read outside the table
        if (threadIdx.x == 0) zai_raise(status, ZAI_ST_TOKEN);
        id = 0;
    }
    const bf16* row = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(row + c);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
        const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]), c2 = __bfloat1622float2(p[2]), d = __bfloat1622float2(p[3]);
        *reinterpret_cast<float4*>(o + c) = make_float4(a.x, a.y, b.x, b.y);
        *reinterpret_cast<float4*>(o + c + 4) = make_float4(c2.x, c2.y, d.x, d.y);
    }
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
    if (table_dtype == ZAI_BF16 && (H & 7) == 0 && ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        const int threads = H >= 1024 ? 128 : (H >= 512 ? 64 : 32);
        return launch_pdl(embed_bf16x8_kernel, dim3(N), dim3(threads), 0, stream, out, (const bf16*)table, ids, H, V, status);
    }
    ZAI_DISPATCH(table_dtype, return launch_pdl(embed_kernel<T>, dim3(N), dim3(256), 0, stream, out, (const T*)table, ids, H, V, status));
}

ZAI_API int zai_gather_add(float* out, const float* h, const void* pending, int pending_dtype, const int* rows,
                           int R, int H, cudaStream_t stream) {
    if (R <= 0) return ZAI_OK;
    ZAI_DISPATCH(pending_dtype,
                 return launch_pdl(gather_add_kernel<T>, dim3(R), dim3(256), 0, stream, out, h, (const T*)pending, rows, H));
}
