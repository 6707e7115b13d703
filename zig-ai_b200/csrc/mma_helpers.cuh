// Small device helpers shared by the tensor-core attention kernels: asynchronous copies,
// ldmatrix, mma.sync m16n8k16 (bfloat16 operands, 32-bit accumulation) and the per-head
// RMSNorm + rotation of one row.
#pragma once
#include "common.cuh"

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;        // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
// d += a (16x16, row) * b (16x8, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}


// 2^x by the special-function unit (2 ulp; x = -inf gives 0, which the masked scores rely on).  The
// library's exp2f costs tens of cycles more per value, which showed as the largest part of a key
// tile's time in the attention kernels.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// one head row: RMSNorm (if gamma) and rotation of the first `rot` dims; `tmp` holds D floats.  The
// row, the norm's weight and the rotation's cosines and sines are all asked for before the first
// of them is used, so the three loads cost one trip to memory, not three.
template <int D>
__device__ __forceinline__ void norm_rotate_row(const bf16* __restrict__ raw, const float* __restrict__ gamma, float eps,
                                                const float2* __restrict__ cs, int rot, float* tmp, bf16* dst, int lane) {
    constexpr int PER = (D + 31) / 32;
    const int half = rot >> 1;
    float v[PER], gm[PER];
    float2 c[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        v[i] = 0.f;
        gm[i] = 1.f;
        c[i] = make_float2(1.f, 0.f);
        if (d < D) {
            v[i] = __bfloat162float(raw[d]);
            if (gamma) gm[i] = gamma[d];
            if (d < rot) c[i] = cs[d < half ? d : d - half];
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) ss += v[i] * v[i];
    float inv = 1.f;
    if (gamma) {
        ss = warp_sum(ss);
        inv = rsqrtf(ss / (float)D + eps);
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        if (d < D) {
            if (gamma) v[i] = v[i] * inv * gm[i];
            tmp[d] = v[i];
        }
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        if (d < D) {
            float r;
            if (d < half) r = v[i] * c[i].x - tmp[d + half] * c[i].y;
            else if (d < rot) r = tmp[d - half] * c[i].y + v[i] * c[i].x;
            else r = v[i];
            dst[d] = __float2bfloat16_rn(r);
        }
    }
    __syncwarp();
}
