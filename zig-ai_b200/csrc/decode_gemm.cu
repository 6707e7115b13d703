// Matrix products for steps of few rows (at most 64): y[M, O] = x[M, K] . W[O, K]^T with bfloat16
// operands and 32-bit accumulation, written for streaming the weights once at memory speed, with
// the work before and after the product fused in:
//
//   before:  x = rmsnorm(h + delta) * gamma      (the block's norm and the residual addition; the
//            32-bit sum h + delta is also written out as the new residual stream), optionally on
//            gathered rows;  or x given in bfloat16
//   after:   bfloat16 store;  32-bit store (logits);  SwiGLU  a = silu(gate) * up  on a stacked
//            gate|up matrix (rows f and F + f are computed by the same warp)
//
// The reference runs a decode token's projections as cublasSgemm with M = 1 and separate norm,
// residual and activation kernels (src/transformer/hybrid_layer.zig:607-672; formulas
// src/transformer/norm.zig:14-32, src/transformer/ffn.zig:23-30).
//
// The weights are the 16-row operand of mma.sync m16n8k16 and the tokens the 8-column operand, so
// 8 tokens cost one instruction per 16 weight rows and 16 k.  Each lane loads 16 bytes (8 k) of a
// weight row straight from global memory into its fragment registers; the matching 8 k of a token
// row come from shared memory with the same lane mapping, so no shuffles are needed (the order of
// k inside a 32-k block is permuted identically for both operands).  A block's warps split K
// between them and add their partial sums through shared memory in a fixed order.
#include "common.cuh"

#define SG_MAX_WARPS 16

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };

struct SkinnyArgs {
    const bf16* W;        // [O, K]
    const bf16* x;        // [M, K] when there is no norm
    const float* h;       // norm: residual stream [rows, K]
    const bf16* delta;    // norm: pending term [rows, K] or null
    const float* gamma;   // norm: [K]
    const int* row_idx;   // norm: source row of each of the M rows, or null for 0..M-1
    float* h_out;         // norm: where block 0 writes h + delta [M, K], or null
    void* y;              // [M, ldy]
    float eps;
    int M, O, K, ldy;
    int F;                // SwiGLU: gate rows 0..F-1, up rows F..2F-1 (O = 2F)
    int n_tiles, tpc, sk; // tiles of 16 weight rows; tiles per block; K slices per tile
    int ring_rounds;      // rounds (of four 32-k blocks) of weights each warp keeps in flight
    int ring_offset;      // byte offset of the weight rings in shared memory (after x)
};

__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;            // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
                 ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;\n" ::); }
// wait until at most n of this thread's committed groups are pending (n is 0..7)
__device__ __forceinline__ void cp_async_wait_rounds(int n) {
    switch (n) {
        case 0: asm volatile("cp.async.wait_group 0;\n" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;\n" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;\n" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;\n" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;\n" ::: "memory"); break;
        case 5: asm volatile("cp.async.wait_group 5;\n" ::: "memory"); break;
        case 6: asm volatile("cp.async.wait_group 6;\n" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 7;\n" ::: "memory"); break;
    }
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, int EPI, bool NORM>
__global__ void __launch_bounds__(SG_MAX_WARPS * 32) skinny_gemm_kernel(const SkinnyArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = a.K, XS = K + 8;
    float* inv_s = reinterpret_cast<float*>(smem_raw);        // [8*MT] 1/rms of each row (64 floats reserved)
    bf16* xs = reinterpret_cast<bf16*>(smem_raw + 256);      // [8*MT][K + 8]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ---- this warp's tile and K slice, and its first weight loads: they depend on no earlier kernel
    const int tile = blockIdx.x * a.tpc + warp / a.sk;
    const int kslice = warp % a.sk;
    const int blocks32 = (K + 31) >> 5;
    const int per = (blocks32 + a.sk - 1) / a.sk;
    const int kb0 = kslice * per, kb1 = min(kb0 + per, blocks32);
    int row_lo, row_hi;                                     // weight rows of fragment rows g and g+8
    if (EPI == EPI_SWIGLU) {
        row_lo = tile * 8 + g;
        row_hi = a.F + tile * 8 + g;
        if (row_lo >= a.F) { row_lo = -1; row_hi = -1; }
    } else {
        row_lo = tile * 16 + g;
        row_hi = row_lo + 8;
        if (row_lo >= a.O) row_lo = -1;
        if (row_hi >= a.O) row_hi = -1;
    }
    const bool active = tile < a.n_tiles;
    if (!active) { row_lo = -1; row_hi = -1; }
    const bf16* w_lo = a.W + (size_t)(row_lo < 0 ? 0 : row_lo) * K + 8 * t;
    const bf16* w_hi = a.W + (size_t)(row_hi < 0 ? 0 : row_hi) * K + 8 * t;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    // ---- the weight stream: each lane copies its own 16-byte fragments of rows g and g+8 into a
    // private ring in shared memory with cp.async, `rounds` rounds of four 32-k blocks ahead of the
    // products, so that a block keeps about 128 KB of loads in flight whatever its register use.
    // Ring layout per warp: [slot][lo|hi][lane] of 16 bytes (a quarter-warp reads 128 contiguous bytes).
    const int depth = a.ring_rounds * 4;                           // slots per warp
    unsigned char* ring = smem_raw + a.ring_offset + (size_t)warp * depth * 1024;
    auto issue_round = [&](int kb) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int blk = kb + u;
            const int k0 = blk << 5;
            const bool ok = blk < kb1 && k0 + 8 * t < K;            // past the slice or past K: zeros
            unsigned char* slot = ring + (size_t)((blk - kb0) % depth) * 1024 + lane * 16;
            cp_async16_zfill(slot, w_lo + k0, ok && row_lo >= 0);
            cp_async16_zfill(slot + 512, w_hi + k0, ok && row_hi >= 0);
        }
        cp_async_commit_group();
    };
    for (int r = 0; r < a.ring_rounds; ++r) issue_round(kb0 + 4 * r);   // all rounds of the ring start at once
    pdl_trigger();
    pdl_wait();

    // ---- x into shared memory.  With the norm, x = (h + delta) * gamma rounded to bfloat16; the
    // row's factor rsqrt(mean((h + delta)^2) + eps) is applied to the sums after the product.
    if (NORM) {
        for (int m = warp; m < 8 * MT; m += nwarps) {
            bf16* dst = xs + (size_t)m * XS;
            if (m >= a.M) {
                for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = zero4;
                if (lane == 0) inv_s[m] = 0.f;
                continue;
            }
            const size_t src = (size_t)(a.row_idx ? a.row_idx[m] : m) * K;
            float ss = 0.f;
            for (int k = lane * 4; k < K; k += 128) {
                float4 v = *reinterpret_cast<const float4*>(a.h + src + k);
                if (a.delta) {
                    const uint2 d = *reinterpret_cast<const uint2*>(a.delta + src + k);
                    const __nv_bfloat162 d0 = *reinterpret_cast<const __nv_bfloat162*>(&d.x);
                    const __nv_bfloat162 d1 = *reinterpret_cast<const __nv_bfloat162*>(&d.y);
                    v.x += __low2float(d0); v.y += __high2float(d0); v.z += __low2float(d1); v.w += __high2float(d1);
                }
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                if (a.h_out && blockIdx.x == 0) *reinterpret_cast<float4*>(a.h_out + (size_t)m * K + k) = v;
                const float4 gm = *reinterpret_cast<const float4*>(a.gamma + k);
                __nv_bfloat162 o0 = __floats2bfloat162_rn(v.x * gm.x, v.y * gm.y);
                __nv_bfloat162 o1 = __floats2bfloat162_rn(v.z * gm.z, v.w * gm.w);
                uint2 o;
                o.x = *reinterpret_cast<uint32_t*>(&o0);
                o.y = *reinterpret_cast<uint32_t*>(&o1);
                *reinterpret_cast<uint2*>(dst + k) = o;
            }
            ss = warp_sum(ss);
            if (lane == 0) inv_s[m] = rsqrtf(ss / (float)K + a.eps);
        }
    } else {
        const int chunks = K >> 3;
        for (int idx = tid; idx < 8 * MT * chunks; idx += blockDim.x) {
            const int m = idx / chunks, c = idx % chunks;
            uint4 v = zero4;
            if (m < a.M) v = *reinterpret_cast<const uint4*>(a.x + (size_t)m * K + c * 8);
            *reinterpret_cast<uint4*>(xs + (size_t)m * XS + c * 8) = v;
        }
    }
    __syncthreads();

    // ---- the product: rounds of four 32-k blocks; a round's slots are refilled as soon as it is used
    float c[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
    {
        const bf16* xrow = xs + (size_t)g * XS + 8 * t;
        for (int kb = kb0; kb < kb1; kb += 4) {
            cp_async_wait_rounds(a.ring_rounds - 1);             // the oldest round in flight has landed
            uint4 wl[4], wh[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const unsigned char* slot = ring + (size_t)((kb + u - kb0) % depth) * 1024 + lane * 16;
                wl[u] = *reinterpret_cast<const uint4*>(slot);
                wh[u] = *reinterpret_cast<const uint4*>(slot + 512);
            }
            issue_round(kb + depth);                              // same slots, `ring_rounds` rounds ahead
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int k0 = (kb + u) << 5;
                const bool kin = (kb + u) < kb1 && k0 + 8 * t < K;
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    const uint4 b = kin ? *reinterpret_cast<const uint4*>(xrow + (size_t)nt * 8 * XS + k0) : zero4;
                    mma16816(c[nt], wl[u].x, wh[u].x, wl[u].y, wh[u].y, b.x, b.y);
                    mma16816(c[nt], wl[u].z, wh[u].z, wl[u].w, wh[u].w, b.z, b.w);
                }
            }
        }
        cp_async_wait_rounds(0);
    }
    float inv_tok[MT][2];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        inv_tok[nt][0] = NORM ? inv_s[nt * 8 + 2 * t] : 1.f;
        inv_tok[nt][1] = NORM ? inv_s[nt * 8 + 2 * t + 1] : 1.f;
    }

    // ---- add the K slices of a tile in a fixed order (shared memory is free again)
    if (a.sk > 1) {
        __syncthreads();
        float* red = reinterpret_cast<float*>(smem_raw);     // [warps][MT*4][32]
        if (kslice > 0) {
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) red[((size_t)warp * MT * 4 + i * 4 + e) * 32 + lane] = c[i][e];
        }
        __syncthreads();
        if (kslice == 0) {
            for (int s = 1; s < a.sk; ++s)
#pragma unroll
                for (int i = 0; i < MT; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) c[i][e] += red[((size_t)(warp + s) * MT * 4 + i * 4 + e) * 32 + lane];
        }
    }
    if (!active || kslice != 0) return;

    // ---- after the product: lane holds rows (g, g+8) x tokens (8 nt + 2t, + 1)
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int tok = nt * 8 + 2 * t + e;
            if (tok >= a.M) continue;
            const float lo = c[nt][e] * inv_tok[nt][e], hi = c[nt][2 + e] * inv_tok[nt][e];
            if (EPI == EPI_SWIGLU) {
                if (row_lo >= 0)
                    reinterpret_cast<bf16*>(a.y)[(size_t)tok * a.ldy + row_lo] = __float2bfloat16_rn(lo / (1.f + expf(-lo)) * hi);
            } else if (EPI == EPI_F32) {
                if (row_lo >= 0) reinterpret_cast<float*>(a.y)[(size_t)tok * a.ldy + row_lo] = lo;
                if (row_hi >= 0) reinterpret_cast<float*>(a.y)[(size_t)tok * a.ldy + row_hi] = hi;
            } else {
                if (row_lo >= 0) reinterpret_cast<bf16*>(a.y)[(size_t)tok * a.ldy + row_lo] = __float2bfloat16_rn(lo);
                if (row_hi >= 0) reinterpret_cast<bf16*>(a.y)[(size_t)tok * a.ldy + row_hi] = __float2bfloat16_rn(hi);
            }
        }
    }
}

static size_t skinny_x_bytes(int mt, int K) {
    return (256 + (size_t)8 * mt * (K + 8) * sizeof(bf16) + 1023) / 1024 * 1024;
}
// Rounds per warp: the warp's whole slice if that keeps the block's rings within 64 KB (so that the
// blocks of the next kernel on the stream fit beside it and can start their own weight stream while
// this kernel still runs), else as many as 64 KB allow, at least one.
static int skinny_ring_rounds(int mt, int K, int warps, int sk) {
    const size_t room = (size_t)216 * 1024 - skinny_x_bytes(mt, K);
    const int fit = (int)(room / ((size_t)warps * 4096));
    const int blocks32 = (K + 31) / 32;
    const int slice_rounds = ((blocks32 + sk - 1) / sk + 3) / 4;
    int r = (int)((size_t)64 * 1024 / ((size_t)warps * 4096));
    if (r < 1) r = 1;
    if (r > slice_rounds) r = slice_rounds;
    if (r > fit) r = fit;
    return r;
}
static size_t skinny_smem(int mt, int K, int warps, int ring_rounds) {
    const size_t main = skinny_x_bytes(mt, K) + (size_t)warps * ring_rounds * 4 * 1024;
    const size_t red = (size_t)warps * mt * 4 * 32 * sizeof(float);
    return main > red ? main : red;
}
// How to cut the work: K slices per tile and tiles per block.  Slices are made short (down to four
// 32-k blocks, one round) until about 2048 warps exist, so that a warp's whole slice is in flight
// from the start and two blocks fit on an SM; long streams (the head) keep one slice per tile.
static void skinny_plan(int n_tiles, int K, int* tpc, int* sk) {
    const int blocks32 = (K + 31) / 32;
    int s = 1;
    while (s < 16 && n_tiles * s < 2048 && blocks32 / (s * 2) >= 4) s *= 2;
    const int warps = s == 16 ? 16 : 8;
    *sk = s;
    *tpc = warps / s;
}

template <int MT, int EPI, bool NORM>
static int skinny_launch(const SkinnyArgs& a, cudaStream_t stream) {
    const int warps = a.tpc * a.sk;
    const size_t smem = skinny_smem(MT, a.K, warps, a.ring_rounds);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MT, EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int grid = (a.n_tiles + a.tpc - 1) / a.tpc;
    return launch_pdl(skinny_gemm_kernel<MT, EPI, NORM>, dim3(grid), dim3(warps * 32), smem, stream, a);
}

template <int EPI, bool NORM>
static int skinny_dispatch_mt(const SkinnyArgs& a, cudaStream_t stream) {
    if (a.M <= 8) return skinny_launch<1, EPI, NORM>(a, stream);
    if (a.M <= 16) return skinny_launch<2, EPI, NORM>(a, stream);
    if (a.M <= 32) return skinny_launch<4, EPI, NORM>(a, stream);
    return skinny_launch<8, EPI, NORM>(a, stream);
}

// 1 if the kernel takes these sizes (else the caller uses the library product and separate kernels)
ZAI_API int zai_skinny_gemm_supports(int M, int O, int K, int epilogue) {
    if (M < 1 || M > 16 || O < 1 || K < 8 || (K & 7)) return 0;    // more rows: the library's product is faster
    if (epilogue == EPI_SWIGLU && (O & 1)) return 0;
    const int mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
    return skinny_ring_rounds(mt, K, SG_MAX_WARPS, 1) >= 1;
}

// y = epilogue(x . W^T).  With `h` given, x = rmsnorm(h[row_idx] + delta[row_idx]) * gamma and, if
// h_out is given, h_out = h + delta (32-bit).  epilogue: 0 bfloat16 [M, O]; 1 float [M, O];
// 2 SwiGLU on W = gate|up stacked, y bfloat16 [M, O/2].
ZAI_API int zai_skinny_gemm(void* y, const void* W, const void* x, const float* h, const void* delta,
                            const float* gamma, const int* row_idx, float* h_out, float eps, int M, int O, int K,
                            int epilogue, cudaStream_t stream) {
    if (!zai_skinny_gemm_supports(M, O, K, epilogue)) return ZAI_BAD_SIZE;
    if (h && (K & 3)) return ZAI_BAD_SIZE;
    SkinnyArgs a;
    a.W = (const bf16*)W; a.x = (const bf16*)x; a.h = h; a.delta = (const bf16*)delta; a.gamma = gamma;
    a.row_idx = row_idx; a.h_out = h_out; a.y = y; a.eps = eps; a.M = M; a.O = O; a.K = K;
    a.F = O / 2;
    a.ldy = epilogue == EPI_SWIGLU ? O / 2 : O;
    a.n_tiles = epilogue == EPI_SWIGLU ? (a.F + 7) / 8 : (O + 15) / 16;
    skinny_plan(a.n_tiles, K, &a.tpc, &a.sk);
    const int mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
    a.ring_rounds = skinny_ring_rounds(mt, K, a.tpc * a.sk, a.sk);
    if (a.ring_rounds < 1) return ZAI_BAD_SIZE;
    a.ring_offset = (int)skinny_x_bytes(mt, K);
    const bool norm = h != nullptr;
    if (epilogue == EPI_BF16) return norm ? skinny_dispatch_mt<EPI_BF16, true>(a, stream) : skinny_dispatch_mt<EPI_BF16, false>(a, stream);
    if (epilogue == EPI_F32) return norm ? skinny_dispatch_mt<EPI_F32, true>(a, stream) : skinny_dispatch_mt<EPI_F32, false>(a, stream);
    if (epilogue == EPI_SWIGLU) return norm ? skinny_dispatch_mt<EPI_SWIGLU, true>(a, stream) : skinny_dispatch_mt<EPI_SWIGLU, false>(a, stream);
    return ZAI_BAD_SIZE;
}
