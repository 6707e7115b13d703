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

#define SG_WARPS 8

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
    int n_tiles, tpc, sk; // tiles of 16 weight rows; tiles per unit; K slices per tile
    int units;            // work units (tpc tiles each), taken round robin by the blocks
    int ring_rounds;      // rounds (of four 32-k blocks) of weights each warp keeps in flight
    int red_offset;       // byte offset of the cross-warp sum buffer in shared memory (after x)
    int ring_offset;      // byte offset of the weight rings (after the sum buffer)
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

// Blocks are persistent: block b takes the work units b, b + gridDim.x, ...; a unit is `tpc` tiles of
// 16 weight rows, each tile's K cut into `sk` slices, one slice per warp (8 warps).  A block uses
// at most half of an SM's shared memory and registers, so the blocks of the next kernel on the stream
// become resident beside it and start their own weight stream while this kernel still runs.
template <int MT, int EPI, bool NORM>
__global__ void __launch_bounds__(SG_WARPS * 32, 2) skinny_gemm_kernel(const SkinnyArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = a.K, XS = K + 8;
    float* inv_s = reinterpret_cast<float*>(smem_raw);        // [8*MT] 1/rms of each row (64 floats reserved)
    bf16* xs = reinterpret_cast<bf16*>(smem_raw + 256);      // [8*MT][K + 8]
    float* red = reinterpret_cast<float*>(smem_raw + a.red_offset);   // [warps][MT*4][32]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ---- this warp's K slice and the sequence of its tiles
    const int kslice = warp % a.sk, tile_in_unit = warp / a.sk;
    const int blocks32 = (K + 31) >> 5;
    const int per = (blocks32 + a.sk - 1) / a.sk;           // 32-k blocks per slice
    const int rpu = (per + 3) >> 2;                         // rounds (of four blocks) per unit
    const int kb0 = kslice * per, kb1 = min(kb0 + per, blocks32);
    const int n_units = ((int)a.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total_rounds = n_units * rpu;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    auto rows_of = [&](int unit_index, int& row_lo, int& row_hi) {
        const int tile = (blockIdx.x + unit_index * gridDim.x) * a.tpc + tile_in_unit;
        if (EPI == EPI_SWIGLU) {
            row_lo = tile * 8 + g;
            row_hi = a.F + tile * 8 + g;
            if (tile >= a.n_tiles || row_lo >= a.F) { row_lo = -1; row_hi = -1; }
        } else {
            row_lo = tile * 16 + g;
            row_hi = row_lo + 8;
            if (tile >= a.n_tiles || row_lo >= a.O) row_lo = -1;
            if (tile >= a.n_tiles || row_hi >= a.O) row_hi = -1;
        }
    };

    // ---- the weight stream: each lane copies its own 16-byte fragments of rows g and g+8 into a
    // private ring in shared memory with cp.async, `ring_rounds` rounds of four 32-k blocks ahead of
    // the products, across the block's units.  Ring layout per warp: [slot][lo|hi][lane] of 16 bytes.
    // Without the norm, x needs no staging: each lane's fragments of the token rows travel through
    // the same ring, right behind the weights of their block (they depend on the kernel before this
    // one, so they are issued after the wait; every warp loads only its own K slice of x).
    constexpr int SLOT = (2 + (NORM ? 0 : MT)) * 512;       // bytes of one 32-k block in a warp's ring
    const int ring_rounds = a.ring_rounds;
    unsigned char* ring = smem_raw + a.ring_offset + (size_t)warp * ring_rounds * 4 * SLOT;
    auto issue_w = [&](int r) {
        if (r < total_rounds) {
            int row_lo, row_hi;
            rows_of(r / rpu, row_lo, row_hi);
            const bf16* w_lo = a.W + (size_t)(row_lo < 0 ? 0 : row_lo) * K + 8 * t;
            const bf16* w_hi = a.W + (size_t)(row_hi < 0 ? 0 : row_hi) * K + 8 * t;
            const int kb = kb0 + (r % rpu) * 4;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int k0 = (kb + u) << 5;
                const bool ok = (kb + u) < kb1 && k0 + 8 * t < K;   // past the slice or past K: zeros
                unsigned char* slot = ring + (size_t)((r % ring_rounds) * 4 + u) * SLOT + lane * 16;
                cp_async16_zfill(slot, w_lo + k0, ok && row_lo >= 0);
                cp_async16_zfill(slot + 512, w_hi + k0, ok && row_hi >= 0);
            }
        }
    };
    auto issue_x = [&](int r) {
        if (!NORM && r < total_rounds) {
            const int kb = kb0 + (r % rpu) * 4;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int k0 = (kb + u) << 5;
                const bool ok = (kb + u) < kb1 && k0 + 8 * t < K;
                unsigned char* slot = ring + (size_t)((r % ring_rounds) * 4 + u) * SLOT + 1024 + lane * 16;
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    const int m = nt * 8 + g;
                    cp_async16_zfill(slot + nt * 512, a.x + (size_t)(m < a.M ? m : 0) * K + k0 + 8 * t, ok && m < a.M);
                }
            }
        }
    };
    for (int r = 0; r < ring_rounds; ++r) {                 // the weights depend on no earlier kernel
        issue_w(r);
        cp_async_commit_group();
    }
    pdl_trigger();
    pdl_wait();
    if (!NORM) {
        for (int r = 0; r < ring_rounds; ++r) issue_x(r);
        cp_async_commit_group();
    }

    // ---- x into shared memory, once per block.  With the norm, x = (h + delta) * gamma rounded to
    // bfloat16; the row's factor rsqrt(mean((h + delta)^2) + eps) is applied to the sums afterwards.
    if (NORM) {
        for (int m = warp; m < 8 * MT; m += SG_WARPS) {
            bf16* dst = xs + (size_t)m * XS;
            if (m >= a.M) {
                for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = zero4;
                if (lane == 0) inv_s[m] = 0.f;
                continue;
            }
            const size_t src = (size_t)(a.row_idx ? a.row_idx[m] : m) * K;
            float ss = 0.f;
            for (int kq = lane * 4; kq < K; kq += 512) {          // four 128-wide pieces at a time, loads first
                float4 v[4], gm[4];
                uint2 d[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int k = kq + u * 128;
                    if (k < K) {
                        v[u] = *reinterpret_cast<const float4*>(a.h + src + k);
                        gm[u] = *reinterpret_cast<const float4*>(a.gamma + k);
                        if (a.delta) d[u] = *reinterpret_cast<const uint2*>(a.delta + src + k);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int k = kq + u * 128;
                    if (k < K) {
                        float4 w = v[u];
                        if (a.delta) {
                            const __nv_bfloat162 d0 = *reinterpret_cast<const __nv_bfloat162*>(&d[u].x);
                            const __nv_bfloat162 d1 = *reinterpret_cast<const __nv_bfloat162*>(&d[u].y);
                            w.x += __low2float(d0); w.y += __high2float(d0); w.z += __low2float(d1); w.w += __high2float(d1);
                        }
                        ss += w.x * w.x + w.y * w.y + w.z * w.z + w.w * w.w;
                        if (a.h_out && blockIdx.x == 0) *reinterpret_cast<float4*>(a.h_out + (size_t)m * K + k) = w;
                        __nv_bfloat162 o0 = __floats2bfloat162_rn(w.x * gm[u].x, w.y * gm[u].y);
                        __nv_bfloat162 o1 = __floats2bfloat162_rn(w.z * gm[u].z, w.w * gm[u].w);
                        uint2 o;
                        o.x = *reinterpret_cast<uint32_t*>(&o0);
                        o.y = *reinterpret_cast<uint32_t*>(&o1);
                        *reinterpret_cast<uint2*>(dst + k) = o;
                    }
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) inv_s[m] = rsqrtf(ss / (float)K + a.eps);
        }
    }
    if (NORM) __syncthreads();
    float inv_tok[MT][2];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        inv_tok[nt][0] = NORM ? inv_s[nt * 8 + 2 * t] : 1.f;
        inv_tok[nt][1] = NORM ? inv_s[nt * 8 + 2 * t + 1] : 1.f;
    }

    const bf16* xrow = xs + (size_t)g * XS + 8 * t;
    for (int unit = 0; unit < n_units; ++unit) {
        // ---- the products of this unit's slice: a round's slots are refilled as soon as it is read
        float c[MT][4];
#pragma unroll
        for (int i = 0; i < MT; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
        for (int q = 0; q < rpu; ++q) {
            const int r = unit * rpu + q;
            const int kb = kb0 + q * 4;
            // round r has landed when at most this many later groups are pending (without the norm
            // the group with the first rounds' x sits between the first weights and the steady rounds)
            cp_async_wait_rounds(NORM ? ring_rounds - 1 : min(r, ring_rounds - 1));
            uint4 wl[4], wh[4], bx[4][MT];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const unsigned char* slot = ring + (size_t)((r % ring_rounds) * 4 + u) * SLOT + lane * 16;
                wl[u] = *reinterpret_cast<const uint4*>(slot);
                wh[u] = *reinterpret_cast<const uint4*>(slot + 512);
                if (!NORM) {
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt) bx[u][nt] = *reinterpret_cast<const uint4*>(slot + 1024 + nt * 512);
                }
            }
            issue_w(r + ring_rounds);
            issue_x(r + ring_rounds);
            cp_async_commit_group();                            // one group per round, used or not
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int k0 = (kb + u) << 5;
                const bool kin = (kb + u) < kb1 && k0 + 8 * t < K;
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    uint4 b4;
                    if (NORM) b4 = kin ? *reinterpret_cast<const uint4*>(xrow + (size_t)nt * 8 * XS + k0) : zero4;
                    else b4 = bx[u][nt];
                    mma16816(c[nt], wl[u].x, wh[u].x, wl[u].y, wh[u].y, b4.x, b4.y);
                    mma16816(c[nt], wl[u].z, wh[u].z, wl[u].w, wh[u].w, b4.z, b4.w);
                }
            }
        }
        // ---- add the K slices of a tile in a fixed order
        if (a.sk > 1) {
            __syncthreads();                                    // the readers of the last unit are done
            if (kslice > 0) {
#pragma unroll
                for (int i = 0; i < MT; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) red[((size_t)warp * MT * 4 + i * 4 + e) * 32 + lane] = c[i][e];
            }
            __syncthreads();
            if (kslice == 0) {
                for (int s2 = 1; s2 < a.sk; ++s2)
#pragma unroll
                    for (int i = 0; i < MT; ++i)
#pragma unroll
                        for (int e = 0; e < 4; ++e) c[i][e] += red[((size_t)(warp + s2) * MT * 4 + i * 4 + e) * 32 + lane];
            }
        }
        if (kslice != 0) continue;
        // ---- after the product: lane holds rows (g, g+8) x tokens (8 nt + 2t, + 1)
        int row_lo, row_hi;
        rows_of(unit, row_lo, row_hi);
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
    cp_async_wait_rounds(0);
}

static int sg_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n < 1) n = 1;
    }
    return n;
}
static size_t skinny_x_bytes(int mt, int K, bool norm) {
    if (!norm) return 1024;                                 // x travels through the rings
    return (256 + (size_t)8 * mt * (K + 8) * sizeof(bf16) + 1023) / 1024 * 1024;
}
static size_t skinny_round_bytes(int mt, bool norm) { return (size_t)SG_WARPS * 4 * (2 + (norm ? 0 : mt)) * 512; }
static size_t skinny_red_bytes(int mt) { return (size_t)SG_WARPS * mt * 4 * 32 * sizeof(float); }
// Rounds per warp in flight: up to 64 KB per block, less when x is large, so that a block stays near
// 112 KB of shared memory and two kernels' blocks fit on an SM together.
static int skinny_ring_rounds(int mt, int K, bool norm) {
    const size_t fixed = skinny_x_bytes(mt, K, norm) + skinny_red_bytes(mt);
    const size_t round = skinny_round_bytes(mt, norm);
    const size_t room_half = fixed < (size_t)112 * 1024 ? (size_t)112 * 1024 - fixed : 0;
    const size_t room_full = fixed < (size_t)216 * 1024 ? (size_t)216 * 1024 - fixed : 0;
    int r = (int)(room_half / round);
    if (r < 2) r = (int)(room_full / round) >= 2 ? 2 : (int)(room_full / round);   // two rounds before co-residency
    if (r > 2) r = 2;
    return r;
}

// How to cut the work: K slices per tile (1, 2, 4 or 8; a slice has at least four 32-k blocks), so that
// the busiest block has the least to do, counting a fixed cost per unit.
static void skinny_plan(int n_tiles, int K, int* tpc, int* sk, int* units) {
    const int blocks32 = (K + 31) / 32;
    int best_sk = 1;
    long best_cost = -1;
    for (int s = 1; s <= SG_WARPS; s *= 2) {
        const int per = (blocks32 + s - 1) / s;
        if (s > 1 && per < 4) break;
        const int u = (n_tiles + SG_WARPS / s - 1) / (SG_WARPS / s);
        const int waves = (u + sg_sm_count() - 1) / sg_sm_count();
        const long cost = (long)waves * (((per + 3) / 4) * 4 + 6);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_sk = s; }
    }
    *sk = best_sk;
    *tpc = SG_WARPS / best_sk;
    *units = (n_tiles + *tpc - 1) / *tpc;
}

template <int MT, int EPI, bool NORM>
static int skinny_launch(const SkinnyArgs& a, cudaStream_t stream) {
    const size_t smem = (size_t)a.ring_offset + skinny_round_bytes(MT, NORM) * a.ring_rounds;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MT, EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int grid = a.units < sg_sm_count() ? a.units : sg_sm_count();
    return launch_pdl(skinny_gemm_kernel<MT, EPI, NORM>, dim3(grid), dim3(SG_WARPS * 32), smem, stream, a);
}

template <int EPI, bool NORM>
static int skinny_dispatch_mt(const SkinnyArgs& a, cudaStream_t stream) {
    if (a.M <= 8) return skinny_launch<1, EPI, NORM>(a, stream);
    return skinny_launch<2, EPI, NORM>(a, stream);
}

// 1 if the kernel takes these sizes (else the caller uses the library product and separate kernels)
ZAI_API int zai_skinny_gemm_supports(int M, int O, int K, int epilogue) {
    if (M < 1 || M > 16 || O < 1 || K < 8 || (K & 7)) return 0;    // more rows: the library's product is faster
    if (epilogue == EPI_SWIGLU && (O & 1)) return 0;
    const int mt = M <= 8 ? 1 : 2;
    return skinny_ring_rounds(mt, K, true) >= 1;
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
    skinny_plan(a.n_tiles, K, &a.tpc, &a.sk, &a.units);
    const int mt = M <= 8 ? 1 : 2;
    const bool norm = h != nullptr;
    a.ring_rounds = skinny_ring_rounds(mt, K, norm);
    if (a.ring_rounds < 1) return ZAI_BAD_SIZE;
    a.red_offset = (int)skinny_x_bytes(mt, K, norm);
    a.ring_offset = a.red_offset + (int)skinny_red_bytes(mt);
    if (epilogue == EPI_BF16) return norm ? skinny_dispatch_mt<EPI_BF16, true>(a, stream) : skinny_dispatch_mt<EPI_BF16, false>(a, stream);
    if (epilogue == EPI_F32) return norm ? skinny_dispatch_mt<EPI_F32, true>(a, stream) : skinny_dispatch_mt<EPI_F32, false>(a, stream);
    if (epilogue == EPI_SWIGLU) return norm ? skinny_dispatch_mt<EPI_SWIGLU, true>(a, stream) : skinny_dispatch_mt<EPI_SWIGLU, false>(a, stream);
    return ZAI_BAD_SIZE;
}
