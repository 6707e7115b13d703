// Matrix products for steps of few rows (at most 64): y[M, O] = x[M, K] . W[O, K]^T with bfloat16
// operands and 32-bit accumulation, written for streaming the weights once at memory speed, with
// the work before and after the product fused in:
//
//   before:  x = rmsnorm(h + delta) * gamma      (the block's norm and the residual addition; the
//            32-bit sum h + delta is also written out as the new residual stream), optionally on
//            gathered rows;  or x given in bfloat16
//   after:   bfloat16 store;  32-bit store (logits);  SwiGLU  a = silu(gate) * up  on a stacked
//            gate|up matrix (rows f and F + f are computed by the same warp);  the short convolution's
//            gates, taps and state update on a stacked B|C|x matrix (rows c, H + c and 2H + c are
//            computed by the same warp; formulas src/cuda/layer_kernels.cu:206-221)
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
#include <cstdlib>
#include "common.cuh"

#define SG_WARPS 8

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_CONV = 3 };
#define SG_CONV_TAPS 4        // the fused convolution takes up to this many taps

// The weights that the product after this one will stream.  Every block asks its share of them into L2,
// so that memory keeps delivering while this kernel stages rows, reduces and drains, and the next
// kernel's rings fill from L2.  `when`: 1 before this kernel's dependency wait (while the kernel before it
// still runs: 0.429 against 0.431 ms a decode step of 8 requests), 2 after it (0.464 ms: the requests
// then compete with this kernel's own stream).
struct NextWeights {
    const unsigned char* base;     // null: none
    unsigned long long bytes;      // a multiple of 16
    unsigned per_block;            // a multiple of 16
    int when;
};
__device__ __forceinline__ void ask_next_weights(const NextWeights& n, int lane) {
    if (!n.base) return;
    const unsigned long long start = (unsigned long long)blockIdx.x * n.per_block;
    if (start >= n.bytes) return;
    const unsigned mine = (unsigned)min((unsigned long long)n.per_block, n.bytes - start);
    for (unsigned off = (unsigned)lane * 2048u; off < mine; off += 32u * 2048u) {
        const uint32_t sz = min(2048u, mine - off);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(n.base + start + off), "r"(sz) : "memory");
    }
}

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
    int half_tiles;       // 1: a tile is 8 weight rows (the other 8 rows of the instruction are zeros), for more units
    int units;            // work units (tpc tiles each), taken round robin by the blocks
    int ring_rounds;      // rounds (of four 32-k blocks) of weights each warp keeps in flight
    int red_offset;       // byte offset of the cross-warp sum buffer in shared memory (after x)
    int ring_offset;      // byte offset of the weight rings (after the sum buffer)
    // convolution epilogue (O = 3F: B rows, C rows, x rows of F channels each)
    const float* conv_w;  // [F, taps]
    const float* conv_b;  // [F] or null
    float* conv_state;    // [slots, state_rows, F]
    const int* slot_ids;  // [M]
    int num_slots;        // slots in conv_state: a slot id outside is read as slot 0 and raises the status word
    int* status;
    int taps, state_rows, write_state;
    int l2_prefetch_bytes; // how much of its weight rows a block asks into L2 before it waits for the kernel before it
    NextWeights next;      // the weights of the product after this one: asked into L2 while this one runs
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
    float* gs = reinterpret_cast<float*>(smem_raw + 256 + (size_t)8 * MT * XS * sizeof(bf16));   // [K] the norm's weight
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
    // weight rows of the lane: (row_lo, row_hi) are rows g and g + 8 of the 16-row operand.  The
    // convolution has two such operands per tile of 8 channels: j = 0: B and C of channel c0 + g;
    // j = 1: x of channel c0 + g (its other 8 rows are zeros).
    auto rows_of = [&](int unit_index, int j, int& row_lo, int& row_hi) {
        const int tile = (blockIdx.x + unit_index * gridDim.x) * a.tpc + tile_in_unit;
        if (EPI == EPI_CONV) {
            const int ch = tile * 8 + g;
            const bool v = tile < a.n_tiles && ch < a.F;
            if (j == 0) { row_lo = v ? ch : -1; row_hi = v ? a.F + ch : -1; }
            else { row_lo = v ? 2 * a.F + ch : -1; row_hi = -1; }
        } else if (EPI == EPI_SWIGLU) {
            row_lo = tile * 8 + g;
            row_hi = a.F + tile * 8 + g;
            if (tile >= a.n_tiles || row_lo >= a.F) { row_lo = -1; row_hi = -1; }
        } else if (a.half_tiles) {
            row_lo = tile * 8 + g;
            row_hi = -1;
            if (tile >= a.n_tiles || row_lo >= a.O) row_lo = -1;
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
    constexpr int NT = EPI == EPI_CONV ? 2 : 1;             // 16-row operands per tile
    constexpr int SLOT = (2 * NT + (NORM ? 0 : MT)) * 512;  // bytes of one 32-k block in a warp's ring
    const int ring_rounds = a.ring_rounds;
    unsigned char* ring = smem_raw + a.ring_offset + (size_t)warp * ring_rounds * 4 * SLOT;
    auto issue_w = [&](int r) {
        if (r < total_rounds) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                int row_lo, row_hi;
                rows_of(r / rpu, j, row_lo, row_hi);
                const bf16* w_lo = a.W + (size_t)(row_lo < 0 ? 0 : row_lo) * K + 8 * t;
                const bf16* w_hi = a.W + (size_t)(row_hi < 0 ? 0 : row_hi) * K + 8 * t;
                const int kb = kb0 + (r % rpu) * 4;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int k0 = (kb + u) << 5;
                    const bool ok = (kb + u) < kb1 && k0 + 8 * t < K;   // past the slice or past K: zeros
                    unsigned char* slot = ring + (size_t)((r % ring_rounds) * 4 + u) * SLOT + j * 1024 + lane * 16;
                    cp_async16_zfill(slot, w_lo + k0, ok && row_lo >= 0);
                    cp_async16_zfill(slot + 512, w_hi + k0, ok && row_hi >= 0);
                }
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
                unsigned char* slot = ring + (size_t)((r % ring_rounds) * 4 + u) * SLOT + NT * 1024 + lane * 16;
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
    // The rest of this block's weight rows are asked into L2 now: this kernel's blocks become resident
    // while the kernel before it on the stream still runs, so the rows arrive from memory meanwhile
    // and the products below find them in L2.
    if (warp == 0 && EPI != EPI_CONV) {
        size_t budget = (size_t)a.l2_prefetch_bytes;
        for (int u = 0; u < n_units && budget > 0; ++u) {
            const int tile_first = (blockIdx.x + u * gridDim.x) * a.tpc;
            const int rows_per_tile = (EPI == EPI_SWIGLU || a.half_tiles) ? 8 : 16;
            const int row0 = tile_first * rows_per_tile;
            const int limit = EPI == EPI_SWIGLU ? a.F : a.O;
            const int nrows = min(limit, row0 + a.tpc * rows_per_tile) - row0;
            if (nrows <= 0) break;
            size_t bytes = (size_t)nrows * K * sizeof(bf16);
            if (bytes > budget) bytes = budget & ~(size_t)15;
            budget -= bytes;
            for (int half = 0; half < (EPI == EPI_SWIGLU ? 2 : 1); ++half) {
                const unsigned char* base = reinterpret_cast<const unsigned char*>(a.W + ((size_t)row0 + (size_t)half * a.F) * K);
                for (size_t off = (size_t)lane * 4096; off < bytes; off += (size_t)32 * 4096) {
                    const uint32_t n = (uint32_t)min((size_t)4096, bytes - off);
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(n) : "memory");
                }
            }
        }
    }
    // ---- the convolution's inputs of a unit (state, taps, bias of the lane's channel and tokens) are
    // asked for at the start of the unit and used in its epilogue, so their way from memory is hidden
    // behind the product (after the wait: the kernel before this one may have written the state)
    float cv_prev[EPI == EPI_CONV ? MT : 1][2][SG_CONV_TAPS - 1], cv_w[SG_CONV_TAPS], cv_b = 0.f;
    int cv_slot[EPI == EPI_CONV ? MT : 1][2];
    auto conv_inputs = [&](int unit) {
        if (EPI != EPI_CONV || kslice != 0) return;
        const int tile = (blockIdx.x + unit * gridDim.x) * a.tpc + tile_in_unit;
        const int ch = tile * 8 + g;
        const bool vc = tile < a.n_tiles && ch < a.F;
        cv_b = (vc && a.conv_b) ? a.conv_b[ch] : 0.f;
#pragma unroll
        for (int j = 0; j < SG_CONV_TAPS; ++j) cv_w[j] = (vc && j < a.taps) ? a.conv_w[(size_t)ch * a.taps + j] : 0.f;
        bool bad_slot = false;                                // (raised once, below: no atomic in the unrolled loops)
#pragma unroll
        for (int nt = 0; nt < (EPI == EPI_CONV ? MT : 1); ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = nt * 8 + 2 * t + e;
                const int slot = tok < a.M ? a.slot_ids[tok] : 0;
                const bool bad = (unsigned)slot >= (unsigned)a.num_slots;     // outside the slots: slot 0, and the step is void
                bad_slot |= bad;
                cv_slot[nt][e] = bad ? 0 : slot;
#pragma unroll
                for (int j = 0; j < SG_CONV_TAPS - 1; ++j)
                    cv_prev[nt][e][j] = (vc && tok < a.M && j < a.taps - 1)
                        ? a.conv_state[((size_t)cv_slot[nt][e] * a.state_rows + j) * a.F + ch] : 0.f;
            }
        if (bad_slot) zai_raise(a.status, ZAI_ST_SLOT);
    };
    // the norm's weight and the rows' source indices are written by no kernel of the step: they are
    // fetched before the wait, the weight into shared memory
    int src_row0 = warp, src_row1 = warp + SG_WARPS;
    if (NORM) {
        for (int k = tid * 4; k < K; k += SG_WARPS * 32 * 4) *reinterpret_cast<float4*>(gs + k) = *reinterpret_cast<const float4*>(a.gamma + k);
        if (a.row_idx) {
            if (src_row0 < a.M) src_row0 = a.row_idx[src_row0];
            if (src_row1 < a.M) src_row1 = a.row_idx[src_row1];
        }
    }
    if (a.next.when == 1 && warp == SG_WARPS - 1) ask_next_weights(a.next, lane);
    pdl_trigger();
    pdl_wait_at(__LINE__, 1 + EPI * 2 + (NORM ? 1 : 0));
    if (a.next.when == 2 && warp == SG_WARPS - 1) ask_next_weights(a.next, lane);
    if (n_units > 0) conv_inputs(0);                         // asked for now, used in the epilogue
    if (NORM) __syncthreads();                               // gs is complete
    if (!NORM) {
        for (int r = 0; r < ring_rounds; ++r) issue_x(r);
        cp_async_commit_group();
    }

    // ---- x into shared memory, once per block.  With the norm, x = (h + delta) * gamma rounded to
    // bfloat16; the row's factor rsqrt(mean((h + delta)^2) + eps) is applied to the sums afterwards.
    // A warp takes a row; a lane asks for up to eight 16-byte pieces of h and of delta before it uses
    // the first, so a row of up to 1024 values costs one trip to memory.
    if (NORM) {
        for (int m = warp; m < 8 * MT; m += SG_WARPS) {
            bf16* dst = xs + (size_t)m * XS;
            if (m >= a.M) {
                for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = zero4;
                if (lane == 0) inv_s[m] = 0.f;
                continue;
            }
            const size_t src = (size_t)(m < SG_WARPS ? src_row0 : src_row1) * K;
            float ss = 0.f;
            for (int kq = lane * 4; kq < K; kq += 1024) {
                float4 v[8];
                uint2 d[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int k = kq + u * 128;
                    if (k < K) {
                        v[u] = *reinterpret_cast<const float4*>(a.h + src + k);
                        if (a.delta) d[u] = *reinterpret_cast<const uint2*>(a.delta + src + k);
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int k = kq + u * 128;
                    if (k < K) {
                        float4 w = v[u];
                        const float4 gm = *reinterpret_cast<const float4*>(gs + k);
                        if (a.delta) {
                            const __nv_bfloat162 d0 = *reinterpret_cast<const __nv_bfloat162*>(&d[u].x);
                            const __nv_bfloat162 d1 = *reinterpret_cast<const __nv_bfloat162*>(&d[u].y);
                            w.x += __low2float(d0); w.y += __high2float(d0); w.z += __low2float(d1); w.w += __high2float(d1);
                        }
                        ss += w.x * w.x + w.y * w.y + w.z * w.z + w.w * w.w;
                        if (a.h_out && blockIdx.x == 0) *reinterpret_cast<float4*>(a.h_out + (size_t)m * K + k) = w;
                        __nv_bfloat162 o0 = __floats2bfloat162_rn(w.x * gm.x, w.y * gm.y);
                        __nv_bfloat162 o1 = __floats2bfloat162_rn(w.z * gm.z, w.w * gm.w);
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
        if (unit > 0) conv_inputs(unit);
        // ---- the products of this unit's slice: a round's slots are refilled as soon as it is read
        float c[NT][MT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < MT; ++i) c[j][i][0] = c[j][i][1] = c[j][i][2] = c[j][i][3] = 0.f;
        for (int q = 0; q < rpu; ++q) {
            const int r = unit * rpu + q;
            const int kb = kb0 + q * 4;
            // round r has landed when at most this many later groups are pending (without the norm
            // the group with the first rounds' x sits between the first weights and the steady rounds)
            cp_async_wait_rounds(NORM ? ring_rounds - 1 : min(r, ring_rounds - 1));
            if (NT == 1) {
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
                        mma16816(c[0][nt], wl[u].x, wh[u].x, wl[u].y, wh[u].y, b4.x, b4.y);
                        mma16816(c[0][nt], wl[u].z, wh[u].z, wl[u].w, wh[u].w, b4.z, b4.w);
                    }
                }
            } else {
                // two operands per 32-k block: read and multiply block by block, refill afterwards
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const unsigned char* slot = ring + (size_t)((r % ring_rounds) * 4 + u) * SLOT + lane * 16;
                    const int k0 = (kb + u) << 5;
                    const bool kin = (kb + u) < kb1 && k0 + 8 * t < K;
                    uint4 b4[MT];
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt) {
                        if (NORM) b4[nt] = kin ? *reinterpret_cast<const uint4*>(xrow + (size_t)nt * 8 * XS + k0) : zero4;
                        else b4[nt] = *reinterpret_cast<const uint4*>(slot + NT * 1024 + nt * 512);
                    }
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        const uint4 wl = *reinterpret_cast<const uint4*>(slot + j * 1024);
                        const uint4 wh = *reinterpret_cast<const uint4*>(slot + j * 1024 + 512);
#pragma unroll
                        for (int nt = 0; nt < MT; ++nt) {
                            mma16816(c[j][nt], wl.x, wh.x, wl.y, wh.y, b4[nt].x, b4[nt].y);
                            mma16816(c[j][nt], wl.z, wh.z, wl.w, wh.w, b4[nt].z, b4[nt].w);
                        }
                    }
                }
                issue_w(r + ring_rounds);
                issue_x(r + ring_rounds);
                cp_async_commit_group();
            }
        }
        // ---- add the K slices of a tile in a fixed order
        if (a.sk > 1) {
            __syncthreads();                                    // the readers of the last unit are done
            if (kslice > 0) {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int i = 0; i < MT; ++i)
#pragma unroll
                        for (int e = 0; e < 4; ++e) red[((size_t)warp * NT * MT * 4 + (j * MT + i) * 4 + e) * 32 + lane] = c[j][i][e];
            }
            __syncthreads();
            if (kslice == 0) {
                for (int s2 = 1; s2 < a.sk; ++s2)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int i = 0; i < MT; ++i)
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                c[j][i][e] += red[((size_t)(warp + s2) * NT * MT * 4 + (j * MT + i) * 4 + e) * 32 + lane];
            }
        }
        if (kslice != 0) continue;
        // ---- after the product: lane holds rows (g, g+8) x tokens (8 nt + 2t, + 1)
        if (EPI == EPI_CONV) {
            const int tile = (blockIdx.x + unit * gridDim.x) * a.tpc + tile_in_unit;
            const int ch = tile * 8 + g;
            if (tile >= a.n_tiles || ch >= a.F) continue;
#pragma unroll
            for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int tok = nt * 8 + 2 * t + e;
                    if (tok >= a.M) continue;
                    const float inv = inv_tok[nt][e];
                    // the three projections rounded as if stored, then the gated convolution in 32-bit
                    const float Bv = __bfloat162float(__float2bfloat16_rn(c[0][nt][e] * inv));
                    const float Cv = __bfloat162float(__float2bfloat16_rn(c[0][nt][2 + e] * inv));
                    const float Xv = __bfloat162float(__float2bfloat16_rn(c[NT - 1][nt][e] * inv));
                    const float u = Bv * Xv;
                    float y = cv_b, w_last = 0.f;
#pragma unroll
                    for (int j = 0; j < SG_CONV_TAPS; ++j) {
                        if (j < a.taps - 1) y += cv_w[j] * cv_prev[nt][e][j < SG_CONV_TAPS - 1 ? j : 0];
                        if (j == a.taps - 1) w_last = cv_w[j];
                    }
                    y += w_last * u;
                    reinterpret_cast<bf16*>(a.y)[(size_t)tok * a.ldy + ch] = __float2bfloat16_rn(Cv * y);
                    if (a.write_state) {
                        float* st = a.conv_state + (size_t)cv_slot[nt][e] * a.state_rows * a.F + ch;
#pragma unroll
                        for (int j = 0; j < SG_CONV_TAPS - 1; ++j)
                            if (j < a.taps - 1) st[(size_t)j * a.F] = (j + 1 < a.taps - 1) ? cv_prev[nt][e][(j + 1) % (SG_CONV_TAPS - 1)] : u;
                    }
                }
            continue;
        }
        int row_lo, row_hi;
        rows_of(unit, 0, row_lo, row_hi);
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = nt * 8 + 2 * t + e;
                if (tok >= a.M) continue;
                const float lo = c[0][nt][e] * inv_tok[nt][e], hi = c[0][nt][2 + e] * inv_tok[nt][e];
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

// ---- long rows (K of several thousand, the feed-forward's second product): K cut across a cluster
//
// With one block per tile, a tile's K slices are the block's 8 warps, and each warp walks its slice
// round by round behind a ring of two rounds: a chain of trips to memory after the wait, and every
// block needs all of x.  Here a tile of 16 weight rows belongs to a cluster of CS blocks; K is cut
// into 8 CS slices, one per warp, short enough that a warp's whole slice of the weights is asked for
// before the wait and its slice of x in one go after it.  The warps of a block add their sums
// through shared memory, the blocks of the cluster through rank 0's shared memory (written by the
// other ranks, then a cluster barrier), both in a fixed order.
#define SK_MAX_BLOCKS 6            // 32-k blocks per warp at most

struct SplitKArgs {
    const bf16* W;        // [O, K]
    const bf16* x;        // [M, K]
    void* y;              // [M, O] bfloat16 or float
    int M, O, K, n_tiles;
    int per;              // 32-k blocks per warp
    int f32_out;
    NextWeights next;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `local` (in this block's shared memory) in the shared memory of block `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(const void* local, uint32_t rank) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(local), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_store_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

template <int MT, int CS>
__global__ void __launch_bounds__(SG_WARPS * 32) skinny_splitk_kernel(const SplitKArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rank = (int)cluster_rank(), tile = blockIdx.x / CS;
    const int K = a.K, per = a.per;
    constexpr int SLOT = (2 + MT) * 512;                     // weights rows g, g+8 and MT token groups of one 32-k block
    unsigned char* mine = smem_raw + (size_t)warp * SK_MAX_BLOCKS * SLOT;
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)SG_WARPS * SK_MAX_BLOCKS * SLOT);   // [warps][MT*4][32]
    float* cred = red + SG_WARPS * MT * 4 * 32;                                                  // [CS][MT*4][32], used on rank 0
    const int blocks32 = (K + 31) >> 5;
    const int kb0 = (rank * SG_WARPS + warp) * per;
    int row_lo = tile * 16 + g, row_hi = row_lo + 8;
    if (row_lo >= a.O) row_lo = -1;
    if (row_hi >= a.O) row_hi = -1;
    const bf16* w_lo = a.W + (size_t)(row_lo < 0 ? 0 : row_lo) * K + 8 * t;
    const bf16* w_hi = a.W + (size_t)(row_hi < 0 ? 0 : row_hi) * K + 8 * t;
#pragma unroll
    for (int u = 0; u < SK_MAX_BLOCKS; ++u) {
        const int k0 = (kb0 + u) << 5;
        const bool ok = u < per && (kb0 + u) < blocks32 && k0 + 8 * t < K;
        cp_async16_zfill(mine + u * SLOT + lane * 16, w_lo + k0, ok && row_lo >= 0);
        cp_async16_zfill(mine + u * SLOT + 512 + lane * 16, w_hi + k0, ok && row_hi >= 0);
    }
    cp_async_commit_group();
    if (a.next.when == 1 && warp == SG_WARPS - 1) ask_next_weights(a.next, lane);
    pdl_trigger();
    pdl_wait();
    if (a.next.when == 2 && warp == SG_WARPS - 1) ask_next_weights(a.next, lane);
#pragma unroll
    for (int u = 0; u < SK_MAX_BLOCKS; ++u) {
        const int k0 = (kb0 + u) << 5;
        const bool ok = u < per && (kb0 + u) < blocks32 && k0 + 8 * t < K;
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            const int m = nt * 8 + g;
            cp_async16_zfill(mine + u * SLOT + 1024 + nt * 512 + lane * 16, a.x + (size_t)(m < a.M ? m : 0) * K + k0 + 8 * t, ok && m < a.M);
        }
    }
    cp_async_commit_group();
    cp_async_wait_rounds(0);
    float c[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
#pragma unroll
    for (int u = 0; u < SK_MAX_BLOCKS; ++u) {
        if (u < per) {
            const uint4 wl = *reinterpret_cast<const uint4*>(mine + u * SLOT + lane * 16);
            const uint4 wh = *reinterpret_cast<const uint4*>(mine + u * SLOT + 512 + lane * 16);
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                const uint4 b4 = *reinterpret_cast<const uint4*>(mine + u * SLOT + 1024 + nt * 512 + lane * 16);
                mma16816(c[nt], wl.x, wh.x, wl.y, wh.y, b4.x, b4.y);
                mma16816(c[nt], wl.z, wh.z, wl.w, wh.w, b4.z, b4.w);
            }
        }
    }
    // ---- the block's warps, in order
    if (warp > 0) {
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) red[((size_t)warp * MT * 4 + i * 4 + e) * 32 + lane] = c[i][e];
    }
    __syncthreads();
    if (warp == 0) {
        for (int w2 = 1; w2 < SG_WARPS; ++w2)
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) c[i][e] += red[((size_t)w2 * MT * 4 + i * 4 + e) * 32 + lane];
        if (rank > 0) {                                     // into rank 0's shared memory
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    cluster_store_f32(cluster_map(cred + ((size_t)rank * MT * 4 + i * 4 + e) * 32 + lane, 0), c[i][e]);
        }
    }
    cluster_sync_all();
    if (rank != 0 || warp != 0) return;
    for (int r2 = 1; r2 < CS; ++r2)
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) c[i][e] += cred[((size_t)r2 * MT * 4 + i * 4 + e) * 32 + lane];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int tok = nt * 8 + 2 * t + e;
            if (tok >= a.M) continue;
            const float lo = c[nt][e], hi = c[nt][2 + e];
            if (a.f32_out) {
                if (row_lo >= 0) reinterpret_cast<float*>(a.y)[(size_t)tok * a.O + row_lo] = lo;
                if (row_hi >= 0) reinterpret_cast<float*>(a.y)[(size_t)tok * a.O + row_hi] = hi;
            } else {
                if (row_lo >= 0) reinterpret_cast<bf16*>(a.y)[(size_t)tok * a.O + row_lo] = __float2bfloat16_rn(lo);
                if (row_hi >= 0) reinterpret_cast<bf16*>(a.y)[(size_t)tok * a.O + row_hi] = __float2bfloat16_rn(hi);
            }
        }
}

// The hint for the next launch of a product kernel from this thread: the weights of the product that
// will follow it.  One launch uses it up.  At most ZAI_NEXT_PREFETCH_MB (24) of them are asked for:
// L2 also has to keep what the running kernel reads.  ZAI_NEXT_PREFETCH=0 ignores hints, 1 (default) asks
// before the dependency wait, 2 after it.
static thread_local const void* hinted_w = nullptr;
static thread_local long long hinted_bytes = 0;
ZAI_API int zai_skinny_hint_next(const void* w, long long bytes) { hinted_w = w; hinted_bytes = bytes; return 0; }
static NextWeights take_hint(int grid) {
    static int when = -1, cap_mb = 24;
    if (when < 0) {
        const char* e = getenv("ZAI_NEXT_PREFETCH");
        when = e ? atoi(e) : 1;
        const char* c = getenv("ZAI_NEXT_PREFETCH_MB");
        if (c) cap_mb = atoi(c);
    }
    NextWeights n = {};
    if (when > 0 && hinted_w && hinted_bytes >= 16 && grid > 0 && ((uintptr_t)hinted_w & 15) == 0) {
        unsigned long long bytes = (unsigned long long)hinted_bytes & ~15ull;
        const unsigned long long cap = (unsigned long long)cap_mb << 20;
        if (bytes > cap) bytes = cap;
        n.base = (const unsigned char*)hinted_w;
        n.bytes = bytes;
        n.per_block = (unsigned)(((bytes + grid - 1) / grid + 15) & ~15ull);
        n.when = when;
    }
    hinted_w = nullptr;
    hinted_bytes = 0;
    return n;
}
template <int MT, int CS>
static int splitk_launch(const SplitKArgs& a, cudaStream_t stream) {
    const size_t smem = (size_t)SG_WARPS * SK_MAX_BLOCKS * (2 + MT) * 512 + (size_t)(SG_WARPS + CS) * MT * 4 * 32 * sizeof(float);
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {
        cudaError_t e = cudaFuncSetAttribute(skinny_splitk_kernel<MT, CS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(a.n_tiles * CS));
    cfg.blockDim = dim3(SG_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    SplitKArgs b = a;
    b.next = take_hint(a.n_tiles * CS);
    return (int)cudaLaunchKernelEx(&cfg, skinny_splitk_kernel<MT, CS>, b);
}

// Cluster size for a plain-input product with rows of K values: 0 = the one-block kernel
static int splitk_cluster(int K) {
    static int off = -1;
    if (off < 0) {
        const char* e = getenv("ZAI_SKINNY_SPLITK");
        off = (e && e[0] == '0') ? 1 : 0;
    }
    if (off) return 0;
    const int blocks32 = (K + 31) / 32;
    if (blocks32 >= 192 && (blocks32 + 31) / 32 > SK_MAX_BLOCKS && (blocks32 + 63) / 64 <= SK_MAX_BLOCKS) return 8;   // K > 6144
    if (blocks32 >= 96 && (blocks32 + 31) / 32 <= SK_MAX_BLOCKS) return 4;      // K >= 3072
    if (blocks32 >= 48 && (blocks32 + 15) / 16 <= SK_MAX_BLOCKS) return 2;      // K >= 1536
    return 0;
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
// Bytes per block asked into L2 ahead of the wait (ZAI_SKINNY_L2_PREFETCH_KB; default 0: measured on
// the LFM2 shapes it gains nothing, the rings already hold what a block needs first)
static int skinny_l2_prefetch_bytes() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("ZAI_SKINNY_L2_PREFETCH_KB");
        v = (e ? atoi(e) : 0) * 1024;
        if (v < 0) v = 0;
    }
    return v;
}
// Blocks of one launch: up to two per SM (a block keeps to half of an SM's shared memory), so that a
// launch with many units has all its weights asked for at once (ZAI_SKINNY_BLOCKS_PER_SM overrides)
static int sg_slots() {
    static int v = 0;
    if (!v) {
        const char* e = getenv("ZAI_SKINNY_BLOCKS_PER_SM");
        int per_sm = e ? atoi(e) : 2;
        if (per_sm < 1) per_sm = 1;
        v = sg_sm_count() * per_sm;
    }
    return v;
}
static size_t skinny_x_bytes(int mt, int K, bool norm) {
    if (!norm) return 1024;                                 // x travels through the rings
    return (256 + (size_t)8 * mt * (K + 8) * sizeof(bf16) + (size_t)K * sizeof(float) + 1023) / 1024 * 1024;
}
static size_t skinny_round_bytes(int mt, bool norm, int nt) { return (size_t)SG_WARPS * 4 * (2 * nt + (norm ? 0 : mt)) * 512; }
static size_t skinny_red_bytes(int mt, int nt) { return (size_t)SG_WARPS * nt * mt * 4 * 32 * sizeof(float); }
// Rounds per warp in flight: up to 64 KB per block, less when x is large, so that a block stays near
// 112 KB of shared memory and two kernels' blocks fit on an SM together.
static int skinny_ring_rounds(int mt, int K, bool norm, int nt) {
    const size_t fixed = skinny_x_bytes(mt, K, norm) + skinny_red_bytes(mt, nt);
    const size_t round = skinny_round_bytes(mt, norm, nt);
    const size_t room_half = fixed < (size_t)112 * 1024 ? (size_t)112 * 1024 - fixed : 0;
    const size_t room_full = fixed < (size_t)216 * 1024 ? (size_t)216 * 1024 - fixed : 0;
    int r = (int)(room_half / round);
    if (r < 2) r = (int)(room_full / round) >= 2 ? 2 : (int)(room_full / round);   // two rounds before co-residency
    if (r > 2) r = 2;
    return r;
}

// How to cut the work: K slices per tile (1, 2, 4 or 8; a slice has at least four 32-k blocks) and
// whole tiles (16 weight rows) or half tiles (8 rows, twice as many units, half the bytes per round),
// so that the busiest block has the least to do, counting a fixed cost per unit.
static void skinny_plan(int rows, bool may_halve, int K, int* n_tiles, int* half, int* tpc, int* sk, int* units, int rows_per_tile = 16) {
    const int blocks32 = (K + 31) / 32;
    long best_cost = -1;
    for (int h = 0; h <= (may_halve ? 1 : 0); ++h) {
        const int tiles = h ? (rows + 7) / 8 : (rows + rows_per_tile - 1) / rows_per_tile;
        for (int s = 1; s <= SG_WARPS; s *= 2) {
            const int per = (blocks32 + s - 1) / s;
            if (s > 1 && per < 4) break;
            const int u = (tiles + SG_WARPS / s - 1) / (SG_WARPS / s);
            const int waves = (u + sg_slots() - 1) / sg_slots();
            const long cost = (long)waves * ((long)((per + 3) / 4) * 4 * (h ? 6 : 10) + 60);
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                *sk = s;
                *half = h;
                *n_tiles = tiles;
            }
        }
    }
    *tpc = SG_WARPS / *sk;
    *units = (*n_tiles + *tpc - 1) / *tpc;
}

template <int MT, int EPI, bool NORM>
static int skinny_launch(const SkinnyArgs& a, cudaStream_t stream) {
    const size_t smem = (size_t)a.ring_offset + skinny_round_bytes(MT, NORM, EPI == EPI_CONV ? 2 : 1) * a.ring_rounds;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<MT, EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int grid = a.units < sg_slots() ? a.units : sg_slots();
    SkinnyArgs b = a;
    b.next = take_hint(grid);
    return launch_pdl(skinny_gemm_kernel<MT, EPI, NORM>, dim3(grid), dim3(SG_WARPS * 32), smem, stream, b);
}

template <int EPI, bool NORM>
static int skinny_dispatch_mt(const SkinnyArgs& a, cudaStream_t stream) {
    if (a.M <= 8) return skinny_launch<1, EPI, NORM>(a, stream);
    return skinny_launch<2, EPI, NORM>(a, stream);
}

// 1 if the kernel takes these sizes (else the caller uses the library product and separate kernels)
// `norm`: x comes as the 32-bit residual stream to be normed (it is staged in shared memory whole,
// which bounds K), not as bfloat16 rows.
ZAI_API int zai_skinny_gemm_supports(int M, int O, int K, int epilogue, int norm) {
    if (M < 1 || M > 16 || O < 1 || K < 8 || (K & 7)) return 0;    // more rows: the library's product is faster
    if (epilogue == EPI_SWIGLU && (O & 1)) return 0;
    if (epilogue == EPI_CONV && O % 3) return 0;
    const int mt = M <= 8 ? 1 : 2;
    return skinny_ring_rounds(mt, K, norm != 0, epilogue == EPI_CONV ? 2 : 1) >= 1;
}

static int skinny_run(SkinnyArgs& a, int epilogue, cudaStream_t stream) {
    const int mt = a.M <= 8 ? 1 : 2, nt = epilogue == EPI_CONV ? 2 : 1;
    const bool norm = a.h != nullptr;
    if (norm && (a.K & 3)) return ZAI_BAD_SIZE;
    a.ring_rounds = skinny_ring_rounds(mt, a.K, norm, nt);
    if (a.ring_rounds < 1) return ZAI_BAD_SIZE;
    {   // no deeper than the busiest block's rounds: shared memory left free lets the next kernel's blocks in
        const int per = ((a.K + 31) / 32 + a.sk - 1) / a.sk, rpu = (per + 3) / 4;
        const int grid = a.units < sg_slots() ? a.units : sg_slots();
        const int rounds = rpu * ((a.units + grid - 1) / grid);
        if (a.ring_rounds > rounds) a.ring_rounds = rounds;
    }
    a.red_offset = (int)skinny_x_bytes(mt, a.K, norm);
    a.ring_offset = a.red_offset + (int)skinny_red_bytes(mt, nt);
    a.l2_prefetch_bytes = skinny_l2_prefetch_bytes();
    if (epilogue == EPI_BF16) return norm ? skinny_dispatch_mt<EPI_BF16, true>(a, stream) : skinny_dispatch_mt<EPI_BF16, false>(a, stream);
    if (epilogue == EPI_F32) return norm ? skinny_dispatch_mt<EPI_F32, true>(a, stream) : skinny_dispatch_mt<EPI_F32, false>(a, stream);
    if (epilogue == EPI_SWIGLU) return norm ? skinny_dispatch_mt<EPI_SWIGLU, true>(a, stream) : skinny_dispatch_mt<EPI_SWIGLU, false>(a, stream);
    if (epilogue == EPI_CONV) return norm ? skinny_dispatch_mt<EPI_CONV, true>(a, stream) : skinny_dispatch_mt<EPI_CONV, false>(a, stream);
    return ZAI_BAD_SIZE;
}

// y = epilogue(x . W^T).  With `h` given, x = rmsnorm(h[row_idx] + delta[row_idx]) * gamma and, if
// h_out is given, h_out = h + delta (32-bit).  epilogue: 0 bfloat16 [M, O]; 1 float [M, O];
// 2 SwiGLU on W = gate|up stacked, y bfloat16 [M, O/2].
ZAI_API int zai_skinny_gemm(void* y, const void* W, const void* x, const float* h, const void* delta,
                            const float* gamma, const int* row_idx, float* h_out, float eps, int M, int O, int K,
                            int epilogue, cudaStream_t stream) {
    if (epilogue == EPI_CONV || !zai_skinny_gemm_supports(M, O, K, epilogue, h != nullptr)) return ZAI_BAD_SIZE;
    const int cs = (!h && (epilogue == EPI_BF16 || epilogue == EPI_F32)) ? splitk_cluster(K) : 0;
    if (cs) {
        SplitKArgs b = {};
        b.W = (const bf16*)W; b.x = (const bf16*)x; b.y = y; b.M = M; b.O = O; b.K = K;
        b.n_tiles = (O + 15) / 16;
        b.per = ((K + 31) / 32 + SG_WARPS * cs - 1) / (SG_WARPS * cs);
        b.f32_out = epilogue == EPI_F32;
        if (cs == 8) return M <= 8 ? splitk_launch<1, 8>(b, stream) : splitk_launch<2, 8>(b, stream);
        if (cs == 4) return M <= 8 ? splitk_launch<1, 4>(b, stream) : splitk_launch<2, 4>(b, stream);
        return M <= 8 ? splitk_launch<1, 2>(b, stream) : splitk_launch<2, 2>(b, stream);
    }
    SkinnyArgs a = {};
    a.W = (const bf16*)W; a.x = (const bf16*)x; a.h = h; a.delta = (const bf16*)delta; a.gamma = gamma;
    a.row_idx = row_idx; a.h_out = h_out; a.y = y; a.eps = eps; a.M = M; a.O = O; a.K = K;
    a.F = O / 2;
    a.ldy = epilogue == EPI_SWIGLU ? O / 2 : O;
    if (epilogue == EPI_SWIGLU) {
        skinny_plan(a.F * 2, false, K, &a.n_tiles, &a.half_tiles, &a.tpc, &a.sk, &a.units);   // 8 gate + 8 up rows per tile
    } else {
        skinny_plan(O, true, K, &a.n_tiles, &a.half_tiles, &a.tpc, &a.sk, &a.units);
    }
    return skinny_run(a, epilogue, stream);
}

// The short convolution's input projection with the convolution as its epilogue, for steps in which
// every row is one token of its own request:  (B, C, x~) = x . W^T with W = [3F, K] stacked;
// u = B x~;  y = bias + sum_j w[c, j] state[j, c] + w[c, taps-1] u;  z = C y (bfloat16 [M, F]);  the
// state of the row's slot moves on by one (if write_state).  B, C and x~ are rounded to bfloat16
// before they are used, as when they are stored.  taps <= 4.
ZAI_API int zai_skinny_conv(void* z, const void* W, const void* x, const float* h, const void* delta, const float* gamma,
                            float* h_out, float eps, const float* conv_w, const float* conv_b, float* state,
                            const int* slot_ids, int M, int F, int K, int taps, int state_rows, int write_state,
                            int num_slots, int* status, cudaStream_t stream) {
    if (F < 1 || taps < 1 || taps > SG_CONV_TAPS || state_rows < taps - 1) return ZAI_BAD_SIZE;
    if (!zai_skinny_gemm_supports(M, 3 * F, K, EPI_CONV, h != nullptr)) return ZAI_BAD_SIZE;
    SkinnyArgs a = {};
    a.W = (const bf16*)W; a.x = (const bf16*)x; a.h = h; a.delta = (const bf16*)delta; a.gamma = gamma;
    a.row_idx = nullptr; a.h_out = h_out; a.y = z; a.eps = eps; a.M = M; a.O = 3 * F; a.K = K;
    a.F = F;
    a.ldy = F;
    a.conv_w = conv_w; a.conv_b = conv_b; a.conv_state = state; a.slot_ids = slot_ids;
    a.num_slots = num_slots; a.status = status;
    a.taps = taps; a.state_rows = state_rows; a.write_state = write_state;
    skinny_plan(F, false, K, &a.n_tiles, &a.half_tiles, &a.tpc, &a.sk, &a.units, 8);   // 8 channels per tile
    return skinny_run(a, EPI_CONV, stream);
}
