// The decode step's attention for head size 64 with the keys and values brought in by TMA.
//
// Same work as decode_fused_kernel (csrc/attention_mma.cu): per-head RMSNorm and rotation of the
// queries and of the new key, the new key and value into their page, attention over the request's
// pages in chunks of keys, and the combination of the chunks by the block that draws the last
// ticket.  What differs is how keys and values reach shared memory: one producer lane issues
// `cp.async.bulk.tensor` loads (no multicast) of whole page-head blocks (page_size rows of 128 bytes, which
// are contiguous in the pool [num_pages, 2, Hkv, page_size, 64]) into a ring of 64-key stages with
// the 128-byte swizzle, each stage signalled by an mbarrier; four consumer warps take the stages in
// turn (a whole 64-key tile per warp), read the fragments with ldmatrix through the swizzle, and
// hand the stage back.  The ring keeps 64 KB of loads in flight per block (three blocks per SM) whatever the
// consumers are doing, which the version with per-lane 16-byte copies could not (its loads stop
// while its warps compute).
//
// Every wait on an mbarrier is bounded; a block whose wait runs out raises the status word, all its
// roles leave their loops and the block still takes its ticket, so nothing hangs.
#include <cuda.h>
#include "common.cuh"
#include "mma_helpers.cuh"

#define TT_D 64
#define TT_TILE 64
#ifndef TT_CONSUMERS
#define TT_CONSUMERS 4
#endif
#define TT_STAGES 4          // a multiple of the consumer warps: a stage always belongs to the same warp
#define TT_THREADS ((TT_CONSUMERS + 1) * 32)
#define TT_SPIN_LIMIT 4000000
#define TT_STAGE_BYTES (2 * TT_TILE * TT_D * 2)       // keys then values: 16 KB

__device__ __forceinline__ void tt_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void tt_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tt_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool tt_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
    const uint32_t a = smem_u32(bar);
    for (int it = 0; it < TT_SPIN_LIMIT; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
        if (*failed) return false;
    }
    *failed = 1;
    return false;
}
__device__ __forceinline__ void tt_tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// Fragments from a 64-row x 128-byte tile stored with the 128-byte swizzle (16-byte chunk c of row r
// lies at chunk c ^ (r & 7)); `rows` points at row 0 of a 16-row group, 1024-byte aligned groups of 8.
__device__ __forceinline__ void qk_16keys_sw(float (&s0)[4], float (&s1)[4], const uint32_t (&qf)[TT_D / 16][4],
                                             const unsigned char* rows, int lane) {
    const int key = ((lane >> 4) << 3) + (lane & 7);
    const int hi = (lane >> 3) & 1;
#pragma unroll
    for (int ks = 0; ks < TT_D / 16; ++ks) {
        uint32_t b[4];
        ldmatrix_x4(b, rows + key * 128 + (((ks * 2 + hi) ^ (key & 7)) << 4));
        mma_bf16(s0, qf[ks], b[0], b[1]);
        mma_bf16(s1, qf[ks], b[2], b[3]);
    }
}
__device__ __forceinline__ void pv_16keys_sw(float (&o)[TT_D / 8][4], const uint32_t (&pf)[4], const unsigned char* rows, int lane) {
    const int key = (((lane >> 3) & 1) << 3) + (lane & 7);
    const int hi = lane >> 4;
#pragma unroll
    for (int dp = 0; dp < TT_D / 16; ++dp) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, rows + key * 128 + (((dp * 2 + hi) ^ (key & 7)) << 4));
        mma_bf16(o[2 * dp], pf, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
    }
}

struct TmaDecodeArgs {
    bf16* out;                 // [B, Hq, 64]
    float* part_o;             // [B, Hq, n_chunks, 64]
    float* part_ml;            // [B, Hq, n_chunks, 2]
    int* tickets;              // [B * Hkv], zero before and after
    int* status;               // the step's status word: a wait that ran out, a page id or position out of bounds
    int num_pages;
    const bf16* qkv;           // [B, qkv_cols]
    const float* q_gamma;
    const float* k_gamma;
    const float2* cs_table;    // [B, rot/2]
    bf16* pages;
    const int* block_table;
    const int* positions;
    float eps, scale_log2;
    int qkv_cols, rot, table_width, page_size, page_shift, Hq, Hkv, window, write_kv, chunk_keys, stages;
    int chunk_fastest;         // the grid is (chunks, Hkv, B) if set, else (Hkv, B, chunks)
};

// (128 registers a thread: three blocks of 160 threads share an SM's 64 K registers; a few more and only two fit)
__global__ void __maxnreg__(128) decode_tma_kernel(const __grid_constant__ CUtensorMap map, const TmaDecodeArgs a) {
    constexpr int D = TT_D, ST = D + 8;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* after = ring + (size_t)a.stages * TT_STAGE_BYTES;
    bf16* sq = reinterpret_cast<bf16*>(after);                      // [16][ST]
    float* tmp = reinterpret_cast<float*>(sq + 16 * ST);             // [4][D]
    bf16* knew = reinterpret_cast<bf16*>(tmp + 4 * D);               // [D], then the new value [D]
    bf16* vnew = knew + D;
    float* snew = reinterpret_cast<float*>(vnew + D);                // [16]
    // the warps' partial outputs lie over the first stages of the ring, which is idle by then
    float* wo = reinterpret_cast<float*>(ring);                      // [4][16][D]
    float* wm = wo + 4 * 16 * D;                                     // [4][16]
    float* wl = wm + 4 * 16;                                         // [4][16]
    __shared__ uint64_t full_bar[12], empty_bar[12];
    __shared__ int s_ticket, failed_flag;
    volatile int* failed = &failed_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // Blocks are handed out in the order of their index, x fastest.  When all of them are resident at
    // once or nearly so, the chunk is the slowest index: the first chunks of every request (all with
    // work) start first, the last chunks (short or empty for most requests) last.  With many more
    // blocks than the SMs hold, the chunk is the fastest index: a request's chunks run together and
    // are combined as the kernel goes, not all at its end.
    const int chunk = a.chunk_fastest ? blockIdx.x : blockIdx.z, hk = a.chunk_fastest ? blockIdx.y : blockIdx.x;
    const int b = a.chunk_fastest ? blockIdx.z : blockIdx.y, n_chunks = a.chunk_fastest ? gridDim.x : gridDim.z;
    const int Hq = a.Hq, Hkv = a.Hkv, G = Hq / Hkv, ps = a.page_size;
    if (tid == 0) {
        failed_flag = 0;
        for (int s = 0; s < a.stages; ++s) {
            tt_mbar_init(&full_bar[s], 1);
            tt_mbar_init(&empty_bar[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();
    // The producer warp reads only what no kernel of this step writes before it (positions, block
    // table, the cached keys and values), so it does not wait for the kernel before this one: its
    // loads fly while that kernel (the qkv projection) still runs.  The consumers need its result.
    // (A layer that only reads a cache which another layer wrote earlier in this step waits, too.)
    // A block without keys waits as a whole: what it stores (its empty partial sum) may lie in memory
    // that a kernel further back in the chain still uses, and nothing is stored before the wait.
    const int pos = a.positions[b];
    const int kstart = a.window > 0 ? max(pos - a.window + 1, 0) : 0;
    const bool has_new = a.write_kv && chunk == pos / a.chunk_keys;
    const int kend = a.write_kv ? pos : pos + 1;
    const int lo = max(chunk * a.chunk_keys, kstart), hi = min((chunk + 1) * a.chunk_keys, kend);
    const bool any_paged = lo < hi;
    if (warp != 0 || !a.write_kv || !(any_paged || has_new)) pdl_wait();
    const int* table = a.block_table + (size_t)b * a.table_width;
    const int tile0 = lo / TT_TILE, tile1 = any_paged ? (hi + TT_TILE - 1) / TT_TILE : tile0;
    const int cw = warp - 1;                                         // consumer index 0..3 (warp 0 produces)

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int g = lane >> 2, tq = lane & 3;

    if (any_paged || has_new) {
        if (warp == 0) {
            // ---- producer warp: a stage per 64-key tile; lane 0 waits for the stage and arms its
            // barrier, then the lanes issue the tile's loads side by side (one per page and per
            // keys/values), so the address work and the issue of the small copies run in parallel
            const int per_tile = TT_TILE / ps;                       // pages of a tile (page_size divides 64)
            int issued = 0;
            for (int t = tile0; t < tile1; ++t) {
                const int i = t - tile0, s = i % a.stages;
                int ok = 1;
                if (lane == 0) {
                    ok = tt_mbar_wait(&empty_bar[s], ((i / a.stages) & 1) ^ 1, failed) ? 1 : 0;
                    if (ok) tt_mbar_expect_tx(&full_bar[s], TT_STAGE_BYTES);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane < 2 * per_tile) {
                    const int p = lane >> 1, kv = lane & 1;
                    unsigned char* st = ring + (size_t)s * TT_STAGE_BYTES;
                    const int idx = ((t * TT_TILE) >> a.page_shift) + p;
                    int page = idx < a.table_width ? table[idx] : 0;               // beyond the table: the null page
                    if ((unsigned)page >= (unsigned)a.num_pages) {                 // outside the pool: page 0, and the step is void
                        zai_raise(a.status, ZAI_ST_PAGE);
                        page = 0;
                    }
                    const int row = ((page * 2 + kv) * Hkv + hk) * ps;
                    tt_tma_load_2d(st + (size_t)kv * TT_TILE * 128 + (size_t)p * ps * 128, &map, 0, row, &full_bar[s]);
                }
                issued = i + 1;
            }
            if (lane == 0 && *failed) {                              // loads already issued still land here: wait for them
                for (int i = max(issued - a.stages, 0); i < issued; ++i) {
                    const uint32_t addr = smem_u32(&full_bar[i % a.stages]);
                    const uint32_t ph = (i / a.stages) & 1;
                    for (int spin = 0; spin < TT_SPIN_LIMIT; ++spin) {
                        uint32_t done;
                        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                     : "=r"(done) : "r"(addr), "r"(ph) : "memory");
                        if (done) break;
                    }
                }
            }
        } else {
            // ---- consumers: first the group's queries, and the new key and value
            const bf16* row = a.qkv + (size_t)b * a.qkv_cols;
            const float2* cs = a.rot ? a.cs_table + (size_t)b * (a.rot >> 1) : nullptr;
            // the rows to prepare (the group's G queries, then the new key) go round the warps
            for (int r = cw; r < 16; r += TT_CONSUMERS) {
                if (r < G) norm_rotate_row<D>(row + (size_t)(hk * G + r) * D, a.q_gamma, a.eps, cs, a.rot, tmp + cw * D, sq + r * ST, lane);
                else for (int d = lane; d < D; d += 32) sq[r * ST + d] = __float2bfloat16_rn(0.f);
            }
            if (has_new && cw == G % TT_CONSUMERS) {
                norm_rotate_row<D>(row + (size_t)(Hq + hk) * D, a.k_gamma, a.eps, cs, a.rot, tmp + cw * D, knew, lane);
                const bf16* vraw = row + (size_t)(Hq + Hkv + hk) * D;
                const int page = zai_checked_page(table, a.table_width, pos < 0 ? -1 : pos >> a.page_shift, a.num_pages,
                                                  lane == 0 ? a.status : nullptr);
                const int off = pos & (ps - 1);
                const size_t page_stride = (size_t)2 * Hkv * ps * D;
                bf16* kdst = a.pages + (size_t)page * page_stride + ((size_t)hk * ps + off) * D;
                bf16* vdst = a.pages + (size_t)page * page_stride + ((size_t)(Hkv + hk) * ps + off) * D;
                for (int d = lane; d < D; d += 32) {
                    const bf16 v = vraw[d];
                    vnew[d] = v;
                    vdst[d] = v;
                    kdst[d] = knew[d];
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(TT_CONSUMERS * 32) : "memory");      // the four consumer warps
            uint32_t qf[D / 16][4];
            {
                const int r = (((lane >> 3) & 1) << 3) + (lane & 7);
                const int dof = (lane >> 4) << 3;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], sq + r * ST + ks * 16 + dof);
            }
            if (has_new && cw == 0 && lane < 16) {
                float dot = 0.f;
                for (int d = 0; d < D; ++d) dot += __bfloat162float(sq[lane * ST + d]) * __bfloat162float(knew[d]);
                snew[lane] = dot;
            }
            // ---- tiles tile0 + cw, tile0 + cw + 4, ...: a whole 64-key tile per warp
            for (int t = tile0 + cw; t < tile1; t += TT_CONSUMERS) {
                const int i = t - tile0, s = i % a.stages;
                if (!tt_mbar_wait(&full_bar[s], (i / a.stages) & 1, failed)) break;
                const unsigned char* kt = ring + (size_t)s * TT_STAGE_BYTES;
                const unsigned char* vt = kt + TT_TILE * 128;
                float sc[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) qk_16keys_sw(sc[2 * kb], sc[2 * kb + 1], qf, kt + kb * 16 * 128, lane);
                float mx0 = -INFINITY, mx1 = -INFINITY;
                const bool edge = t * TT_TILE < lo || (t + 1) * TT_TILE > hi;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    if (edge) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int j = t * TT_TILE + nt * 8 + 2 * tq + e;
                            if (j < lo || j >= hi) { sc[nt][e] = -INFINITY; sc[nt][2 + e] = -INFINITY; }
                        }
                    }
                    mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1]));
                    mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);       // finite: the tile has a visible key
                const float u0 = n0 * a.scale_log2, u1 = n1 * a.scale_log2;
                const float c0 = fast_exp2(m0 * a.scale_log2 - u0), c1 = fast_exp2(m1 * a.scale_log2 - u1);
                m0 = n0;
                m1 = n1;
                l0 *= c0;
                l1 *= c1;
#pragma unroll
                for (int j = 0; j < D / 8; ++j) {
                    o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1;
                }
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    // a masked score is -inf: exp2f gives 0 (a value row of a never-written page is zeros, finite)
                    sc[nt][0] = fast_exp2(sc[nt][0] * a.scale_log2 - u0);
                    sc[nt][1] = fast_exp2(sc[nt][1] * a.scale_log2 - u0);
                    sc[nt][2] = fast_exp2(sc[nt][2] * a.scale_log2 - u1);
                    sc[nt][3] = fast_exp2(sc[nt][3] * a.scale_log2 - u1);
                    l0 += sc[nt][0] + sc[nt][1];
                    l1 += sc[nt][2] + sc[nt][3];
                }
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) {
                    uint32_t pf[4];
                    pf[0] = pack_bf16(sc[2 * kb][0], sc[2 * kb][1]);
                    pf[1] = pack_bf16(sc[2 * kb][2], sc[2 * kb][3]);
                    pf[2] = pack_bf16(sc[2 * kb + 1][0], sc[2 * kb + 1][1]);
                    pf[3] = pack_bf16(sc[2 * kb + 1][2], sc[2 * kb + 1][3]);
                    pv_16keys_sw(o, pf, vt + kb * 16 * 128, lane);
                }
                __syncwarp();
                if (lane == 0) tt_mbar_arrive(&empty_bar[s]);                // the stage may be filled again
            }
            // every consumer is done with the ring (its first stages are reused for the partial sums
            // below), and snew, vnew are visible to the first consumer
            asm volatile("bar.sync 1, %0;" ::"n"(TT_CONSUMERS * 32) : "memory");
            if (has_new && cw == 0) {                                          // fold the new key into this warp's sums
                const float s0 = snew[g], s1 = snew[g + 8];
                const float n0 = fmaxf(m0, s0), n1 = fmaxf(m1, s1);
                const float c0 = fast_exp2(m0 * a.scale_log2 - n0 * a.scale_log2), c1 = fast_exp2(m1 * a.scale_log2 - n1 * a.scale_log2);
                const float p0 = fast_exp2(s0 * a.scale_log2 - n0 * a.scale_log2), p1 = fast_exp2(s1 * a.scale_log2 - n1 * a.scale_log2);
                m0 = n0;
                m1 = n1;
                l0 = l0 * c0 + (tq == 0 ? p0 : 0.f);
                l1 = l1 * c1 + (tq == 0 ? p1 : 0.f);
#pragma unroll
                for (int j = 0; j < D / 8; ++j) {
                    const float v0 = __bfloat162float(vnew[j * 8 + 2 * tq]), v1 = __bfloat162float(vnew[j * 8 + 2 * tq + 1]);
                    o[j][0] = o[j][0] * c0 + p0 * v0; o[j][1] = o[j][1] * c0 + p0 * v1;
                    o[j][2] = o[j][2] * c1 + p1 * v0; o[j][3] = o[j][3] * c1 + p1 * v1;
                }
            }
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
            l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                const int d = j * 8 + 2 * tq;
                wo[(cw * 16 + g) * D + d] = o[j][0];
                wo[(cw * 16 + g) * D + d + 1] = o[j][1];
                wo[(cw * 16 + g + 8) * D + d] = o[j][2];
                wo[(cw * 16 + g + 8) * D + d + 1] = o[j][3];
            }
            if (tq == 0) {
                wm[cw * 16 + g] = m0 == -INFINITY ? -INFINITY : m0 * a.scale_log2;
                wm[cw * 16 + g + 8] = m1 == -INFINITY ? -INFINITY : m1 * a.scale_log2;
                wl[cw * 16 + g] = l0;
                wl[cw * 16 + g + 8] = l1;
            }
        }
        __syncthreads();
        if (!failed_flag) {
            for (int idx = tid; idx < G * D; idx += TT_THREADS) {
                const int r = idx / D, d = idx % D;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < TT_CONSUMERS; ++w) M = fmaxf(M, wm[w * 16 + r]);
                float acc = 0.f, L = 0.f;
#pragma unroll
                for (int w = 0; w < TT_CONSUMERS; ++w) {
                    const float mw = wm[w * 16 + r];
                    const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
                    acc += wo[(w * 16 + r) * D + d] * f;
                    L += wl[w * 16 + r] * f;
                }
                const size_t base = ((size_t)b * Hq + hk * G + r) * n_chunks + chunk;
                a.part_o[base * D + d] = acc;
                if (d == 0) {
                    a.part_ml[base * 2] = M;
                    a.part_ml[base * 2 + 1] = L;
                }
            }
        } else if (tid < G) {
            float* ml = a.part_ml + (((size_t)b * Hq + hk * G + tid) * n_chunks + chunk) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.f;
        }
    } else if (tid < G) {
        float* ml = a.part_ml + (((size_t)b * Hq + hk * G + tid) * n_chunks + chunk) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
    }
    if (tid == 0 && failed_flag) zai_raise(a.status, ZAI_ST_WAIT);

    // ---- the last block of this (request, key/value head) combines the chunks
    // (one fence, by the thread that takes the ticket, behind the block's barrier: the barrier puts every
    // thread's stores before it and the fence is cumulative; a fence in every thread costs each of them the
    // wait for the memory system, which is busy with the other blocks' keys)
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        s_ticket = atomicAdd(&a.tickets[b * Hkv + hk], 1);
    }
    __syncthreads();
    if (s_ticket != n_chunks - 1) return;
    __threadfence();
    for (int idx = tid; idx < G * D; idx += TT_THREADS) {
        const int r = idx / D, d = idx % D;
        const size_t bh = (size_t)b * Hq + hk * G + r;
        const float* ml = a.part_ml + bh * n_chunks * 2;
        float M = -INFINITY;
        for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, __ldcg(ml + 2 * c));
        float acc = 0.f, L = 0.f;
        for (int c = 0; c < n_chunks; ++c) {
            const float mc = __ldcg(ml + 2 * c);
            if (mc == -INFINITY) continue;
            const float f = fast_exp2(mc - M);
            acc += __ldcg(a.part_o + (bh * n_chunks + c) * D + d) * f;
            L += __ldcg(ml + 2 * c + 1) * f;
        }
        a.out[bh * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
    if (tid == 0) a.tickets[b * Hkv + hk] = 0;
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*TtEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TtEncodeTiledFn tt_encode_tiled() {
    static TtEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (TtEncodeTiledFn)p;
    }
    return fn;
}

static int tt_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n < 1) n = 1;
    }
    return n;
}

// 1 if this kernel takes the sizes: head size 64, a page size that is a power of two from 8 to 64,
// at most 16 query heads per key/value head
ZAI_API int zai_decode_attention_tma_supports(int D, int Hq, int Hkv, int page_size) {
    if (D != TT_D || Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16) return 0;
    if (page_size < 8 || page_size > 64 || (page_size & (page_size - 1))) return 0;
    return tt_encode_tiled() != nullptr;
}

// Arguments as zai_decode_attention_fused, plus the number of pages of the pool (with the null
// page) and a status word that a block raises to 1 if one of its waits ran out.
ZAI_API int zai_decode_attention_tma(void* out, float* part_o, float* part_ml, int* tickets, int* status, const void* qkv,
                                     int qkv_cols, const float* q_gamma, const float* k_gamma, float eps,
                                     const float2* cs_table, int rot, void* pages, int num_pages, const int* block_table,
                                     int table_width, const int* positions, int B, int n_chunks, int page_size, int Hq,
                                     int Hkv, int D, float scale, int window, int write_kv, int chunk_keys,
                                     cudaStream_t stream) {
    if (B <= 0) return ZAI_OK;
    if (!zai_decode_attention_tma_supports(D, Hq, Hkv, page_size)) return ZAI_BAD_SIZE;
    if (chunk_keys < TT_TILE || chunk_keys % TT_TILE || n_chunks < 1 || Hkv > 65535 || B > 65535 || n_chunks > 65535 || rot < 0 || rot > D || (rot & 1))
        return ZAI_BAD_SIZE;
    if (reinterpret_cast<uintptr_t>(pages) & 15) return ZAI_BAD_SIZE;
    // the pool as rows of 64 elements: [num_pages * 2 * Hkv * page_size, 64]; a box is one page-head block
    CUtensorMap map;
    const cuuint64_t dims[2] = {TT_D, (cuuint64_t)num_pages * 2 * Hkv * page_size};
    const cuuint64_t strides[1] = {TT_D * 2};
    const cuuint32_t box[2] = {TT_D, (cuuint32_t)page_size};
    const cuuint32_t estr[2] = {1, 1};
    if (tt_encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, pages, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return -6;
    TmaDecodeArgs a;
    a.out = (bf16*)out; a.part_o = part_o; a.part_ml = part_ml; a.tickets = tickets; a.status = status; a.num_pages = num_pages; a.qkv = (const bf16*)qkv;
    a.q_gamma = q_gamma; a.k_gamma = k_gamma; a.cs_table = cs_table; a.pages = (bf16*)pages; a.block_table = block_table;
    a.positions = positions; a.eps = eps; a.scale_log2 = scale * 1.4426950408889634f; a.qkv_cols = qkv_cols; a.rot = rot;
    a.table_width = table_width; a.page_size = page_size; a.Hq = Hq; a.Hkv = Hkv; a.window = window; a.write_kv = write_kv;
    a.chunk_keys = chunk_keys;
    a.page_shift = 0;
    while ((1 << a.page_shift) < page_size) ++a.page_shift;
    const int tiles = chunk_keys / TT_TILE;
    // As many stages as consumer warps (fewer only if the chunk has fewer tiles and the ring never
    // wraps): then a stage is always read by the same warp, which sees its phases in order.  With a
    // stage count that the warps do not divide, the warp that reads a stage's next round could test
    // the barrier while the round before is still in flight, and a parity test cannot tell "two
    // phases behind" from "done".
    static_assert(TT_STAGES % TT_CONSUMERS == 0, "a stage must always be read by the same warp");
    a.stages = tiles < TT_STAGES ? (tiles < 2 ? 2 : tiles) : TT_STAGES;
    const size_t tail = (size_t)16 * (TT_D + 8) * 2 + (size_t)4 * TT_D * 4 + (size_t)2 * TT_D * 2 + 16 * 4;
    const size_t smem = 1024 + (size_t)a.stages * TT_STAGE_BYTES + tail;
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {                // once per device, for the longest ring
        const size_t most = 1024 + (size_t)TT_STAGES * TT_STAGE_BYTES + tail;
        cudaError_t e = cudaFuncSetAttribute(decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
        if (e != cudaSuccess) return (int)e;
    }
    a.chunk_fastest = (long long)B * Hkv * n_chunks > 6 * (long long)tt_sm_count();    // more than two rounds of three blocks per SM
    const dim3 grid = a.chunk_fastest ? dim3(n_chunks, Hkv, B) : dim3(Hkv, B, n_chunks);
    return launch_pdl(decode_tma_kernel, grid, dim3(TT_THREADS), smem, stream, map, a);
}
