// Matrix products for steps of 17 to 128 rows (decode steps of many requests, short prompt portions)
// on the 5th-generation tensor cores, built to stream the weights once at the memory system's speed:
//
//     y[N, O] = epilogue( x[N, K] . W[O, K]^T ),   bfloat16 operands, 32-bit accumulation in TMEM
//
// With so few rows the product is bound by reading W, and for the small matrices of a layer by the
// latency of a dependent launch.  So:
//   * The weights are the M operand of tcgen05.mma (a tile of 128 weight rows per block), all of the
//     step's rows are the N operand (32, 64 or 128 columns): every weight is read once.
//   * When there are fewer tiles than SMs, K is cut across a thread-block cluster of 2, 4 or 8 blocks;
//     the partial sums are exchanged through distributed shared memory (each block receives the
//     columns of its share of the rows, sums them in rank order, and finishes those rows).
//   * A block's TMA loads of its weights do not depend on the kernel before it and are issued before
//     the dependency wait (programmatic dependent launch); only the loads of x come after it.
//   * What follows the product in the layer is its epilogue:
//       0 bfloat16 store;  1 32-bit store (logits);
//       2 SwiGLU  a = silu(gate) * up  with gate and up stacked as [2F, K]: a tile holds 64 gate rows
//         and the 64 up rows of the same features, two warps hand the up values to the other two
//         through shared memory;
//       3 ShortConv for steps of single tokens: W = [3C, K] stacked as B, C-gate, x~; a tile holds
//         the three rows of 32 channels; u = B x~, y = bias + sum_j w[c, j] state[j, c] + w[c, L-1] u,
//         z = Cgate y, and the state of the row's slot moves on by one
//         (src/cuda/layer_kernels.cu:192-222 for the taps' indexing; the LFM2 gating around it).
// The reference runs each of these as cublasSgemm plus separate kernels (src/matmul/cublas.zig:515-548,
// src/transformer/hybrid_layer.zig:661-669, src/cuda/layer_kernels.cu:62-70).
//
// A block has 192 threads: warp 0 (one lane) issues the TMA loads into a ring of 64-k stages with
// 128-byte swizzle, warp 1 (one lane) issues tcgen05.mma from shared-memory descriptors and commits
// each stage back to the ring, warps 2-5 read the accumulator with tcgen05.ld (a thread owns one
// weight row's sums for all columns) and run the exchange and the epilogue.  No load is multicast.
// Every wait on an mbarrier is bounded: when one runs out the block raises the status word, all its
// roles leave their loops, it still meets its cluster at the barriers, frees its TMEM and returns.
#include <cuda.h>
#include "common.cuh"

#define SG_BM 128
#define SG_BK 64
#define SG_THREADS 192
#define SG_SPIN_LIMIT 4000000
#define SG_MAX_STAGES 12
#define SG_CONV_MAX_TAPS 4

enum { ST_EPI_BF16 = 0, ST_EPI_F32 = 1, ST_EPI_SWIGLU = 2, ST_EPI_CONV = 3 };

__device__ __forceinline__ uint32_t st_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void st_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(st_smem(bar)), "r"(count));
}
__device__ __forceinline__ void st_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(st_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool st_mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(st_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity; gives up after SG_SPIN_LIMIT polls or when another role
// of the block has already given up.  Returns false then.
__device__ __forceinline__ bool st_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
    for (int it = 0; it < SG_SPIN_LIMIT; ++it) {
        if (st_mbar_try(bar, parity)) return true;
        if (*failed) return false;
    }
    *failed = 1;
    return false;
}
__device__ __forceinline__ void st_tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(st_smem(dst)), "l"(map), "r"(st_smem(bar)), "r"(c0), "r"(c1) : "memory");
}
// K-major operand tile with 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t st_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void st_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void st_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(st_smem(bar)) : "memory");
}
// 32 columns of this warp's lanes into registers; the caller waits (tcgen05.wait::ld) once for all its loads
__device__ __forceinline__ void st_tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ uint32_t st_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void st_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t st_cluster_map(uint32_t local_saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_store4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ unsigned long long st_now() {
    return (unsigned long long)clock64();          // cycles of this SM (cheap to read; the global timer is not)
}
#define ST_DBG(slot) do { if (a.dbg && blockIdx.x == 0) a.dbg[slot] = st_now(); } while (0)
__device__ __forceinline__ float st_bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct StreamArgs {
    void* y;
    int* status;
    int N, O, K, ldy;
    int F;                 // SwiGLU: features (O = 2F); ShortConv: channels (O = 3F)
    int R, r_shift;        // weight rows per part in a tile (a power of two): a tile holds PARTS x R rows
    int a_bytes;           // bytes of a stage that the weight rows take (a multiple of 1024)
    int pad_bytes;         // bytes behind the ring that the last stage's product may read past its weight rows
    int ks;                // blocks of a cluster (1: no cluster); K is cut into ks ranges of kb_per 64-k slices
    int kb_per, num_kb;
    int stages;
    // ShortConv epilogue
    const float* conv_w;   // [F, taps]
    const float* conv_b;   // [F] or null
    float* conv_state;     // [slots, state_rows, F]
    const int* slot_ids;   // [N]
    int taps, state_rows, write_state, num_slots;
    unsigned long long* dbg;   // development aid: cycle counts at the steps of block 0's roles (null: none)
};

// A tile's weight rows are PARTS groups of R consecutive rows (one TMA box each): PARTS = 1 for a plain
// product, 2 for SwiGLU (R gate rows and the R up rows of the same features), 3 for the ShortConv
// (the B, C-gate and x~ rows of R channels).  The product instruction always computes 128 rows (TMEM
// lanes); lanes from PARTS x R on hold nothing.  With a small R there are many tiles, so that every
// SM streams a share of a small matrix; every block reads all of x (from L2).
// Shared memory: [ring: stages x (weight rows | BN x 128 B of x)] [16 KB that the last stage's product
// may read past its weight rows] [exchange / hand-over area: 128 x BN floats].
template <int BN, int EPI>
__global__ void __launch_bounds__(SG_THREADS) stream_gemm_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                 const __grid_constant__ CUtensorMap map_x, const StreamArgs a) {
    constexpr int PARTS = EPI == ST_EPI_SWIGLU ? 2 : (EPI == ST_EPI_CONV ? 3 : 1);
    constexpr uint32_t B_BYTES = BN * SG_BK * 2;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_bytes = (uint32_t)a.a_bytes, stage_bytes = a_bytes + B_BYTES;
    float* xch = reinterpret_cast<float*>(ring + (size_t)a.stages * stage_bytes + a.pad_bytes);
    __shared__ uint64_t full_bar[SG_MAX_STAGES], empty_bar[SG_MAX_STAGES], acc_bar;
    __shared__ uint32_t tmem_base_holder;
    __shared__ int failed_flag;
    volatile int* failed = &failed_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ks = a.ks, rank = ks > 1 ? (int)st_cluster_rank() : 0, tile = blockIdx.x / ks;
    const int kb0 = rank * a.kb_per, kb1 = min(kb0 + a.kb_per, a.num_kb), n_kb = max(kb1 - kb0, 0);
    const int stages = a.stages;
    const int R = a.R, o0 = tile * R;                          // the tile's first row inside each part
    const uint32_t loaded = (uint32_t)(PARTS * R * SG_BK * 2) + B_BYTES;      // bytes a stage receives

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        failed_flag = 0;
        for (int s = 0; s < stages; ++s) {
            st_mbar_init(&full_bar[s], 1);
            st_mbar_init(&empty_bar[s], 1);
        }
        st_mbar_init(&acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(st_smem(&tmem_base_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_holder;
    if (threadIdx.x == 0) ST_DBG(0);
    pdl_trigger();
    if (ks > 1) st_cluster_arrive();          // phase 1: "this block runs" (others may write to its shared memory after it)

    auto load_weights = [&](unsigned char* st, int kb, uint64_t* bar) {
#pragma unroll
        for (int p = 0; p < PARTS; ++p)
            st_tma_load_2d(st + (size_t)p * R * SG_BK * 2, &map_w, kb * SG_BK, p * a.F + o0, bar);
    };

    if (warp == 0) {
        if (lane == 0) {
            // the first ring of weights does not depend on the kernel before this one: ask for it now
            const int first = n_kb < stages ? n_kb : stages;
            for (int i = 0; i < first; ++i) {
                st_mbar_expect_tx(&full_bar[i], loaded);
                load_weights(ring + (size_t)i * stage_bytes, kb0 + i, &full_bar[i]);
            }
            ST_DBG(1);
            pdl_wait();
            ST_DBG(2);
            for (int i = 0; i < first; ++i)
                st_tma_load_2d(ring + (size_t)i * stage_bytes + a_bytes, &map_x, (kb0 + i) * SG_BK, 0, &full_bar[i]);
            int issued = first;
            for (int i = first; i < n_kb; ++i) {
                const int s = i % stages;
                if (!st_mbar_wait(&empty_bar[s], ((i / stages) & 1) ^ 1, failed)) break;
                unsigned char* st = ring + (size_t)s * stage_bytes;
                st_mbar_expect_tx(&full_bar[s], loaded);
                load_weights(st, kb0 + i, &full_bar[s]);
                st_tma_load_2d(st + a_bytes, &map_x, (kb0 + i) * SG_BK, 0, &full_bar[s]);
                issued = i + 1;
            }
            ST_DBG(3);
            if (*failed) {
                // copies already issued still land in this block's shared memory: wait for them (bounded)
                for (int i = max(issued - stages, 0); i < issued; ++i)
                    for (int spin = 0; spin < SG_SPIN_LIMIT; ++spin)
                        if (st_mbar_try(&full_bar[i % stages], (i / stages) & 1)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D 32-bit, A and B bfloat16, both K-major, N = BN, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(SG_BM >> 4) << 24);
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % stages;
                if (!st_mbar_wait(&full_bar[s], (i / stages) & 1, failed)) break;
                if (i < 8) ST_DBG(8 + i);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = st_smem(ring + (size_t)s * stage_bytes), sb = sa + a_bytes;
#pragma unroll
                for (int k = 0; k < SG_BK / 16; ++k)
                    st_mma(tmem_base, st_desc(sa + k * 32), st_desc(sb + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
                st_commit(&empty_bar[s]);
                if (i < 8) ST_DBG(16 + i);
            }
            st_commit(&acc_bar);                               // (also after a failure, so that the epilogue wakes)
            ST_DBG(4);
        }
    }

    // ---- the accumulator: a thread of warps 2-5 owns one weight row (TMEM lane) and all BN columns
    const bool epi_warp = warp >= 2;
    const int q = warp & 3, row = q * 32 + lane;
    const int part = row >> a.r_shift, r = row & (R - 1);      // which part's row this lane holds (part >= PARTS: none)
    const bool holds = part < PARTS;
    const int cols_per = BN / (ks > 1 ? ks : 1);               // columns (rows of the step) this block finishes: a power of two
    const int cols_shift = 31 - __clz(cols_per);
    const int c_first = rank * cols_per;
    float acc[BN];                                             // ks == 1: all columns; else only [0, cols_per) are used after the exchange
    if (epi_warp) {
        pdl_wait();
        const bool have = n_kb > 0 && st_mbar_wait(&acc_bar, 0, failed) && !*failed;
        if (threadIdx.x == 64) ST_DBG(5);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
        uint32_t raw[BN];
        if (have && q * 32 < PARTS * R) {                      // (a warp whose lanes all hold nothing skips the loads)
#pragma unroll
            for (int c = 0; c < BN; c += 32) st_tmem_ld32(taddr + c, raw + c);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int c = 0; c < BN; ++c) acc[c] = holds ? __uint_as_float(raw[c]) : 0.f;
        } else {
#pragma unroll
            for (int c = 0; c < BN; ++c) acc[c] = 0.f;
        }
    }
    __syncwarp();                                              // (the lanes of warps 0 and 1 meet again before the aligned barriers)
    if (ks > 1) {
        st_cluster_wait();                                     // phase 1 over: every block of the cluster runs
        // column c of this block's partial sums belongs to block c / cols_per, which keeps the partial sums it
        // receives as [src rank][4 columns][128 rows][4]: a warp's store is 512 contiguous bytes
        if (epi_warp && holds) {
#pragma unroll
            for (int c = 0; c < BN; c += 4) {
                const int dst = c >> cols_shift, c4 = (c & (cols_per - 1)) >> 2;
                const uint32_t mine = st_smem(xch + (((size_t)rank * (cols_per >> 2) + c4) * SG_BM + row) * 4);
                st_cluster_store4(st_cluster_map(mine, (uint32_t)dst), acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
            }
        }
        __syncwarp();
        st_cluster_arrive();                                   // phase 2: all partial sums are written
        st_cluster_wait();
        if (epi_warp) {
#pragma unroll
            for (int c = 0; c < BN; ++c) acc[c] = 0.f;
            if (holds) {
                for (int src = 0; src < ks; ++src) {           // in rank order, whoever ran first
#pragma unroll
                    for (int c4 = 0; c4 < BN / 4; ++c4) {
                        if (c4 * 4 < cols_per) {
                            const float4 v = *reinterpret_cast<const float4*>(xch + (((size_t)src * (cols_per >> 2) + c4) * SG_BM + row) * 4);
                            acc[c4 * 4] += v.x; acc[c4 * 4 + 1] += v.y; acc[c4 * 4 + 2] += v.z; acc[c4 * 4 + 3] += v.w;
                        }
                    }
                }
            }
        }
    }

    // ---- epilogue over the columns this block finishes: step rows c_first .. c_first + cols_per - 1
    if (threadIdx.x == 64) ST_DBG(6);
    if (EPI == ST_EPI_BF16 || EPI == ST_EPI_F32) {
        if (epi_warp && holds) {
            const int o = o0 + r;
            if (o < a.O) {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int n = c_first + c;
                    if (c < cols_per && n < a.N) {
                        if (EPI == ST_EPI_F32) reinterpret_cast<float*>(a.y)[(size_t)n * a.ldy + o] = acc[c];
                        else reinterpret_cast<bf16*>(a.y)[(size_t)n * a.ldy + o] = __float2bfloat16_rn(acc[c]);
                    }
                }
            }
        }
    } else if (epi_warp) {
        // the lanes hand each other their parts' values through shared memory: [column][part][R] floats, in the
        // exchange area (after an exchange its partial sums are in registers by now)
        float* hand = xch;
        if (ks > 1) asm volatile("bar.sync 1, 128;" ::: "memory");            // the four warps have read the partial sums
        const bool giver = EPI == ST_EPI_SWIGLU ? part == 1 : part < 2;         // up rows; B and C-gate rows
        if (giver) {
            const int slot = EPI == ST_EPI_SWIGLU ? 0 : part;
#pragma unroll
            for (int c = 0; c < BN; ++c)
                if (c < cols_per) hand[((size_t)c * 2 + slot) * R + r] = acc[c];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (EPI == ST_EPI_SWIGLU) {
            const int f = o0 + r;
            if (part == 0 && f < a.F) {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int n = c_first + c;
                    if (c < cols_per && n < a.N) {
                        const float g = acc[c], up = hand[(size_t)c * 2 * R + r];
                        reinterpret_cast<bf16*>(a.y)[(size_t)n * a.ldy + f] = __float2bfloat16_rn(__fdividef(g, 1.f + __expf(-g)) * up);
                    }
                }
            }
        } else {
            const int ch = o0 + r;
            if (part == 2 && ch < a.F) {                                       // the x~ rows' lanes finish the channels
                float w[SG_CONV_MAX_TAPS];
#pragma unroll
                for (int j = 0; j < SG_CONV_MAX_TAPS; ++j) w[j] = j < a.taps ? a.conv_w[(size_t)ch * a.taps + j] : 0.f;
                const float bias = a.conv_b ? a.conv_b[ch] : 0.f;
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int n = c_first + c;
                    if (c < cols_per && n < a.N) {
                        // B, C-gate and x~ are rounded to bfloat16 before they are used, as when they are stored
                        const float bv = st_bf16_round(hand[((size_t)c * 2) * R + r]);
                        const float cv = st_bf16_round(hand[((size_t)c * 2 + 1) * R + r]);
                        const float u = bv * st_bf16_round(acc[c]);
                        float* st = a.conv_state + ((size_t)zai_checked_slot(a.slot_ids[n], a.num_slots, a.status) * a.state_rows) * a.F + ch;
                        float prev[SG_CONV_MAX_TAPS - 1];
                        float yv = bias;
#pragma unroll
                        for (int j = 0; j < SG_CONV_MAX_TAPS - 1; ++j) {
                            prev[j] = j < a.taps - 1 ? st[(size_t)j * a.F] : 0.f;
                            if (j < a.taps - 1) yv += w[j] * prev[j];
                        }
#pragma unroll
                        for (int j = 0; j < SG_CONV_MAX_TAPS; ++j)
                            if (j == a.taps - 1) yv += w[j] * u;
                        reinterpret_cast<bf16*>(a.y)[(size_t)n * a.ldy + ch] = __float2bfloat16_rn(cv * yv);
                        if (a.write_state) {
#pragma unroll
                            for (int j = 0; j < SG_CONV_MAX_TAPS - 1; ++j)
                                if (j < a.taps - 1) st[(size_t)j * a.F] = (j + 1 < a.taps - 1) ? prev[j + 1] : u;
                        }
                    }
                }
            }
        }
    }

    if (threadIdx.x == 64) ST_DBG(7);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed_flag) zai_raise(a.status, ZAI_ST_WAIT);
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*StEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static StEncodeTiledFn st_encode_tiled() {
    static StEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (StEncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bfloat16 row-major matrix as a tensor map with boxes of 64 k x box_rows rows, 128-byte swizzle;
// what lies outside the matrix reads as zero.
static int st_make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    StEncodeTiledFn enc = st_encode_tiled();
    if (!enc) return -5;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {SG_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -6;
}

static int st_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n < 1) n = 1;
    }
    return n;
}

static int st_forced_cluster = -1, st_forced_rows = 0;
static unsigned long long* st_debug_times = nullptr;
ZAI_API int zai_stream_debug(unsigned long long* device_buffer) {     // 16 times of block 0's roles per launch, or null
    st_debug_times = device_buffer;
    return 0;
}
ZAI_API int zai_stream_force_cluster(int ks) {          // 0: the launcher chooses (tests use the other values)
    st_forced_cluster = ks;
    return 0;
}
ZAI_API int zai_stream_force_rows(int rows) {           // rows per part of a tile; 0: the launcher chooses
    st_forced_rows = rows;
    return 0;
}

// How a product is cut into blocks: `rows` weight rows per part and tile (a power of two, 8..128 / parts) and
// `ks` blocks per cluster along K.  Enough tiles for every SM where the matrix allows, the largest
// rows that give them; a long K (the feed-forward's second product) is cut across a cluster instead,
// so that a block does not read all of a long x.
static void st_plan(int part_rows, int num_kb, int parts, int bn, int* rows, int* ks) {
    if (st_forced_cluster < 0) {
        const char* e = getenv("ZAI_STREAM_KSPLIT");
        st_forced_cluster = e ? atoi(e) : 0;
    }
    const int sms = st_sm_count();
    const int most = parts == 1 ? 128 : (parts == 2 ? 64 : 32);
    auto tiles_of = [&](int r) { return (part_rows + r - 1) / r; };
    int r = most, k = 1;
    if (parts == 1 && num_kb >= 32) {
        r = part_rows >= 128 * sms ? 128 : 64;
        while (k < 8 && tiles_of(r) * k * 2 <= sms + sms / 8 && num_kb / (k * 2) >= 4 && bn / (k * 2) >= 4) k *= 2;
    } else {
        while (r > 8 && tiles_of(r) < sms - sms / 5) r >>= 1;
    }
    if (st_forced_rows >= 8 && st_forced_rows <= most && (st_forced_rows & (st_forced_rows - 1)) == 0) r = st_forced_rows;
    if (st_forced_cluster == 1 || st_forced_cluster == 2 || st_forced_cluster == 4 || st_forced_cluster == 8) {
        k = parts == 1 ? st_forced_cluster : 1;
        while (k > 1 && (k > num_kb || bn / k < 4)) k /= 2;
    }
    *rows = r;
    *ks = k;
}

template <int BN, int EPI>
static int st_launch(const CUtensorMap& mw, const CUtensorMap& mx, StreamArgs a, int tiles, cudaStream_t stream) {
    constexpr int PARTS = EPI == ST_EPI_SWIGLU ? 2 : (EPI == ST_EPI_CONV ? 3 : 1);
    const size_t stage = (size_t)a.a_bytes + (size_t)BN * SG_BK * 2;
    a.pad_bytes = a.a_bytes < SG_BM * SG_BK * 2 ? SG_BM * SG_BK * 2 : 0;
    const size_t xch = (a.ks > 1 || PARTS > 1) ? (size_t)SG_BM * BN * sizeof(float) : 0;
    const size_t fixed = 1024 + (size_t)a.pad_bytes + xch;
    int stages = a.kb_per < SG_MAX_STAGES ? a.kb_per : SG_MAX_STAGES;
    // several blocks per SM (each issues its own loads and products, and the next kernel's blocks can start
    // their weight loads while this kernel's still run) where that leaves a ring of three stages or the whole
    // K range; else as deep a ring as one block may have
    const size_t small = 108 * 1024, large = 210 * 1024;
    if (fixed + stage * (stages < 3 ? stages : 3) <= small) {
        while (stages > 3 && fixed + stage * stages > small / 2) --stages;      // four blocks if three stages fit in half
        while (fixed + stage * stages > small) --stages;
    } else {
        while (stages > 1 && fixed + stage * stages > large) --stages;
    }
    if (fixed + stage * stages > 220 * 1024) return ZAI_BAD_SIZE;
    a.stages = stages;
    const size_t smem = fixed + stage * stages;
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {
        cudaError_t e = cudaFuncSetAttribute(stream_gemm_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * a.ks));
    cfg.blockDim = dim3(SG_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (a.ks > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = a.ks;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    return (int)cudaLaunchKernelEx(&cfg, stream_gemm_kernel<BN, EPI>, mw, mx, a);
}

// 1 if zai_stream_gemm takes these sizes: 17..128 rows (any count from 1 works, the few-rows kernel is the
// better one below 17), K a multiple of 8, and for the two stacked forms an O that divides.
ZAI_API int zai_stream_gemm_supports(int N, int O, int K, int epilogue) {
    if (N < 1 || N > 128 || O < 1 || K < 8 || (K & 7)) return 0;
    if (epilogue < 0 || epilogue > ST_EPI_CONV) return 0;
    if (epilogue == ST_EPI_SWIGLU && (O & 1)) return 0;
    if (epilogue == ST_EPI_CONV && (O % 3)) return 0;
    return st_encode_tiled() != nullptr;
}

static int st_run(void* y, const void* W, const void* x, int* status, int N, int O, int K, int epilogue, StreamArgs a,
                  cudaStream_t stream) {
    if ((reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return ZAI_BAD_SIZE;
    const int bn = N <= 32 ? 32 : (N <= 64 ? 64 : 128);
    const int parts = epilogue == ST_EPI_SWIGLU ? 2 : (epilogue == ST_EPI_CONV ? 3 : 1);
    a.y = y; a.status = status; a.N = N; a.O = O; a.K = K;
    a.F = parts > 1 ? O / parts : 0;
    a.ldy = parts > 1 ? a.F : O;
    a.num_kb = (K + SG_BK - 1) / SG_BK;
    st_plan(O / parts, a.num_kb, parts, bn, &a.R, &a.ks);
    a.r_shift = 0;
    while ((1 << a.r_shift) < a.R) ++a.r_shift;
    a.a_bytes = (parts * a.R * SG_BK * 2 + 1023) / 1024 * 1024;
    a.kb_per = (a.num_kb + a.ks - 1) / a.ks;
    a.dbg = st_debug_times;
    const int tiles = (O / parts + a.R - 1) / a.R;
    CUtensorMap mw, mx;
    int e = st_make_map(&mw, W, O, K, a.R);
    if (e) return e;
    e = st_make_map(&mx, x, N, K, bn);
    if (e) return e;
#define ST_CASE(BNV, EPIV) if (bn == BNV && epilogue == EPIV) return st_launch<BNV, EPIV>(mw, mx, a, tiles, stream);
    ST_CASE(32, ST_EPI_BF16) ST_CASE(64, ST_EPI_BF16) ST_CASE(128, ST_EPI_BF16)
    ST_CASE(32, ST_EPI_F32) ST_CASE(64, ST_EPI_F32) ST_CASE(128, ST_EPI_F32)
    ST_CASE(32, ST_EPI_SWIGLU) ST_CASE(64, ST_EPI_SWIGLU) ST_CASE(128, ST_EPI_SWIGLU)
    ST_CASE(32, ST_EPI_CONV) ST_CASE(64, ST_EPI_CONV) ST_CASE(128, ST_EPI_CONV)
#undef ST_CASE
    return ZAI_BAD_SIZE;
}

// y = epilogue(x . W^T); x [N, K], W [O, K] bfloat16, both contiguous and 16-byte aligned, N <= 128.
// epilogue 0: y bfloat16 [N, O]; 1: y float [N, O]; 2: SwiGLU, W = gate|up stacked, y bfloat16 [N, O/2].
// `status`: the step's status word (a wait that ran out raises ZAI_ST_WAIT).
ZAI_API int zai_stream_gemm(void* y, const void* W, const void* x, int* status, int N, int O, int K, int epilogue,
                            cudaStream_t stream) {
    if (epilogue == ST_EPI_CONV || !zai_stream_gemm_supports(N, O, K, epilogue)) return ZAI_BAD_SIZE;
    StreamArgs a = {};
    return st_run(y, W, x, status, N, O, K, epilogue, a, stream);
}

// The short convolution's input projection with the convolution as its epilogue, for steps in which every
// row is one token of its own request: W = [3F, K] stacked as B, C-gate, x~; z bfloat16 [N, F]; the state
// [num_slots, state_rows, F] of row n's slot slot_ids[n] moves on by one if write_state.  taps <= 4.
ZAI_API int zai_stream_conv(void* z, const void* W, const void* x, int* status, const float* conv_w, const float* conv_b,
                            float* state, const int* slot_ids, int N, int F, int K, int taps, int state_rows,
                            int write_state, int num_slots, cudaStream_t stream) {
    if (F < 1 || taps < 1 || taps > SG_CONV_MAX_TAPS || state_rows < taps - 1 || num_slots < 1) return ZAI_BAD_SIZE;
    if (!zai_stream_gemm_supports(N, 3 * F, K, ST_EPI_CONV)) return ZAI_BAD_SIZE;
    StreamArgs a = {};
    a.conv_w = conv_w; a.conv_b = conv_b; a.conv_state = state; a.slot_ids = slot_ids;
    a.taps = taps; a.state_rows = state_rows; a.write_state = write_state; a.num_slots = num_slots;
    return st_run(z, W, x, status, N, 3 * F, K, ST_EPI_CONV, a, stream);
}
