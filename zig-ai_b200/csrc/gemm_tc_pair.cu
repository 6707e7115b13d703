// Matrix products for steps of many rows on the 5th-generation tensor cores, two blocks to a tile:
//
//     y[N, O] = epilogue( x[N, K] . W[O, K]^T ),   bfloat16 operands, 32-bit accumulation in TMEM
//
// A cluster of two blocks (on two SMs) owns a tile of 256 tokens x 256 (or 128) weight rows.  The
// tokens are the M operand of tcgen05.mma.cta_group::2: each block loads its 128 tokens and keeps
// their 128 accumulator rows in its own TMEM lanes.  The weight rows are the N operand, and each
// block loads only half of them: the tensor cores of both SMs read both halves.  So a block brings
// 32 KB per 64-k slice for 128 x 256 x 64 products, where a one-block tile of the same size needs
// 48 KB: the operand traffic from L2, which bounds the one-block kernel, falls by a third.
//
// Epilogues: bfloat16 store; 32-bit store; SwiGLU a = silu(gate) * up with the gate and up matrices
// stacked as [2F, K]: the first block of the pair loads 128 gate rows, the second the 128 up rows of
// the same outputs, so the accumulator columns 0..127 are gates, 128..255 the matching ups, and one
// thread (one token) holds both values of an output and stores 32 neighbouring outputs at a time.
//
// The reference runs these products as cublasSgemm followed by a separate activation kernel
// (src/matmul/cublas.zig:515-548, src/transformer/hybrid_layer.zig:661-669, src/cuda/layer_kernels.cu:62-70).
//
// Structure of a block (192 threads), both blocks of a pair alike unless said:
//   warp 0, one lane   TMA producer: loads this block's token tile and its half of the weight tile
//                      of every 64-k slice into a ring of stages (128-byte swizzle).  Both blocks'
//                      loads count on the FIRST block's "full" barrier of the stage.
//   warp 1, one lane   first block only: waits for a stage, issues four tcgen05.mma.cta_group::2
//                      (M 256, N 256 or 128, K 16); tcgen05.commit frees the stage in both blocks
//                      and, after the last slice, wakes both blocks' epilogues
//   warps 2-5          read this block's accumulator rows with tcgen05.ld, apply the epilogue, store;
//                      then tell the first block that the accumulator buffer is free
// Pairs are persistent (tiles taken round robin); TMEM holds the accumulators of two tiles, so a
// tile's epilogue overlaps the next tile's products.  No load is sent to more than one block.
// Every wait on an mbarrier is bounded: when it runs out the block raises an error word in global
// memory, every role leaves its loop, the pair meets at a cluster barrier, TMEM is freed and the
// blocks return; the host reports the error.
#include <cuda.h>
#include <cstdlib>
#include "common.cuh"

#define TP_BM 128
#define TP_BK 64
#define TP_THREADS 192
#define TP_SPIN_LIMIT 4000000

enum { TP_EPI_BF16 = 0, TP_EPI_F32 = 1, TP_EPI_SWIGLU = 2 };

__device__ __forceinline__ uint32_t tp_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t tp_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void tp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of this block's shared-memory location `a` in block `rank` of the cluster
__device__ __forceinline__ uint32_t tp_map_to(uint32_t a, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ void tp_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tp_smem(bar)), "r"(count));
}
__device__ __forceinline__ void tp_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tp_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tp_mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Waits for the phase with the given parity of a barrier of this block; gives up after
// TP_SPIN_LIMIT polls or when another role of the block has already failed.  Returns false then.
__device__ __forceinline__ bool tp_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
    const uint32_t a = tp_smem(bar);
    for (int it = 0; it < TP_SPIN_LIMIT; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
        if (*failed) return false;
    }
    *failed = 1;
    return false;
}
// One block's tile into its own shared memory; the bytes count on the barrier at `bar_cluster_addr`,
// which may lie in the other block of the pair.
__device__ __forceinline__ void tp_tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(tp_smem(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
// asks for a tile to be brought into L2 (no destination, nothing to wait for)
__device__ __forceinline__ void tp_tma_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}
// K-major operand tile with 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t tp_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tp_mma_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the products issued so far are done, on the barrier at this offset in both blocks
__device__ __forceinline__ void tp_commit_both(uint64_t* bar) {
    asm volatile("{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
                 "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
                 ::"r"(tp_smem(bar)) : "memory");
}
__device__ __forceinline__ void tp_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ uint32_t tp_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct TpArgs {
    void* y;
    int* status;          // set to 1 by a block whose wait ran out
    int N, O, K, ldy;
    int F;                // SwiGLU: gate rows 0..F-1, up rows F..2F-1
    int stages, prefetch;
    int tiles_m, tiles;   // tiles along the tokens; all tiles (tile t: token tile t % tiles_m, weight tile t / tiles_m)
};

// 32 neighbouring outputs of one token: as 16-byte stores when the row allows it
template <int EPI>
__device__ __forceinline__ void tp_store32(const TpArgs& a, int row, int col0, int col_limit, const float (&v)[32]) {
    if (EPI == TP_EPI_F32) {
        float* dst = reinterpret_cast<float*>(a.y) + (size_t)row * a.ldy + col0;
        if (col0 + 32 <= col_limit && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
            for (int j = 0; j < 32 && col0 + j < col_limit; ++j) dst[j] = v[j];
        }
    } else {
        bf16* dst = reinterpret_cast<bf16*>(a.y) + (size_t)row * a.ldy + col0;
        if (col0 + 32 <= col_limit && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8)
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(tp_pack(v[j], v[j + 1]), tp_pack(v[j + 2], v[j + 3]),
                                                                tp_pack(v[j + 4], v[j + 5]), tp_pack(v[j + 6], v[j + 7]));
        } else {
            for (int j = 0; j < 32 && col0 + j < col_limit; ++j) dst[j] = __float2bfloat16_rn(v[j]);
        }
    }
}

// WR: weight rows that one block loads per tile (the pair's accumulator has 2 WR columns)
template <int WR, int EPI>
__global__ void __launch_bounds__(TP_THREADS) gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                                                               const __grid_constant__ CUtensorMap map_w, const TpArgs a) {
    constexpr uint32_t A_BYTES = TP_BM * TP_BK * 2, B_BYTES = WR * TP_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t BN = 2 * WR;                            // accumulator columns of a tile
    constexpr uint32_t TMEM_COLS = 2 * BN;                     // two tiles: 512 or 256
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // (static shared memory lies at the same offsets in both blocks, which the two-block commit relies on)
    __shared__ uint64_t full_bar[8], empty_bar[8], acc_full_bar[2], acc_empty_bar[2];
    __shared__ uint32_t tmem_base_holder;
    __shared__ int failed_flag;
    volatile int* failed = &failed_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tp_cluster_rank();                   // 0: the block that issues the products
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int stages = a.stages;
    const int num_kb = (a.K + TP_BK - 1) / TP_BK;

    if (threadIdx.x == 0) {
        failed_flag = 0;
        for (int s = 0; s < stages; ++s) {
            tp_mbar_init(&full_bar[s], 1);                     // the first block's: its own expect_tx arrival
            tp_mbar_init(&empty_bar[s], 1);                    // one commit
        }
        for (int i = 0; i < 2; ++i) {
            tp_mbar_init(&acc_full_bar[i], 1);                 // one commit
            tp_mbar_init(&acc_empty_bar[i], 8);                // the first block's: four epilogue warps of each block
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                           // the same warp of both blocks allocates the pair's columns
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tp_smem(&tmem_base_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    tp_cluster_sync();                                         // both blocks' barriers exist before either is used
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_holder;
    pdl_trigger();
    // The weights are no kernel's output: the producer asks for its first tile's weight rows to be
    // brought into L2 while the kernel before this one still runs.  (Later tiles' rows are asked for
    // one tile ahead, below: a load that misses L2 takes twice as long to land, and the ring holds
    // too few bytes to cover that.)
    auto weight_row = [&](int t) {
        const int nt = t / a.tiles_m;
        return EPI == TP_EPI_SWIGLU ? (rank == 0 ? nt * WR : a.F + nt * WR) : nt * (2 * WR) + (int)rank * WR;
    };
    if (a.prefetch && warp == 0 && lane == 0 && pair < a.tiles) {
        const int w_row = weight_row(pair);
        for (int kb = 0; kb < num_kb; ++kb) tp_tma_prefetch_2d(&map_w, kb * TP_BK, w_row);
    }
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            int it = 0, issued = 0;                            // `it` counts k-blocks over all of this pair's tiles
            bool ok = true;
            for (int t = pair; t < a.tiles && ok; t += n_pairs) {
                const int m0 = (t % a.tiles_m) * (2 * TP_BM) + (int)rank * TP_BM;
                const int w_row = weight_row(t);
                const int next_row = (a.prefetch && t + n_pairs < a.tiles) ? weight_row(t + n_pairs) : -1;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    if (next_row >= 0 && next_row != w_row) tp_tma_prefetch_2d(&map_w, kb * TP_BK, next_row);
                    const int s = it % stages;
                    const uint32_t ph = (it / stages) & 1;
                    if (!tp_mbar_wait(&empty_bar[s], ph ^ 1, failed)) { ok = false; break; }
                    unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                    if (rank == 0) tp_mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
                    const uint32_t bar = tp_map_to(tp_smem(&full_bar[s]), 0);
                    tp_tma_load_2d(st, &map_x, kb * TP_BK, m0, bar);
                    tp_tma_load_2d(st + A_BYTES, &map_w, kb * TP_BK, w_row, bar);
                    issued = it + 1;
                }
            }
            if (*failed && rank == 0) {
                // copies already issued still land in the pair's shared memory and count on this block's
                // barriers: wait for them (bounded) before the pair goes on to its end
                for (int i = max(issued - stages, 0); i < issued; ++i) {
                    const uint32_t a_ = tp_smem(&full_bar[i % stages]);
                    const uint32_t ph = (i / stages) & 1;
                    for (int spin = 0; spin < TP_SPIN_LIMIT; ++spin) {
                        uint32_t done;
                        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                     : "=r"(done) : "r"(a_), "r"(ph) : "memory");
                        if (done) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // instruction descriptor: D fp32, A and B bfloat16, both K-major, N = BN, M = 256 over the pair
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * TP_BM) >> 4) << 24);
            bool ok = true;
            int it = 0, local = 0;
            for (int t = pair; t < a.tiles && ok; t += n_pairs, ++local) {
                const int buf = local & 1;
                const uint32_t acc = tmem_base + buf * BN;
                // both blocks' epilogues must have drained this buffer (two tiles ago)
                ok = tp_mbar_wait(&acc_empty_bar[buf], ((local >> 1) & 1) ^ 1, failed);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % stages;
                    const uint32_t ph = (it / stages) & 1;
                    ok = tp_mbar_wait(&full_bar[s], ph, failed);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = tp_smem(tiles + (size_t)s * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int k = 0; k < TP_BK / 16; ++k)
                        tp_mma_pair(acc, tp_desc(sa + k * 32), tp_desc(sb + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tp_commit_both(&empty_bar[s]);             // the stage is free in both blocks once these products are done
                }
                tp_commit_both(&acc_full_bar[buf]);            // (also after a failure, so that the epilogues wake)
            }
        }
    } else {
        const int q = warp & 3;                                // this warp's quarter of the TMEM lanes
        const uint32_t acc_empty0 = tp_map_to(tp_smem(&acc_empty_bar[0]), 0);
        const uint32_t acc_empty1 = tp_map_to(tp_smem(&acc_empty_bar[1]), 0);
        int local = 0;
        for (int t = pair; t < a.tiles; t += n_pairs, ++local) {
            const int buf = local & 1;
            const int row = (t % a.tiles_m) * (2 * TP_BM) + (int)rank * TP_BM + q * 32 + lane, nt = t / a.tiles_m;
            if (!tp_mbar_wait(&acc_full_bar[buf], (local >> 1) & 1, failed) || *failed) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
            constexpr int OUT_COLS = EPI == TP_EPI_SWIGLU ? WR : (int)BN;
            const int col_base = nt * OUT_COLS, col_limit = EPI == TP_EPI_SWIGLU ? a.F : a.O;
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += 32) {
                uint32_t r[32];
                float v[32];
                tp_tmem_ld32(acc + c0, r);
                if (EPI == TP_EPI_SWIGLU) {
                    uint32_t u[32];
                    tp_tmem_ld32(acc + WR + c0, u);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float g = __uint_as_float(r[j]);
                        v[j] = __fdividef(g, 1.f + __expf(-g)) * __uint_as_float(u[j]);
                    }
                } else {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                }
                if (c0 + 32 >= OUT_COLS) {                     // everything of this buffer is in registers now
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) tp_mbar_arrive_cluster(buf ? acc_empty1 : acc_empty0);
                }
                if (row < a.N && col_base + c0 < col_limit) tp_store32<EPI>(a, row, col_base + c0, col_limit, v);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    tp_cluster_sync();                 // neither block leaves while the other may still read its tiles or signal its barriers
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed_flag) zai_raise(a.status, ZAI_ST_WAIT);
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*TpEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TpEncodeTiledFn tp_encode_tiled() {
    static TpEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (TpEncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bfloat16 row-major matrix as a tensor map with boxes of 64 k x box_rows rows, 128-byte swizzle.
static int tp_make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    TpEncodeTiledFn enc = tp_encode_tiled();
    if (!enc) return -5;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {TP_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -6;
}

static int tp_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n < 2) n = 2;
    }
    return n;
}

template <int WR, int EPI>
static int tp_launch(const CUtensorMap& mx, const CUtensorMap& mw, TpArgs a, int w_tiles, cudaStream_t stream) {
    const size_t stage = (size_t)TP_BM * TP_BK * 2 + (size_t)WR * TP_BK * 2;
    static const int budget_kb = getenv("ZAI_PAIR_SMEM_KB") ? atoi(getenv("ZAI_PAIR_SMEM_KB")) : 196;
    static const int prefetch = getenv("ZAI_PAIR_PREFETCH") ? atoi(getenv("ZAI_PAIR_PREFETCH")) : 1;
    int stages = (int)(((size_t)budget_kb * 1024) / stage);
    if (stages > 8) stages = 8;
    if (stages < 2) return ZAI_BAD_SIZE;
    a.stages = stages;
    a.prefetch = prefetch;
    const size_t smem = stage * stages + 1024;
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<WR, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    a.tiles_m = (a.N + 2 * TP_BM - 1) / (2 * TP_BM);
    a.tiles = a.tiles_m * w_tiles;
    const int pairs = a.tiles < tp_sm_count() / 2 ? a.tiles : tp_sm_count() / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(TP_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, gemm_pair_kernel<WR, EPI>, mx, mw, a);
}

ZAI_API int zai_gemm_pair_supports(int N, int O, int K, int epilogue) {
    if (N < 1 || O < 1 || K < 8 || (K & 7)) return 0;        // TMA wants rows of a multiple of 16 bytes
    if (epilogue < 0 || epilogue > 2 || (epilogue == TP_EPI_SWIGLU && (O & 1))) return 0;
    return tp_encode_tiled() != nullptr;
}

// y = epilogue(x . W^T); x [N, K], W [O, K] bfloat16, both contiguous and 16-byte aligned.
// epilogue 0: y bfloat16 [N, O]; 1: y float [N, O]; 2: SwiGLU, W = gate|up stacked, y bfloat16 [N, O/2].
// `wide`: 1 = tiles of 256 weight rows (128 outputs for SwiGLU), 0 = 128 (64), -1 = chosen here.
// `status` is a device int that a block sets to 1 if one of its waits ran out.
ZAI_API int zai_gemm_pair(void* y, const void* W, const void* x, int* status, int N, int O, int K, int epilogue, int wide,
                          cudaStream_t stream) {
    if (!zai_gemm_pair_supports(N, O, K, epilogue)) return ZAI_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return ZAI_BAD_SIZE;
    const int out_cols = epilogue == TP_EPI_SWIGLU ? O / 2 : O;
    const int per_wide = epilogue == TP_EPI_SWIGLU ? 128 : 256;              // outputs of a wide tile
    const int tiles_m = (N + 2 * TP_BM - 1) / (2 * TP_BM);
    if (wide < 0) {
        // wide tiles need a third less operand traffic; narrow ones when wide ones leave pairs idle
        // or fill the last round badly
        const int pairs = tp_sm_count() / 2;
        const int tw = tiles_m * ((out_cols + per_wide - 1) / per_wide), tn = tiles_m * ((out_cols + per_wide / 2 - 1) / (per_wide / 2));
        const double rounds_w = (double)((tw + pairs - 1) / pairs), rounds_n = 0.5 * 1.25 * (double)((tn + pairs - 1) / pairs);
        wide = rounds_w <= rounds_n ? 1 : 0;
    }
    const int wr = wide ? 128 : 64;
    CUtensorMap mx, mw;
    int e = tp_make_map(&mx, x, N, K, TP_BM);
    if (e) return e;
    e = tp_make_map(&mw, W, O, K, wr);
    if (e) return e;
    TpArgs a;
    a.y = y; a.status = status; a.N = N; a.O = O; a.K = K;
    a.F = O / 2;
    a.ldy = out_cols;
    a.stages = 0; a.prefetch = 0; a.tiles_m = 0; a.tiles = 0;
    const int per = wide ? per_wide : per_wide / 2;
    const int w_tiles = (out_cols + per - 1) / per;
#define TP_CASE(WRV, EPIV) if (wr == WRV && epilogue == EPIV) return tp_launch<WRV, EPIV>(mx, mw, a, w_tiles, stream);
    TP_CASE(128, TP_EPI_BF16) TP_CASE(64, TP_EPI_BF16)
    TP_CASE(128, TP_EPI_F32) TP_CASE(64, TP_EPI_F32)
    TP_CASE(128, TP_EPI_SWIGLU) TP_CASE(64, TP_EPI_SWIGLU)
#undef TP_CASE
    return ZAI_BAD_SIZE;
}
