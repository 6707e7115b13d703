// Matrix products for steps of many rows on the 5th-generation tensor cores:
//
//     y[N, O] = epilogue( x[N, K] . W[O, K]^T ),   bfloat16 operands, 32-bit accumulation in TMEM
//
// The weights are the M operand of tcgen05.mma (128 rows per tile) and the tokens the N operand
// (128 or 256 per tile), so the accumulator D[o, token] has one weight row per TMEM lane and one
// token per TMEM column.  Epilogues: bfloat16 store; 32-bit store; SwiGLU a = silu(gate) * up with
// the gate and up matrices stacked as [2F, K] (each tile accumulates the gate rows f0..f0+127 and
// the up rows F+f0.. into two accumulators, so one thread holds both values of an output).
//
// The reference runs these products as cublasSgemm followed by a separate activation kernel
// (src/matmul/cublas.zig:515-548, src/transformer/hybrid_layer.zig:661-669, src/cuda/layer_kernels.cu:62-70).
//
// Structure of a block (192 threads):
//   warp 0, one lane   TMA producer: cp.async.bulk.tensor loads of 64-k slices of the weight and
//                      token tiles into a ring of shared-memory stages (128-byte swizzle), each
//                      stage signalled by an mbarrier with the expected byte count
//   warp 1, one lane   issues tcgen05.mma (kind::f16, cta_group::1, M = 128, N = tile's tokens,
//                      K = 16, four per stage and accumulator) from shared-memory descriptors;
//                      tcgen05.commit frees the stage, and after the last slice signals the epilogue
//   warps 2-5          read the accumulators with tcgen05.ld (each warp its quarter of the lanes),
//                      apply the epilogue and store
// Blocks are persistent (one per SM, tiles taken round robin) and TMEM holds the accumulators of two
// tiles, so a tile's epilogue overlaps the next tile's products.
// TMA loads are never multicast.  Every wait on an mbarrier is bounded: when it runs out the block
// raises an error word in global memory, every role leaves its loop, TMEM is freed and the block
// returns; the host reports the error.
#include <cuda.h>
#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_SPIN_LIMIT 4000000

enum { TC_EPI_BF16 = 0, TC_EPI_F32 = 1, TC_EPI_SWIGLU = 2 };

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// Waits for the phase with the given parity; gives up after TC_SPIN_LIMIT polls or when another
// role has already failed.  Returns false then.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
    const uint32_t a = smem_addr(bar);
    for (int it = 0; it < TC_SPIN_LIMIT; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
        if (*failed) return false;
    }
    *failed = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1) : "memory");
}
// K-major operand tile with 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}

struct TcArgs {
    void* y;
    int* status;          // set to 1 by a block whose wait ran out
    int N, O, K, ldy;
    int F;                // SwiGLU: gate rows 0..F-1, up rows F..2F-1
    int stages;
    int tiles_o, tiles;   // tiles along the weight rows; all tiles (tile t: o tile t % tiles_o, token tile t / tiles_o)
};

// Blocks are persistent: block b takes tiles b, b + gridDim.x, ...  The accumulator memory holds two
// tiles, so the epilogue of one tile runs while the products of the next are issued.
template <int BN, int EPI, int ACC_BUFS>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                             const __grid_constant__ CUtensorMap map_x, const TcArgs a) {
    constexpr int NA = EPI == TC_EPI_SWIGLU ? 2 : 1;           // accumulators per tile (weight tiles per stage)
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = NA * A_BYTES + B_BYTES;
    constexpr uint32_t TILE_COLS = NA * BN;                    // TMEM columns of one tile's accumulators
    constexpr uint32_t TMEM_COLS = ACC_BUFS * TILE_COLS;       // one or two tiles: 128..512, a power of two
    static_assert(TMEM_COLS <= 512, "the accumulators must fit the 512 TMEM columns");
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_bar[8], empty_bar[8], acc_full_bar[2], acc_empty_bar[2];
    __shared__ uint32_t tmem_base_holder;
    __shared__ int failed_flag;
    volatile int* failed = &failed_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages = a.stages;
    const int num_kb = (a.K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        failed_flag = 0;
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full_bar[i], 1);
            mbar_init(&acc_empty_bar[i], 4);                   // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                           // one warp allocates the accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(&tmem_base_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_holder;
    pdl_trigger();
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0, it = 0;                            // `it` counts k-blocks over all of this block's tiles
            bool ok = true;
            for (int t = blockIdx.x; t < a.tiles && ok; t += gridDim.x) {
                const int o0 = (t % a.tiles_o) * TC_BM, n0 = (t / a.tiles_o) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % stages;
                    const uint32_t ph = (it / stages) & 1;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1, failed)) { ok = false; break; }
                    unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                    tma_load_2d(st, &map_w, kb * TC_BK, o0, &full_bar[s]);
                    if (NA == 2) tma_load_2d(st + A_BYTES, &map_w, kb * TC_BK, a.F + o0, &full_bar[s]);
                    tma_load_2d(st + NA * A_BYTES, &map_x, kb * TC_BK, n0, &full_bar[s]);
                    issued = it + 1;
                }
            }
            if (*failed) {
                // copies already issued still land in this block's shared memory: wait for them (bounded)
                for (int i = max(issued - stages, 0); i < issued; ++i) {
                    const uint32_t a_ = smem_addr(&full_bar[i % stages]);
                    const uint32_t ph = (i / stages) & 1;
                    for (int spin = 0; spin < TC_SPIN_LIMIT; ++spin) {
                        uint32_t done;
                        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                     : "=r"(done) : "r"(a_), "r"(ph) : "memory");
                        if (done) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D fp32, A and B bfloat16, both K-major, N = BN, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            bool ok = true;
            int it = 0, local = 0;
            for (int t = blockIdx.x; t < a.tiles && ok; t += gridDim.x, ++local) {
                const int buf = local % ACC_BUFS;
                const uint32_t acc = tmem_base + buf * TILE_COLS;
                // the epilogue must have drained this buffer (ACC_BUFS tiles ago)
                ok = mbar_wait(&acc_empty_bar[buf], ((local / ACC_BUFS) & 1) ^ 1, failed);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % stages;
                    const uint32_t ph = (it / stages) & 1;
                    ok = mbar_wait(&full_bar[s], ph, failed);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = smem_addr(tiles + (size_t)s * STAGE_BYTES);
                    const uint32_t sb = sa + NA * A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        const uint64_t db = umma_desc(sb + k * 32);
                        umma_bf16(acc, umma_desc(sa + k * 32), db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        if (NA == 2) umma_bf16(acc + BN, umma_desc(sa + A_BYTES + k * 32), db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);                // the stage is free once these products are done
                }
                umma_commit(&acc_full_bar[buf]);               // (also after a failure, so that the epilogue wakes)
            }
        }
    } else {
        const int q = warp & 3;                                // this warp's quarter of the TMEM lanes
        const int row = q * 32 + lane;
        const int o_limit = EPI == TC_EPI_SWIGLU ? a.F : a.O;
        int local = 0;
        for (int t = blockIdx.x; t < a.tiles; t += gridDim.x, ++local) {
            const int buf = local % ACC_BUFS;
            const int o = (t % a.tiles_o) * TC_BM + row, n0 = (t / a.tiles_o) * BN;
            if (!mbar_wait(&acc_full_bar[buf], (local / ACC_BUFS) & 1, failed) || *failed) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_base + buf * TILE_COLS + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32], u[32];
                tmem_ld32(acc + c0, r);
                if (EPI == TC_EPI_SWIGLU) tmem_ld32(acc + BN + c0, u);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c0 + 32 >= BN) {                           // everything of this buffer is in registers now
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&acc_empty_bar[buf])) : "memory");
                }
                if (o < o_limit && n0 + c0 < a.N) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int n = n0 + c0 + j;
                        if (n >= a.N) break;
                        const float v = __uint_as_float(r[j]);
                        if (EPI == TC_EPI_SWIGLU) {
                            const float up = __uint_as_float(u[j]);
                            reinterpret_cast<bf16*>(a.y)[(size_t)n * a.ldy + o] =
                                __float2bfloat16_rn(__fdividef(v, 1.f + __expf(-v)) * up);
                        } else if (EPI == TC_EPI_F32) {
                            reinterpret_cast<float*>(a.y)[(size_t)n * a.ldy + o] = v;
                        } else {
                            reinterpret_cast<bf16*>(a.y)[(size_t)n * a.ldy + o] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed_flag) zai_raise(a.status, ZAI_ST_WAIT);
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bfloat16 row-major matrix as a tensor map with boxes of 64 k x box_rows rows, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return -5;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -6;
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n < 1) n = 1;
    }
    return n;
}

template <int BN, int EPI, int ACC_BUFS>
static int tc_launch(const CUtensorMap& mw, const CUtensorMap& mx, TcArgs a, int o_tiles, cudaStream_t stream) {
    constexpr int NA = EPI == TC_EPI_SWIGLU ? 2 : 1;
    const size_t stage = (size_t)NA * TC_BM * TC_BK * 2 + (size_t)BN * TC_BK * 2;
    int stages = (int)(((size_t)200 * 1024) / stage);
    if (stages > 8) stages = 8;
    if (stages < 2) return ZAI_BAD_SIZE;
    a.stages = stages;
    const size_t smem = stage * stages + 1024;
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, ACC_BUFS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    a.tiles_o = o_tiles;
    a.tiles = o_tiles * ((a.N + BN - 1) / BN);
    const int grid = a.tiles < sm_count() ? a.tiles : sm_count();
    return launch_pdl(gemm_tc_kernel<BN, EPI, ACC_BUFS>, dim3(grid), dim3(TC_THREADS), smem, stream, mw, mx, a);
}

ZAI_API int zai_gemm_tc_supports(int N, int O, int K, int epilogue) {
    if (N < 1 || O < 1 || K < 8 || (K & 7)) return 0;        // TMA wants rows of a multiple of 16 bytes
    if (epilogue == TC_EPI_SWIGLU && (O & 1)) return 0;
    return encode_tiled() != nullptr;
}

// y = epilogue(x . W^T); x [N, K], W [O, K] bfloat16, both contiguous and 16-byte aligned.
// epilogue 0: y bfloat16 [N, O]; 1: y float [N, O]; 2: SwiGLU, W = gate|up stacked, y bfloat16 [N, O/2].
// `status` is a device int that a block sets to 1 if one of its waits ran out.
ZAI_API int zai_gemm_tc(void* y, const void* W, const void* x, int* status, int N, int O, int K, int epilogue,
                        cudaStream_t stream) {
    if (!zai_gemm_tc_supports(N, O, K, epilogue)) return ZAI_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return ZAI_BAD_SIZE;
    // two tiles' accumulators share the 512 TMEM columns: 256 tokens per tile, 128 when a tile has two
    // accumulators; 128 also when 256 would leave SMs without a tile
    // (for SwiGLU a tile of 256 tokens would fill all 512 columns and its epilogue could not overlap
    // the next tile's products; measured no faster, so 128)
    const int o_rows = epilogue == TC_EPI_SWIGLU ? O / 2 : O;
    int bn = (N > 128 && epilogue != TC_EPI_SWIGLU) ? 256 : 128;
    if (bn == 256 && ((o_rows + TC_BM - 1) / TC_BM) * ((N + 255) / 256) < sm_count()) bn = 128;
    CUtensorMap mw, mx;
    int e = make_map(&mw, W, O, K, TC_BM);
    if (e) return e;
    e = make_map(&mx, x, N, K, bn);
    if (e) return e;
    TcArgs a;
    a.y = y; a.status = status; a.N = N; a.O = O; a.K = K;
    a.F = O / 2;
    a.ldy = epilogue == TC_EPI_SWIGLU ? O / 2 : O;
    a.stages = 0; a.tiles_o = 0; a.tiles = 0;
    const int o_tiles = ((epilogue == TC_EPI_SWIGLU ? a.F : O) + TC_BM - 1) / TC_BM;
#define TC_CASE(BNV, EPIV, BUFS) if (bn == BNV && epilogue == EPIV) return tc_launch<BNV, EPIV, BUFS>(mw, mx, a, o_tiles, stream);
    TC_CASE(128, TC_EPI_BF16, 2) TC_CASE(256, TC_EPI_BF16, 2)
    TC_CASE(128, TC_EPI_F32, 2) TC_CASE(256, TC_EPI_F32, 2)
    TC_CASE(128, TC_EPI_SWIGLU, 2) TC_CASE(256, TC_EPI_SWIGLU, 1)
#undef TC_CASE
    return ZAI_BAD_SIZE;
}
