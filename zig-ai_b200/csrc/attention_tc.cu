// Prefill attention for head size 64 on the 5th-generation tensor cores.
//
// Same result as prefill_mma_kernel (csrc/attention_mma.cu): causal attention of a step's query rows
// over their requests' pages (cached positions and the step's own), optionally with a window, by
// the online-softmax recurrence over tiles of keys (the reference computes the same sums with one
// thread block per query row and head, src/cuda/paged_attention.cu:230-337).  What differs is where the products
// run: a block owns 128 query rows of one head; per tile of 64 keys
//
//     S = Q K^T      tcgen05.mma, M = 128 (query rows = TMEM lanes), N = 64 keys, K = 64, into TMEM
//     P = exp2(..)   four warps, one query row per thread: the row's 64 scores come from TMEM with
//                    tcgen05.ld (no shuffles: a thread owns its row), the load of the next 32 columns
//                    in flight while these are worked on; P goes back into TMEM (tcgen05.st, two
//                    bfloat16 a column) as the next product's A operand
//     O_t = P V      tcgen05.mma with A in TMEM, N = 64, K = 64 keys, V read straight from its page
//                    layout [key][64] as an MN-major operand, accumulated into O in TMEM; the threads
//                    rescale O there only when a row's reference maximum has to move
//
// TMEM holds two score buffers and two P buffers (tile i uses buffer i & 1), so the products run a
// tile ahead of the softmax: the scores of tile i + 2 are issued when the softmax has read those of
// tile i, and the softmax of tile i + 1 finds its scores ready when it has written P of tile i.
//
// After a row's first tile the threads do not look for a tile's maximum first: they compute P against
// the reference as it is and find the maximum on the way; only if it lies more than 2^8 above the
// reference in some row of the warp does the reference move and the tile get walked again.
//
// Q, K and V reach shared memory by TMA (cp.async.bulk.tensor, no multicast), K and V page by page
// through the block table into six stages of 16 KB.  Roles: warp 0 one lane issues the loads, warp 1
// one lane the products, warps 2-5 are the softmax.
//
// Blocks are handed out heads first, tiles of query rows from the last rows backwards: under the causal
// mask the last rows of a long span walk many more key tiles than the first, a block's tiles are a chain
// (scores, softmax, P, product), and the longest blocks of every head should start first.
// Every wait on an mbarrier is bounded; a block whose wait runs out raises the status word, its roles
// leave their loops, TMEM is freed and the block returns.
#include <cuda.h>
#include "common.cuh"

#define AT_D 64
#define AT_BM 128
#define AT_BN 64
#define AT_THREADS 192
#define AT_STAGES 6
#define AT_SPIN_LIMIT 4000000
#define AT_Q_BYTES (AT_BM * AT_D * 2)                 // 16 KB
#define AT_KV_BYTES (2 * AT_BN * AT_D * 2)            // keys then values: 16 KB
#define AT_TMEM_COLS 256                              // two score buffers in columns 0..127, O in 128..191, two P buffers in 192..255
#define AT_COL_O (2 * AT_BN)
#define AT_COL_P (2 * AT_BN + AT_D)

__device__ __forceinline__ uint32_t at_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ bool at_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
    const uint32_t a = at_smem(bar);
    for (int it = 0; it < AT_SPIN_LIMIT; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
        if (*failed) return false;
    }
    *failed = 1;
    return false;
}
// A warp's wait: lane 0 watches the barrier, the others hear the outcome.
__device__ __forceinline__ bool at_mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* failed) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = at_mbar_wait(bar, parity, failed) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void at_tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(c0), "r"(c1) : "memory");
}
// Operand tile of 128-byte rows with the 128-byte swizzle, groups of 8 rows 1024 bytes apart.  For a
// K-major operand a row is a matrix row (64 k); for an MN-major one a row is one k (64 n).
__device__ __forceinline__ uint64_t at_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void at_umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void at_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 2^x by the special-function unit (x <= 0 here; -inf gives 0)
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void at_tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void at_tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}

__device__ __forceinline__ void at_tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
// A product whose A operand lies in TMEM (row = lane, two bfloat16 of k per 32-bit column)
__device__ __forceinline__ void at_umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// The wait for a thread's TMEM loads, tied to the registers of one of them: what is computed from those
// registers cannot be scheduled ahead of the wait, while another load may stay in flight across it.
__device__ __forceinline__ void at_tmem_wait_ld(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                   "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :: "memory");
}

struct AtArgs {
    bf16* out;                  // [rows of the step, Hq, 64]
    const int* block_table;     // [S, table_width]
    const int* cu_q;            // [S + 1] first row of each request's span
    const int* ctx_lens;        // [S] positions cached before the step
    int* status;                // the step's status word: a wait that ran out, a page id outside the pool
    int num_pages;
    int table_width, S, page_size, page_shift, Hq, Hkv, window;
    float scale_log2;
    // With few tiles of query rows and long contexts, `splits` blocks (grid z) share a tile's key range; each
    // leaves its O [64][128], its rows' references and sums here, and the one that takes the last ticket of
    // the tile combines them (no block waits for another).
    int splits;
    float* part_o;              // [tiles of query rows x heads x splits][64][128]
    float* part_ml;             // [tiles of query rows x heads x splits][2][128]: reference (in the exponent's units), sum
    int* tickets;               // [tiles of query rows x heads], zero between launches
};

template <bool SHARED>               // several blocks (grid z) share a tile of query rows' keys
__global__ void __launch_bounds__(AT_THREADS) prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                const __grid_constant__ CUtensorMap map_kv, const AtArgs a) {
    // All shared memory is dynamic and the tiles come first: 112 KB of tiles, 256 bytes of barriers and
    // words, and the 1 KB the system reserves per block make 115,968 bytes, so that two blocks fit
    // an SM's 233,472 (with a kilobyte of static variables or of alignment slack they would not).
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = smem_raw;
    unsigned char* sQ = base;
    unsigned char* sKV = base + AT_Q_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + AT_STAGES * AT_KV_BYTES);
    uint64_t& q_full = bars[0];
    uint64_t* kv_full = bars + 1;                               // [AT_STAGES]
    uint64_t* kv_empty = bars + 1 + AT_STAGES;                  // [AT_STAGES]
    uint64_t* s_ready = bars + 1 + 2 * AT_STAGES;               // [2] scores of tile i in buffer i & 1
    uint64_t* p_ready = bars + 3 + 2 * AT_STAGES;               // [2] P of tile i in buffer i & 1
    uint64_t* o_ready = bars + 5 + 2 * AT_STAGES;               // [2] the product of tile i has read P buffer i & 1 and added to O
    uint32_t& tmem_base_holder = *reinterpret_cast<uint32_t*>(bars + 7 + 2 * AT_STAGES);
    int* words = reinterpret_cast<int*>(bars + 8 + 2 * AT_STAGES);
    int& failed_flag = words[0];
    int& s_seq = words[1];
    int& s_i0 = words[2];
    volatile int* failed = &failed_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        failed_flag = (at_smem(base) & 1023u) ? 1 : 0;          // the swizzled tiles need 1024-byte alignment
        at_mbar_init(&q_full, 1);
        for (int s = 0; s < AT_STAGES; ++s) {
            at_mbar_init(&kv_full[s], 1);
            at_mbar_init(&kv_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            at_mbar_init(&s_ready[b], 1);
            at_mbar_init(&p_ready[b], 4);                       // one arrival per softmax warp
            at_mbar_init(&o_ready[b], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(at_smem(&tmem_base_holder)), "r"(AT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_holder;
    pdl_trigger();
    pdl_wait();
    if (tid == 0) {
        // Blocks are handed out x fastest, so the heads are x and the tiles of query rows y, numbered from
        // the last rows of the last request backwards: under the causal mask later rows have more keys
        // to walk, and the longest blocks of every head should start first
        int t = (int)gridDim.y - 1 - (int)blockIdx.y, s = 0;
        for (; s < a.S; ++s) {
            const int nt = (a.cu_q[s + 1] - a.cu_q[s] + AT_BM - 1) / AT_BM;
            if (t < nt) break;
            t -= nt;
        }
        s_seq = s;
        s_i0 = t * AT_BM;
    }
    __syncthreads();
    const int s = s_seq, i0 = s_i0;
    const int h = blockIdx.x;
    // the softmax threads' state, kept past the roles for a shared tile's combination
    float m = -INFINITY, l = 0.f;                               // m: the row's reference, in units of the scores
    bool have_o = false;                                        // the row's O in TMEM is complete
    int row0 = 0, rows = 0;
    if (s < a.S && !failed_flag) {
        const int hk = h / (a.Hq / a.Hkv);
        row0 = a.cu_q[s];
        const int q_len = a.cu_q[s + 1] - row0, ctx = a.ctx_lens[s];
        rows = min(AT_BM, q_len - i0);                              // valid query rows of this block
        const int kend = ctx + i0 + rows;                           // one past the last visible key of the block
        const int kbeg = a.window > 0 ? max(ctx + i0 - a.window + 1, 0) : 0;
        int tile0 = kbeg / AT_BN, tile1 = (kend + AT_BN - 1) / AT_BN;
        if (SHARED) {                                               // this block's share of the key tiles
            const int per = (tile1 - tile0 + a.splits - 1) / a.splits;
            tile0 = min(tile0 + (int)blockIdx.z * per, tile1);
            tile1 = min(tile0 + per, tile1);
        }
        const int n_tiles = tile1 - tile0;

        if (warp == 0) {
            if (lane == 0 && n_tiles > 0) {
                // ---- loads: the block's queries, then a stage of keys and values per tile, page by page
                const int* table = a.block_table + (size_t)s * a.table_width;
                const int ps = a.page_size, box_rows = ps < AT_BN ? ps : AT_BN, per_tile = AT_BN / box_rows;
                at_mbar_expect_tx(&q_full, AT_Q_BYTES);
                at_tma_load_2d(sQ, &map_q, h * AT_D, row0 + i0, &q_full);
                int issued = 0;
                for (int i = 0; i < n_tiles; ++i) {
                    const int st = i % AT_STAGES;
                    if (!at_mbar_wait(&kv_empty[st], ((i / AT_STAGES) & 1) ^ 1, failed)) break;
                    at_mbar_expect_tx(&kv_full[st], AT_KV_BYTES);
                    unsigned char* dst = sKV + (size_t)st * AT_KV_BYTES;
                    for (int p = 0; p < per_tile; ++p) {
                        const int key0 = (tile0 + i) * AT_BN + p * box_rows;
                        const int idx = key0 >> a.page_shift, off = key0 & (ps - 1);
                        int page = idx < a.table_width ? table[idx] : 0;              // beyond the table: the null page
                        if ((unsigned)page >= (unsigned)a.num_pages) {                // outside the pool: page 0, and the step is void
                            zai_raise(a.status, ZAI_ST_PAGE);
                            page = 0;
                        }
                        const int krow = ((page * 2 + 0) * a.Hkv + hk) * ps + off;
                        const int vrow = ((page * 2 + 1) * a.Hkv + hk) * ps + off;
                        at_tma_load_2d(dst + (size_t)p * box_rows * 128, &map_kv, 0, krow, &kv_full[st]);
                        at_tma_load_2d(dst + AT_BN * 128 + (size_t)p * box_rows * 128, &map_kv, 0, vrow, &kv_full[st]);
                    }
                    issued = i + 1;
                }
                if (*failed) {                                  // loads already issued still land here: wait for them
                    for (int i = max(issued - AT_STAGES, 0); i < issued; ++i) {
                        const uint32_t addr = at_smem(&kv_full[i % AT_STAGES]);
                        const uint32_t ph = (i / AT_STAGES) & 1;
                        for (int spin = 0; spin < AT_SPIN_LIMIT; ++spin) {
                            uint32_t done;
                            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                         : "=r"(done) : "r"(addr), "r"(ph) : "memory");
                            if (done) break;
                        }
                    }
                    const uint32_t addr = at_smem(&q_full);
                    for (int spin = 0; spin < AT_SPIN_LIMIT; ++spin) {
                        uint32_t done;
                        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                     : "=r"(done) : "r"(addr), "r"(0u) : "memory");
                        if (done) break;
                    }
                }
            }
        } else if (warp == 1) {
            if (lane == 0 && n_tiles > 0) {
                // ---- products.  Instruction descriptors: D 32-bit, A and B bfloat16, M = 128, N = 64; the
                // scores have both operands K-major; O_t has A (P) in TMEM and B (the values) MN-major.
                constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BN >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
                constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(AT_D >> 3) << 17) |
                                             ((uint32_t)(AT_BM >> 4) << 24);
                const uint32_t tS = tmem_base, tO = tmem_base + AT_COL_O, tP = tmem_base + AT_COL_P;
                const uint32_t aQ = at_smem(sQ);
                bool ok = at_mbar_wait(&q_full, 0, failed);
                auto scores = [&](int i) {                      // S = Q K^T of tile i into score buffer i & 1
                    const int st = i % AT_STAGES;
                    if (!at_mbar_wait(&kv_full[st], (i / AT_STAGES) & 1, failed)) return false;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t aK = at_smem(sKV + (size_t)st * AT_KV_BYTES);
#pragma unroll
                    for (int k = 0; k < AT_D / 16; ++k)
                        at_umma(tS + (i & 1) * AT_BN, at_desc(aQ + k * 32), at_desc(aK + k * 32), idesc_s, k > 0 ? 1u : 0u);
                    at_commit(&s_ready[i & 1]);
                    return true;
                };
                // the scores run a tile ahead of the softmax: those of tile i + 2 are issued when the softmax
                // has read those of tile i (same buffer), so tile i + 1's are ready when the softmax of
                // tile i ends
                if (ok) ok = scores(0);
                if (ok && n_tiles > 1) ok = scores(1);
                for (int i = 0; i < n_tiles && ok; ++i) {
                    const int st = i % AT_STAGES;
                    ok = at_mbar_wait(&p_ready[i & 1], (i >> 1) & 1, failed);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t aV = at_smem(sKV + (size_t)st * AT_KV_BYTES + AT_BN * 128);
#pragma unroll
                    for (int kk = 0; kk < AT_BN / 16; ++kk)     // 16 keys a step: eight columns of P, two groups of 8 keys of V
                        at_umma_ts(tO, tP + (i & 1) * (AT_BN / 2) + kk * 8, at_desc(aV + kk * 2048), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
                    at_commit(&o_ready[i & 1]);
                    at_commit(&kv_empty[st]);
                    if (i + 2 < n_tiles) ok = scores(i + 2);
                }
            }
        } else if (n_tiles > 0) {
            // ---- softmax: thread = query row.  O stays in TMEM (the products add to it); the row's
            // reference maximum is only moved, and O and the sum rescaled, when a tile's maximum exceeds
            // it by more than 2^8 (P then stays below 256, exact enough in bfloat16 and 32-bit sums; the
            // result O / l does not depend on the reference).
            const int qd = warp & 3;                            // this warp's quarter of the TMEM lanes
            const int row = qd * 32 + lane;
            const bool valid = row < rows;
            const int qpos = ctx + i0 + row;                    // the row's position: keys 0..qpos are visible
            const int klo = a.window > 0 ? max(qpos - a.window + 1, 0) : 0;
            const uint32_t tS = tmem_base + ((uint32_t)(qd * 32) << 16), tO = tS + AT_COL_O, tP = tS + AT_COL_P;
            const float c = a.scale_log2;
            bool alive = true;
            for (int i = 0; i < n_tiles && alive; ++i) {
                const int key0 = (tile0 + i) * AT_BN;
                if (!at_mbar_wait_warp(&s_ready[i & 1], (i >> 1) & 1, failed)) { alive = false; break; }    // (the warp leaves together)
                const uint32_t tSi = tS + (i & 1) * AT_BN, tPi = tP + (i & 1) * (AT_BN / 2);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // keys of this tile that the row sees: [lo, hi)
                const int lo = valid ? max(klo - key0, 0) : AT_BN, hi = valid ? min(qpos + 1 - key0, AT_BN) : 0;
                const bool full = lo <= 0 && hi >= AT_BN;       // the row sees the whole tile: no masking needed
                // one walk over the row's 64 scores in chunks of 32 columns, the load of the next chunk in
                // flight while this one is worked on: the maximum of the visible scores (`mx`), and with
                // `emit` the probabilities against `ref` into P and their sum (`lt`)
                auto walk = [&](bool emit, float ref, float& mx, float& lt) {
                    uint32_t r[2][32];
                    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, lt4[4] = {0.f, 0.f, 0.f, 0.f};   // four chains each, not one of 64 links
                    at_tmem_ld32_nowait(tSi, r[0]);
#pragma unroll
                    for (int k = 0; k < AT_BN / 32; ++k) {
                        at_tmem_wait_ld(r[k & 1]);
                        if (k + 1 < AT_BN / 32) at_tmem_ld32_nowait(tSi + 32 * (k + 1), r[(k + 1) & 1]);
                        const uint32_t (&x)[32] = r[k & 1];
                        const int c0 = 32 * k;
                        if (!emit) {
                            if (full) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(x[j]));
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                    if (c0 + j >= lo && c0 + j < hi) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(x[j]));
                            }
                            continue;
                        }
                        uint32_t pk[16];
                        if (full) {
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                const float s0 = __uint_as_float(x[j]), s1 = __uint_as_float(x[j + 1]);
                                mx4[(j >> 1) & 3] = fmaxf(mx4[(j >> 1) & 3], fmaxf(s0, s1));
                                const float p0 = at_exp2(s0 * c - ref), p1 = at_exp2(s1 * c - ref);
                                lt4[(j >> 1) & 3] += p0 + p1;
                                __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                                pk[j >> 1] = *reinterpret_cast<uint32_t*>(&v);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                // (a hidden score may be anything, also NaN: it is replaced before the exponential)
                                const int k0 = c0 + j;
                                const bool v0 = k0 >= lo && k0 < hi, v1 = k0 + 1 >= lo && k0 + 1 < hi;
                                const float s0 = v0 ? __uint_as_float(x[j]) : -INFINITY, s1 = v1 ? __uint_as_float(x[j + 1]) : -INFINITY;
                                mx4[(j >> 1) & 3] = fmaxf(mx4[(j >> 1) & 3], fmaxf(s0, s1));
                                const float p0 = at_exp2(s0 * c - ref), p1 = at_exp2(s1 * c - ref);
                                lt4[(j >> 1) & 3] += p0 + p1;
                                __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                                pk[j >> 1] = *reinterpret_cast<uint32_t*>(&v);
                            }
                        }
                        // (This P buffer was read by the product of the tile two before.  That product was issued
                        // before this tile's scores, and the commit behind the scores covers every product issued
                        // before it: the scores being ready says the buffer is free.)
                        at_tmem_st16(tPi + 16 * k, pk);         // 32 keys = 16 columns of P
                    }
                    mx = fmaxf(mx, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
                    lt += (lt4[0] + lt4[1]) + (lt4[2] + lt4[3]);
                };
                // With a reference in every row of the warp, the tile is walked once against it; else the
                // maximum is found first, as a walk of its own.
                const bool speculate = i > 0 && __all_sync(0xffffffffu, m != -INFINITY || !valid);
                float mx = -INFINITY, lt = 0.f;
                if (speculate) walk(true, m == -INFINITY ? 0.f : m * c, mx, lt);
                else walk(false, 0.f, mx, lt);
                if (!alive) break;
                // move the reference?  (warp-wide decision: the TMEM accesses below are the whole warp's)
                float alpha = 1.f;
                if (m == -INFINITY) {
                    m = mx;                                     // nothing summed so far (O and l are 0, or this is the first tile)
                } else if (mx * c > m * c + 8.f) {
                    alpha = at_exp2(m * c - mx * c);
                    m = mx;
                }
                const bool moved = __any_sync(0xffffffffu, alpha != 1.f);
                if (i > 0 && moved) {
                    if (!at_mbar_wait_warp(&o_ready[(i - 1) & 1], ((i - 1) >> 1) & 1, failed)) { alive = false; break; }   // the product before (and with it all before) has added to O
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int c0 = 0; c0 < AT_D; c0 += 32) {
                        uint32_t r[32];
                        at_tmem_ld32(tO + c0, r);
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
                        at_tmem_st32(tO + c0, r);
                    }
                    l *= alpha;
                }
                if (!speculate || moved) {
                    lt = 0.f;
                    float again = -INFINITY;
                    walk(true, m == -INFINITY ? 0.f : m * c, again, lt);   // no key seen so far: every p is 0
                    if (!alive) break;
                }
                l += lt;
                // P (and a rescaled O) are in TMEM before the product-issuing thread hears of it
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) at_mbar_arrive(&p_ready[i & 1]);
            }
            if (alive && at_mbar_wait_warp(&o_ready[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, failed)) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                have_o = true;
                const float inv = l > 0.f ? 1.f / l : 0.f;
                bf16* dst = a.out + ((size_t)(row0 + i0 + row) * a.Hq + h) * AT_D;
#pragma unroll
                for (int c0 = 0; c0 < AT_D && !SHARED; c0 += 32) {
                    uint32_t r[32];
                    at_tmem_ld32(tO + c0, r);
                    if (valid) {
#pragma unroll
                        for (int d = 0; d < 32; d += 8) {
                            uint4 v;
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[d]) * inv, __uint_as_float(r[d + 1]) * inv);
                            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[d + 2]) * inv, __uint_as_float(r[d + 3]) * inv);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[d + 4]) * inv, __uint_as_float(r[d + 5]) * inv);
                            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[d + 6]) * inv, __uint_as_float(r[d + 7]) * inv);
                            v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                            v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                            *reinterpret_cast<uint4*>(dst + c0 + d) = v;
                        }
                    }
                }
            }
        }
    }
    if (SHARED && s < a.S && warp >= 2) {
        // ---- a shared tile of query rows: this block's part into memory, a ticket, and the last one combines
        const int qd = warp & 3, row = qd * 32 + lane;
        const uint32_t tO = tmem_base + ((uint32_t)(qd * 32) << 16) + AT_COL_O;
        const int slot = ((int)gridDim.y - 1 - (int)blockIdx.y) * a.Hq + h;
        const size_t mine = (size_t)slot * a.splits + blockIdx.z;
        float* po = a.part_o + mine * (AT_D * AT_BM);
        float* pml = a.part_ml + mine * (2 * AT_BM);
        const bool ok = have_o && !failed_flag;                 // (a block without key tiles, or one that gave up, has no part)
        pml[row] = (ok && m != -INFINITY) ? m * a.scale_log2 : -INFINITY;
        pml[AT_BM + row] = ok ? l : 0.f;
        if (ok) {
#pragma unroll
            for (int c0 = 0; c0 < AT_D; c0 += 32) {
                uint32_t r[32];
                at_tmem_ld32(tO + c0, r);
#pragma unroll
                for (int j = 0; j < 32; ++j) po[(c0 + j) * AT_BM + row] = __uint_as_float(r[j]);
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");          // the four softmax warps
        if (tid == 64) {
            __threadfence();                                    // (one fence behind the barrier: it is cumulative)
            s_seq = atomicAdd(a.tickets + slot, 1);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s_seq == a.splits - 1) {
            __threadfence();
            float top = -INFINITY, sum = 0.f, acc[AT_D];
#pragma unroll
            for (int d = 0; d < AT_D; ++d) acc[d] = 0.f;
            for (int z = 0; z < a.splits; ++z) {
                const size_t other = (size_t)slot * a.splits + z;
                const volatile float* qml = a.part_ml + other * (2 * AT_BM);
                const float mz = qml[row], lz = qml[AT_BM + row];
                if (mz == -INFINITY) continue;                  // nothing from this part (its O may be unwritten)
                const float ntop = fmaxf(top, mz);
                const float f_old = top == -INFINITY ? 0.f : at_exp2(top - ntop), f_new = at_exp2(mz - ntop);
                const volatile float* qo = a.part_o + other * (AT_D * AT_BM);
                sum = sum * f_old + lz * f_new;
#pragma unroll
                for (int d = 0; d < AT_D; ++d) acc[d] = acc[d] * f_old + qo[d * AT_BM + row] * f_new;
                top = ntop;
            }
            const float inv = sum > 0.f ? 1.f / sum : 0.f;
            if (row < rows) {
                bf16* dst = a.out + ((size_t)(row0 + i0 + row) * a.Hq + h) * AT_D;
#pragma unroll
                for (int d = 0; d < AT_D; d += 8) {
                    uint4 v;
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[d] * inv, acc[d + 1] * inv), p1 = __floats2bfloat162_rn(acc[d + 2] * inv, acc[d + 3] * inv);
                    __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[d + 4] * inv, acc[d + 5] * inv), p3 = __floats2bfloat162_rn(acc[d + 6] * inv, acc[d + 7] * inv);
                    v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                    v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                    *reinterpret_cast<uint4*>(dst + d) = v;
                }
            }
            if (tid == 64) a.tickets[slot] = 0;                 // ready for the next launch
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(AT_TMEM_COLS) : "memory");
    }
    if (tid == 0 && failed_flag) zai_raise(a.status, ZAI_ST_WAIT);
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*AtEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AtEncodeTiledFn at_encode_tiled() {
    static AtEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (AtEncodeTiledFn)p;
    }
    return fn;
}
static int at_make_map(CUtensorMap* map, const void* ptr, cuuint64_t cols, cuuint64_t rows, cuuint32_t box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {AT_D, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return at_encode_tiled()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -6;
}

// 1 if this kernel takes the sizes: head size 64, a page size that is a power of two from 8 to 128 (a tile
// of 64 keys is loaded page by page, or as half of a page of 128)
ZAI_API int zai_prefill_attention_tc_supports(int D, int Hq, int Hkv, int page_size) {
    if (D != AT_D || Hkv < 1 || Hq % Hkv != 0 || Hq > 32767) return 0;
    if (page_size < 8 || page_size > 128 || (page_size & (page_size - 1))) return 0;
    return at_encode_tiled() != nullptr;
}

// How many blocks should share a tile of query rows' keys: 1 when the tiles alone fill the SMs (two blocks
// each) or the contexts are short; else enough to fill them, with at least eight key tiles for each at the
// longest context a block-table row holds, and 16 at most.
ZAI_API int zai_prefill_attention_tc_splits(int n_tiles, int Hq, int table_width, int page_size) {
    static int sms = 0;
    if (!sms) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) sms = n;
        else sms = 148;
    }
    const long long blocks = (long long)n_tiles * Hq, places = 2LL * sms;
    if (blocks <= 0 || 2 * blocks > places) return 1;
    long long want = (places + blocks - 1) / blocks;
    const long long key_tiles = ((long long)table_width * page_size + AT_BN - 1) / AT_BN;
    if (want > key_tiles / 8) want = key_tiles / 8;
    if (want > 16) want = 16;
    return want < 2 ? 1 : (int)want;
}

// out [N, Hq, 64] = attention of q [N, Hq, 64] (N rows in all, `n_tiles` blocks of 128 rows over the
// requests' spans) over the pages [num_pages, 2, Hkv, page_size, 64]; arguments as
// zai_prefill_attention_mma, plus the row and page counts and the status word that a block raises
// if one of its waits ran out or a page id lay outside the pool.  With splits > 1 (zai_prefill_attention_tc_splits
// proposes a number) the caller gives the scratch for the parts: part_o [n_tiles * Hq * splits * 64 * 128]
// and part_ml [n_tiles * Hq * splits * 2 * 128] floats, and tickets [n_tiles * Hq] ints that are zero.
ZAI_API int zai_prefill_attention_tc(void* out, const void* q, const void* pages, int num_pages, int* status,
                                     const int* block_table, int table_width, const int* cu_q, const int* ctx_lens, int N,
                                     int S, int n_tiles, int page_size, int Hq, int Hkv, int D, float scale, int window,
                                     int splits, float* part_o, float* part_ml, int* tickets, cudaStream_t stream) {
    if (N <= 0 || S <= 0 || n_tiles <= 0) return ZAI_OK;
    if (!zai_prefill_attention_tc_supports(D, Hq, Hkv, page_size) || n_tiles > 65535) return ZAI_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(pages) | reinterpret_cast<uintptr_t>(out)) & 15) return ZAI_BAD_SIZE;
    CUtensorMap mq, mkv;
    int e = at_make_map(&mq, q, (cuuint64_t)Hq * AT_D, (cuuint64_t)N, AT_BM);
    if (e) return e;
    e = at_make_map(&mkv, pages, AT_D, (cuuint64_t)num_pages * 2 * Hkv * page_size, (cuuint32_t)(page_size < AT_BN ? page_size : AT_BN));
    if (e) return e;
    AtArgs a;
    a.out = (bf16*)out; a.block_table = block_table; a.cu_q = cu_q; a.ctx_lens = ctx_lens; a.status = status; a.num_pages = num_pages;
    a.table_width = table_width; a.S = S; a.page_size = page_size; a.Hq = Hq; a.Hkv = Hkv; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    if (splits < 1 || splits > 64 || (splits > 1 && (!part_o || !part_ml || !tickets))) return ZAI_BAD_SIZE;
    a.splits = splits; a.part_o = part_o; a.part_ml = part_ml; a.tickets = tickets;
    a.page_shift = 0;
    while ((1 << a.page_shift) < page_size) ++a.page_shift;
    const size_t smem = AT_Q_BYTES + (size_t)AT_STAGES * AT_KV_BYTES + 256;
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {
        cudaError_t err = cudaFuncSetAttribute(prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        // two blocks per SM: ask for the largest shared-memory carve-out
        if (err == cudaSuccess) err = cudaFuncSetAttribute(prefill_tc_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(prefill_tc_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (err != cudaSuccess) return (int)err;
    }
    if (splits > 1) return launch_pdl(prefill_tc_kernel<true>, dim3(Hq, n_tiles, splits), dim3(AT_THREADS), smem, stream, mq, mkv, a);
    return launch_pdl(prefill_tc_kernel<false>, dim3(Hq, n_tiles), dim3(AT_THREADS), smem, stream, mq, mkv, a);
}
