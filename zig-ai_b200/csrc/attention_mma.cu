// Paged attention on the tensor cores (bfloat16 operands, 32-bit accumulation and softmax):
//
//   * prefill: a flash-style kernel over block tables.  One block takes 128 consecutive query rows
//     of one request and one query head (eight warps of 16 rows); it walks the request's cached keys in tiles of 64 (the
//     cached prefix and the rows of this very step, which are already in the pages), keeps the
//     running maximum, the running sum and the unnormalised output of each row in registers and
//     never writes scores to memory.  Spans of one token are handled too, so a mixed step needs no
//     second kernel.
//   * decode: every row is one token.  One block takes one request, one key/value head and one
//     chunk of 256 keys; the query heads that share the key/value head are the rows of one 16-row
//     tile, so keys and values are read once per group.  Each of the four warps takes 16 keys of
//     every 64-key tile.  Blocks write unnormalised partial outputs with their maximum and sum to
//     scratch memory and a second kernel combines the chunks (no block waits on another).
//
// The reference's kernels give one warp to each (token, head) and walk all keys serially
// (src/cuda/paged_attention.cu:121-225 decode, :230-337 prefill).  Same mathematics: scores
// q.k/sqrt(D) (src/transformer/hybrid_attn.zig:571), causal bound on the absolute position (:587),
// max-subtracted softmax (:578-600), query head h reads key/value head h / (Hq/Hkv)
// (src/cuda/paged_attention.cu:142).
//
// Key tiles start at multiples of 64 counted from position 0 and chunks at multiples of 256, so a
// row's sums are formed in the same order however the request was cut into steps and whatever
// else is in the batch.  Pages: [num_pages, 2, Hkv, page_size, D].
#include "common.cuh"
#include "mma_helpers.cuh"

#define TILE 64              // keys per tile, query rows per prefill block
#define CHUNK 256            // keys per decode block
#define NTHREADS 128
#ifndef ZAI_DECODE_STAGES
#define ZAI_DECODE_STAGES 2
#endif

// Rows t0 .. t0+63 of the keys (kv = 0) or values (kv = 1) of one head into shared memory, row
// stride D + 8 elements; rows outside [kstart, kend) are filled with zeros.  `page_shift` is
// log2(page_size) if that is a power of two, else -1.
template <int D, int NT>
__device__ __forceinline__ void load_kv_tile(bf16* dst, const bf16* __restrict__ pages, const ZaiTableRow& table,
                                             int t0, int kstart, int kend, int page_size, int page_shift,
                                             size_t page_stride, size_t head_off, int tid) {
    constexpr int CH = D / 8;
    for (int idx = tid; idx < TILE * CH; idx += NT) {
        const int r = idx / CH, c = idx % CH;
        const int j = t0 + r;
        const bool valid = j >= kstart && j < kend;
        const bf16* src = pages;
        if (valid) {
            int page, off;
            if (page_shift >= 0) {
                page = table.page(j >> page_shift);
                off = j & (page_size - 1);
            } else {
                page = table.page(j / page_size);
                off = j % page_size;
            }
            src = pages + (size_t)page * page_stride + head_off + (size_t)off * D + c * 8;
        }
        cp_async16(dst + r * (D + 8) + c * 8, src, valid);
    }
}

// The same for one warp alone: rows t0 .. t0+63 of keys and values of one head, each row's page
// looked up once for both.
template <int D>
__device__ __forceinline__ void load_kv_tile_warp(bf16* kdst, bf16* vdst, const bf16* __restrict__ pages,
                                                  const ZaiTableRow& table, int t0, int kstart, int kend,
                                                  int page_size, int page_shift, size_t page_stride, size_t k_off,
                                                  size_t v_off, int lane) {
    constexpr int CH = D / 8;
    for (int idx = lane; idx < TILE * CH; idx += 32) {
        const int r = idx / CH, c = idx % CH;
        const int j = t0 + r;
        const bool valid = j >= kstart && j < kend;
        const bf16* src = pages;
        if (valid) {
            int page, off;
            if (page_shift >= 0) {
                page = table.page(j >> page_shift);
                off = j & (page_size - 1);
            } else {
                page = table.page(j / page_size);
                off = j % page_size;
            }
            src = pages + (size_t)page * page_stride + (size_t)off * D + c * 8;
        }
        cp_async16(kdst + r * (D + 8) + c * 8, src + (valid ? k_off : 0), valid);
        cp_async16(vdst + r * (D + 8) + c * 8, src + (valid ? v_off : 0), valid);
    }
}

// S[16 x 16 keys] += Q (A fragments of all D/16 steps) . K^T for the 16 keys at `krows` (shared, stride D+8)
template <int D>
__device__ __forceinline__ void qk_16keys(float (&s0)[4], float (&s1)[4], const uint32_t (&qf)[D / 16][4],
                                          const bf16* krows, int lane) {
    const int key = ((lane >> 4) << 3) + (lane & 7);       // matrices 0,1: keys 0-7; 2,3: keys 8-15
    const int dof = ((lane >> 3) & 1) << 3;                // matrices 1,3: dims +8
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t b[4];
        ldmatrix_x4(b, krows + key * (D + 8) + ks * 16 + dof);
        mma_bf16(s0, qf[ks], b[0], b[1]);
        mma_bf16(s1, qf[ks], b[2], b[3]);
    }
}

// O[16 x D] += P (one A fragment: 16 rows x 16 keys) . V for the 16 keys at `vrows`
template <int D>
__device__ __forceinline__ void pv_16keys(float (&o)[D / 8][4], const uint32_t (&pf)[4], const bf16* vrows, int lane) {
    const int key = (((lane >> 3) & 1) << 3) + (lane & 7);  // matrices 1,3: keys 8-15
    const int dof = (lane >> 4) << 3;                       // matrices 2,3: dims +8
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vrows + key * (D + 8) + dp * 16 + dof);
        mma_bf16(o[2 * dp], pf, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
    }
}

// ------------------------------------------------------------------------------------------ prefill
#define PREFILL_WARPS 8
#define PREFILL_ROWS (16 * PREFILL_WARPS)      // query rows per block

template <int D>
__global__ void __launch_bounds__(PREFILL_WARPS * 32) prefill_mma_kernel(
    bf16* __restrict__ out, const bf16* __restrict__ q, const bf16* __restrict__ pages,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ cu_q,
    const int* __restrict__ ctx_lens, int S, int page_size, int Hq, int Hkv, float scale_log2, int window,
    int num_pages, int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int ST = D + 8, NT = PREFILL_WARPS * 32, QR = PREFILL_ROWS;
    bf16* sq = reinterpret_cast<bf16*>(smem_raw);           // [QR][ST]
    bf16* sk = sq + QR * ST;                                // [2][64][ST]
    bf16* sv = sk + 2 * TILE * ST;                          // [2][64][ST]
    __shared__ int s_seq, s_i0;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    pdl_trigger();
    pdl_wait();
    if (tid == 0) {
        // blocks are numbered from the last rows of the last request backwards: under the causal
        // mask later rows have more keys to walk, and the longest blocks should start first
        int t = gridDim.x - 1 - blockIdx.x, s = 0;
        for (; s < S; ++s) {
            const int nt = (cu_q[s + 1] - cu_q[s] + QR - 1) / QR;
            if (t < nt) break;
            t -= nt;
        }
        s_seq = s;
        s_i0 = t * QR;
    }
    __syncthreads();
    const int s = s_seq, i0 = s_i0;
    if (s >= S) return;
    const int h = blockIdx.y, hk = h / (Hq / Hkv);
    const int row0 = cu_q[s], q_len = cu_q[s + 1] - row0, ctx = ctx_lens[s];
    const int rows = min(QR, q_len - i0);                   // valid query rows of this block
    const ZaiTableRow table{block_table + (size_t)s * table_width, table_width, num_pages, status};
    const size_t page_stride = (size_t)2 * Hkv * page_size * D;
    const size_t k_off = (size_t)hk * page_size * D, v_off = ((size_t)Hkv + hk) * page_size * D;
    const int kend = ctx + i0 + rows;                       // one past the last visible key of the block
    int kbeg = 0;
    if (window > 0) kbeg = max(ctx + i0 - window + 1, 0);
    const int tile0 = kbeg / TILE, tile1 = (kend + TILE - 1) / TILE;

    // queries of the block: rows beyond the span are zeros
    for (int idx = tid; idx < QR * (D / 8); idx += NT) {
        const int r = idx / (D / 8), c = idx % (D / 8);
        const bool valid = r < rows;
        const bf16* src = valid ? q + ((size_t)(row0 + i0 + r) * Hq + h) * D + c * 8 : q;
        cp_async16(sq + r * ST + c * 8, src, valid);
    }
    load_kv_tile<D, NT>(sk, pages, table, tile0 * TILE, kbeg, kend, page_size, page_shift, page_stride, k_off, tid);
    load_kv_tile<D, NT>(sv, pages, table, tile0 * TILE, kbeg, kend, page_size, page_shift, page_stride, v_off, tid);
    cp_async_commit();

    uint32_t qf[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;       // rows g and g+8 of the warp's 16
    const int g = lane >> 2, tq = lane & 3;
    const int p0 = ctx + i0 + warp * 16 + g, p1 = p0 + 8;          // positions of the two rows
    const int lo0 = window > 0 ? p0 - window + 1 : 0, lo1 = window > 0 ? p1 - window + 1 : 0;
    const bool warp_has_rows = warp * 16 < rows;

    for (int t = tile0; t < tile1; ++t) {
        const int buf = (t - tile0) & 1;
        if (t + 1 < tile1) {
            load_kv_tile<D, NT>(sk + (buf ^ 1) * TILE * ST, pages, table, (t + 1) * TILE, kbeg, kend, page_size,
                                page_shift, page_stride, k_off, tid);
            load_kv_tile<D, NT>(sv + (buf ^ 1) * TILE * ST, pages, table, (t + 1) * TILE, kbeg, kend, page_size,
                                page_shift, page_stride, v_off, tid);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (t == tile0) {
            const int r = warp * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
            const int dof = (lane >> 4) << 3;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], sq + r * ST + ks * 16 + dof);
        }
        const bf16* kt = sk + buf * TILE * ST;
        const bf16* vt = sv + buf * TILE * ST;
        // a warp whose rows all lie before this tile's first key, or that has no rows, skips the tile
        const int warp_last_pos = ctx + i0 + warp * 16 + 15;
        const int warp_first_lo = window > 0 ? ctx + i0 + warp * 16 - window + 1 : 0;
        if (warp_has_rows && t * TILE <= warp_last_pos && (t + 1) * TILE > warp_first_lo) {
            float sc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) qk_16keys<D>(sc[2 * kb], sc[2 * kb + 1], qf, kt + kb * 16 * ST, lane);
            float mx0 = -INFINITY, mx1 = -INFINITY;
            const bool diag = (t + 1) * TILE - 1 > ctx + i0 + warp * 16 || window > 0;   // some element may be masked
            if (diag) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int j = t * TILE + nt * 8 + 2 * tq + e;
                        if (j > p0 || j < lo0) sc[nt][e] = -INFINITY;
                        if (j > p1 || j < lo1) sc[nt][2 + e] = -INFINITY;
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
            const float u0 = n0 == -INFINITY ? 0.f : n0 * scale_log2;    // a row with nothing visible yet
            const float u1 = n1 == -INFINITY ? 0.f : n1 * scale_log2;
            const float c0 = fast_exp2(m0 * scale_log2 - u0), c1 = fast_exp2(m1 * scale_log2 - u1);
            m0 = n0;
            m1 = n1;
            l0 *= c0;
            l1 *= c1;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                sc[nt][0] = fast_exp2(sc[nt][0] * scale_log2 - u0);
                sc[nt][1] = fast_exp2(sc[nt][1] * scale_log2 - u0);
                sc[nt][2] = fast_exp2(sc[nt][2] * scale_log2 - u1);
                sc[nt][3] = fast_exp2(sc[nt][3] * scale_log2 - u1);
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
                pv_16keys<D>(o, pf, vt + kb * 16 * ST, lane);
            }
        }
        __syncthreads();                                    // the buffer is loaded again two tiles on
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int d = i * 8 + 2 * tq;
        if (r0 < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + i0 + r0) * Hq + h) * D + d) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
        if (r1 < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + i0 + r1) * Hq + h) * D + d) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

// ------------------------------------------------------------------------------------------ decode
// part_o [B, Hq, n_chunks, D] unnormalised outputs; part_ml [B, Hq, n_chunks, 2]: maximum (in log2
// units, already scaled) and sum.  A chunk with no visible key writes (-inf, 0).
template <int D> struct DecodeStages { static constexpr int N = ZAI_DECODE_STAGES; };   // tiles in flight + 1

template <int D>
__global__ void __launch_bounds__(NTHREADS) decode_mma_kernel(
    float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q,
    const bf16* __restrict__ pages, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ positions, int page_size, int Hq, int Hkv, float scale_log2, int window,
    int num_pages, int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int ST = D + 8, NS = DecodeStages<D>::N;
    bf16* sq = reinterpret_cast<bf16*>(smem_raw);           // [16][ST]
    bf16* sk = sq + 16 * ST;                                // [NS][64][ST]
    bf16* sv = sk + NS * TILE * ST;                         // [NS][64][ST]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z, n_chunks = gridDim.x;
    const int G = Hq / Hkv;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    pdl_trigger();
    pdl_wait();
    const int pos = positions[b];
    const int kend = pos + 1;
    const int kstart = window > 0 ? max(pos - window + 1, 0) : 0;
    const int lo = max(chunk * CHUNK, kstart), hi = min((chunk + 1) * CHUNK, kend);
    if (lo >= hi) {
        if (tid < G) {
            float* ml = part_ml + (((size_t)b * Hq + hk * G + tid) * n_chunks + chunk) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.f;
        }
        return;
    }
    const ZaiTableRow table{block_table + (size_t)b * table_width, table_width, num_pages, status};
    const size_t page_stride = (size_t)2 * Hkv * page_size * D;
    const size_t k_off = (size_t)hk * page_size * D, v_off = ((size_t)Hkv + hk) * page_size * D;
    const int tile0 = lo / TILE, tile1 = (hi + TILE - 1) / TILE;

    for (int idx = tid; idx < 16 * (D / 8); idx += NTHREADS) {
        const int r = idx / (D / 8), c = idx % (D / 8);
        const bool valid = r < G;
        const bf16* src = valid ? q + ((size_t)b * Hq + hk * G + r) * D + c * 8 : q;
        cp_async16(sq + r * ST + c * 8, src, valid);
    }
    // the first NS-1 tiles start moving at once; one group is committed per tile slot, used or not
#pragma unroll
    for (int s = 0; s < NS - 1; ++s) {
        if (tile0 + s < tile1) {
            load_kv_tile<D, NTHREADS>(sk + s * TILE * ST, pages, table, (tile0 + s) * TILE, lo, hi, page_size, page_shift, page_stride, k_off, tid);
            load_kv_tile<D, NTHREADS>(sv + s * TILE * ST, pages, table, (tile0 + s) * TILE, lo, hi, page_size, page_shift, page_stride, v_off, tid);
        }
        cp_async_commit();
    }

    uint32_t qf[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int g = lane >> 2, tq = lane & 3;

    for (int t = tile0; t < tile1; ++t) {
        const int buf = (t - tile0) % NS;
        cp_async_wait<NS - 2>();                            // tile t has arrived
        __syncthreads();                                    // and everyone is done with tile t-1
        {
            const int nxt = t + NS - 1;
            if (nxt < tile1) {
                const int nb = (nxt - tile0) % NS;
                load_kv_tile<D, NTHREADS>(sk + nb * TILE * ST, pages, table, nxt * TILE, lo, hi, page_size, page_shift, page_stride, k_off, tid);
                load_kv_tile<D, NTHREADS>(sv + nb * TILE * ST, pages, table, nxt * TILE, lo, hi, page_size, page_shift, page_stride, v_off, tid);
            }
            cp_async_commit();
        }
        if (t == tile0) {
            const int r = (((lane >> 3) & 1) << 3) + (lane & 7);
            const int dof = (lane >> 4) << 3;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], sq + r * ST + ks * 16 + dof);
        }
        const int j0 = t * TILE + warp * 16;                // this warp's 16 keys of the tile
        if (j0 < hi && j0 + 16 > lo) {
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
            qk_16keys<D>(s0, s1, qf, sk + (buf * TILE + warp * 16) * ST, lane);
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int ja = j0 + 2 * tq + e, jb = ja + 8;
                if (ja < lo || ja >= hi) { s0[e] = -INFINITY; s0[2 + e] = -INFINITY; }
                if (jb < lo || jb >= hi) { s1[e] = -INFINITY; s1[2 + e] = -INFINITY; }
                mx0 = fmaxf(mx0, fmaxf(s0[e], s1[e]));
                mx1 = fmaxf(mx1, fmaxf(s0[2 + e], s1[2 + e]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);   // finite: the warp has a visible key
            const float u0 = n0 * scale_log2, u1 = n1 * scale_log2;
            const float c0 = fast_exp2(m0 * scale_log2 - u0), c1 = fast_exp2(m1 * scale_log2 - u1);
            m0 = n0;
            m1 = n1;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
            }
            s0[0] = fast_exp2(s0[0] * scale_log2 - u0); s0[1] = fast_exp2(s0[1] * scale_log2 - u0);
            s0[2] = fast_exp2(s0[2] * scale_log2 - u1); s0[3] = fast_exp2(s0[3] * scale_log2 - u1);
            s1[0] = fast_exp2(s1[0] * scale_log2 - u0); s1[1] = fast_exp2(s1[1] * scale_log2 - u0);
            s1[2] = fast_exp2(s1[2] * scale_log2 - u1); s1[3] = fast_exp2(s1[3] * scale_log2 - u1);
            l0 = l0 * c0 + s0[0] + s0[1] + s1[0] + s1[1];
            l1 = l1 * c1 + s0[2] + s0[3] + s1[2] + s1[3];
            uint32_t pf[4];
            pf[0] = pack_bf16(s0[0], s0[1]);
            pf[1] = pack_bf16(s0[2], s0[3]);
            pf[2] = pack_bf16(s1[0], s1[1]);
            pf[3] = pack_bf16(s1[2], s1[3]);
            pv_16keys<D>(o, pf, sv + (buf * TILE + warp * 16) * ST, lane);
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                        // the tiles are no longer needed
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // combine the four warps through shared memory (the tiles are no longer needed)
    float* wo = reinterpret_cast<float*>(sk);               // [4][16][D]
    float* wm = wo + 4 * 16 * D;                            // [4][16] maxima (log2 units)
    float* wl = wm + 4 * 16;                                // [4][16] sums
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int d = i * 8 + 2 * tq;
        wo[(warp * 16 + g) * D + d] = o[i][0];
        wo[(warp * 16 + g) * D + d + 1] = o[i][1];
        wo[(warp * 16 + g + 8) * D + d] = o[i][2];
        wo[(warp * 16 + g + 8) * D + d + 1] = o[i][3];
    }
    if (tq == 0) {
        wm[warp * 16 + g] = m0 == -INFINITY ? -INFINITY : m0 * scale_log2;
        wm[warp * 16 + g + 8] = m1 == -INFINITY ? -INFINITY : m1 * scale_log2;
        wl[warp * 16 + g] = l0;
        wl[warp * 16 + g + 8] = l1;
    }
    __syncthreads();
    for (int idx = tid; idx < G * D; idx += NTHREADS) {
        const int r = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, wm[w * 16 + r]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = wm[w * 16 + r];
            const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
            acc += wo[(w * 16 + r) * D + d] * f;
            L += wl[w * 16 + r] * f;
        }
        const size_t base = ((size_t)b * Hq + hk * G + r) * n_chunks + chunk;
        part_o[base * D + d] = acc;
        if (d == 0) {
            part_ml[base * 2] = M;
            part_ml[base * 2 + 1] = L;
        }
    }
}

template <int D>
__global__ void decode_combine_kernel(bf16* __restrict__ out, const float* __restrict__ part_o,
                                      const float* __restrict__ part_ml, int n_chunks) {
    pdl_trigger();
    pdl_wait();
    const size_t bh = blockIdx.x;                           // b * Hq + h
    const float* ml = part_ml + bh * n_chunks * 2;
    float M = -INFINITY;
    for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, ml[2 * c]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f, L = 0.f;
        for (int c = 0; c < n_chunks; ++c) {
            const float mc = ml[2 * c];
            if (mc == -INFINITY) continue;
            const float f = fast_exp2(mc - M);
            acc += part_o[(bh * n_chunks + c) * D + d] * f;
            L += ml[2 * c + 1] * f;
        }
        out[bh * D + d] = __float2bfloat16_rn(acc / L);
    }
}

template <int D> static size_t decode_smem();

// ------------------------------------------------------------------------------------------ fused decode
// The decode step's whole attention in one kernel, from the raw qkv projection to the output:
//   * the block normalises (per-head RMSNorm) and rotates its group's query rows itself;
//   * the block whose chunk holds the new position does the same for the new key, writes key and
//     value into the request's page, and folds that one key into its sums directly (it is not read
//     back from the page in this step);
//   * blocks write their partial sums as before, take a ticket per (request, key/value head), and
//     the block that draws the last ticket combines all chunks and writes the output (no block waits
//     for another; the ticket counter is left at zero for the next call).
// This replaces three kernels of the unfused path (q/k norm + rotary + page write, the chunk
// kernel, the combine kernel; the reference has one kernel each for norm, rotary, append and
// attention, src/transformer/hybrid_attn.zig:710-764).
struct FusedDecodeArgs {
    bf16* out;                 // [B, Hq, D]
    float* part_o;             // [B, Hq, n_chunks, D]
    float* part_ml;            // [B, Hq, n_chunks, 2]
    int* tickets;              // [B * Hkv], zero before and after
    const bf16* qkv;           // [B, qkv_cols] = q heads | k heads | v heads
    const float* q_gamma;      // [D] or null
    const float* k_gamma;      // [D] or null
    const float2* cs_table;    // [B, rot/2] (cos, sin) of each row's position, or null when rot == 0
    bf16* pages;
    const int* block_table;
    const int* positions;
    float eps, scale_log2;
    int qkv_cols, rot, table_width, page_size, Hq, Hkv, window, write_kv;
    int num_pages;             // pages in `pages`: a table entry outside is read as page 0 and raises the status word
    int* status;
    int chunk_keys;            // keys per block: a multiple of 64
};

template <int D>
__global__ void __launch_bounds__(NTHREADS) decode_fused_kernel(const FusedDecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int ST = D + 8;
    bf16* sq = reinterpret_cast<bf16*>(smem_raw);           // [16][ST]
    bf16* sk = sq + 16 * ST;                                // [4 warps][64][ST]: each warp loads and reads its own tiles
    bf16* sv = sk + 4 * TILE * ST;                          // [4 warps][64][ST]
    float* tmp = reinterpret_cast<float*>(sv + 4 * TILE * ST);    // [4][D] scratch of the four warps
    bf16* knew = reinterpret_cast<bf16*>(tmp + 4 * D);      // [D] the new key, [D] the new value
    bf16* vnew = knew + D;
    float* snew = reinterpret_cast<float*>(vnew + D);       // [16] scores of the new key
    __shared__ int s_ticket;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z, n_chunks = gridDim.x;
    const int Hq = a.Hq, Hkv = a.Hkv, G = Hq / Hkv, page_size = a.page_size;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    pdl_trigger();
    pdl_wait();
    const int pos = a.positions[b];
    const int kstart = a.window > 0 ? max(pos - a.window + 1, 0) : 0;
    const bool has_new = a.write_kv && chunk == pos / a.chunk_keys;        // this block owns the new key
    const int kend = a.write_kv ? pos : pos + 1;                    // keys read from the pages
    const int lo = max(chunk * a.chunk_keys, kstart), hi = min((chunk + 1) * a.chunk_keys, kend);
    const bool any_paged = lo < hi;
    const ZaiTableRow table{a.block_table + (size_t)b * a.table_width, a.table_width, a.num_pages, a.status};
    const size_t page_stride = (size_t)2 * Hkv * page_size * D;
    const size_t k_off = (size_t)hk * page_size * D, v_off = ((size_t)Hkv + hk) * page_size * D;
    const int tile0 = lo / TILE, tile1 = any_paged ? (hi + TILE - 1) / TILE : tile0;

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int g = lane >> 2, tq = lane & 3;

    if (any_paged || has_new) {
        // each warp takes the tiles tile0 + warp, tile0 + warp + 4, ... of the chunk and loads them
        // itself (no block-wide barrier per tile); the first one starts moving now
        bf16* wk = sk + warp * TILE * ST;
        bf16* wv = sv + warp * TILE * ST;
        if (tile0 + warp < tile1)
            load_kv_tile_warp<D>(wk, wv, a.pages, table, (tile0 + warp) * TILE, lo, hi, page_size, page_shift, page_stride, k_off, v_off, lane);
        cp_async_commit();
        // meanwhile: the group's queries, and the new key and value
        const bf16* row = a.qkv + (size_t)b * a.qkv_cols;
        const float2* cs = a.rot ? a.cs_table + (size_t)b * (a.rot >> 1) : nullptr;
        for (int r = warp; r < 16; r += 4) {
            if (r < G) norm_rotate_row<D>(row + (size_t)(hk * G + r) * D, a.q_gamma, a.eps, cs, a.rot, tmp + warp * D, sq + r * ST, lane);
            else for (int d = lane; d < D; d += 32) sq[r * ST + d] = __float2bfloat16_rn(0.f);
        }
        if (has_new && warp == 0) {
            norm_rotate_row<D>(row + (size_t)(Hq + hk) * D, a.k_gamma, a.eps, cs, a.rot, tmp, knew, lane);
            const bf16* vraw = row + (size_t)(Hq + Hkv + hk) * D;
            int page, off;
            if (page_shift >= 0) { page = table.page(pos >> page_shift); off = pos & (page_size - 1); }
            else { page = table.page(pos / page_size); off = pos % page_size; }
            bf16* kdst = a.pages + (size_t)page * page_stride + k_off + (size_t)off * D;
            bf16* vdst = a.pages + (size_t)page * page_stride + v_off + (size_t)off * D;
            for (int d = lane; d < D; d += 32) {
                const bf16 v = vraw[d];
                vnew[d] = v;
                vdst[d] = v;
                kdst[d] = knew[d];
            }
        }
        __syncthreads();
        uint32_t qf[D / 16][4];
        {
            const int r = (((lane >> 3) & 1) << 3) + (lane & 7);
            const int dof = (lane >> 4) << 3;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], sq + r * ST + ks * 16 + dof);
        }
        if (has_new && warp == 0 && lane < 16) {             // scores of the new key, one query row per lane
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot += __bfloat162float(sq[lane * ST + d]) * __bfloat162float(knew[d]);
            snew[lane] = dot;
        }

        for (int t = tile0 + warp; t < tile1; t += 4) {
            cp_async_wait<0>();
            __syncwarp();                                       // this warp's tile t has arrived
            float sc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) qk_16keys<D>(sc[2 * kb], sc[2 * kb + 1], qf, wk + kb * 16 * ST, lane);
            float mx0 = -INFINITY, mx1 = -INFINITY;
            const bool edge = t * TILE < lo || (t + 1) * TILE > hi;      // some keys of the tile are not visible
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                if (edge) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int j = t * TILE + nt * 8 + 2 * tq + e;
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
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);   // finite: the tile has a visible key
            const float u0 = n0 * a.scale_log2, u1 = n1 * a.scale_log2;
            const float c0 = fast_exp2(m0 * a.scale_log2 - u0), c1 = fast_exp2(m1 * a.scale_log2 - u1);
            m0 = n0;
            m1 = n1;
            l0 *= c0;
            l1 *= c1;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
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
                pv_16keys<D>(o, pf, wv + kb * 16 * ST, lane);
            }
            __syncwarp();                                       // the buffers are read; the next tile may land
            if (t + 4 < tile1)
                load_kv_tile_warp<D>(wk, wv, a.pages, table, (t + 4) * TILE, lo, hi, page_size, page_shift, page_stride, k_off, v_off, lane);
            cp_async_commit();
        }
        cp_async_wait<0>();
        __syncthreads();                                        // tiles done; snew, vnew visible
        if (has_new && warp == 0) {                             // fold the new key into warp 0's sums
            const float s0 = snew[g], s1 = snew[g + 8];
            const float n0 = fmaxf(m0, s0), n1 = fmaxf(m1, s1);
            const float c0 = fast_exp2(m0 * a.scale_log2 - n0 * a.scale_log2), c1 = fast_exp2(m1 * a.scale_log2 - n1 * a.scale_log2);
            const float p0 = fast_exp2(s0 * a.scale_log2 - n0 * a.scale_log2), p1 = fast_exp2(s1 * a.scale_log2 - n1 * a.scale_log2);
            m0 = n0;
            m1 = n1;
            l0 = l0 * c0 + (tq == 0 ? p0 : 0.f);                // the row's sum is spread over the four lanes of a quad
            l1 = l1 * c1 + (tq == 0 ? p1 : 0.f);
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                const float v0 = __bfloat162float(vnew[i * 8 + 2 * tq]), v1 = __bfloat162float(vnew[i * 8 + 2 * tq + 1]);
                o[i][0] = o[i][0] * c0 + p0 * v0; o[i][1] = o[i][1] * c0 + p0 * v1;
                o[i][2] = o[i][2] * c1 + p1 * v0; o[i][3] = o[i][3] * c1 + p1 * v1;
            }
        }
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

        // combine the four warps through shared memory (the tiles are no longer needed)
        float* wo = reinterpret_cast<float*>(sk);               // [4][16][D]
        float* wm = wo + 4 * 16 * D;                            // [4][16] maxima (log2 units)
        float* wl = wm + 4 * 16;                                // [4][16] sums
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            const int d = i * 8 + 2 * tq;
            wo[(warp * 16 + g) * D + d] = o[i][0];
            wo[(warp * 16 + g) * D + d + 1] = o[i][1];
            wo[(warp * 16 + g + 8) * D + d] = o[i][2];
            wo[(warp * 16 + g + 8) * D + d + 1] = o[i][3];
        }
        if (tq == 0) {
            wm[warp * 16 + g] = m0 == -INFINITY ? -INFINITY : m0 * a.scale_log2;
            wm[warp * 16 + g + 8] = m1 == -INFINITY ? -INFINITY : m1 * a.scale_log2;
            wl[warp * 16 + g] = l0;
            wl[warp * 16 + g + 8] = l1;
        }
        __syncthreads();
        for (int idx = tid; idx < G * D; idx += NTHREADS) {
            const int r = idx / D, d = idx % D;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) M = fmaxf(M, wm[w * 16 + r]);
            float acc = 0.f, L = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
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

    // ---- the last block of this (request, key/value head) combines the chunks
    // (one fence, by the thread that takes the ticket, behind the block's barrier: the fence is cumulative)
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        s_ticket = atomicAdd(&a.tickets[b * Hkv + hk], 1);
    }
    __syncthreads();
    if (s_ticket != n_chunks - 1) return;
    __threadfence();
    for (int idx = tid; idx < G * D; idx += NTHREADS) {
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
        a.out[bh * D + d] = __float2bfloat16_rn(acc / L);
    }
    if (tid == 0) a.tickets[b * Hkv + hk] = 0;
}

template <int D> static size_t decode_fused_smem() {
    const size_t tiles = (size_t)(16 + 2 * 4 * TILE) * (D + 8) * sizeof(bf16);
    return tiles + (size_t)4 * D * sizeof(float) + (size_t)2 * D * sizeof(bf16) + 16 * sizeof(float) + 64;
}

template <int D>
static int launch_decode_fused(const FusedDecodeArgs& a, int B, int n_chunks, cudaStream_t stream) {
    const size_t smem = decode_fused_smem<D>();
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {
        cudaError_t e = cudaFuncSetAttribute(decode_fused_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(decode_fused_kernel<D>, dim3(n_chunks, a.Hkv, B), dim3(NTHREADS), smem, stream, a);
}

template <int D> static size_t prefill_smem() { return (size_t)(PREFILL_ROWS + 4 * TILE) * (D + 8) * sizeof(bf16); }
template <int D> size_t decode_smem() {
    const size_t tiles = (size_t)(16 + 2 * DecodeStages<D>::N * TILE) * (D + 8) * sizeof(bf16);
    const size_t comb = 16 * (D + 8) * sizeof(bf16) + (size_t)(4 * 16 * D + 2 * 4 * 16) * sizeof(float);
    return tiles > comb ? tiles : comb;
}

template <int D>
static int launch_prefill(bf16* out, const bf16* q, const bf16* pages, const int* block_table, int table_width,
                          const int* cu_q, const int* ctx_lens, int S, int n_tiles, int page_size, int Hq, int Hkv,
                          float scale, int window, int num_pages, int* status, cudaStream_t stream) {
    const size_t smem = prefill_smem<D>();
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {
        cudaError_t e = cudaFuncSetAttribute(prefill_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(prefill_mma_kernel<D>, dim3(n_tiles, Hq), dim3(PREFILL_WARPS * 32), smem, stream,
                      out, q, pages, block_table, table_width, cu_q, ctx_lens, S, page_size, Hq, Hkv,
                      scale * 1.4426950408889634f, window, num_pages, status);
}

template <int D>
static int launch_decode(bf16* out, float* part_o, float* part_ml, const bf16* q, const bf16* pages,
                         const int* block_table, int table_width, const int* positions, int B, int n_chunks,
                         int page_size, int Hq, int Hkv, float scale, int window, int num_pages, int* status,
                         cudaStream_t stream) {
    const size_t smem = decode_smem<D>();
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {
        cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    int e = launch_pdl(decode_mma_kernel<D>, dim3(n_chunks, Hkv, B), dim3(NTHREADS), smem, stream,
                       part_o, part_ml, q, pages, block_table, table_width, positions, page_size, Hq, Hkv,
                       scale * 1.4426950408889634f, window, num_pages, status);
    if (e) return e;
    return launch_pdl(decode_combine_kernel<D>, dim3(B * Hq), dim3(D <= 64 ? 64 : 128), 0, stream,
                      out, (const float*)part_o, (const float*)part_ml, n_chunks);
}

#define ZAI_HEAD_DIMS(X) X(16) X(32) X(48) X(64) X(80) X(96) X(128)

// 1 if the tensor-core kernels take this head size (bfloat16 only; others use the general kernel)
ZAI_API int zai_attention_mma_supports(int D, int Hq, int Hkv) {
    if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16) return 0;
#define X(d) if (D == d) return 1;
    ZAI_HEAD_DIMS(X)
#undef X
    return 0;
}

ZAI_API int zai_prefill_attention_mma(void* out, const void* q, const void* pages, const int* block_table,
                                      int table_width, const int* cu_q, const int* ctx_lens, int S, int n_tiles,
                                      int page_size, int Hq, int Hkv, int D, float scale, int window,
                                      int num_pages, int* status, cudaStream_t stream) {
    if (S <= 0 || n_tiles <= 0) return ZAI_OK;
    if (Hq > 65535) return ZAI_BAD_SIZE;
#define X(d) if (D == d) return launch_prefill<d>((bf16*)out, (const bf16*)q, (const bf16*)pages, block_table, table_width, \
                                                  cu_q, ctx_lens, S, n_tiles, page_size, Hq, Hkv, scale, window, num_pages, status, stream);
    ZAI_HEAD_DIMS(X)
#undef X
    return ZAI_BAD_SIZE;
}

// Scratch: part_o holds B*Hq*n_chunks*D floats, part_ml B*Hq*n_chunks*2 floats; n_chunks covers the
// longest request, ceil(max(pos + 1) / 256).
ZAI_API int zai_decode_attention_mma(void* out, float* part_o, float* part_ml, const void* q, const void* pages,
                                     const int* block_table, int table_width, const int* positions, int B,
                                     int n_chunks, int page_size, int Hq, int Hkv, int D, float scale, int window,
                                     int num_pages, int* status, cudaStream_t stream) {
    if (B <= 0) return ZAI_OK;
    if (n_chunks < 1 || Hkv < 1 || Hkv > 65535 || B > 65535 || Hq % Hkv != 0 || Hq / Hkv > 16) return ZAI_BAD_SIZE;
#define X(d) if (D == d) return launch_decode<d>((bf16*)out, part_o, part_ml, (const bf16*)q, (const bf16*)pages, block_table, \
                                                 table_width, positions, B, n_chunks, page_size, Hq, Hkv, scale, window, num_pages, status, stream);
    ZAI_HEAD_DIMS(X)
#undef X
    return ZAI_BAD_SIZE;
}

// The decode step's attention from the raw qkv rows: see decode_fused_kernel.  `tickets` holds
// B * Hkv zeros (and again after the call).
ZAI_API int zai_decode_attention_fused(void* out, float* part_o, float* part_ml, int* tickets, const void* qkv,
                                       int qkv_cols, const float* q_gamma, const float* k_gamma, float eps,
                                       const float2* cs_table, int rot, void* pages, const int* block_table,
                                       int table_width, const int* positions, int B, int n_chunks, int page_size,
                                       int Hq, int Hkv, int D, float scale, int window, int write_kv, int chunk_keys,
                                       int num_pages, int* status, cudaStream_t stream) {
    if (B <= 0) return ZAI_OK;
    if (chunk_keys < TILE || chunk_keys % TILE) return ZAI_BAD_SIZE;
    if (n_chunks < 1 || Hkv < 1 || Hkv > 65535 || B > 65535 || Hq % Hkv != 0 || Hq / Hkv > 16 || rot < 0 || rot > D || (rot & 1))
        return ZAI_BAD_SIZE;
    FusedDecodeArgs a;
    a.out = (bf16*)out; a.part_o = part_o; a.part_ml = part_ml; a.tickets = tickets; a.qkv = (const bf16*)qkv;
    a.q_gamma = q_gamma; a.k_gamma = k_gamma; a.cs_table = cs_table; a.pages = (bf16*)pages; a.block_table = block_table;
    a.positions = positions; a.eps = eps; a.scale_log2 = scale * 1.4426950408889634f; a.qkv_cols = qkv_cols; a.rot = rot;
    a.table_width = table_width; a.page_size = page_size; a.Hq = Hq; a.Hkv = Hkv; a.window = window; a.write_kv = write_kv; a.chunk_keys = chunk_keys;
    a.num_pages = num_pages; a.status = status;
#define X(d) if (D == d) return launch_decode_fused<d>(a, B, n_chunks, stream);
    ZAI_HEAD_DIMS(X)
#undef X
    return ZAI_BAD_SIZE;
}

ZAI_API int zai_decode_chunk_keys() { return CHUNK; }
ZAI_API int zai_prefill_block_rows() { return PREFILL_ROWS; }

// ------------------------------------------------------------------------------------------ no allocation
// The same two kernels with their scratch in a static device array; see attention_no_alloc.h for
// who needs this, its cost and its limits.
#include "attention_no_alloc.h"

static __device__ __align__(256) float zai_static_scratch[ZAI_STATIC_SCRATCH_FLOATS];

#define ZAI_MAX_DEVICES 64
static float* zai_static_scratch_ptr[ZAI_MAX_DEVICES];   // device address of the array, per device

// In host code the array's name is only a handle; its device address has to be asked for, once per
// device, with that device current.
static int static_scratch_address(float** ptr) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= ZAI_MAX_DEVICES) return ZAI_SCRATCH_SETUP_FAILED;
    if (zai_static_scratch_ptr[dev] == nullptr) {
        float* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, zai_static_scratch) != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            return ZAI_SCRATCH_SETUP_FAILED;
        }
        zai_static_scratch_ptr[dev] = p;
    }
    *ptr = zai_static_scratch_ptr[dev];
    return ZAI_OK;
}

ZAI_API int zai_decode_attention_static(void* out, const void* q, const void* pages, const int* block_table,
                                        int table_width, const int* positions, int B, int n_chunks, int page_size,
                                        int Hq, int Hkv, int D, float scale, int window, cudaStream_t stream) {
    if (B <= 0) return ZAI_OK;
    if (n_chunks < 1 || Hq < 1 || Hkv < 1 || D < 1) return ZAI_BAD_SIZE;
    const unsigned long long rows = (unsigned long long)B * Hq * n_chunks;
    if (rows * (unsigned long long)(D + 2) > (unsigned long long)ZAI_STATIC_SCRATCH_FLOATS) return ZAI_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    const int e = static_scratch_address(&scratch);
    if (e != ZAI_OK) return e;
    float* part_o = scratch;                              // [B, Hq, n_chunks, D]
    float* part_ml = scratch + rows * D;                  // [B, Hq, n_chunks, 2]
    // (this entry point's caller vouches for its block tables: no bound on the page ids, no status word)
    return zai_decode_attention_mma(out, part_o, part_ml, q, pages, block_table, table_width, positions, B, n_chunks,
                                    page_size, Hq, Hkv, D, scale, window, 0x7fffffff, nullptr, stream);
}

ZAI_API const char* zai_decode_attention_static_error(int code) {
    switch (code) {
        case ZAI_OK: return "ok";
        case ZAI_BAD_DTYPE: return "element type not supported";
        case ZAI_BAD_SIZE: return "a size is outside what the kernel supports";
        case ZAI_SCRATCH_TOO_SMALL:
            return "B * Hq * n_chunks * (D + 2) floats of scratch are needed, more than the static array of "
                   "1048576 floats holds; use zai_decode_attention_mma with scratch of your own";
        case ZAI_SCRATCH_SETUP_FAILED: return "the device address of the static scratch array could not be obtained";
        default: return "CUDA error at launch";
    }
}
