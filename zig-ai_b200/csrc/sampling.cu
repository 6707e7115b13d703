// Sampling on the device from 32-bit logits [R, V], one block per row.
//
// Greedy: the first index of the maximum (src/transformer/pipeline.zig:153-181).
// Otherwise the reference's order (pipeline.zig:25-151): repetition penalty on the tokens of the
// history (a positive logit is divided, a negative one multiplied, once for every occurrence,
// :60-67), division by the temperature (:75-76), top-k keeps the values >= the k-th largest
// (:79-99), top-p keeps the most probable tokens until their mass reaches p (:102-138), and the
// token is the first index whose cumulative probability reaches u times the kept mass (:39-52,
// :141-149), u being a uniform number in [0, 1) that the caller supplies for the row.  The scan
// runs in index order over the kept set (the reference scans its nucleus in sorted order; the
// distribution is the same).  No sort: the k-th largest value (or the 4096-th, a bound on the nucleus) is
// found by a radix selection over the ordered bit patterns, the values at or above it are laid into
// shared memory in index order, and the nucleus and the inverse CDF run on that list; ties at a
// threshold are all kept.  A row whose kept set does not fit the list (a top-k above 4096, many ties,
// a nucleus of more than 4096 tokens) takes the general way, thresholds by bisection over the row.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned ordered_key(float f) {          // monotone map float -> unsigned
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(unsigned k) {
    const unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(u);
}

struct MaxIdx { float v; int i; };
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ MaxIdx block_argmax(MaxIdx x, MaxIdx* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    __syncthreads();
    if (lane == 0) red[warp] = x;
    __syncthreads();
    if (warp == 0) {
        MaxIdx y = lane < nwarp ? red[lane] : MaxIdx{-INFINITY, 0x7fffffff};
        for (int o = 16; o > 0; o >>= 1) {
            MaxIdx z;
            z.v = __shfl_xor_sync(0xffffffffu, y.v, o);
            z.i = __shfl_xor_sync(0xffffffffu, y.i, o);
            y = better(y, z);
        }
        if (lane == 0) red[32] = y;
    }
    __syncthreads();
    return red[32];
}

// The thread's best (value, first index) over a row, scanned with 16-byte loads, several in flight.
__device__ __forceinline__ MaxIdx scan_row(const float* __restrict__ row, int V) {
    MaxIdx x{-INFINITY, 0x7fffffff};
    if ((V & 3) == 0 && (reinterpret_cast<size_t>(row) & 15) == 0) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int n4 = V >> 2;
        for (int i = threadIdx.x; i < n4; i += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = i + u * blockDim.x;
                v[u] = j < n4 ? r4[j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {                   // indices rise with u, then within the float4
                const int j = (i + u * blockDim.x) << 2;
                if (v[u].x > x.v) { x.v = v[u].x; x.i = j; }
                if (v[u].y > x.v) { x.v = v[u].y; x.i = j + 1; }
                if (v[u].z > x.v) { x.v = v[u].z; x.i = j + 2; }
                if (v[u].w > x.v) { x.v = v[u].w; x.i = j + 3; }
            }
        }
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (v > x.v) { x.v = v; x.i = i; }              // a strided scan visits indices in rising order
        }
    }
    return x;
}

// `status`, if given, is the step's status word: block 0 copies it behind the R token ids (out[R]), so that one
// copy to the host brings both.
__global__ void argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, const int* __restrict__ status) {
    __shared__ MaxIdx red[33];
    pdl_trigger();
    pdl_wait();
    if (status && blockIdx.x == 0 && threadIdx.x == 0) out[gridDim.x] = *status;
    const float* row = logits + (size_t)blockIdx.x * V;
    MaxIdx x = scan_row(row, V);
    x = block_argmax(x, red);
    if (threadIdx.x == 0) out[blockIdx.x] = x.i == 0x7fffffff ? 0 : x.i;
}

// logits[r, token] is scaled `count` times: divided by the penalty if positive, multiplied if negative.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, const int* __restrict__ tokens,
                                          const int* __restrict__ counts, const int* __restrict__ offsets,
                                          const float* __restrict__ penalty, int V) {
    const int r = blockIdx.x;
    const float p = penalty[r];
    if (p == 1.f) return;
    float* row = logits + (size_t)r * V;
    for (int i = offsets[r] + threadIdx.x; i < offsets[r + 1]; i += blockDim.x) {
        const int tok = tokens[i];
        if (tok < 0 || tok >= V) continue;
        float v = row[tok];
        for (int c = 0; c < counts[i]; ++c) v = v > 0.f ? v / p : (v < 0.f ? v * p : v);
        row[tok] = v;
    }
}

// The same penalty from a table of counts on the device: counts[slot, token] is how often the request in that
// slot has produced the token.  A row whose slot is negative (or whose penalty is 1) is copied as it is.
__global__ void repetition_penalty_counts_kernel(float* __restrict__ out, const float* __restrict__ logits,
                                                 const int* __restrict__ counts, const int* __restrict__ slots,
                                                 const float* __restrict__ penalty, int V) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int slot = slots[r];
    const float p = penalty[r];
    const float* row = logits + (size_t)r * V;
    float* dst = out + (size_t)r * V;
    const int* cnt = (slot >= 0 && p != 1.f) ? counts + (size_t)slot * V : nullptr;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < V; i += gridDim.y * blockDim.x) {
        float v = row[i];
        if (cnt) {
            const int c = cnt[i];
            for (int k = 0; k < c; ++k) v = v > 0.f ? v / p : (v < 0.f ? v * p : v);
        }
        dst[i] = v;
    }
}

// counts[slots[r], ids[r]] += 1 for the rows with a slot: the tokens just sampled join their requests' histories.
__global__ void count_tokens_kernel(int* __restrict__ counts, const int* __restrict__ ids, const int* __restrict__ slots, int R, int V) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    const int slot = slots[r], id = ids[r];
    if (slot >= 0 && id >= 0 && id < V) counts[(size_t)slot * V + id] += 1;      // (a slot belongs to one row)
}

// The general way, for rows whose kept set may be large (a top-k above SAMPLE_CAP, many ties, a nucleus that the
// SAMPLE_CAP largest values do not cover): thresholds by bisection over the bit patterns, about seventy walks over
// the row.  `x` is the row's maximum and its first index.
__device__ __noinline__ void sample_row_by_bisection(int* __restrict__ out, const float* __restrict__ row, float T, int k, float tp,
                                                     float u, int V, int r, MaxIdx x) {
    __shared__ float red[33];
    __shared__ float scan[SAMPLE_THREADS];
    __shared__ int chosen;
    const int tid = threadIdx.x;
    const float inv_t = 1.f / T;
    const float mx = x.v * inv_t;
    // top-k: the k-th largest scaled value, by bisection on the ordered bit pattern
    float floor_val = -INFINITY;
    if (k > 0 && k < V) {
        unsigned lo = 0u, hi = 0xffffffffu;           // largest key with count(key >= .) >= k
        while (lo < hi) {
            const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1) >> 1);
            float cnt = 0.f;
            for (int i = tid; i < V; i += blockDim.x) cnt += ordered_key(row[i] * inv_t) >= mid ? 1.f : 0.f;
            cnt = block_sum(cnt, red);
            if (cnt >= (float)k) lo = mid; else hi = mid - 1;
        }
        floor_val = key_to_float(lo);
    }
    // probabilities (unnormalised) of the kept set
    float part = 0.f;
    for (int i = tid; i < V; i += blockDim.x) {
        const float w = row[i] * inv_t;
        if (w >= floor_val) part += expf(w - mx);
    }
    float mass = block_sum(part, red);
    // top-p: the largest threshold whose kept mass still reaches p * mass
    float p_floor = 0.f;
    if (tp < 1.f) {
        const float target = tp * mass;
        unsigned lo = ordered_key(0.f), hi = ordered_key(1.f);
        while (lo < hi) {
            const unsigned mid = lo + ((hi - lo + 1) >> 1);
            const float th = key_to_float(mid);
            float s = 0.f;
            for (int i = tid; i < V; i += blockDim.x) {
                const float w = row[i] * inv_t;
                if (w >= floor_val) {
                    const float e = expf(w - mx);
                    if (e >= th) s += e;
                }
            }
            s = block_sum(s, red);
            if (s >= target) lo = mid; else hi = mid - 1;
        }
        p_floor = key_to_float(lo);
        part = 0.f;
        for (int i = tid; i < V; i += blockDim.x) {
            const float w = row[i] * inv_t;
            if (w >= floor_val) {
                const float e = expf(w - mx);
                if (e >= p_floor) part += e;
            }
        }
        mass = block_sum(part, red);
    }
    // inverse CDF in index order: each thread owns a contiguous piece of the row
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int a = min(tid * per, V), b = min(a + per, V);
    float mine = 0.f;
    for (int i = a; i < b; ++i) {
        const float w = row[i] * inv_t;
        if (w >= floor_val) {
            const float e = expf(w - mx);
            if (e >= p_floor) mine += e;
        }
    }
    scan[tid] = mine;
    if (tid == 0) chosen = 0x7fffffff;
    __syncthreads();
    // exclusive prefix over the pieces, serially by one warp-free thread per 32: small (1024 entries)
    if (tid == 0) {
        float run = 0.f;
        for (int i = 0; i < (int)blockDim.x; ++i) { const float v = scan[i]; scan[i] = run; run += v; }
        red[0] = run;
    }
    __syncthreads();
    const float total = red[0];
    const float target = u * total;
    float cum = scan[tid];
    if (target >= cum) {      // later pieces start past the target; the lowest pick wins
        int pick = -1;
        for (int i = a; i < b; ++i) {
            const float w = row[i] * inv_t;
            if (w >= floor_val) {
                const float e = expf(w - mx);
                if (e >= p_floor) {
                    cum += e;
                    if (target <= cum) { pick = i; break; }
                }
            }
        }
        if (pick >= 0) atomicMin(&chosen, pick);
    }
    __syncthreads();
    if (tid == 0) {
        int c = chosen;
        if (c == 0x7fffffff) c = x.i;                // rounding left the target past the last kept token
        out[r] = c;
    }
}


// ---- the quick way.  The kept set is almost always small: top-k says so, and a nucleus seldom has more than a
// few thousand tokens.  So the SAMPLE_CAP largest values (or the k largest) are found by a radix selection over
// the ordered bit patterns (four walks over the row, counting by byte; the first also finds the maximum), the
// values at or above that floor are laid into shared memory in index order, and the rest (masses, the nucleus,
// the inverse CDF) runs on that list, in one warp.  A warp owns a contiguous range of the row and reads it 32
// consecutive values at a time, so every walk is coalesced and what a warp counts is what lies in its range.
// Probabilities are summed as integers (exp(w - max) in units of 2^-40), so a sum does not depend on the order
// in which it is taken and the same row with the same u gives the same token in whatever batch it runs.
#define SAMPLE_CAP 4096
#define SAMPLE_UNIT 1099511627776.f                     // 2^40
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)
#define SAMPLE_BATCH 8                                  // loads of a lane in flight in a walk
// a walk over this warp's range [ra, rb): BODY sees the index `i` and the value `v`, eight loads asked for at once
#define SAMPLE_WALK(BODY)                                                        \
    for (int i0_ = ra + lane; i0_ < rb; i0_ += 32 * SAMPLE_BATCH) {              \
        float v_[SAMPLE_BATCH];                                                  \
        _Pragma("unroll") for (int u_ = 0; u_ < SAMPLE_BATCH; ++u_) {            \
            const int i_ = i0_ + 32 * u_;                                        \
            v_[u_] = i_ < rb ? row[i_] : 0.f;                                    \
        }                                                                        \
        _Pragma("unroll") for (int u_ = 0; u_ < SAMPLE_BATCH; ++u_) {            \
            const int i = i0_ + 32 * u_;                                         \
            const float v = v_[u_];                                              \
            if (i < rb) { BODY }                                                 \
        }                                                                        \
    }

typedef unsigned long long u64;

__device__ __forceinline__ u64 unit_of(float e) { return __float2ull_rz(e * SAMPLE_UNIT); }
__device__ __forceinline__ u64 warp_sum_u64(u64 v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// inclusive prefix over the lanes of a warp
__device__ __forceinline__ u64 warp_scan_u64(u64 v, int lane) {
    for (int o = 1; o < 32; o <<= 1) {
        const u64 y = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += y;
    }
    return v;
}

// What is left once the kept values lie in a list in index order (le: exp(w - max), li: index; n entries), for a
// block of WARPS warps: the list's mass, the nucleus if top-p is set, the inverse CDF.  Returns the token, or
// 0x7fffffff if rounding left the target past the last kept token, or -1 if the list does not hold the nucleus
// (top-p without top-k: `all_mass` is the row's).  Every thread of the block calls it and gets the same answer.
struct ListScratch {
    u64* wmass;                 // [WARPS]
    unsigned* word;             // one word
    int* chosen;
    int* pick_warp;
    u64* pick_before;
    u64* pick_target;
    u64* hist64;                // [n_hist][256]: weighted histograms
    int n_hist;
};
template <int WARPS>
__device__ __forceinline__ int pick_from_list(const float* le, const int* li, int n, bool use_k, bool use_p, float tp, float u,
                                              u64 all_mass, const ListScratch sc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lrange = ((n + WARPS - 1) / WARPS + 31) / 32 * 32;    // a warp owns a contiguous part of the list
    const int la = min(warp * lrange, n), lb = min(la + lrange, n);
    auto block_sum = [&](u64 v) {                            // over the block, to every thread
        v = warp_sum_u64(v);
        if (lane == 0) sc.wmass[warp] = v;
        __syncthreads();
        u64 t = 0;
        for (int w2 = 0; w2 < WARPS; ++w2) t += sc.wmass[w2];
        __syncthreads();
        return t;
    };
    u64 part = 0;
    for (int j = la + lane; j < lb; j += 32) part += unit_of(le[j]);
    const u64 list_mass = block_sum(part);
    float p_floor = 0.f;
    if (use_p) {
        const u64 base = use_k ? list_mass : all_mass;
        const u64 target = (u64)((double)tp * (double)base);
        if (list_mass < target) return -1;                   // with top-p alone the list has to hold the whole nucleus
        // the largest threshold on exp(w - max) whose tokens still hold p of the mass (positive floats order as their bits do)
        unsigned lo = __float_as_uint(0.f), hi = __float_as_uint(1.f);
        if (n <= 1024) {                                     // a short list: one warp, no block-wide sums
            if (warp == 0) {
                while (lo < hi) {
                    const unsigned mid = lo + ((hi - lo + 1) >> 1);
                    const float th = __uint_as_float(mid);
                    u64 s2 = 0;
                    for (int j = lane; j < n; j += 32) {
                        const float e = le[j];
                        if (e >= th) s2 += unit_of(e);
                    }
                    if (warp_sum_u64(s2) >= target) lo = mid; else hi = mid - 1;
                }
                if (lane == 0) *sc.word = lo;
            }
            __syncthreads();
            lo = *sc.word;
        } else {
            // a long list: the threshold's bit pattern byte by byte from the top, each time from a histogram of
            // the masses by that byte (of the entries that agree with the bytes found so far)
            const u64 need = target ? target : 1ull;         // (at least the largest entry is kept)
            unsigned prefix = 0;
            u64 carried = 0;                                 // mass of the entries above the bytes found so far
            u64* mine_hist = sc.hist64 + (size_t)(warp % sc.n_hist) * 256;
            for (int byte = 3; byte >= 0; --byte) {
                const int shift = byte * 8;
                const unsigned high_mask = byte == 3 ? 0u : (0xffffffffu << (shift + 8));
                for (int j = tid; j < sc.n_hist * 256; j += WARPS * 32) sc.hist64[j] = 0ull;
                __syncthreads();
                for (int j = la + lane; j < lb; j += 32) {
                    const float e = le[j];
                    const unsigned key = __float_as_uint(e);
                    if ((key & high_mask) == (prefix & high_mask)) atomicAdd(mine_hist + ((key >> shift) & 255u), unit_of(e));
                }
                __syncthreads();
                if (tid < 256) {
                    u64 t = 0;
                    for (int h = 0; h < sc.n_hist; ++h) t += sc.hist64[(size_t)h * 256 + tid];
                    sc.hist64[tid] = t;                      // (histogram 0 becomes the sum; its own part was read first)
                }
                __syncthreads();
                if (warp == 0) {
                    // lane l owns bins 8l..8l+7; the digit is the highest bin at which the mass from the top reaches `need`
                    u64 mine = 0;
                    for (int j = 0; j < 8; ++j) mine += sc.hist64[lane * 8 + j];
                    u64 incl = mine;
                    for (int o = 1; o < 32; o <<= 1) {
                        const u64 y = __shfl_down_sync(0xffffffffu, incl, o);
                        if (lane + o < 32) incl += y;
                    }
                    const u64 higher = carried + incl - mine;
                    if (higher < need && need <= higher + mine) {
                        u64 cum = higher;
                        for (int j = 7; j >= 0; --j) {
                            const u64 m = sc.hist64[lane * 8 + j];
                            if (cum + m >= need) { *sc.word = (unsigned)(lane * 8 + j); *sc.pick_before = cum; break; }
                            cum += m;
                        }
                    }
                }
                __syncthreads();
                prefix |= *sc.word << shift;
                carried = *sc.pick_before;
                __syncthreads();
            }
            lo = prefix;
        }
        p_floor = __uint_as_float(lo);
    }
    // the kept mass of every part, then the part that holds the target walks again (the list is in index order)
    part = 0;
    for (int j = la + lane; j < lb; j += 32) {
        const float e = le[j];
        if (e >= p_floor) part += unit_of(e);
    }
    part = warp_sum_u64(part);
    if (lane == 0) sc.wmass[warp] = part;
    if (tid == 0) *sc.chosen = 0x7fffffff;
    __syncthreads();
    if (warp == 0) {
        const u64 mine = lane < WARPS ? sc.wmass[lane] : 0ull;
        const u64 incl = warp_scan_u64(mine, lane);
        const u64 total = __shfl_sync(0xffffffffu, incl, 31);
        const u64 target = (u64)((double)u * (double)total);
        const unsigned hit = __ballot_sync(0xffffffffu, mine > 0 && target <= incl);
        if (lane == 0) {
            *sc.pick_warp = hit ? __ffs(hit) - 1 : -1;
            *sc.pick_target = target;
        }
        if (hit && lane == __ffs(hit) - 1) *sc.pick_before = incl - mine;
    }
    __syncthreads();
    if (warp == *sc.pick_warp) {
        u64 cum = *sc.pick_before;
        const u64 target = *sc.pick_target;
        for (int j0 = la; j0 < lb; j0 += 32) {
            const int j = j0 + lane;
            const float e = j < lb ? le[j] : 0.f;
            const u64 ei = (j < lb && e >= p_floor) ? unit_of(e) : 0ull;
            const u64 incl = warp_scan_u64(ei, lane) + cum;
            const unsigned hit = __ballot_sync(0xffffffffu, ei > 0 && target <= incl);
            if (hit) {
                if (lane == 0) *sc.chosen = li[j0 + __ffs(hit) - 1];
                break;
            }
            cum = __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();
    return *sc.chosen;
}

struct SampleShared {
    unsigned whist[SAMPLE_WARPS][256];                  // a histogram per warp (= per range of the row)
    unsigned hist[256];
    float le[SAMPLE_CAP];                               // the list: exp(w - max),
    int li[SAMPLE_CAP];                                 //   index
    u64 wmass[SAMPLE_WARPS];                            // per range: mass
    unsigned wcount[SAMPLE_WARPS];                      // per range: values above the floor's first three bytes
    unsigned woffset[SAMPLE_WARPS];                     // per range: where its kept values start in the list
    MaxIdx redm[33];
    unsigned sel_digit, sel_above;
    int chosen, pick_warp;
    u64 pick_before, pick_target;
};

// One count into a warp's histogram, with runs of the same bin counted in a register first (the top bytes of a
// row's values are nearly all the same, and atomics of a warp on one address are served one after the other).
struct RunCount {
    unsigned bin, n;
    __device__ __forceinline__ void add(unsigned* hist, unsigned b) {
        if (b == bin) { ++n; return; }
        if (n) atomicAdd(hist + bin, n);
        bin = b;
        n = 1;
    }
    __device__ __forceinline__ void flush(unsigned* hist) { if (n) atomicAdd(hist + bin, n); n = 0; }
};

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
                              const float* __restrict__ temperature, const int* __restrict__ top_k,
                              const float* __restrict__ top_p, const float* __restrict__ uniform, int V,
                              const int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char sample_smem[];
    SampleShared& sh = *reinterpret_cast<SampleShared*>(sample_smem);
    pdl_trigger();
    pdl_wait();
    if (status && blockIdx.x == 0 && threadIdx.x == 0) out[gridDim.x] = *status;
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = logits + (size_t)r * V;
    const float T = temperature[r];
    if (T <= 0.f) {
        MaxIdx x = scan_row(row, V);
        x = block_argmax(x, sh.redm);
        if (tid == 0) out[r] = x.i == 0x7fffffff ? 0 : x.i;
        return;
    }
    const float inv_t = 1.f / T, u = uniform[r], tp = top_p[r];
    const int k = top_k[r];
    const bool use_k = k > 0 && k < V, use_p = tp < 1.f;
    // this warp's range of the row: [ra, rb), a multiple of 32 long (but for the row's end)
    const int range = ((V + SAMPLE_WARPS - 1) / SAMPLE_WARPS + 31) / 32 * 32;
    const int ra = min(warp * range, V), rb = min(ra + range, V);
    const int want = use_k ? k : min(SAMPLE_CAP, V);
    const bool select = (use_k || use_p) && want <= SAMPLE_CAP;

    // ---- walk one: the maximum and its first index, and the count by the top byte of the key
    for (int j = lane; j < 256; j += 32) sh.whist[warp][j] = 0;
    __syncwarp();
    MaxIdx x{-INFINITY, 0x7fffffff};
    {
        RunCount rc{0u, 0u};
        SAMPLE_WALK(
            if (v > x.v) { x.v = v; x.i = i; }               // (a lane's indices rise)
            if (select) rc.add(sh.whist[warp], ordered_key(v * inv_t) >> 24);
        )
        rc.flush(sh.whist[warp]);
    }
    x = block_argmax(x, sh.redm);                            // (syncs the block)
    const float mx = x.v * inv_t;

    // the floor: the key of the `want`-th largest scaled value, byte by byte from the top
    unsigned floor_key = 0, n_keep = 0;
    u64 all_mass = 0;                                        // of the whole row
    bool quick = select;
    if (select) {
        unsigned prefix = 0, remaining = (unsigned)want, above = 0;
        for (int byte = 3; byte >= 0; --byte) {
            const int shift = byte * 8;
            if (byte < 3) {
                for (int j = lane; j < 256; j += 32) sh.whist[warp][j] = 0;
                __syncwarp();
                const unsigned high_mask = 0xffffffffu << (shift + 8);
                RunCount rc{0u, 0u};
                u64 part = 0;
                unsigned gt = 0;
                SAMPLE_WALK(
                    const float w = v * inv_t;
                    const unsigned key = ordered_key(w);
                    if ((key & high_mask) == (prefix & high_mask)) rc.add(sh.whist[warp], (key >> shift) & 255u);
                    if (byte == 2) part += unit_of(expf(w - mx));
                    if (byte == 0) gt += (key & high_mask) > (prefix & high_mask) ? 1u : 0u;
                )
                rc.flush(sh.whist[warp]);
                if (byte == 2) {
                    part = warp_sum_u64(part);
                    if (lane == 0) sh.wmass[warp] = part;
                }
                if (byte == 0) {
                    gt = __reduce_add_sync(0xffffffffu, gt);
                    if (lane == 0) sh.wcount[warp] = gt;
                }
            }
            __syncthreads();
            if (tid < 256) {
                unsigned c = 0;
                for (int w2 = 0; w2 < SAMPLE_WARPS; ++w2) c += sh.whist[w2][tid];
                sh.hist[tid] = c;
            }
            __syncthreads();
            if (warp == 0) {
                // lane l owns bins 8l..8l+7; the digit is the highest bin at which the count from the top reaches `remaining`
                unsigned mine = 0;
                for (int j = 0; j < 8; ++j) mine += sh.hist[lane * 8 + j];
                unsigned incl = mine;                        // sum over lanes >= this one
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned y = __shfl_down_sync(0xffffffffu, incl, o);
                    if (lane + o < 32) incl += y;
                }
                const unsigned higher = incl - mine;         // in the lanes above this one
                if (higher < remaining && remaining <= incl) {
                    unsigned cum = higher;
                    for (int j = 7; j >= 0; --j) {
                        const unsigned c = sh.hist[lane * 8 + j];
                        if (cum + c >= remaining) { sh.sel_digit = (unsigned)(lane * 8 + j); sh.sel_above = cum; break; }
                        cum += c;
                    }
                }
            }
            __syncthreads();
            prefix |= sh.sel_digit << shift;
            above += sh.sel_above;                            // values whose key is larger in this byte (and equal above it)
            remaining -= sh.sel_above;
            if (byte == 0) n_keep = above + sh.hist[sh.sel_digit];
            if (byte == 2) {
                for (int w2 = 0; w2 < SAMPLE_WARPS; ++w2) all_mass += sh.wmass[w2];
            }
            if (byte > 0) __syncthreads();                   // (the last walk's histograms are still needed below)
        }
        floor_key = prefix;
        quick = n_keep <= SAMPLE_CAP;                        // (ties at the floor are all kept)
    }
    if (select && !quick) {
        sample_row_by_bisection(out, row, T, k, tp, u, V, r, x);
        return;
    }

    if (!select) {
        if (use_k || use_p) {                                // a top-k above what the list holds
            sample_row_by_bisection(out, row, T, k, tp, u, V, r, x);
            return;
        }
        // ---- nothing to select: the inverse CDF over the whole row.  The ranges' masses, then the range that
        // holds the target walks again.
        u64 part = 0;
        SAMPLE_WALK(part += unit_of(expf(v * inv_t - mx));)
        part = warp_sum_u64(part);
        if (lane == 0) sh.wmass[warp] = part;
        if (tid == 0) sh.chosen = 0x7fffffff;
        __syncthreads();
        if (warp == 0) {
            const u64 mine = lane < SAMPLE_WARPS ? sh.wmass[lane] : 0ull;
            const u64 incl = warp_scan_u64(mine, lane);
            const u64 total = __shfl_sync(0xffffffffu, incl, 31);
            const u64 target = (u64)((double)u * (double)total);
            // the first range whose cumulative mass reaches the target (and that has mass)
            const unsigned hit = __ballot_sync(0xffffffffu, mine > 0 && target <= incl);
            if (lane == 0) {
                sh.pick_warp = hit ? __ffs(hit) - 1 : -1;
                sh.pick_target = target;
            }
            if (hit && lane == __ffs(hit) - 1) sh.pick_before = incl - mine;
        }
        __syncthreads();
        if (warp == sh.pick_warp) {
            u64 cum = sh.pick_before;
            const u64 target = sh.pick_target;
            for (int i0 = ra; i0 < rb; i0 += 32) {
                const int i = i0 + lane;
                const u64 e = i < rb ? unit_of(expf(row[i] * inv_t - mx)) : 0ull;
                const u64 incl = warp_scan_u64(e, lane) + cum;
                const unsigned hit = __ballot_sync(0xffffffffu, e > 0 && target <= incl);
                if (hit) {
                    if (lane == 0) sh.chosen = i0 + __ffs(hit) - 1;
                    break;
                }
                cum = __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        __syncthreads();
        if (tid == 0) out[r] = sh.chosen == 0x7fffffff ? x.i : sh.chosen;   // (rounding left the target past the last token)
        return;
    }

    // ---- the list, in index order: a range's kept values follow those of the ranges before it
    {
        unsigned mine = 0;                                   // kept in this range: above the floor's first bytes, or at them with a last byte >= the floor's
        const unsigned digit = floor_key & 255u;
        for (int j = lane; j < 256; j += 32) mine += (unsigned)j >= digit ? sh.whist[warp][j] : 0u;
        mine = __reduce_add_sync(0xffffffffu, mine) + sh.wcount[warp];
        if (lane == 0) sh.woffset[warp] = mine;
        __syncthreads();
        if (warp == 0) {
            const unsigned c = lane < SAMPLE_WARPS ? sh.woffset[lane] : 0u;
            unsigned incl = c;
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned y = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += y;
            }
            if (lane < SAMPLE_WARPS) sh.woffset[lane] = incl - c;
        }
        __syncthreads();
        unsigned at = sh.woffset[warp];
        for (int i0 = ra; i0 < rb; i0 += 32 * SAMPLE_BATCH) {
            float v[SAMPLE_BATCH];
#pragma unroll
            for (int q = 0; q < SAMPLE_BATCH; ++q) {
                const int i = i0 + 32 * q + lane;
                v[q] = i < rb ? row[i] : 0.f;
            }
#pragma unroll
            for (int q = 0; q < SAMPLE_BATCH; ++q) {
                const int i = i0 + 32 * q + lane;
                const float w = v[q] * inv_t;
                const bool keep = i < rb && ordered_key(w) >= floor_key;
                const unsigned m = __ballot_sync(0xffffffffu, keep);
                if (keep) {
                    const unsigned pos = at + __popc(m & ((1u << lane) - 1u));
                    if (pos < SAMPLE_CAP) {
                        sh.le[pos] = expf(w - mx);
                        sh.li[pos] = i;
                    }
                }
                at += __popc(m);
            }
        }
        __syncthreads();
    }
    // ---- on the list: its mass, the nucleus, the inverse CDF
    const ListScratch scratch{sh.wmass, &sh.sel_digit, &sh.chosen, &sh.pick_warp, &sh.pick_before, &sh.pick_target,
                              reinterpret_cast<u64*>(&sh.whist[0][0]), (int)(sizeof(sh.whist) / (256 * sizeof(u64)))};
    const int token = pick_from_list<SAMPLE_WARPS>(sh.le, sh.li, (int)n_keep, use_k, use_p, tp, u, all_mass, scratch);
    if (token == -1) {                                       // the nucleus is larger than the list
        sample_row_by_bisection(out, row, T, k, tp, u, V, r, x);
        return;
    }
    if (tid == 0) out[r] = token == 0x7fffffff ? x.i : token;       // (rounding left the target past the last kept token)
}

// ---- the same for a large vocabulary, by a cluster of eight blocks a row.  One block walks a row of 65 536
// values in 2-3 us, and the quick way walks it five times; with few rows most SMs idle meanwhile.  Here every
// block of the cluster owns an eighth of the row; what all of them must know (the maximum, the histogram of a
// byte, masses, counts) each block writes into the shared memory of all eight, a cluster barrier follows,
// and every block computes the same decision from the same numbers.  The kept values go into block 0's list,
// which finishes alone.  Rows that need the general way are done by block 0.
#define SC_CTAS 8
#define SC_THREADS 512
#define SC_WARPS (SC_THREADS / 32)

struct ClusterShared {
    unsigned whist[SC_WARPS][256];                      // a histogram per warp
    unsigned ghist[2][SC_CTAS][256];                    // every block's histogram, in every block (two in turn)
    float le[SAMPLE_CAP];                               // the list (block 0's is the one that is used)
    int li[SAMPLE_CAP];
    u64 gmass[SC_CTAS];                                 // per block: mass of its part of the row
    unsigned gcount[SC_CTAS];                           // per block: kept values
    MaxIdx gmax[SC_CTAS];                               // per block: maximum
    u64 wmass[SC_WARPS];
    unsigned wcount[SC_WARPS], woffset[SC_WARPS];
    MaxIdx redm[33];
    unsigned sel_digit, sel_above;
    int chosen, pick_warp;
    u64 pick_before, pick_target;
};

__device__ __forceinline__ unsigned sc_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void sc_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of `local` (in this block's shared memory) in block `rank` of the cluster
__device__ __forceinline__ unsigned sc_map(const void* local, unsigned rank) {
    unsigned a = (unsigned)__cvta_generic_to_shared(local), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ void sc_store_u32(unsigned addr, unsigned v) { asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void sc_store_f32(unsigned addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void sc_store_u64(unsigned addr, u64 v) { asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory"); }

__global__ void __launch_bounds__(SC_THREADS) sample_cluster_kernel(int* __restrict__ out, const float* __restrict__ logits,
                              const float* __restrict__ temperature, const int* __restrict__ top_k,
                              const float* __restrict__ top_p, const float* __restrict__ uniform, int V,
                              const int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char sample_smem[];
    ClusterShared& sh = *reinterpret_cast<ClusterShared*>(sample_smem);
    __shared__ unsigned hist[256];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned c = sc_rank();
    const int r = blockIdx.x / SC_CTAS;
    if (status && blockIdx.x == 0 && tid == 0) out[gridDim.x / SC_CTAS] = *status;
    const float* row = logits + (size_t)r * V;
    const float T = temperature[r];
    const bool greedy = T <= 0.f;
    const float inv_t = greedy ? 1.f : 1.f / T, u = uniform[r], tp = top_p[r];
    const int k = top_k[r];
    const bool use_k = !greedy && k > 0 && k < V, use_p = !greedy && tp < 1.f;
    // the cluster's 128 warps in index order: warp (block c, w) owns [ra, rb), a multiple of 32 long
    const int range = ((V + SC_CTAS * SC_WARPS - 1) / (SC_CTAS * SC_WARPS) + 31) / 32 * 32;
    const int ra = min((int)(c * SC_WARPS + warp) * range, V), rb = min(ra + range, V);
    const int want = use_k ? k : min(SAMPLE_CAP, V);
    const bool select = (use_k || use_p) && want <= SAMPLE_CAP;
    // this block's copy of a gathered field, as seen by block q
    auto everywhere_u32 = [&](unsigned* field, unsigned v) {
        for (unsigned q = 0; q < SC_CTAS; ++q) sc_store_u32(sc_map(field, q), v);
    };

    // ---- walk one: the maximum and its first index, and the count by the top byte of the key
    for (int j = lane; j < 256; j += 32) sh.whist[warp][j] = 0;
    __syncwarp();
    MaxIdx x{-INFINITY, 0x7fffffff};
    {
        RunCount rc{0u, 0u};
        SAMPLE_WALK(
            if (v > x.v) { x.v = v; x.i = i; }
            if (select) rc.add(sh.whist[warp], ordered_key(v * inv_t) >> 24);
        )
        rc.flush(sh.whist[warp]);
    }
    x = block_argmax(x, sh.redm);                            // (syncs the block)
    if (tid == 0) {
        everywhere_u32(reinterpret_cast<unsigned*>(&sh.gmax[c].v), __float_as_uint(x.v));
        everywhere_u32(reinterpret_cast<unsigned*>(&sh.gmax[c].i), (unsigned)x.i);
    }
    if (select && tid < 256) {
        unsigned n = 0;
        for (int w2 = 0; w2 < SC_WARPS; ++w2) n += sh.whist[w2][tid];
        everywhere_u32(&sh.ghist[0][c][tid], n);
    }
    sc_sync();
    x = sh.gmax[0];
    for (int q = 1; q < SC_CTAS; ++q) x = better(x, sh.gmax[q]);
    if (greedy) {
        if (c == 0 && tid == 0) out[r] = x.i == 0x7fffffff ? 0 : x.i;
        return;
    }
    const float mx = x.v * inv_t;

    // the floor: the key of the `want`-th largest scaled value, byte by byte from the top
    unsigned floor_key = 0, n_keep = 0;
    u64 all_mass = 0;
    if (select) {
        unsigned prefix = 0, remaining = (unsigned)want, above = 0;
        for (int byte = 3; byte >= 0; --byte) {
            const int shift = byte * 8, buf = (3 - byte) & 1;
            if (byte < 3) {
                for (int j = lane; j < 256; j += 32) sh.whist[warp][j] = 0;
                __syncwarp();
                const unsigned high_mask = 0xffffffffu << (shift + 8);
                RunCount rc{0u, 0u};
                u64 part = 0;
                unsigned gt = 0;
                SAMPLE_WALK(
                    const float w = v * inv_t;
                    const unsigned key = ordered_key(w);
                    if ((key & high_mask) == (prefix & high_mask)) rc.add(sh.whist[warp], (key >> shift) & 255u);
                    if (byte == 2) part += unit_of(expf(w - mx));
                    if (byte == 0) gt += (key & high_mask) > (prefix & high_mask) ? 1u : 0u;
                )
                rc.flush(sh.whist[warp]);
                if (byte == 2) {
                    part = warp_sum_u64(part);
                    if (lane == 0) sh.wmass[warp] = part;
                }
                if (byte == 0) {
                    gt = __reduce_add_sync(0xffffffffu, gt);
                    if (lane == 0) sh.wcount[warp] = gt;
                }
                __syncthreads();
                if (tid < 256) {
                    unsigned n = 0;
                    for (int w2 = 0; w2 < SC_WARPS; ++w2) n += sh.whist[w2][tid];
                    everywhere_u32(&sh.ghist[buf][c][tid], n);
                }
                if (byte == 2 && tid == 0) {
                    u64 m = 0;
                    for (int w2 = 0; w2 < SC_WARPS; ++w2) m += sh.wmass[w2];
                    for (unsigned q = 0; q < SC_CTAS; ++q) sc_store_u64(sc_map(&sh.gmass[c], q), m);
                }
                sc_sync();
            }
            if (tid < 256) {
                unsigned n = 0;
                for (int q = 0; q < SC_CTAS; ++q) n += sh.ghist[buf][q][tid];
                hist[tid] = n;
            }
            __syncthreads();
            if (warp == 0) {
                // lane l owns bins 8l..8l+7; the digit is the highest bin at which the count from the top reaches `remaining`
                unsigned mine = 0;
                for (int j = 0; j < 8; ++j) mine += hist[lane * 8 + j];
                unsigned incl = mine;
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned y = __shfl_down_sync(0xffffffffu, incl, o);
                    if (lane + o < 32) incl += y;
                }
                const unsigned higher = incl - mine;
                if (higher < remaining && remaining <= incl) {
                    unsigned cum = higher;
                    for (int j = 7; j >= 0; --j) {
                        const unsigned n = hist[lane * 8 + j];
                        if (cum + n >= remaining) { sh.sel_digit = (unsigned)(lane * 8 + j); sh.sel_above = cum; break; }
                        cum += n;
                    }
                }
            }
            __syncthreads();
            prefix |= sh.sel_digit << shift;
            above += sh.sel_above;
            remaining -= sh.sel_above;
            if (byte == 0) n_keep = above + hist[sh.sel_digit];
            if (byte == 2) {
                for (int q = 0; q < SC_CTAS; ++q) all_mass += sh.gmass[q];
            }
            __syncthreads();
        }
        floor_key = prefix;
    }
    if (!select) {
        if (use_k || use_p) {                                // a top-k above what the list holds
            if (c == 0) sample_row_by_bisection(out, row, T, k, tp, u, V, r, x);
            return;
        }
        // ---- nothing to select: the inverse CDF over the whole row.  The blocks' masses to every block, then the
        // block that holds the target finds the warp and the warp walks again.
        u64 part = 0;
        SAMPLE_WALK(part += unit_of(expf(v * inv_t - mx));)
        part = warp_sum_u64(part);
        if (lane == 0) sh.wmass[warp] = part;
        __syncthreads();
        if (tid == 0) {
            u64 m = 0;
            for (int w2 = 0; w2 < SC_WARPS; ++w2) m += sh.wmass[w2];
            for (unsigned q = 0; q < SC_CTAS; ++q) sc_store_u64(sc_map(&sh.gmass[c], q), m);
        }
        sc_sync();
        u64 total = 0, before = 0;
        for (unsigned q = 0; q < SC_CTAS; ++q) {
            if (q < c) before += sh.gmass[q];
            total += sh.gmass[q];
        }
        const u64 target = (u64)((double)u * (double)total);
        // the first block whose cumulative mass reaches the target (and that has mass) is the one
        int owner = -1;
        {
            u64 cum = 0;
            for (int q = 0; q < SC_CTAS; ++q) {
                cum += sh.gmass[q];
                if (sh.gmass[q] > 0 && target <= cum) { owner = q; break; }
            }
        }
        if (owner < 0) {
            if (c == 0 && tid == 0) out[r] = x.i;             // (rounding left the target past the last token)
            return;
        }
        if ((int)c != owner) return;
        if (tid == 0) sh.chosen = 0x7fffffff;
        __syncthreads();
        if (warp == 0) {
            const u64 mine = lane < SC_WARPS ? sh.wmass[lane] : 0ull;
            const u64 incl = warp_scan_u64(mine, lane) + before;
            const unsigned hit = __ballot_sync(0xffffffffu, mine > 0 && target <= incl);
            if (lane == 0) sh.pick_warp = hit ? __ffs(hit) - 1 : -1;
            if (hit && lane == __ffs(hit) - 1) sh.pick_before = incl - mine;
        }
        __syncthreads();
        if (warp == sh.pick_warp) {
            u64 cum = sh.pick_before;
            for (int i0 = ra; i0 < rb; i0 += 32) {
                const int i = i0 + lane;
                const u64 e = i < rb ? unit_of(expf(row[i] * inv_t - mx)) : 0ull;
                const u64 incl = warp_scan_u64(e, lane) + cum;
                const unsigned hit = __ballot_sync(0xffffffffu, e > 0 && target <= incl);
                if (hit) {
                    if (lane == 0) sh.chosen = i0 + __ffs(hit) - 1;
                    break;
                }
                cum = __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        __syncthreads();
        if (tid == 0) out[r] = sh.chosen == 0x7fffffff ? x.i : sh.chosen;
        return;
    }
    if (n_keep > SAMPLE_CAP) {                               // (ties at the floor are all kept)
        if (c == 0) sample_row_by_bisection(out, row, T, k, tp, u, V, r, x);
        return;
    }

    // ---- the list, in block 0, in index order: every block's kept count to every block, then each warp writes its
    // kept values behind those of the warps (and blocks) before it
    {
        unsigned mine = 0;
        const unsigned digit = floor_key & 255u;
        for (int j = lane; j < 256; j += 32) mine += (unsigned)j >= digit ? sh.whist[warp][j] : 0u;
        mine = __reduce_add_sync(0xffffffffu, mine) + sh.wcount[warp];
        if (lane == 0) sh.woffset[warp] = mine;
        __syncthreads();
        if (warp == 0) {
            const unsigned n = lane < SC_WARPS ? sh.woffset[lane] : 0u;
            unsigned incl = n;
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned y = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += y;
            }
            if (lane < SC_WARPS) sh.woffset[lane] = incl - n;
            if (lane == 31) everywhere_u32(&sh.gcount[c], incl);
        }
        sc_sync();
        unsigned at = sh.woffset[warp];
        for (unsigned q = 0; q < c; ++q) at += sh.gcount[q];
        const unsigned le0 = sc_map(sh.le, 0), li0 = sc_map(sh.li, 0);
        for (int i0 = ra; i0 < rb; i0 += 32 * SAMPLE_BATCH) {
            float v[SAMPLE_BATCH];
#pragma unroll
            for (int q = 0; q < SAMPLE_BATCH; ++q) {
                const int i = i0 + 32 * q + lane;
                v[q] = i < rb ? row[i] : 0.f;
            }
#pragma unroll
            for (int q = 0; q < SAMPLE_BATCH; ++q) {
                const int i = i0 + 32 * q + lane;
                const float w = v[q] * inv_t;
                const bool keep = i < rb && ordered_key(w) >= floor_key;
                const unsigned m = __ballot_sync(0xffffffffu, keep);
                if (keep) {
                    const unsigned pos = at + __popc(m & ((1u << lane) - 1u));
                    if (pos < SAMPLE_CAP) {
                        sc_store_f32(le0 + 4u * pos, expf(w - mx));
                        sc_store_u32(li0 + 4u * pos, (unsigned)i);
                    }
                }
                at += __popc(m);
            }
        }
        sc_sync();
    }
    if (c != 0) return;
    const ListScratch scratch{sh.wmass, &sh.sel_digit, &sh.chosen, &sh.pick_warp, &sh.pick_before, &sh.pick_target,
                              reinterpret_cast<u64*>(&sh.whist[0][0]), (int)(sizeof(sh.whist) / (256 * sizeof(u64)))};
    const int token = pick_from_list<SC_WARPS>(sh.le, sh.li, (int)n_keep, use_k, use_p, tp, u, all_mass, scratch);
    if (token == -1) {                                       // the nucleus is larger than the list
        sample_row_by_bisection(out, row, T, k, tp, u, V, r, x);
        return;
    }
    if (tid == 0) out[r] = token == 0x7fffffff ? x.i : token;
}

// out holds R ids, and the status word behind them if `status` is given (R + 1 ints then).
ZAI_API int zai_argmax(int* out, const float* logits, int R, int V, const int* status, cudaStream_t stream) {
    if (R <= 0) return ZAI_OK;
    return launch_pdl(argmax_kernel, dim3(R), dim3(1024), 0, stream, out, logits, V, status);
}

ZAI_API int zai_repetition_penalty(float* logits, const int* tokens, const int* counts, const int* offsets,
                                   const float* penalty, int R, int V, cudaStream_t stream) {
    if (R <= 0) return ZAI_OK;
    repetition_penalty_kernel<<<R, 128, 0, stream>>>(logits, tokens, counts, offsets, penalty, V);
    return launch_status();
}

// out [R, V] = logits [R, V] with the penalty applied from the table of counts [slots, V]; slots [R] (negative: none)
ZAI_API int zai_repetition_penalty_counts(float* out, const float* logits, const int* counts, const int* slots,
                                          const float* penalty, int R, int V, cudaStream_t stream) {
    if (R <= 0) return ZAI_OK;
    const int by = (V + 256 * 8 - 1) / (256 * 8);
    return launch_pdl(repetition_penalty_counts_kernel, dim3(R, by < 1 ? 1 : by), dim3(256), 0, stream, out, logits, counts, slots,
                      penalty, V);
}

ZAI_API int zai_count_tokens(int* counts, const int* ids, const int* slots, int R, int V, cudaStream_t stream) {
    if (R <= 0) return ZAI_OK;
    return launch_pdl(count_tokens_kernel, dim3((R + 127) / 128), dim3(128), 0, stream, counts, ids, slots, R, V);
}

ZAI_API int zai_sample(int* out, const float* logits, const float* temperature, const int* top_k, const float* top_p,
                       const float* uniform, int R, int V, const int* status, cudaStream_t stream) {
    if (R <= 0) return ZAI_OK;
    static int use_cluster = -1;
    if (use_cluster < 0) {
        const char* e = getenv("ZAI_SAMPLE_CLUSTER");
        use_cluster = e ? atoi(e) : 1;
    }
    if (use_cluster && V >= 16384 && R <= 32) {                // (with more rows the SMs are busy anyway)
        // a cluster of eight blocks a row
        const size_t smem = sizeof(ClusterShared);
        static unsigned long long configured = 0;
        if (zai_first_on_device(&configured)) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)R * SC_CTAS);
        cfg.blockDim = dim3(SC_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = SC_CTAS;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        return (int)cudaLaunchKernelEx(&cfg, sample_cluster_kernel, out, logits, temperature, top_k, top_p, uniform, V, status);
    }
    const size_t smem = sizeof(SampleShared);
    static unsigned long long configured = 0;
    if (zai_first_on_device(&configured)) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), smem, stream, out, logits, temperature, top_k, top_p, uniform, V,
                      status);
}
