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
// distribution is the same).  Thresholds of top-k and top-p are found by bisection over the bit
// patterns of the values, so no sort is needed; ties at a threshold are all kept.
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

__global__ void sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
                              const float* __restrict__ temperature, const int* __restrict__ top_k,
                              const float* __restrict__ top_p, const float* __restrict__ uniform, int V,
                              const int* __restrict__ status) {
    __shared__ MaxIdx redm[33];
    __shared__ float red[33];
    __shared__ float scan[SAMPLE_THREADS];
    __shared__ int chosen;
    pdl_trigger();
    pdl_wait();
    if (status && blockIdx.x == 0 && threadIdx.x == 0) out[gridDim.x] = *status;
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * V;
    const float T = temperature[r];
    MaxIdx x = scan_row(row, V);
    x = block_argmax(x, redm);
    if (T <= 0.f) {
        if (tid == 0) out[r] = x.i == 0x7fffffff ? 0 : x.i;
        return;
    }
    const float inv_t = 1.f / T;
    const float mx = x.v * inv_t;
    // top-k: the k-th largest scaled value, by bisection on the ordered bit pattern
    float floor_val = -INFINITY;
    const int k = top_k[r];
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
    const float tp = top_p[r];
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
    const float target = uniform[r] * total;
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

ZAI_API int zai_sample(int* out, const float* logits, const float* temperature, const int* top_k, const float* top_p,
                       const float* uniform, int R, int V, const int* status, cudaStream_t stream) {
    if (R <= 0) return ZAI_OK;
    return launch_pdl(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, out, logits, temperature, top_k, top_p, uniform, V,
                      status);
}
