// The ShortConv mixer between its two projections: u = B * x~, a causal depthwise convolution of u
// over the request's conv state followed by this step's rows, and the gate z = C * y.
//
//   y[t, c] = sum_j w[c, j] * u_[i + j, c] (+ b[c]),   u_ = state rows 0..L-2 ++ u rows of the span
//
// with i the row's index inside its request's span, so tap L-1 multiplies the current token (the
// indexing of the reference's conv1dSiluKernel, src/cuda/layer_kernels.cu:206-213, which adds a
// SiLU that the LFM2 operator does not have).  The new state is the last L-1 rows of u_
// (ibid. :216-221).  The reference passes one buffer as old and new state although its kernel
// forbids that (src/transformer/short_conv.zig:408-415 against layer_kernels.cu:191); here the
// rows are computed by one kernel that only reads the state, and the state is replaced by a second
// kernel in which each thread first reads everything it needs and then writes.  When every span
// is a single token both happen in one kernel, thread by thread.
// The state is 32-bit and holds u exactly as the products of the stored B and x~, so a row's
// result does not depend on whether its neighbours come from the state or from the same step.
#include "common.cuh"

#define ZAI_MAX_TAPS 16

template <typename T>
__global__ void conv_rows_kernel(T* __restrict__ z, const T* __restrict__ bcx, const float* __restrict__ w,
                                 const float* __restrict__ bias, const float* __restrict__ state,
                                 const int* __restrict__ seq_idx, const int* __restrict__ cu_q,
                                 const int* __restrict__ slot_ids, int C, int L, int state_rows, int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = seq_idx[t];
    const int i = t - cu_q[s];
    const float* st = state + ((size_t)zai_checked_slot(slot_ids[s], num_slots, status) * state_rows) * C;
    float y = bias ? bias[c] : 0.f;
    for (int j = 0; j < L; ++j) {
        const int r = i + j - (L - 1);                    // row of the span, negative: from the state
        float u;
        if (r >= 0) {
            const T* row = bcx + (size_t)(t - i + r) * 3 * C;
            u = to_float(row[c]) * to_float(row[2 * C + c]);
        } else {
            u = st[(size_t)(i + j) * C + c];
        }
        y += w[(size_t)c * L + j] * u;
    }
    const float gate = to_float(bcx[(size_t)t * 3 * C + C + c]);
    z[(size_t)t * C + c] = from_float<T>(gate * y);
}

// bfloat16, C a multiple of 8: one thread per (row, 8 channels), 16-byte loads of B, C and x~
__global__ void conv_rows_bf16x8_kernel(bf16* __restrict__ z, const bf16* __restrict__ bcx, const float* __restrict__ w,
                                        const float* __restrict__ bias, const float* __restrict__ state,
                                        const int* __restrict__ seq_idx, const int* __restrict__ cu_q,
                                        const int* __restrict__ slot_ids, int C, int L, int state_rows, int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int s = seq_idx[t];
    const int i = t - cu_q[s];
    const float* st = state + ((size_t)zai_checked_slot(slot_ids[s], num_slots, status) * state_rows) * C;
    float y[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = bias ? bias[c + e] : 0.f;
    for (int j = 0; j < L; ++j) {
        const int r = i + j - (L - 1);
        float u[8];
        if (r >= 0) {
            const bf16* row = bcx + (size_t)(t - i + r) * 3 * C;
            const uint4 b4 = *reinterpret_cast<const uint4*>(row + c);
            const uint4 x4 = *reinterpret_cast<const uint4*>(row + 2 * C + c);
            const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b4);
            const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 b = __bfloat1622float2(bp[e]), x = __bfloat1622float2(xp[e]);
                u[2 * e] = b.x * x.x;
                u[2 * e + 1] = b.y * x.y;
            }
        } else {
            const float4 a = *reinterpret_cast<const float4*>(st + (size_t)(i + j) * C + c);
            const float4 b = *reinterpret_cast<const float4*>(st + (size_t)(i + j) * C + c + 4);
            u[0] = a.x; u[1] = a.y; u[2] = a.z; u[3] = a.w; u[4] = b.x; u[5] = b.y; u[6] = b.z; u[7] = b.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] += w[(size_t)(c + e) * L + j] * u[e];
    }
    const uint4 g4 = *reinterpret_cast<const uint4*>(bcx + (size_t)t * 3 * C + C + c);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
    uint4 o4;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 gte = __bfloat1622float2(gp[e]);
        op[e] = __floats2bfloat162_rn(gte.x * y[2 * e], gte.y * y[2 * e + 1]);
    }
    *reinterpret_cast<uint4*>(z + (size_t)t * C + c) = o4;
}

// bfloat16, C a multiple of 8, L taps (1..4): one thread per (4 consecutive rows, 8 channels).  The
// rows' B, C and x~ (twelve 16-byte loads) are asked for at once; the products u = B x~ of earlier
// rows stay in registers while the thread walks down its rows, so a row is read once; only a
// thread's first row (or a row that starts a request's span) fetches its L - 1 predecessors or the
// request's state.
#define CONV_R 4
template <int L>
__global__ void __launch_bounds__(128) conv_rows_bf16x8_walk_kernel(
    bf16* __restrict__ z, const bf16* __restrict__ bcx, const float* __restrict__ w, const float* __restrict__ bias,
    const float* __restrict__ state, const int* __restrict__ seq_idx, const int* __restrict__ cu_q,
    const int* __restrict__ slot_ids, int N, int C, int state_rows, int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t0 = blockIdx.x * CONV_R;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= C || t0 >= N) return;
    const int rows = min(CONV_R, N - t0);
    uint4 b4[CONV_R], g4[CONV_R], x4[CONV_R];
    int sq[CONV_R];
#pragma unroll
    for (int r = 0; r < CONV_R; ++r) {
        if (r < rows) {
            const bf16* row = bcx + (size_t)(t0 + r) * 3 * C + c;
            b4[r] = *reinterpret_cast<const uint4*>(row);
            g4[r] = *reinterpret_cast<const uint4*>(row + C);
            x4[r] = *reinterpret_cast<const uint4*>(row + 2 * C);
            sq[r] = seq_idx[t0 + r];
        }
    }
    float wt[8][L], bs[8];
    {
        float flat[8 * L];
#pragma unroll
        for (int q = 0; q < 2 * L; ++q) {
            const float4 v = *reinterpret_cast<const float4*>(w + (size_t)c * L + 4 * q);
            flat[4 * q] = v.x; flat[4 * q + 1] = v.y; flat[4 * q + 2] = v.z; flat[4 * q + 3] = v.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e)
#pragma unroll
            for (int j = 0; j < L; ++j) wt[e][j] = flat[e * L + j];
#pragma unroll
        for (int e = 0; e < 8; ++e) bs[e] = bias ? bias[c + e] : 0.f;
    }
    float hist[L > 1 ? L - 1 : 1][8];                         // u of the L-1 rows before the current one, oldest first
    int prev_seq = -1;
#pragma unroll
    for (int r = 0; r < CONV_R; ++r) {
        if (r >= rows) break;
        const int t = t0 + r, s = sq[r];
        const int i = t - cu_q[s];                                // the row's place in its span
        if (L > 1 && (s != prev_seq || i == 0)) {                // (re)build the history: earlier rows, or the state
            const float* st = state + ((size_t)zai_checked_slot(slot_ids[s], num_slots, status) * state_rows) * C;
#pragma unroll
            for (int j = 0; j < L - 1; ++j) {
                const int rr = i + j - (L - 1);
                if (rr >= 0) {
                    const bf16* row = bcx + (size_t)(t - i + rr) * 3 * C + c;
                    const uint4 pb = *reinterpret_cast<const uint4*>(row), px = *reinterpret_cast<const uint4*>(row + 2 * C);
                    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&pb);
                    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&px);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 b = __bfloat1622float2(bp[e]), x = __bfloat1622float2(xp[e]);
                        hist[j][2 * e] = b.x * x.x;
                        hist[j][2 * e + 1] = b.y * x.y;
                    }
                } else {
                    const float4 a = *reinterpret_cast<const float4*>(st + (size_t)(i + j) * C + c);
                    const float4 b = *reinterpret_cast<const float4*>(st + (size_t)(i + j) * C + c + 4);
                    hist[j][0] = a.x; hist[j][1] = a.y; hist[j][2] = a.z; hist[j][3] = a.w;
                    hist[j][4] = b.x; hist[j][5] = b.y; hist[j][6] = b.z; hist[j][7] = b.w;
                }
            }
        }
        prev_seq = s;
        float u[8];
        {
            const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b4[r]);
            const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x4[r]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 b = __bfloat1622float2(bp[e]), x = __bfloat1622float2(xp[e]);
                u[2 * e] = b.x * x.x;
                u[2 * e + 1] = b.y * x.y;
            }
        }
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            y[e] = bs[e];
#pragma unroll
            for (int j = 0; j < L - 1; ++j) y[e] += wt[e][j] * hist[j][e];
            y[e] += wt[e][L - 1] * u[e];
        }
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4[r]);
        uint4 o4;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 gte = __bfloat1622float2(gp[e]);
            op[e] = __floats2bfloat162_rn(gte.x * y[2 * e], gte.y * y[2 * e + 1]);
        }
        *reinterpret_cast<uint4*>(z + (size_t)t * C + c) = o4;
#pragma unroll
        for (int j = 0; j + 1 < L - 1; ++j)
#pragma unroll
            for (int e = 0; e < 8; ++e) hist[j][e] = hist[j + 1][e];
        if (L > 1) {
#pragma unroll
            for (int e = 0; e < 8; ++e) hist[L - 2][e] = u[e];
        }
    }
}

template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ bcx, float* __restrict__ state,
                                  const int* __restrict__ cu_q, const int* __restrict__ slot_ids,
                                  int C, int L, int state_rows, int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int a = cu_q[s], n = cu_q[s + 1] - a;
    float* st = state + ((size_t)zai_checked_slot(slot_ids[s], num_slots, status) * state_rows) * C;
    float keep[ZAI_MAX_TAPS];
#pragma unroll
    for (int r = 0; r < ZAI_MAX_TAPS; ++r) {
        if (r < L - 1) {
            const int src = n + r;                         // index into u_ = state ++ u
            if (src < L - 1) {
                keep[r] = st[(size_t)src * C + c];
            } else {
                const T* row = bcx + (size_t)(a + src - (L - 1)) * 3 * C;
                keep[r] = to_float(row[c]) * to_float(row[2 * C + c]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ZAI_MAX_TAPS; ++r)
        if (r < L - 1) st[(size_t)r * C + c] = keep[r];
}

// Every span is one token: row s belongs to request s.
template <typename T>
__global__ void conv_decode_kernel(T* __restrict__ z, const T* __restrict__ bcx, const float* __restrict__ w,
                                   const float* __restrict__ bias, float* __restrict__ state,
                                   const int* __restrict__ slot_ids, int C, int L, int state_rows, int write_state, int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float* st = state + ((size_t)zai_checked_slot(slot_ids[s], num_slots, status) * state_rows) * C;
    const T* row = bcx + (size_t)s * 3 * C;
    const float u = to_float(row[c]) * to_float(row[2 * C + c]);
    float y = bias ? bias[c] : 0.f;
    float prev[ZAI_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < ZAI_MAX_TAPS; ++j)
        if (j < L - 1) {
            prev[j] = st[(size_t)j * C + c];
            y += w[(size_t)c * L + j] * prev[j];
        }
    y += w[(size_t)c * L + (L - 1)] * u;
    z[(size_t)s * C + c] = from_float<T>(to_float(row[C + c]) * y);
    if (write_state) {
#pragma unroll
        for (int j = 0; j < ZAI_MAX_TAPS; ++j)
            if (j < L - 1) st[(size_t)j * C + c] = (j + 1 < L - 1) ? prev[j + 1] : u;
    }
}

ZAI_API int zai_short_conv(void* z, const void* bcx, int dtype, const float* w, const float* bias, float* state,
                           const int* seq_idx, const int* cu_q, const int* slot_ids, int N, int S, int C, int L,
                           int state_rows, int decode_only, int write_state, int num_slots, int* status, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (L < 1 || L > ZAI_MAX_TAPS || state_rows < L - 1) return ZAI_BAD_SIZE;
    const int threads = 128;
    const unsigned bx = (unsigned)((C + threads - 1) / threads);
    if (decode_only) {
        ZAI_DISPATCH(dtype, return launch_pdl(conv_decode_kernel<T>, dim3(S, bx), dim3(threads), 0, stream,
            (T*)z, (const T*)bcx, w, bias, state, slot_ids, C, L, state_rows, write_state, num_slots, status));
    }
    int e = 0;
    const bool aligned = ((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(bcx) | reinterpret_cast<uintptr_t>(w) |
                           reinterpret_cast<uintptr_t>(state)) & 15) == 0;
    if (dtype == ZAI_BF16 && (C & 7) == 0 && aligned) {
        const int c8 = C / 8, th = c8 < 128 ? ((c8 + 31) / 32) * 32 : 128;
        const dim3 walk((N + CONV_R - 1) / CONV_R, (c8 + th - 1) / th);
#define ZAI_CONV_WALK(l) if (L == l) e = launch_pdl(conv_rows_bf16x8_walk_kernel<l>, walk, dim3(th), 0, stream, (bf16*)z, \
        (const bf16*)bcx, w, bias, (const float*)state, seq_idx, cu_q, slot_ids, N, C, state_rows, num_slots, status);
        ZAI_CONV_WALK(1) ZAI_CONV_WALK(2) ZAI_CONV_WALK(3) ZAI_CONV_WALK(4)
#undef ZAI_CONV_WALK
        if (L > 4)
            e = launch_pdl(conv_rows_bf16x8_kernel, dim3(N, (c8 + th - 1) / th), dim3(th), 0, stream, (bf16*)z, (const bf16*)bcx, w,
                           bias, (const float*)state, seq_idx, cu_q, slot_ids, C, L, state_rows, num_slots, status);
    } else
    ZAI_DISPATCH(dtype, e = launch_pdl(conv_rows_kernel<T>, dim3(N, bx), dim3(threads), 0, stream,
        (T*)z, (const T*)bcx, w, bias, (const float*)state, seq_idx, cu_q, slot_ids, C, L, state_rows, num_slots, status));
    if (e || !write_state || L == 1) return e;
    ZAI_DISPATCH(dtype, return launch_pdl(conv_state_kernel<T>, dim3(S, bx), dim3(threads), 0, stream,
        (const T*)bcx, state, cu_q, slot_ids, C, L, state_rows, num_slots, status));
}
