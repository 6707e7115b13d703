// Shared helpers of the sm_100a kernels: element types, warp and block reductions, and the C ABI
// conventions of the launchers (every launcher takes raw device pointers and a stream, launches on
// that stream and returns the CUDA error code of the launch, 0 for success).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define ZAI_API extern "C" __attribute__((visibility("default")))

enum ZaiDtype { ZAI_F32 = 0, ZAI_BF16 = 1 };
enum ZaiError { ZAI_OK = 0, ZAI_BAD_DTYPE = -1, ZAI_BAD_SIZE = -2 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // `red` may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// ---- the status word of a step: one device int that kernels OR bits into and the host reads with the
// step's results.  A kernel never traps and never touches memory outside the tensors it was given: an
// id outside its bound is replaced by id 0 (page 0 and slot 0 are never handed to a request, padding
// rows use them), the bit is raised and the step's results are to be thrown away by the host.
enum ZaiStatusBit {
    ZAI_ST_WAIT = 1,        // a bounded wait (mbarrier, ticket) ran out
    ZAI_ST_TOKEN = 2,       // a token id outside the vocabulary
    ZAI_ST_PAGE = 4,        // a block-table entry outside the pool
    ZAI_ST_SLOT = 8,        // a state slot outside the slots
    ZAI_ST_POSITION = 16    // a position outside the request's block-table row
};
__device__ __forceinline__ void zai_raise(int* status, int bit) {
    if (status) atomicOr(status, bit);
}
// The page that holds logical page `idx` of a request whose block-table row is `table_row`.
__device__ __forceinline__ int zai_checked_page(const int* __restrict__ table_row, int table_width, int idx,
                                                int num_pages, int* status) {
    if ((unsigned)idx >= (unsigned)table_width) {
        zai_raise(status, ZAI_ST_POSITION);
        return 0;
    }
    const int page = table_row[idx];
    if ((unsigned)page >= (unsigned)num_pages) {
        zai_raise(status, ZAI_ST_PAGE);
        return 0;
    }
    return page;
}
// A request's row of a block table with its bounds: page(idx) is the checked lookup above.
struct ZaiTableRow {
    const int* row;
    int width, num_pages;
    int* status;
    __device__ __forceinline__ int page(int idx) const { return zai_checked_page(row, width, idx, num_pages, status); }
};
__device__ __forceinline__ int zai_checked_slot(int slot, int num_slots, int* status) {
    if ((unsigned)slot >= (unsigned)num_slots) {
        zai_raise(status, ZAI_ST_SLOT);
        return 0;
    }
    return slot;
}

// ---- programmatic dependent launch: a kernel launched this way may start while the kernel before
// it on the stream still runs.  It must call pdl_wait() before it reads anything an earlier kernel
// wrote and before it writes anything an earlier kernel may still read (so: before its first global
// write); what it does before that (address arithmetic, loads of weights) overlaps the predecessor.
// pdl_trigger() lets the kernel after this one begin its own start-up.  Both are no-ops in a kernel
// launched the ordinary way.  ZAI_PDL=0 in the environment launches everything the ordinary way.
//
// Built with -DZAI_TIMELINE (ZAI_TIMELINE=1 in the environment when the libraries are built), the
// last thread of every kernel's first block notes the global timer before and after the wait, so a
// step's kernels can be laid out on one time axis without a profiler's serialisation:
// zai_timeline_read() returns the records (id, time at the wait, time after it); the id is the
// source line of the wait times 256 plus a number the kernel may add (a template variant).
#ifdef ZAI_TIMELINE
#define ZAI_TIMELINE_RECORDS 16384
static __device__ unsigned long long zai_tl_records[ZAI_TIMELINE_RECORDS * 3];
static __device__ unsigned int zai_tl_count;
__device__ __forceinline__ unsigned long long zai_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void zai_tl_put(unsigned long long id, unsigned long long t0, unsigned long long t1) {
    const unsigned int i = atomicAdd(&zai_tl_count, 1u);
    if (i < ZAI_TIMELINE_RECORDS) {
        zai_tl_records[3 * i] = id;
        zai_tl_records[3 * i + 1] = t0;
        zai_tl_records[3 * i + 2] = t1;
    }
}
__device__ __forceinline__ bool zai_tl_thread() {
    return blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == blockDim.x - 1 && threadIdx.y == 0;
}
#endif
__device__ __forceinline__ void pdl_wait_at(int line, int variant) {
#ifdef ZAI_TIMELINE
    const bool rec = zai_tl_thread();
    unsigned long long t0 = 0;
    if (rec) t0 = zai_global_ns();
#endif
    asm volatile("griddepcontrol.wait;" ::: "memory");
#ifdef ZAI_TIMELINE
    if (rec) zai_tl_put((unsigned long long)line * 256 + (unsigned long long)(variant & 255), t0, zai_global_ns());
#else
    (void)line;
    (void)variant;
#endif
}
#define pdl_wait() pdl_wait_at(__LINE__, 0)
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// A further point on the time axis from inside a kernel (same thread as above): a record with both
// times equal and the id (1 << 32) + mark.  Compiles to nothing without ZAI_TIMELINE.
__device__ __forceinline__ void zai_mark(int mark) {
#ifdef ZAI_TIMELINE
    if (zai_tl_thread()) {
        const unsigned long long t = zai_global_ns();
        zai_tl_put((1ull << 32) + (unsigned long long)(mark & 255), t, t);
    }
#else
    (void)mark;
#endif
}
// The life of every block of a kernel (not only the first): call at the block's start, keep the value,
// and hand it back at the block's end; a record with the id (2 << 32) + the block's linear index.
__device__ __forceinline__ unsigned long long zai_block_begin() {
#ifdef ZAI_TIMELINE
    return zai_global_ns();
#else
    return 0;
#endif
}
__device__ __forceinline__ void zai_block_end(unsigned long long t_begin) {
#ifdef ZAI_TIMELINE
    if (threadIdx.x == 0 && threadIdx.y == 0)
        zai_tl_put((2ull << 32) + blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z),
                   t_begin, zai_global_ns());
#else
    (void)t_begin;
#endif
}
#ifdef ZAI_TIMELINE
// Copies up to `max_records` (id, t_wait, t_after) triples to `out` and empties the list; returns how many.
ZAI_API int zai_timeline_read(unsigned long long* out, int max_records) {
    unsigned int n = 0;
    if (cudaMemcpyFromSymbol(&n, zai_tl_count, sizeof(n)) != cudaSuccess) return -1;
    if (n > ZAI_TIMELINE_RECORDS) n = ZAI_TIMELINE_RECORDS;
    if ((int)n > max_records) n = (unsigned int)max_records;
    if (n && cudaMemcpyFromSymbol(out, zai_tl_records, (size_t)n * 3 * sizeof(unsigned long long)) != cudaSuccess) return -1;
    const unsigned int zero = 0;
    cudaMemcpyToSymbol(zai_tl_count, &zero, sizeof(zero));
    return (int)n;
}
#endif

#include <stdlib.h>
static inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("ZAI_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// True the first time it is called with `*done` on each device: a kernel's attributes (its dynamic
// shared-memory limit) are set per device, so a launcher sets them on its first launch on every device.
static inline bool zai_first_on_device(unsigned long long* done) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if ((*done >> dev) & 1ull) return false;
    *done |= 1ull << dev;
    return true;
}

template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Calls `expr` with T bound to the element type that `dtype` names.
#define ZAI_DISPATCH(dtype, ...)                                   \
    do {                                                           \
        if ((dtype) == ZAI_F32) { typedef float T; __VA_ARGS__; }  \
        else if ((dtype) == ZAI_BF16) { typedef bf16 T; __VA_ARGS__; } \
        else return ZAI_BAD_DTYPE;                                 \
    } while (0)
