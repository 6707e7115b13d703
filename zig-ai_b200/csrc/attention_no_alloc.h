// Split-key decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (samooth/zig-ai allocates what its kernels
// need from its own pools before it launches them); it exists for users of this library only.
//
// Who needs it.  The regular entry point, zai_decode_attention_mma, wants two scratch buffers from
// its caller, and the Python wrapper gets them from PyTorch's allocator.  Some callers have no
// allocator to ask: a host program that drives these libraries through their C symbols without
// PyTorch; a server that handed the whole device to its own arena at start-up and may not grow;
// a step loop in which a cudaMalloc, which synchronises the device, would stall every stream.
// For them the scratch lives inside the library, in a file-scope `static __device__` array.
//
// What it costs and what it limits.
//   * The array holds ZAI_STATIC_SCRATCH_FLOATS 32-bit floats (4 MiB).  Every GPU on which the
//     library is loaded keeps that memory until the process ends, whether or not this entry point
//     is ever called.
//   * A call needs B * Hq * n_chunks * (D + 2) floats.  A larger call is refused with
//     ZAI_SCRATCH_TOO_SMALL (-3) and launches nothing; zai_decode_attention_static_error() gives the
//     text for a code.  For the LFM2 shapes (16 or 32 query heads of size 64) and requests up to
//     4096 positions (16 chunks) this allows batches of 62 and 31 requests.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and remembers it; make that first call before any stream capture begins.
//     The call itself uses cudaMalloc, cudaFree or any other allocating routine at no time.
//   * All calls share the one array, and it keeps what the last call left.  Nothing in it has to
//     start at zero: every chunk's maximum and sum are rewritten by each call before they are read,
//     and outputs of chunks without visible keys are never read.  Two calls that overlap on the GPU
//     (different streams, or different host threads) race on the array: serialise them.
//
// Arguments are those of zai_decode_attention_mma without the two scratch pointers: inputs and
// outputs still come from the caller.  bfloat16 only.  Returns 0, a negative ZaiError, or the
// CUDA error code of the launch.
#pragma once
#include <cuda_runtime.h>

#define ZAI_STATIC_SCRATCH_FLOATS (1 << 20)
#define ZAI_SCRATCH_TOO_SMALL (-3)
#define ZAI_SCRATCH_SETUP_FAILED (-4)

#ifdef __cplusplus
extern "C" {
#endif

int zai_decode_attention_static(void* out, const void* q, const void* pages, const int* block_table,
                                int table_width, const int* positions, int B, int n_chunks, int page_size,
                                int Hq, int Hkv, int D, float scale, int window, cudaStream_t stream);

// Text for a code returned by zai_decode_attention_static.
const char* zai_decode_attention_static_error(int code);

#ifdef __cplusplus
}
#endif
