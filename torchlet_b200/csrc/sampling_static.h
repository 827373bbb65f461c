// Token selection that allocates nothing.
//
// This entry point has no counterpart in the reference (4mengy/torchlet samples with
// torch's argmax and lets PyTorch allocate whatever it needs).  It exists for callers
// that cannot allocate device memory at the moment they need a token: code that runs
// inside a region where cudaMalloc is forbidden or would synchronize the device (while a
// stream is being captured into a CUDA graph, inside a latency-critical serving loop that
// must not touch the allocator, in a process whose memory pool is owned by another
// component and may not be grown).
//
// tl_sample_static does what tl_sample does -- argmax, or a seeded Gumbel-max draw from
// softmax(logits / temperature), one token per row of float32 logits [rows, vocab] -- but
// the intermediate results of the blocks that share a row live in a fixed array inside
// the library instead of a buffer supplied by the caller:
//
//   * the array is file-scope device memory of TL_SAMPLE_STATIC_MAX_PARTIALS entries
//     (8 bytes each, 256 KiB in all); every GPU that loads the library holds it until the
//     process exits;
//   * rows * ceil(vocab / 8192) must not exceed TL_SAMPLE_STATIC_MAX_PARTIALS; larger
//     problems are refused with TL_SAMPLE_STATIC_TOO_LARGE and nothing is launched;
//   * the first call on a device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current) and keeps it; make that first call
//     before any stream capture begins;
//   * all calls share the one array and it keeps the last call's contents.  Nothing in it
//     has to start at zero: every entry a call reads has been written by that call first.
//     Two calls that overlap on the GPU (different streams, or one graph replayed while
//     another call runs) race on it: keep calls on one device ordered.
//
// The caller still passes inputs and outputs (device pointers); no cudaMalloc, cudaFree or
// other allocating routine is called.
#pragma once
#include <cuda_runtime.h>

#define TL_SAMPLE_STATIC_MAX_PARTIALS 32768
#define TL_SAMPLE_STATIC_TOO_LARGE 10002

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, TL_SAMPLE_STATIC_TOO_LARGE, 10001 (bad arguments) or a cudaError_t.
// temperature / seed / counter may all be null: every row is then greedy.  A non-null
// temperature needs a seed and a counter as well (a row with temperature > 0 reads both);
// with either missing the call is refused with 10001 and nothing is launched.
int tl_sample_static(const float* logits, long long row_stride, int rows, int vocab, const float* temperature,
                     const long long* seed, const int* counter, int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
