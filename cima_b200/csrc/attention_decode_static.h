// cima_attention_decode_static: the split-KV decode attention without any allocation.
//
// This entry point has no counterpart in the reference.  It exists for callers that are not allowed
// to obtain device memory at the time they need attention: code that runs inside a host program
// whose device memory was handed out once at start-up and is owned by someone else (an inference
// server's plug-in, an embedded runtime with a fixed arena), or a latency-critical loop in which an
// allocation would stall the device.  Such callers can supply the inputs and the output, which they
// own anyway, but not the float32 scratch that the merge of the key splits needs.
//
// Here that scratch is a fixed array in the library's own device image
// (CIMA_DECODE_STATIC_FLOATS float32 values, 8 MiB, held by every GPU that loads the library until
// the process ends).  The arguments are those of cima_attention_decode without part_o and part_ml.
//
// Rules of use:
//   * Sizes whose scratch, B * heads * n_splits * (head_dim + 2) floats, exceeds the array are
//     refused with CIMA_E_SIZE and a sentence in cima_last_error(); nothing is launched.
//   * The first call on a device looks the array's device address up (one cudaGetSymbolAddress,
//     with that device current) and remembers it; make that first call before any stream capture.
//   * All calls share the one array and it keeps what the last call left.  Nothing in it needs to
//     start at zero: every (sequence, head, split) cell that the merge reads is written by the same
//     call first, empty splits included.  Two calls that overlap on the GPU (different streams)
//     race on the array; serialise them.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any path.
#pragma once
#include <cuda_runtime.h>

#define CIMA_DECODE_STATIC_FLOATS (1 << 21)

#ifdef __cplusplus
extern "C" {
#endif
int cima_attention_decode_static(const void* qkv, int ld, const void* cache, const int* table, int table_width,
                                 int ring, int page_size, const int* seq_slot, const int* seq_len, void* out, int ldo,
                                 int B, int nh, int nkv, int hd, float scale, int window, int n_splits,
                                 cudaStream_t stream);
#ifdef __cplusplus
}
#endif
