// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (Foundation Model Stack is pure PyTorch and leaves
// all memory to torch's allocator).  It exists for hosts that embed these kernels where cudaMalloc is not
// an option: a process that runs under a fixed memory budget handed out at start-up, a real-time or
// safety-reviewed loop in which an allocation (a possible device synchronisation, a possible failure) may
// not happen once the loop has started, or a plug-in whose host application owns the allocator.
//
// fms_attention_decode (attention.cu) needs scratch memory for the partial results of its key splits and
// expects the caller to provide it.  fms_attention_decode_no_alloc is the same computation — the same two
// kernels, the same launch shapes, bit-identical results (as long as fms_attention_decode is not given what lets
// it pick its streaming kernel) — but takes its scratch from an array that is
// part of the library image itself:
//
//     static __device__ __align__(256) unsigned char g_decode_scratch[FMS_NO_ALLOC_SCRATCH_BYTES];
//
// Limit.  FMS_NO_ALLOC_SCRATCH_BYTES is 8 MiB.  A call needs
//     n_seqs * nheads * n_splits * (head_dim + 2) * 4 bytes
// (e.g. 8 sequences x 32 heads x 8 splits of 256 keys x 130 floats = 1.0 MiB); a larger call is refused
// with an error and nothing is launched.  Every GPU on which the library's kernels get loaded holds the
// 8 MiB until the process exits, whether or not this entry point is ever called.  The attention source is built
// once per head size (libfms_attention_hd64, _hd128, ...), and each of these libraries carries an array of its
// own: a process that loads three of them holds 24 MiB per GPU.
//
// Precondition.  n_splits * 256 must be at least every sequence's length after the step (len_after lives on the
// device, so this function cannot check it).  This entry point has no error word on the device: a longer sequence
// silently loses its keys beyond n_splits * 256.  Nothing outside the array is read or written in that case.
//
// Set-up.  The array's name is a host-side handle, not a device address.  The first call on each device
// (with that device current: the address is taken for the current device, not for the device of `stream`, so
// make the stream's device current before every call) asks the runtime for the address with cudaGetSymbolAddress, checks the
// result and remembers it per device; later calls on that device reuse it.  Make that first call before
// any stream capture begins.  The function calls no cudaMalloc, cudaFree or other allocating routine.
//
// Sharing.  All calls on a device use the same array, and it keeps what the last call left.  Nothing in it
// has to start at zero: every entry that the combining kernel reads was written by the split kernel of the
// same call.  Two calls whose kernels can overlap on the GPU (different streams without an ordering
// between them, or several host threads) race on the array; serialise them.
//
// Arguments are those of fms_attention_decode without the two scratch pointers and without what only its
// streaming kernel needs (the pool size, the total length, a work counter, the error flag): this entry point
// always takes the kernels with one block of threads per split.  Inputs and outputs are still the caller's.  Returns 0, or non-zero with the reason in fms_last_error().
#pragma once

#include <cuda_runtime.h>

#define FMS_NO_ALLOC_SCRATCH_BYTES (8u << 20)

extern "C" int fms_attention_decode_no_alloc(const void* q, void* out, int dtype, const void* keys, const void* values,
                                             const int* table, int table_stride, int block_tokens, const int* slots,
                                             const int* first_row, const int* len_after, int n_seqs, int n_splits,
                                             int nheads, int kvheads, int head_dim, float scale, int window,
                                             cudaStream_t stream);
