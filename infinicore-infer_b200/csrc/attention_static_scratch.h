// An entry point of the decode attention kernel that allocates nothing.
//
// This function has NO COUNTERPART IN THE REFERENCE (InfiniCore-Infer takes every buffer from
// its pooled allocator, src/allocator/memory_allocator.cpp); it exists for callers of this
// library's C symbols that cannot allocate device memory at the moment of the call:
//   * a serving loop that may not stall: cudaMalloc and cudaFree synchronise the whole device,
//     so one allocation in the decode path holds up every stream;
//   * a process whose device memory has been handed to the page pool down to the last page,
//     where an allocation, however small, would fail;
//   * a C or ctypes caller that has no tensor library at hand to allocate with.
// `jk_attention_decode` needs scratch memory for the partial results of its key splits and takes
// it from the caller.  `jk_attention_decode_static` is the same computation with the same inputs
// and outputs, minus that argument: the partials go to an array that is part of the library's
// own image.
//
// What a caller has to know:
//   * The array holds JK_STATIC_SCRATCH_FLOATS floats (4 MiB).  Every GPU on which the library is
//     loaded holds it until the process ends.  A call that needs more
//     (nrows * nh * splits * (dh + 2) floats when splits > 1) is refused with JK_BAD_ARGUMENT and a
//     message; nothing is launched.
//   * The FIRST call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and remembers it.  Make that first call before any stream capture
//     begins on that device.
//   * The function calls no cudaMalloc, cudaFree or other allocating routine.
//   * All calls share the one array, and it keeps what the last call left.  Nothing in it has to
//     start at zero: every slot a call reads was written by that same call first.  Two calls whose
//     kernels overlap on the GPU (different streams) would overwrite each other's partials: keep
//     calls on one stream, or order them yourself.
#pragma once

#include <cuda_runtime.h>

#define JK_STATIC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments as jk_attention_decode without `scratch`; returns 0 on success, else a status
// code (the message is available from jk_attention_last_error()).
int jk_attention_decode_static(const void *q, const void *k_pages, const void *v_pages, void *out,
                               const int *rows, int nrows, const int *positions, const int *row_req,
                               const int *block_table, int max_blocks, int page_size, int nh, int nkvh,
                               int dh, float scale, int window, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
