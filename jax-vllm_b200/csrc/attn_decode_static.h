// Split decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (alec-tschantz/jax-vllm has no native
// code at all); it exists for users of this library whose code runs where allocation is
// not possible or not allowed: inside a region that is being recorded into a CUDA graph by
// someone else's framework, in a process whose memory pool was sized up front and sealed, or
// from a host thread that may not call into an allocator.  Everything else in this package
// gets its scratch memory from the caller (torch's allocator); this function gets it from a
// fixed array that is part of the library image.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Bytes of the fixed scratch array.  Every GPU on which this library is loaded holds that much
// device memory from load to exit, whether or not the function is ever called.
#define JV_ATTN_STATIC_SCRATCH_BYTES (16u << 20)

// The first JV_ATTN_STATIC_COUNTERS words of the array are arrival counters, one per
// (token, kv head, group of 16 query heads); the rest holds the partial results.
#define JV_ATTN_STATIC_COUNTERS 16384u

// Floats of scratch that a call needs: n_work * n_q_heads * n_splits * (head_dim + 2); they must fit
// into the array less its counters, and n_work * n_kv_heads * ceil(G / 16) into the counters.
long long jv_attn_decode_static_scratch_floats(int n_work, int n_q_heads, int n_splits, int head_dim);

// Attention of single decoded tokens over the paged cache, keys split into `n_splits` ranges of
// `split_size` positions; the same computation as jv_attn_mma with n_splits > 0 (bfloat16, head
// sizes 16/32/64/128), with the same arguments except that no scratch pointers are passed.
//
// Returns 0 on success; 2 if the sizes are not supported or the call needs more scratch than
// JV_ATTN_STATIC_SCRATCH_BYTES (nothing is launched then); 1 if a launch failed; 3 if the address
// of the scratch array could not be obtained.
//
// The function calls no cudaMalloc, no cudaFree and no allocating library routine.  Its first
// call on each device looks up the device address of the scratch array (cudaGetSymbolAddress)
// and opts the kernel into its shared-memory size; make that first call outside any stream
// capture.  All calls on a device share the one array, which keeps what the last call left in
// it; the partial results need no clearing, because every element a call reads was written by the
// same call before, and the counters are cleared by the call itself (a memset on `stream`).  For the same reason two calls whose kernels may overlap on the GPU (different streams
// without an ordering between them) race on the array: order them.
int jv_attn_decode_static(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                          const void* v_cache, const int* block_table, int table_width, const int* cu_seqlens,
                          const int* start_pos, const int* work, int n_work, int n_q_heads, int n_kv_heads,
                          int head_dim, int page_size, int num_pages, int window, float scale, int split_size,
                          int n_splits, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
