// Embedding row gather: out[n, :] = table[ids[n], :], written as 32-bit floats (the
// residual stream of the engine is 32-bit in every mode).
#include "common.cuh"

template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int hidden, int vocab,
                                    int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int id = ids[n];
  float* dst = out + (size_t)n * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, JV_STATUS_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(src[i]);
}

// table: [vocab, hidden] of dtype `dtype`; ids: [n] int32; out: [n, hidden] float.
JV_EXPORT int jv_embed_gather(const void* table, int dtype, const int* ids, float* out, int n,
                              int hidden, int vocab, int* status, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  const int threads = hidden >= 1024 ? 256 : 128;
  JV_DISPATCH_DTYPE(dtype, T, return jv_launch(embed_gather_kernel<T>, dim3(n), dim3(threads), 0, stream,
                                                (const T*)table, ids, out, hidden, vocab, status));
  return JV_ERR_UNSUPPORTED;
}
