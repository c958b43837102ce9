// Gated activation of the feed-forward: act[n, i] = silu(gu[n, i]) * gu[n, inter + i],
// with silu(z) = z * sigmoid(z) evaluated in 32-bit.  `gu` holds the gate columns
// first and the up columns after them, as the packed gate|up projection writes them.
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const size_t n = idx / inter;
    const int i = (int)(idx - n * inter);
    const float g = to_f32(gu[n * 2 * inter + i]);
    const float u = to_f32(gu[n * 2 * inter + inter + i]);
    const float s = g / (1.f + expf(-g));
    act[idx] = from_f32<T>(s * u);
  }
}

// gu: [n, 2*inter]; act: [n, inter]; both of dtype `dtype`.
JV_EXPORT int jv_swiglu(const void* gu, void* act, int dtype, int n, int inter, cudaStream_t stream) {
  const size_t total = (size_t)n * inter;
  if (total == 0) return JV_OK;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  JV_DISPATCH_DTYPE(dtype, T, (swiglu_kernel<T><<<(int)blocks, 256, 0, stream>>>(
                                  (const T*)gu, (T*)act, inter, total)));
  return jv_check_launch();
}
