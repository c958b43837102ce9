// Gated activation of the feed-forward: act[n, i] = silu(gate_i) * up_i with silu(z) = z * sigmoid(z)
// evaluated in 32-bit.  `gu` is what the packed gate|up projection writes: blocks of `block` gate
// columns followed by the `block` up columns of the same indices (block == inter: all gate columns,
// then all up columns), so gate_i = gu[n, (i / block) * 2 * block + i % block] and up_i is `block`
// columns further.
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter, int block, size_t total) {
  pdl_trigger();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const size_t n = idx / inter;
    const int i = (int)(idx - n * inter);
    const size_t col = (size_t)(i / block) * 2 * block + (i % block);
    const float g = to_f32(gu[n * 2 * inter + col]);
    const float u = to_f32(gu[n * 2 * inter + col + block]);
    const float s = g / (1.f + expf(-g));
    act[idx] = from_f32<T>(s * u);
  }
}

// Same, 16 bytes per access (block a multiple of the vector length, rows 16-byte aligned).
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter, int block, size_t total_vec) {
  pdl_trigger();
  pdl_wait();
  constexpr int V = 16 / sizeof(T);
  const int vec_per_row = inter / V;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total_vec; idx += stride) {
    const size_t n = idx / vec_per_row;
    const int i = (int)(idx - n * vec_per_row) * V;
    const size_t col = (size_t)(i / block) * 2 * block + (i % block);
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + n * 2 * inter + col);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + n * 2 * inter + col + block);
    const T* g = reinterpret_cast<const T*>(&g4);
    const T* u = reinterpret_cast<const T*>(&u4);
    uint4 o4;
    T* o = reinterpret_cast<T*>(&o4);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float gv = to_f32(g[k]);
      o[k] = from_f32<T>(gv / (1.f + expf(-gv)) * to_f32(u[k]));
    }
    *reinterpret_cast<uint4*>(act + n * inter + i) = o4;
  }
}

// gu: [n, 2*inter]; act: [n, inter]; both of dtype `dtype`; block: see above (a divisor of inter).
JV_EXPORT int jv_swiglu(const void* gu, void* act, int dtype, int n, int inter, int block, cudaStream_t stream) {
  const size_t total = (size_t)n * inter;
  if (total == 0) return JV_OK;
  if (block < 1 || inter % block) return JV_ERR_UNSUPPORTED;
  const int vec = dtype == 0 ? 4 : 8;
  if (block % vec == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)act % 16) == 0) {
    const size_t total_vec = total / vec;
    size_t blocks = (total_vec + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    JV_DISPATCH_DTYPE(dtype, T, return jv_launch(swiglu_vec_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                                  (const T*)gu, (T*)act, inter, block, total_vec));
    return JV_ERR_UNSUPPORTED;
  }
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  JV_DISPATCH_DTYPE(dtype, T, return jv_launch(swiglu_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                                (const T*)gu, (T*)act, inter, block, total));
  return JV_ERR_UNSUPPORTED;
}
