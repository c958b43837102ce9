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

// The same for a gate|up given as `parts` 32-bit tensors [n, 2*inter] `part_stride` elements apart, whose sum it is
// (the sums over the parts of k that a split product leaves), four columns per thread and pass.
template <typename T>
__global__ void swiglu_parts_kernel(const float* __restrict__ gu, T* __restrict__ act, int inter, int block, size_t total_vec,
                                    int parts, size_t part_stride) {
  pdl_trigger();
  pdl_wait();
  const int vec_per_row = inter / 4;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total_vec; idx += stride) {
    const size_t n = idx / vec_per_row;
    const int i = (int)(idx - n * vec_per_row) * 4;
    const size_t col = (size_t)(i / block) * 2 * block + (i % block);
    const float* src = gu + n * 2 * inter + col;
    float4 g = *reinterpret_cast<const float4*>(src), u = *reinterpret_cast<const float4*>(src + block);
    // up to eight parts ask for their loads together; they are added in the order of the parts
    float4 gp[7], up[7];
#pragma unroll
    for (int s = 1; s < 8; ++s)
      if (s < parts) {
        gp[s - 1] = *reinterpret_cast<const float4*>(src + s * part_stride);
        up[s - 1] = *reinterpret_cast<const float4*>(src + s * part_stride + block);
      }
#pragma unroll
    for (int s = 1; s < 8; ++s)
      if (s < parts) {
        g.x += gp[s - 1].x; g.y += gp[s - 1].y; g.z += gp[s - 1].z; g.w += gp[s - 1].w;
        u.x += up[s - 1].x; u.y += up[s - 1].y; u.z += up[s - 1].z; u.w += up[s - 1].w;
      }
    for (int s = 8; s < parts; ++s) {
      const float4 g2 = *reinterpret_cast<const float4*>(src + s * part_stride);
      const float4 u2 = *reinterpret_cast<const float4*>(src + s * part_stride + block);
      g.x += g2.x; g.y += g2.y; g.z += g2.z; g.w += g2.w;
      u.x += u2.x; u.y += u2.y; u.z += u2.z; u.w += u2.w;
    }
    T* dst = act + n * inter + i;
    dst[0] = from_f32<T>(g.x / (1.f + expf(-g.x)) * u.x);
    dst[1] = from_f32<T>(g.y / (1.f + expf(-g.y)) * u.y);
    dst[2] = from_f32<T>(g.z / (1.f + expf(-g.z)) * u.z);
    dst[3] = from_f32<T>(g.w / (1.f + expf(-g.w)) * u.w);
  }
}

// gu: [n, 2*inter]; act: [n, inter]; both of dtype `dtype`; block: see above (a divisor of inter).
// parts > 1: gu is `parts` float tensors [n, 2*inter], part_stride elements apart, and act is of dtype `dtype`
// (block and part_stride multiples of 4, gu 16-byte aligned).
JV_EXPORT int jv_swiglu(const void* gu, void* act, int dtype, int n, int inter, int block, int parts, long long part_stride,
                        cudaStream_t stream) {
  const size_t total = (size_t)n * inter;
  if (total == 0) return JV_OK;
  if (block < 1 || inter % block || parts < 1) return JV_ERR_UNSUPPORTED;
  if (parts > 1) {
    if ((block % 4) || (part_stride % 4) || ((uintptr_t)gu % 16)) return JV_ERR_UNSUPPORTED;
    const size_t total_vec = total / 4;
    size_t blocks = (total_vec + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    JV_DISPATCH_DTYPE(dtype, T, return jv_launch(swiglu_parts_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                                  (const float*)gu, (T*)act, inter, block, total_vec, parts, (size_t)part_stride));
    return JV_ERR_UNSUPPORTED;
  }
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
