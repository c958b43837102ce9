// RMSNorm over rows of the 32-bit residual stream, optionally fused with the residual
// sum that precedes it and with a row gather.
//
//   h[r, :] += delta[r, :]           (if delta is given; the sum is kept in 32-bit.  delta may come as
//                                     `parts` tensors `part_stride` elements apart, added in order: the
//                                     sums over the parts of k that a split product leaves)
//   y[i, :]  = h[r, :] * rsqrt(mean(h[r, :]^2) + eps) * weight[:]
//
// with r = rows[i] if `rows` is given, else r = i.  When `rows` is given the sum is
// not written back to h (the gathered rows are the last use of the stream).  Squares,
// mean, rsqrt and the scaling are 32-bit; the result is rounded once, to the output
// type.
#include "common.cuh"

template <typename TD, typename TW, typename TY>
__global__ void rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                               const int* __restrict__ rows, const TW* __restrict__ weight,
                               TY* __restrict__ y, int hidden, float eps, int n_rows_total,
                               int* __restrict__ status, int parts, size_t part_stride) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  int r = i;
  if (rows != nullptr) {
    r = rows[i];
    if (r < 0 || r >= n_rows_total) {
      if (threadIdx.x == 0) atomicOr(status, JV_STATUS_BAD_ROW);
      for (int c = threadIdx.x; c < hidden; c += blockDim.x) y[(size_t)i * hidden + c] = from_f32<TY>(0.f);
      return;
    }
  }
  float* hr = h + (size_t)r * hidden;
  const TD* dr = delta ? delta + (size_t)r * hidden : nullptr;
  const bool write_back = (dr != nullptr) && (rows == nullptr);
  float ss = 0.f;
  auto delta_at = [&](int c) {
    float d = to_f32(dr[c]);
    for (int s = 1; s < parts; ++s) d += to_f32(dr[s * part_stride + c]);
    return d;
  };
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = hr[c];
    if (dr) v += delta_at(c);
    if (write_back) hr[c] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TY* yr = y + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = hr[c];                          // this thread's own write, if any
    if (dr && !write_back) v += delta_at(c);
    yr[c] = from_f32<TY>(v * inv * to_f32(weight[c]));
  }
}

// The same with the row held in registers and 8 elements per thread and pass (hidden a multiple
// of 8, at most blockDim.x * 8 * RM_ITERS): one read of the stream, no second read for the scaling.
constexpr int RM_ITERS = 4;

template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) { const float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 a;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = a;
}

// ITERS: passes per thread (1 for rows of up to 640 vectors of 8, else RM_ITERS).  TOGETHER: how many parts of a
// sum ask for their loads at once: 8 for a few rows (a decode step waits for this kernel, and one trip to the L2
// per part is most of its time), 1 for many rows, where registers are better spent on more blocks per
// multiprocessor.
template <typename TD, typename TW, typename TY, int ITERS, int TOGETHER>
__global__ void __launch_bounds__(ITERS == 1 ? 640 : 1024) rmsnorm_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const int* __restrict__ rows, const TW* __restrict__ weight,
                                   TY* __restrict__ y, int hidden, float eps, int n_rows_total,
                                   int* __restrict__ status, int parts, size_t part_stride) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  int r = i;
  if (rows != nullptr) {
    r = rows[i];
    if (r < 0 || r >= n_rows_total) {
      if (threadIdx.x == 0) atomicOr(status, JV_STATUS_BAD_ROW);
      for (int c = threadIdx.x; c < hidden; c += blockDim.x) y[(size_t)i * hidden + c] = from_f32<TY>(0.f);
      return;
    }
  }
  float* hr = h + (size_t)r * hidden;
  const TD* dr = delta ? delta + (size_t)r * hidden : nullptr;
  const bool write_back = (dr != nullptr) && (rows == nullptr);
  float v[ITERS][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c < hidden) {
      load8<float>(hr + c, v[it]);
      if (dr) {
        // the parts of a sum (eight at most ask for their loads together, then add in the order of the parts)
        float d[8];
        load8<TD>(dr + c, d);
        float e[TOGETHER][8];
#pragma unroll
        for (int s = 1; s < TOGETHER; ++s)
          if (s < parts) load8<TD>(dr + s * part_stride + c, e[s]);
#pragma unroll
        for (int s = 1; s < TOGETHER; ++s)
          if (s < parts) {
#pragma unroll
            for (int k = 0; k < 8; ++k) d[k] += e[s][k];
          }
        for (int s = TOGETHER; s < parts; ++s) {
          float f[8];
          load8<TD>(dr + s * part_stride + c, f);
#pragma unroll
          for (int k = 0; k < 8; ++k) d[k] += f[k];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) v[it][k] += d[k];
        if (write_back) store8<float>(hr + c, v[it]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += v[it][k] * v[it][k];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TY* yr = y + (size_t)i * hidden;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c < hidden) {
      float w[8];
      load8<TW>(weight + c, w);
#pragma unroll
      for (int k = 0; k < 8; ++k) w[k] = v[it][k] * inv * w[k];
      store8<TY>(yr + c, w);
    }
  }
}

// h: [n_total, hidden] float (updated in place when delta is given and rows is null);
// delta: [n_total, hidden] of dtype `delta_dtype` or null, or `delta_parts` such tensors `delta_part_stride`
// elements apart whose sum it is; rows: [n_out] int32 or null;
// weight: [hidden] of dtype `weight_dtype`; y: [n_out, hidden] of dtype `out_dtype`.
JV_EXPORT int jv_rmsnorm(float* h, const void* delta, int delta_dtype, const int* rows,
                         const void* weight, int weight_dtype, void* y, int out_dtype, int n_out,
                         int n_total, int hidden, float eps, int delta_parts, long long delta_part_stride, int* status,
                         cudaStream_t stream) {
  if (n_out == 0) return JV_OK;
  if (delta_parts < 1 || (delta_part_stride % 8)) return JV_ERR_UNSUPPORTED;
  const int parts = delta_parts;
  const size_t part_stride = (size_t)delta_part_stride;
  const bool aligned = ((uintptr_t)h % 16) == 0 && ((uintptr_t)delta % 16) == 0 && ((uintptr_t)weight % 16) == 0 &&
                       ((uintptr_t)y % 16) == 0;
  if (hidden % 8 == 0 && hidden <= 1024 * 8 * RM_ITERS && aligned) {
    const int vecs = hidden / 8;
    int iters = vecs <= 640 ? 1 : (vecs + 511) / 512;     // up to 640 threads, then more passes per thread
    if (iters > RM_ITERS) iters = RM_ITERS;
    int vthreads = ((vecs + iters - 1) / iters + 31) / 32 * 32;
    if (vthreads > 1024) vthreads = 1024;
    if (iters == 1 && parts > 1 && n_out <= 256)
      JV_DISPATCH_DTYPE(out_dtype, TY, JV_DISPATCH_DTYPE(weight_dtype, TW, JV_DISPATCH_DTYPE(delta_dtype, TD,
          return jv_launch(rmsnorm_vec_kernel<TD, TW, TY, 1, 8>, dim3(n_out), dim3(vthreads), 0, stream,
                           h, (const TD*)delta, rows, (const TW*)weight, (TY*)y, hidden, eps, n_total, status, parts, part_stride))));
    if (iters == 1)
      JV_DISPATCH_DTYPE(out_dtype, TY, JV_DISPATCH_DTYPE(weight_dtype, TW, JV_DISPATCH_DTYPE(delta_dtype, TD,
          return jv_launch(rmsnorm_vec_kernel<TD, TW, TY, 1, 1>, dim3(n_out), dim3(vthreads), 0, stream,
                           h, (const TD*)delta, rows, (const TW*)weight, (TY*)y, hidden, eps, n_total, status, parts, part_stride))));
    JV_DISPATCH_DTYPE(out_dtype, TY, JV_DISPATCH_DTYPE(weight_dtype, TW, JV_DISPATCH_DTYPE(delta_dtype, TD,
        return jv_launch(rmsnorm_vec_kernel<TD, TW, TY, RM_ITERS, 1>, dim3(n_out), dim3(vthreads), 0, stream,
                         h, (const TD*)delta, rows, (const TW*)weight, (TY*)y, hidden, eps, n_total, status, parts, part_stride))));
    return JV_ERR_UNSUPPORTED;
  }
  int threads = 32;
  while (threads < 512 && threads * 4 < hidden) threads *= 2;
  JV_DISPATCH_DTYPE(out_dtype, TY, JV_DISPATCH_DTYPE(weight_dtype, TW, JV_DISPATCH_DTYPE(delta_dtype, TD,
      return jv_launch(rmsnorm_kernel<TD, TW, TY>, dim3(n_out), dim3(threads), 0, stream,
                       h, (const TD*)delta, rows, (const TW*)weight, (TY*)y, hidden, eps, n_total, status, parts, part_stride))));
  return JV_ERR_UNSUPPORTED;
}

// Adds delta into the 32-bit stream without a norm: h[r, :] += delta[r, :].
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ h, const TD* __restrict__ delta, size_t n, int parts,
                                    size_t part_stride) {
  pdl_trigger();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float d = to_f32(delta[i]);
    for (int s = 1; s < parts; ++s) d += to_f32(delta[s * part_stride + i]);
    h[i] += d;
  }
}

// delta as for jv_rmsnorm: one tensor (delta_parts 1) or the parts of a sum.
JV_EXPORT int jv_residual_add(float* h, const void* delta, int delta_dtype, long long n, int delta_parts,
                              long long delta_part_stride, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  if (delta_parts < 1) return JV_ERR_UNSUPPORTED;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  JV_DISPATCH_DTYPE(delta_dtype, TD, return jv_launch(residual_add_kernel<TD>, dim3((int)blocks), dim3(256), 0, stream,
                                                      h, (const TD*)delta, (size_t)n, delta_parts,
                                                      (size_t)delta_part_stride));
  return JV_ERR_UNSUPPORTED;
}
