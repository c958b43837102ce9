// What is done to a query or key head before attention, written once for every kernel that does it
// (rope_kv.cu for any batch; the prepare path of attn_decode_tcgen05.cu for steps of single tokens):
//
//   per-head RMSNorm (optional):  u <- u * rsqrt(mean(u^2) + eps) * weight          jllm/model/common.py:44-48,107-111
//   rotation ("half-split"):      a_j = float(position) * table[j]                   jllm/model/common.py:51-66
//                                 u'[j]        = u[j] * cos(a_j) - u[j + half] * sin(a_j)
//                                 u'[j + half] = u[j + half] * cos(a_j) + u[j] * sin(a_j),   j < half
//
// all in 32-bit, angles, cosines and sines included.  The kernels differ in how they spread a head over a warp
// (registers or shared memory); the arithmetic is these functions and nothing else, so another family of position
// encodings (another map from position and table entry to angle, another pairing) is written here once.
#pragma once

#include "common.cuh"

// Cosine and sine of the rotation of pair j at a position: the angle is position * table[j].
__device__ __forceinline__ void qk_rotation(int position, float table_j, float* sn, float* cs) {
  sincosf((float)position * table_j, sn, cs);
}

// The rotated pair (first-half element, its partner in the second half).
__device__ __forceinline__ void qk_rotate_pair(float first, float second, float cs, float sn, float* first_out, float* second_out) {
  *first_out = first * cs - second * sn;
  *second_out = second * cs + first * sn;
}

// The factor that RMSNorm multiplies a head with, from the sum of squares over its `dim` elements.
__device__ __forceinline__ float qk_norm_factor(float sum_of_squares, int dim, float eps) {
  return rsqrtf(sum_of_squares / (float)dim + eps);
}

// A warp's share of one head in registers: lane l holds E consecutive elements d0 .. d0+E-1 of the first half in `a`
// and their partners half+d0 .. in `b` (d0 = l * E, half = 32 * E).  Normalises with the weight given by
// `weight_at(index)` if `normed`, then rotates with this lane's cosines and sines.
template <int E, typename WeightAt>
__device__ __forceinline__ void qk_prepare_head(float (&a)[E], float (&b)[E], int d0, int half, bool normed, float eps,
                                                WeightAt weight_at, const float (&cs)[E], const float (&sn)[E]) {
  if (normed) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < E; ++i) ss += a[i] * a[i] + b[i] * b[i];
    ss = warp_sum(ss);
    const float inv = qk_norm_factor(ss, 2 * half, eps);
#pragma unroll
    for (int i = 0; i < E; ++i) {
      a[i] = a[i] * inv * weight_at(d0 + i);
      b[i] = b[i] * inv * weight_at(half + d0 + i);
    }
  }
#pragma unroll
  for (int i = 0; i < E; ++i) qk_rotate_pair(a[i], b[i], cs[i], sn[i], &a[i], &b[i]);
}
