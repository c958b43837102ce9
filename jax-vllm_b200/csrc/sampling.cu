// Token choice from 32-bit logits, one block per row.
//   temperature == 0: the index of the largest logit (the lowest index among equals).
//   temperature  > 0: a draw from softmax(logits / temperature) by the Gumbel-max rule,
//       argmax_v(logits[v] / temperature - log(-log(u_v))), with u_v in (0, 1) from a
//       counter-based generator keyed by (seed of the request, index of the output token,
//       v).  The draw therefore depends on the request and the place in its output only,
//       not on the batch it was sampled in.
#include "common.cuh"
#include <math.h>

__host__ __device__ __forceinline__ unsigned long long jv_mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

// Uniform in (0, 1) with 24 random bits.
__host__ __device__ __forceinline__ float jv_uniform(unsigned long long seed, unsigned long long counter,
                                                     unsigned long long v) {
  unsigned long long h = jv_mix64(seed + 0x9E3779B97F4A7C15ULL * (counter + 1));
  h = jv_mix64(h ^ (v * 0xD1342543DE82EF95ULL + 0x2545F4914F6CDD1DULL));
  return ((float)(unsigned)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

__global__ void sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                              const long long* __restrict__ seeds, const long long* __restrict__ counters,
                              int* __restrict__ out) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const int row = blockIdx.x;
  const float* lr = logits + (size_t)row * vocab;
  const float temp = temperature[row];
  const unsigned long long seed = (unsigned long long)seeds[row];
  const unsigned long long counter = (unsigned long long)counters[row];
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
    float x = lr[v];
    if (temp > 0.f) {
      const float u = jv_uniform(seed, counter, (unsigned long long)v);
      x = x / temp - logf(-logf(u));
    }
    if (x > bv || (x == bv && v < bi)) { bv = x; bi = v; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nwarps = blockDim.x >> 5;
    bv = lane < nwarps ? best_v[lane] : -INFINITY;
    bi = lane < nwarps ? best_i[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;
  }
}

// logits: [rows, vocab] float; temperature: [rows] float; seeds, counters: [rows] int64;
// out: [rows] int32.
JV_EXPORT int jv_sample(const float* logits, int rows, int vocab, const float* temperature,
                        const long long* seeds, const long long* counters, int* out,
                        cudaStream_t stream) {
  if (rows == 0) return JV_OK;
  sample_kernel<<<rows, 512, 0, stream>>>(logits, vocab, temperature, seeds, counters, out);
  return jv_check_launch();
}
