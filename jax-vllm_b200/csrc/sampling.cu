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

// (value, index) ordering: larger value wins, the lower index among equal values.
__device__ __forceinline__ void take_better(float& bv, int& bi, float ov, int oi) {
  if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

__device__ __forceinline__ void block_best(float& bv, int& bi, float* sv, int* si) {
  for (int o = 16; o > 0; o >>= 1)
    take_better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nwarps = blockDim.x >> 5;
    bv = lane < nwarps ? sv[lane] : -INFINITY;
    bi = lane < nwarps ? si[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1)
      take_better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  }
}

// Stage 1: block (chunk, row) finds the best entry of its part of the vocabulary.
__global__ void sample_partial_kernel(const float* __restrict__ logits, int vocab, int chunk,
                                      const float* __restrict__ temperature, const long long* __restrict__ seeds,
                                      const long long* __restrict__ counters, float* __restrict__ part_v,
                                      int* __restrict__ part_i) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.y;
  const float* lr = logits + (size_t)row * vocab;
  const float temp = temperature[row];
  const unsigned long long seed = (unsigned long long)seeds[row];
  const unsigned long long counter = (unsigned long long)counters[row];
  const int begin = blockIdx.x * chunk, end = min(vocab, begin + chunk);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int v = begin + threadIdx.x; v < end; v += blockDim.x) {
    float x = lr[v];
    if (temp > 0.f) x = x / temp - logf(-logf(jv_uniform(seed, counter, (unsigned long long)v)));
    take_better(bv, bi, x, v);
  }
  block_best(bv, bi, sv, si);
  if (threadIdx.x == 0) {
    part_v[(size_t)row * gridDim.x + blockIdx.x] = bv;
    part_i[(size_t)row * gridDim.x + blockIdx.x] = bi;
  }
}

// Stage 2: one warp per row over the chunk winners.
__global__ void sample_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int n_chunks,
                                    int* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < n_chunks; c += 32)
    take_better(bv, bi, part_v[(size_t)row * n_chunks + c], part_i[(size_t)row * n_chunks + c]);
  for (int o = 16; o > 0; o >>= 1)
    take_better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (threadIdx.x == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;
}

// Chunks that the vocabulary is cut into (scratch: rows * chunks floats and ints).
JV_EXPORT int jv_sample_chunks(int vocab) {
  int c = (vocab + 2047) / 2048;
  return c < 1 ? 1 : (c > 128 ? 128 : c);
}

// logits: [rows, vocab] float; temperature: [rows] float; seeds, counters: [rows] int64;
// part_v/part_i: scratch of rows * jv_sample_chunks(vocab) elements; out: [rows] int32.
JV_EXPORT int jv_sample(const float* logits, int rows, int vocab, const float* temperature,
                        const long long* seeds, const long long* counters, float* part_v, int* part_i,
                        int* out, cudaStream_t stream) {
  if (rows == 0) return JV_OK;
  const int chunks = jv_sample_chunks(vocab);
  const int chunk = (vocab + chunks - 1) / chunks;
  if (jv_launch(sample_partial_kernel, dim3(chunks, rows), dim3(256), 0, stream, logits, vocab, chunk, temperature,
                seeds, counters, part_v, part_i) != JV_OK)
    return JV_ERR_LAUNCH;
  return jv_launch(sample_final_kernel, dim3(rows), dim3(32), 0, stream, (const float*)part_v, (const int*)part_i, chunks,
                   out);
}
