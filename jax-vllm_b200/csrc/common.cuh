// Shared device helpers for the sm_100a kernels of this engine.
//
// Every kernel file is plain CUDA with `extern "C"` launchers that take raw device
// pointers, sizes and a stream; nothing here includes a framework header, so a file
// compiles in seconds.  Arithmetic that the engine promises in 32-bit (norms,
// softmax, rotation angles, the residual sum) is done on `float` values obtained
// through `to_f32`/`from_f32`, whatever the storage type is.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define JV_EXPORT extern "C" __attribute__((visibility("default")))

// Error codes returned by launchers (0 = launched).
enum : int {
  JV_OK = 0,
  JV_ERR_LAUNCH = 1,       // cudaGetLastError() after the launch was not cudaSuccess
  JV_ERR_UNSUPPORTED = 2,  // the sizes given are outside what the kernel handles
};

// Bits of the device-side status word (a kernel that meets an index outside its
// tables sets a bit, skips the access and goes on; the host reads the word after the
// step and raises).
enum : int {
  JV_STATUS_BAD_TOKEN = 1,   // token id outside the embedding table
  JV_STATUS_BAD_PAGE = 2,    // page id outside the pool, or a missing table entry
  JV_STATUS_BAD_ROW = 4,     // row index outside the batch
  JV_STATUS_WAIT_EXPIRED = 8 // a bounded wait on a barrier ran out
};

template <typename T> struct DType;
template <> struct DType<float> { static constexpr int code = 0; };
template <> struct DType<__nv_bfloat16> { static constexpr int code = 1; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over all threads of a block (blockDim.x a multiple of 32, at most 1024).
// `scratch` holds at least 33 floats of shared memory.  Every thread gets the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// Programmatic dependent launch.  A kernel launched through jv_launch may be made resident while the
// kernel before it in the stream is still finishing; whatever it does before `pdl_wait()` (index
// arithmetic, prefetching weights that no kernel writes) overlaps that kernel's tail, and everything
// after `pdl_wait()` sees all of its results.  `pdl_trigger()` says that the next kernel may be made
// resident; kernels call it first thing.  No kernel reads activations or writes anything before its
// `pdl_wait()`.  JAX_VLLM_B200_PDL=0 in the environment launches plainly instead.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>
static inline bool jv_pdl_enabled() {
  static int state = -1;
  if (state < 0) {
    const char* v = std::getenv("JAX_VLLM_B200_PDL");
    state = (v != nullptr && v[0] == '0') ? 0 : 1;
  }
  return state == 1;
}

template <typename... KArgs, typename... Args>
static inline int jv_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = jv_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...) == cudaSuccess ? JV_OK : JV_ERR_LAUNCH;
}

// One-time set-up per device (function attributes are per device): runs `setup` the first time it is reached
// with a given device current; false if the device cannot be told or `setup` returns false.  Launchers call it
// before their first launch, which keeps the attribute calls out of stream captures.
#define JV_MAX_DEVICES 64
template <typename F>
static inline bool jv_once_per_device(bool (&done)[JV_MAX_DEVICES], F&& setup) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= JV_MAX_DEVICES) return false;
  if (!done[dev]) {
    if (!setup()) return false;
    done[dev] = true;
  }
  return true;
}

static inline int jv_check_launch() {
  return cudaGetLastError() == cudaSuccess ? JV_OK : JV_ERR_LAUNCH;
}

// Dispatch on a dtype code: 0 = float, 1 = bfloat16.
#define JV_DISPATCH_DTYPE(code, T, ...)                        \
  do {                                                         \
    if ((code) == 0) { using T = float; __VA_ARGS__; }         \
    else if ((code) == 1) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return JV_ERR_UNSUPPORTED;                            \
  } while (0)
