// Shared helpers for the KV-cache kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "jpt_b200.h"

namespace jpt {

// Thread-local description of the last failure, returned by
// jpt_last_error_string().
char* last_error_buffer();
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);
long long launch_count();

#define JPT_REQUIRE(cond, code, ...)       \
  do {                                     \
    if (!(cond)) return ::jpt::fail((code), __VA_ARGS__); \
  } while (0)

inline bool aligned(const void* p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) % a) == 0;
}

inline int dtype_bytes(int dt) {
  return dt == JPT_BF16 ? 2 : dt == JPT_F32 ? 4 : dt == JPT_INT8 ? 1 : 0;
}

// Element load / store with conversion through fp32.
template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x);
}
template <>
__device__ __forceinline__ float to_f32<int8_t>(int8_t x) { return (float)x; }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// Round an fp32 intermediate to the storage type T and widen again: the
// "every op rounds to the tensor dtype" rule of eager execution.
template <typename T>
__device__ __forceinline__ float round_to(float x) {
  return to_f32<T>(from_f32<T>(x));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide max; `red` is shared scratch of at least 33 floats.  Every thread
// of the block must call it.
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float x = lane < nwarps ? red[lane] : 0.f;
    x = warp_max(x);
    if (lane == 0) red[32] = x;
  }
  __syncthreads();
  return red[32];
}

// Decode quantiser (truncate) and insert quantiser (round half even), both with
// every intermediate rounded to the storage type T of the input.
template <typename T>
__device__ __forceinline__ float decode_scale(float amax) {
  return round_to<T>(__fdiv_rn(amax, 127.0f));
}
template <typename T>
__device__ __forceinline__ int8_t decode_code(float x, float scale) {
  float t = round_to<T>(__fdiv_rn(x, scale));
  if (t != t) t = 0.f;  // 0/0 for an all-zero token
  t = truncf(t);
  t = fminf(fmaxf(t, -128.f), 127.f);
  return (int8_t)(int)t;
}
template <typename T>
__device__ __forceinline__ float insert_scale(float amax) {
  const float eps = round_to<T>(1e-5f);
  return round_to<T>(__fdiv_rn(fmaxf(amax, eps), 127.0f));
}
template <typename T>
__device__ __forceinline__ float insert_recip(float scale) {
  return round_to<T>(__fdiv_rn(1.0f, scale));
}
template <typename T>
__device__ __forceinline__ int8_t insert_code(float x, float recip) {
  const float t = round_to<T>(__fmul_rn(x, recip));
  // one conversion instruction: round half to even, saturating; then the clamp on the integer
  const int q = __float2int_rn(t);
  return (int8_t)max(-128, min(127, q));
}

// Programmatic dependent launch: a kernel launched with launch_after_previous()
// may start (CTA launch ramp, set-up that touches no global data) while the
// kernel before it in the stream is still running; grid_dependency_wait() blocks
// until that kernel has completed and its writes are visible, and is a no-op for
// an ordinary launch.  grid_dependency_trigger() lets the kernel after this one
// start the same way.  The attribute is left out while the stream is being captured into a
// graph, and with JPT_NO_PDL=1 in the environment.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_after_previous(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                         Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // Inside a CUDA graph the launch gaps are already short and the early start measured slower
  // (59.1 against 57.0 us per decode layer); eager launches gain from it (12 % end to end).
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &capturing) != cudaSuccess) capturing = cudaStreamCaptureStatusNone;
  cfg.numAttrs = (pdl_enabled() && capturing == cudaStreamCaptureStatusNone) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace jpt
