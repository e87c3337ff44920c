// Shared helpers of the sm_100a kernels: element types, status codes, reductions.
//
// Every launcher in this library is a plain C function that takes raw device
// pointers, sizes and a stream, validates the sizes, launches, and returns
// GG_OK or an error code; gg_last_error() gives the message.  Nothing here
// allocates device memory: the caller owns inputs, outputs and scratch.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

enum GgStatus { GG_OK = 0, GG_ERR_INVALID = 1, GG_ERR_CUDA = 2, GG_ERR_UNSUPPORTED = 3 };
enum GgDtype { GG_F32 = 0, GG_BF16 = 1 };

// Sets the calling thread's error message (printf style) and returns `code`.
int gg_fail(int code, const char* fmt, ...);
// Returns GG_OK if no launch error is pending on this thread, else records it.
int gg_check_launch(const char* what);

#define GG_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return gg_fail(GG_ERR_INVALID, __VA_ARGS__);   \
  } while (0)

// Programmatic dependent launch.  Every kernel of this library is launched so that it
// may start while its predecessor in the stream is still draining: its blocks are
// scheduled (and may read data no kernel writes, such as weights) and then block in
// pdl_wait() until the predecessor has completed and its writes are visible.  A
// kernel calls pdl_wait() before it reads anything another kernel produced and
// before its first write, and pdl_trigger() once the grid that follows may be
// scheduled.  Without a predecessor launched this way both are no-ops.
// What a kernel reads BEFORE pdl_wait() must not be written by a kernel of this library that
// is directly ahead of it: weights, and the step's packed lists (positions, cache slots, row
// and tile lists, block tables, context lengths), which the host copies in before the step's
// first kernel.  Launchers say so where an argument is read that early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// True unless GOLLMGO_B200_NO_PDL is set in the environment.
bool gg_pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t gg_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gg_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
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

// Sum over the whole block in a fixed order (same result on every run).
// `red` is shared memory of at least 33 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
