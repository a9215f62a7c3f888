// Shared device helpers of the velox_b200 kernels (sm_100a).
//
// Conventions of every launcher in this directory:
//  * plain C ABI (`extern "C"`), raw device pointers, a `cudaStream_t` last; the return value is
//    the cudaError_t of the launch (0 = launched);
//  * `dtype` arguments: 0 = float32, 1 = bfloat16;
//  * a kernel that checks its indices never traps: it skips the bad access and sets a bit in a
//    device status word that the host reads at its next synchronisation point.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define VX_DTYPE_F32 0
#define VX_DTYPE_BF16 1

// Bits of the device status word.
#define VX_STATUS_BAD_TOKEN_ID 1
#define VX_STATUS_BAD_POSITION 2
#define VX_STATUS_BAD_SLOT 4
#define VX_STATUS_BAD_PAGE 8
#define VX_STATUS_WAIT_TIMEOUT 16

#define VX_API extern "C" __attribute__((visibility("default")))

namespace vx {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of the
// additions depends only on the block size, never on what else runs.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int num_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  if (warp == 0) {
    total = lane < num_warps ? scratch[lane] : 0.f;
    total = warp_sum(total);
    if (lane == 0) scratch[0] = total;
  }
  __syncthreads();
  total = scratch[0];
  __syncthreads();
  return total;
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of a step is launched with the attribute that
// lets it start while its predecessor in the stream is still running; it may then do work that
// does not depend on the predecessor (set up barriers, prefetch weights) and must call
// grid_dependency_wait() before it reads or writes anything another kernel of the stream
// touches.  The wait returns once the predecessor has completed and its writes are visible.
// allow_dependents() tells the scheduler that the successor may be started.
// Launched without the attribute, both calls do nothing.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void allow_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  // VELOX_B200_NO_PDL=1 launches every kernel fully serialised (for bisecting a fault).
  static const bool serialised = [] {
    const char* value = getenv("VELOX_B200_NO_PDL");
    return value != nullptr && value[0] == '1';
  }();
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = serialised ? 0 : 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

}  // namespace vx
