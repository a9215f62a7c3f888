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
#define VX_STATUS_BAD_PARTIAL_ROW 32

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
// mbarrier helpers (shared::cta).  Every wait is bounded: after about two seconds without a
// phase flip the waiter records VX_STATUS_WAIT_TIMEOUT and gives up instead of hanging.
// ---------------------------------------------------------------------------------------------
constexpr unsigned long long VX_WAIT_CYCLES = 4000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false (and records it) if the barrier did not flip within `limit`
// cycles of the SM's clock.
__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, int* status,
                                                  unsigned long long limit) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - start > limit) {
      atomicOr(status, VX_STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
  return mbar_wait_limited(bar, parity, status, VX_WAIT_CYCLES);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Bulk copy global -> shared (16-byte aligned, size a multiple of 16) that signals `bar`.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
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

// ---------------------------------------------------------------------------------------------
// Timeline tracing, compiled in with -DVX_TRACE only (VELOX_B200_TRACE=1 at build time).  Every
// CTA appends (kernel id, grid size, block, SM, start ns, end ns) to a buffer the host set up;
// the host groups the events by launch.  A build without the flag contains none of this.
// ---------------------------------------------------------------------------------------------
#ifdef VX_TRACE
struct TraceEvent {
  unsigned long long t0, t1;
  int kernel, grid, block, sm;
  unsigned long long marks[4];  // optional points inside the kernel, 0 if never reached
};
// One buffer per translation unit (each .cu file is its own device module).
static __device__ TraceEvent* g_trace_events = nullptr;
static __device__ unsigned int g_trace_capacity = 0;
static __device__ unsigned int g_trace_cursor = 0;

__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct TraceScope {
  unsigned long long t0;
  unsigned long long marks[4];
  int kernel;
  __device__ __forceinline__ explicit TraceScope(int id) : t0(0), kernel(id) {
    marks[0] = marks[1] = marks[2] = marks[3] = 0;
    if (threadIdx.x == 0) t0 = trace_now();
  }
  __device__ __forceinline__ void mark(int i) {
    if (threadIdx.x == 0) marks[i] = trace_now();
  }
  // A figure of the kernel's own (cycles spent in a phase, say) in the place of a time.
  __device__ __forceinline__ void set(int i, unsigned long long value) {
    if (threadIdx.x == 0) marks[i] = value;
  }
  __device__ __forceinline__ ~TraceScope() {
    if (threadIdx.x != 0 || g_trace_events == nullptr) return;
    const unsigned int slot = atomicAdd(&g_trace_cursor, 1u);
    if (slot >= g_trace_capacity) return;
    unsigned int sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    TraceEvent e;
    e.t0 = t0;
    e.t1 = trace_now();
    e.kernel = kernel;
    e.grid = (int)(gridDim.x * gridDim.y * gridDim.z);
    e.block = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
    e.sm = (int)sm;
    for (int i = 0; i < 4; ++i) e.marks[i] = marks[i];
    g_trace_events[slot] = e;
  }
};
#define VX_TRACE_SCOPE(id) vx::TraceScope vx_trace_scope_(id)
#define VX_TRACE_MARK(i) vx_trace_scope_.mark(i)
#define VX_TRACE_SET(i, value) vx_trace_scope_.set(i, value)
#else
#define VX_TRACE_SCOPE(id)
#define VX_TRACE_MARK(i)
#define VX_TRACE_SET(i, value)
#endif

}  // namespace vx

#ifdef VX_TRACE
// Host side of the trace: point this library's kernels at a device buffer of 64-byte events.
#define VX_TRACE_API(prefix)                                                                      \
  VX_API int prefix##_trace_setup(void* events, unsigned int capacity) {                          \
    vx::TraceEvent* p = (vx::TraceEvent*)events;                                                  \
    unsigned int zero = 0;                                                                        \
    cudaError_t e = cudaMemcpyToSymbol(vx::g_trace_events, &p, sizeof(p));                        \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(vx::g_trace_capacity, &capacity, sizeof(capacity)); \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(vx::g_trace_cursor, &zero, sizeof(zero));         \
    return (int)e;                                                                                \
  }                                                                                               \
  VX_API int prefix##_trace_count(unsigned int* count) {                                          \
    return (int)cudaMemcpyFromSymbol(count, vx::g_trace_cursor, sizeof(unsigned int));            \
  }
#else
#define VX_TRACE_API(prefix)
#endif
