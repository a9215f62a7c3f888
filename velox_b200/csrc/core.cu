// Row-wise kernels of the model step: embedding, fused residual-add + RMSNorm, rotate-half RoPE
// fused with the K/V write into the paged cache, SwiGLU, and a float32 SIMT GEMM for the true
// 32-bit path.  All arithmetic that the engine promises in 32-bit (norm statistics, rotation,
// the residual sum, SiLU) is float32 here whatever the storage type.
//
// Formulas follow the reference engine (paths inside that project):
//   RMSNorm            src/rmsnorm.py:20-28      x * rsqrt(mean(x^2) + eps) * w
//   RoPE               src/rope_inplace.py:25-47 lo' = lo*cos - hi*sin ; hi' = lo*sin + hi*cos
//   cache write        src/paged_kv_cache.py:122-123  flat[slot] = k / v of the token
//   SwiGLU             src/mlp.py:13-15          silu(gate) * up on the halves of [T, 2I]
// The residual stream is kept in float32 (the reference adds in the model dtype,
// src/decoder_layer.py:49,54).
#include "common.cuh"

namespace vx {

// ---------------------------------------------------------------------------------------------
// Embedding: resid[t, :] = float(table[ids[t], :])
// With `fed` given, an id of -1 - r stands for "the token the sampler drew for row r of the step
// before": it is read from fed[r] here, so a step can be queued before the host has seen the
// tokens of the step before it.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ resid, int hidden, int vocab, int* status,
                             const int* __restrict__ fed, int fed_rows) {
  VX_TRACE_SCOPE(1);
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && fed != nullptr && -1 - id < fed_rows) id = fed[-1 - id];
  const bool bad = id < 0 || id >= vocab;
  if (bad) {
    if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_TOKEN_ID);
    id = 0;
  }
  const T* row = table + (size_t)id * hidden;
  float* dst = resid + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = bad ? 0.f : to_float(row[i]);
}

// ---------------------------------------------------------------------------------------------
// Fused residual add + RMSNorm.
//   v = resid[r] + delta[r]   (delta may be null)
//   if write_resid: resid[r] = v
//   out[o] = v * (1 / sqrt(mean(v^2) + eps)) * weight
// `rows` (may be null) selects the rows to normalise: out row o comes from input row rows[o].
// ---------------------------------------------------------------------------------------------
constexpr int NORM_MAX_PER_THREAD = 8;

template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const float* __restrict__ weight, float eps,
                                   T* __restrict__ out, const int* __restrict__ rows, int hidden,
                                   int write_resid) {
  __shared__ float scratch[32];
  VX_TRACE_SCOPE(2);
  allow_dependents();
  grid_dependency_wait();
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* x = resid + (size_t)r * hidden;
  const T* d = delta ? delta + (size_t)r * hidden : nullptr;
  auto value = [&](int i) { return d ? x[i] + to_float(d[i]) : x[i]; };

  // A row of up to 8 elements per thread is read once and kept in registers, and so is the
  // norm weight: nothing is fetched after the reduction.
  const bool cached = hidden <= NORM_MAX_PER_THREAD * (int)blockDim.x;
  float vals[NORM_MAX_PER_THREAD], wts[NORM_MAX_PER_THREAD];
  float ss = 0.f;
  if (cached) {
#pragma unroll
    for (int j = 0; j < NORM_MAX_PER_THREAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      vals[j] = i < hidden ? value(i) : 0.f;
      wts[j] = i < hidden ? weight[i] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < NORM_MAX_PER_THREAD; ++j) ss += vals[j] * vals[j];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = value(i);
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* y = out + (size_t)o * hidden;
  if (cached) {
#pragma unroll
    for (int j = 0; j < NORM_MAX_PER_THREAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < hidden) {
        if (write_resid) x[i] = vals[j];
        y[i] = from_float<T>(vals[j] * inv * wts[j]);
      }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = value(i);
      if (write_resid) x[i] = v;
      y[i] = from_float<T>(v * inv * weight[i]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RoPE on q (in place) and on k, fused with the write of k and v into the paged cache.
//   qkv row layout: [H*D q | G*D k | G*D v]; the first `rot` dims of every head rotate as two
//   halves (rot = 0: no rotation), cos/sin are float32 tables [max_pos, rot/2].
//   slots[t] is the flat cache index (page * page_size + offset); a negative slot skips the
//   write (padding rows).  write_cache = 0 rotates q only (a layer that reads another's cache).
//   One block per (token, head of q|k|v).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                        const float* __restrict__ cos_t,
                                        const float* __restrict__ sin_t,
                                        const int* __restrict__ slots, T* __restrict__ k_cache,
                                        T* __restrict__ v_cache, int H, int G, int D, int rot,
                                        int max_pos, long long num_slots, int write_cache,
                                        int* status) {
  VX_TRACE_SCOPE(3);
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // 0..H-1 q, H..H+G-1 k, H+G.. v
  const int half = rot >> 1;
  const bool is_q = head < H, is_k = !is_q && head < H + G;
  if (!is_q && !write_cache) return;
  int pos = positions[t];
  if (rot > 0 && (pos < 0 || pos >= max_pos)) {
    if (threadIdx.x == 0 && head == 0) atomicOr(status, VX_STATUS_BAD_POSITION);
    pos = 0;
  }
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;
  const size_t width = (size_t)(H + 2 * G) * D;
  T* row = qkv + (size_t)t * width + (size_t)head * D;
  auto load = [&](int e) { return to_float(row[e]); };

  T* dst = row;  // q is rotated in place
  if (!is_q) {
    const int slot = slots[t];
    if (slot < 0) return;
    if ((long long)slot >= num_slots) {
      if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_SLOT);
      return;
    }
    const int g = is_k ? head - H : head - H - G;
    dst = (is_k ? k_cache : v_cache) + ((size_t)slot * G + g) * D;
  }
  if (is_q || is_k) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float lo = load(i), hi = load(i + half);
      dst[i] = from_float<T>(lo * c[i] - hi * s[i]);
      dst[i + half] = from_float<T>(lo * s[i] + hi * c[i]);
    }
    // Dims that do not rotate stay where they are for q and are copied for k.
    if (is_k) {
      for (int i = rot + threadIdx.x; i < D; i += blockDim.x) dst[i] = from_float<T>(load(i));
    }
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = from_float<T>(load(i));
  }
}

// ---------------------------------------------------------------------------------------------
// 16-byte vectors of the storage type: 4 floats or 8 bfloat16.
// ---------------------------------------------------------------------------------------------
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void unpack(float (&v)[4]) const {
    v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
  }
  __device__ __forceinline__ void pack(const float (&v)[4]) { raw = make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ void unpack(float (&v)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  __device__ __forceinline__ void pack(const float (&v)[8]) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  }
};

template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* p) {
  Vec16<T> v;
  v.raw = *reinterpret_cast<const decltype(v.raw)*>(p);
  return v;
}
template <typename T>
__device__ __forceinline__ void store16(T* p, const Vec16<T>& v) {
  *reinterpret_cast<decltype(v.raw)*>(p) = v.raw;
}

// ---------------------------------------------------------------------------------------------
// The same rotation and cache write, 16 bytes at a time: one block per token, one thread per
// 16-byte chunk of the token's q|k|v row.  For head sizes, rotary widths whose half and vector
// sizes divide evenly (the launcher checks); otherwise the kernel above runs.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_vec_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                            const float* __restrict__ cos_t,
                                            const float* __restrict__ sin_t,
                                            const int* __restrict__ slots, T* __restrict__ k_cache,
                                            T* __restrict__ v_cache, int H, int G, int D, int rot,
                                            int max_pos, long long num_slots, int write_cache,
                                            int* status) {
  constexpr int N = Vec16<T>::N;
  VX_TRACE_SCOPE(3);
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int half = rot >> 1;
  const int chunks = D / N;  // per head
  int pos = positions[t];
  if (rot > 0 && (pos < 0 || pos >= max_pos)) {
    if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_POSITION);
    pos = 0;
  }
  const int slot = write_cache ? slots[t] : -1;
  const bool slot_ok = slot >= 0 && (long long)slot < num_slots;
  if (write_cache && slot >= 0 && !slot_ok && threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_SLOT);
  T* row = qkv + (size_t)t * (size_t)(H + 2 * G) * D;
  const int total = (H + 2 * G) * chunks;
  for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const int head = idx / chunks, d = (idx - head * chunks) * N;
    const bool is_q = head < H, is_k = !is_q && head < H + G;
    T* src = row + (size_t)head * D;
    T* dst = src;
    if (!is_q) {
      if (!slot_ok) continue;
      const int g = is_k ? head - H : head - H - G;
      dst = (is_k ? k_cache : v_cache) + ((size_t)slot * G + g) * D;
    }
    if ((is_q || is_k) && d < rot) {
      if (d >= half) continue;  // the high half is written with its low partner
      float lo[N], hi[N], c[N], s[N], out_lo[N], out_hi[N];
      load16(src + d).unpack(lo);
      load16(src + d + half).unpack(hi);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        c[k] = cos_t[(size_t)pos * half + d + k];
        s[k] = sin_t[(size_t)pos * half + d + k];
        out_lo[k] = lo[k] * c[k] - hi[k] * s[k];
        out_hi[k] = lo[k] * s[k] + hi[k] * c[k];
      }
      Vec16<T> a, b;
      a.pack(out_lo);
      b.pack(out_hi);
      store16(dst + d, a);
      store16(dst + d + half, b);
    } else if (!is_q) {
      store16(dst + d, load16(src + d));  // dims of k that do not rotate, and all of v
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The rotation over the whole head (rot == D), 16 bytes at a time, with no idle threads: a
// thread takes a chunk of the low half and its partner in the high half of one head (for v: the
// two chunks as they are), the angles as vectors.  Same arithmetic as the kernels above.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_pair_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                             const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                             const int* __restrict__ slots, T* __restrict__ k_cache,
                                             T* __restrict__ v_cache, int H, int G, int D, int max_pos,
                                             long long num_slots, int write_cache, int num_tokens, int* status) {
  constexpr int N = Vec16<T>::N;
  VX_TRACE_SCOPE(3);
  allow_dependents();
  grid_dependency_wait();
  const int half = D >> 1;
  const int pairs = half / N;              // per head
  const int per_token = (H + 2 * G) * pairs;
  const long long total = (long long)num_tokens * per_token;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / per_token);
    const int within = (int)(idx - (long long)t * per_token);
    const int head = within / pairs, d = (within - head * pairs) * N;
    const bool is_q = head < H, is_k = !is_q && head < H + G;
    T* src = qkv + (size_t)t * (size_t)(H + 2 * G) * D + (size_t)head * D;
    T* dst = src;
    if (!is_q) {
      if (!write_cache) continue;
      const int slot = slots[t];
      if (slot < 0) continue;
      if ((long long)slot >= num_slots) {
        if (d == 0) atomicOr(status, VX_STATUS_BAD_SLOT);
        continue;
      }
      const int g = is_k ? head - H : head - H - G;
      dst = (is_k ? k_cache : v_cache) + ((size_t)slot * G + g) * D;
    }
    const Vec16<T> a = load16(src + d), b = load16(src + d + half);
    if (is_q || is_k) {
      int pos = positions[t];
      if (pos < 0 || pos >= max_pos) {
        if (within == 0) atomicOr(status, VX_STATUS_BAD_POSITION);
        pos = 0;
      }
      float lo[N], hi[N], c[N], s[N], out_lo[N], out_hi[N];
      a.unpack(lo);
      b.unpack(hi);
      const float4* cp = reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + d);
      const float4* sp = reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + d);
#pragma unroll
      for (int v4 = 0; v4 < N / 4; ++v4) {
        const float4 cv = __ldg(cp + v4), sv = __ldg(sp + v4);
        c[4 * v4] = cv.x, c[4 * v4 + 1] = cv.y, c[4 * v4 + 2] = cv.z, c[4 * v4 + 3] = cv.w;
        s[4 * v4] = sv.x, s[4 * v4 + 1] = sv.y, s[4 * v4 + 2] = sv.z, s[4 * v4 + 3] = sv.w;
      }
#pragma unroll
      for (int k = 0; k < N; ++k) {
        out_lo[k] = lo[k] * c[k] - hi[k] * s[k];
        out_hi[k] = lo[k] * s[k] + hi[k] * c[k];
      }
      Vec16<T> ra, rb;
      ra.pack(out_lo);
      rb.pack(out_hi);
      store16(dst + d, ra);
      store16(dst + d + half, rb);
    } else {
      store16(dst + d, a);
      store16(dst + d + half, b);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i], float32 inside, one rounding.
// The vector kernel (16 bytes per thread) serves widths that are a multiple of the vector.
// ---------------------------------------------------------------------------------------------
// A thread takes SWIGLU_PER_THREAD chunks of 16 bytes, a block's width apart, and asks for all
// of its gate and up values before it computes: eight loads under way per thread.
constexpr int SWIGLU_PER_THREAD = 4;

template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
  constexpr int N = Vec16<T>::N;
  allow_dependents();
  grid_dependency_wait();
  const size_t t = blockIdx.y;
  const T* gate = gate_up + t * 2 * inter;
  const T* up = gate + inter;
  const int first = (blockIdx.x * SWIGLU_PER_THREAD * blockDim.x + threadIdx.x) * N;
  Vec16<T> gv[SWIGLU_PER_THREAD], uv[SWIGLU_PER_THREAD];
#pragma unroll
  for (int j = 0; j < SWIGLU_PER_THREAD; ++j) {
    const int i = first + j * (int)blockDim.x * N;
    if (i < inter) {
      gv[j] = load16(gate + i);
      uv[j] = load16(up + i);
    }
  }
#pragma unroll
  for (int j = 0; j < SWIGLU_PER_THREAD; ++j) {
    const int i = first + j * (int)blockDim.x * N;
    if (i >= inter) continue;
    float g[N], u[N], r[N];
    gv[j].unpack(g);
    uv[j].unpack(u);
    // The result is rounded to bfloat16 right away: the fast exponential and division (a few
    // units in the last place of float32) are far below that; float32 rows take the exact ones.
#pragma unroll
    for (int k = 0; k < N; ++k)
      r[k] = sizeof(T) == 2 ? __fdividef(g[k], 1.0f + __expf(-g[k])) * u[k] : g[k] / (1.0f + expf(-g[k])) * u[k];
    Vec16<T> o;
    o.pack(r);
    store16(out + t * inter + i, o);
  }
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total,
                              int inter) {
  allow_dependents();
  grid_dependency_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += stride) {
    const long long t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_float(gate_up[t * 2 * inter + i]);
    const float u = to_float(gate_up[t * 2 * inter + inter + i]);
    const float silu = g / (1.0f + expf(-g));
    out[idx] = from_float<T>(silu * u);
  }
}

// ---------------------------------------------------------------------------------------------
// float32 GEMM on the FP32 pipes (no tensor cores, no TF32): C[M,N] = A[M,K] * W[N,K]^T + bias.
// Every output element is summed over k = 0..K-1 in order by one thread, so a row's result does
// not depend on M or on where the row sits in the batch.
// ---------------------------------------------------------------------------------------------
constexpr int GF_BM = 64, GF_BN = 64, GF_BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                const float* __restrict__ bias, float* __restrict__ C, int M, int N, int K) {
  allow_dependents();
  grid_dependency_wait();
  __shared__ float As[GF_BK][GF_BM + 4];
  __shared__ float Ws[GF_BK][GF_BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
  const int ty = tid >> 4, tx = tid & 15;
  const int load_row = tid >> 2, load_k = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GF_BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + load_k + j;
      const int am = m0 + load_row, wn = n0 + load_row;
      As[load_k + j][load_row] = (am < M && k < K) ? A[(size_t)am * K + k] : 0.f;
      Ws[load_k + j][load_row] = (wn < N && k < K) ? W[(size_t)wn * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GF_BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * N + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

// bf16 -> float32 copy of selected rows (logits of the bfloat16 path are returned as float32).
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in,
                                        float* __restrict__ out, long long total) {
  allow_dependents();
  grid_dependency_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += stride)
    out[idx] = __bfloat162float(in[idx]);
}

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded wait: one CTA arms a barrier that nobody will ever arrive at and
// waits for it through the helper every kernel of this package waits with, with a short limit.
// The wait has to run out, set VX_STATUS_WAIT_TIMEOUT and let the kernel return normally.
// ---------------------------------------------------------------------------------------------
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_cycles, int* returned) {
  __shared__ __align__(8) uint64_t never;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&never), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const bool flipped = mbar_wait_limited(smem_u32(&never), 0u, status, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0) *returned = flipped ? 2 : 1;
}

}  // namespace vx

// =============================================================================================
// Launchers
// =============================================================================================
using namespace vx;

VX_TRACE_API(vx_core)

VX_API int vx_embed(const void* table, int dtype, const int* ids, float* resid, int num_tokens,
                    int hidden, int vocab, int* status, const int* fed, int fed_rows, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == VX_DTYPE_F32)
    launch_pdl(embed_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)table, ids, resid,
               hidden, vocab, status, fed, fed_rows);
  else
    launch_pdl(embed_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream,
               (const __nv_bfloat16*)table, ids, resid, hidden, vocab, status, fed, fed_rows);
  return (int)cudaGetLastError();
}

// The same for rows whose length is a multiple of 4: a thread takes chunks of four consecutive
// elements (16-byte loads of the residual and the weight, 8- or 16-byte loads of the delta),
// at most NORM_VEC_CHUNKS of them, kept in registers across the reduction.
constexpr int NORM_VEC_CHUNKS = 2;

template <typename T>
__device__ __forceinline__ float4 load4_as_float(const T* p);
template <>
__device__ __forceinline__ float4 load4_as_float<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T>
__device__ __forceinline__ void store4_from_float(T* p, float4 v);
template <>
__device__ __forceinline__ void store4_from_float<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4_from_float<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&a);
  raw.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       const float* __restrict__ weight, float eps,
                                       T* __restrict__ out, const int* __restrict__ rows, int hidden,
                                       int write_resid) {
  __shared__ float scratch[32];
  VX_TRACE_SCOPE(2);
  allow_dependents();
  const int chunks = hidden >> 2;
  // The weight does not depend on the kernel before.
  float4 wts[NORM_VEC_CHUNKS];
#pragma unroll
  for (int j = 0; j < NORM_VEC_CHUNKS; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    wts[j] = c < chunks ? *reinterpret_cast<const float4*>(weight + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  grid_dependency_wait();
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* x = resid + (size_t)r * hidden;
  const T* d = delta ? delta + (size_t)r * hidden : nullptr;
  float4 vals[NORM_VEC_CHUNKS];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NORM_VEC_CHUNKS; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < chunks) {
      v = *reinterpret_cast<const float4*>(x + 4 * c);
      if (d) {
        const float4 e = load4_as_float<T>(d + 4 * c);
        v.x += e.x;
        v.y += e.y;
        v.z += e.z;
        v.w += e.w;
      }
    }
    vals[j] = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* y = out + (size_t)o * hidden;
#pragma unroll
  for (int j = 0; j < NORM_VEC_CHUNKS; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < chunks) {
      const float4 v = vals[j];
      if (write_resid && d) *reinterpret_cast<float4*>(x + 4 * c) = v;
      store4_from_float<T>(y + 4 * c, make_float4(v.x * inv * wts[j].x, v.y * inv * wts[j].y,
                                                   v.z * inv * wts[j].z, v.w * inv * wts[j].w));
    }
  }
}

// The same with a few warps per row, for steps of many rows: a lane keeps its share of the row
// (chunks idx, idx + lanes, ... of four elements) in registers and has all its loads under way
// at once, the sum of squares goes through shuffles and one exchange between the row's warps,
// and a block (two rows) meets once between its loads and its stores.  (One block per row reached
// about half of the memory bandwidth at 2,048 rows: three waves of blocks that each load, meet,
// and store.)
template <typename T, int MAX_CHUNKS, int WPR>
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ weight,
                        float eps, T* __restrict__ out, const int* __restrict__ rows, int hidden, int write_resid,
                        int num_rows) {
  // WPR warps share a row (their 32 * WPR lanes take chunks idx, idx + 32 * WPR, ...):
  // fewer instructions per warp, whose chain is what a launch of one wave takes, and the weights
  // are asked for together with the row, not after the sum.
  constexpr int LANES = 32 * WPR;
  __shared__ float warp_sums[8];
  VX_TRACE_SCOPE(2);
  allow_dependents();
  grid_dependency_wait();
  const int warp = threadIdx.x >> 5;
  const int idx = threadIdx.x % LANES;
  const int o = blockIdx.x * (blockDim.x / LANES) + (threadIdx.x / LANES);
  const bool live = o < num_rows;
  const int r = live ? (rows ? rows[o] : o) : 0;
  const int chunks = live ? hidden >> 2 : 0;
  float* x = resid + (size_t)r * hidden;
  const T* d = delta ? delta + (size_t)r * hidden : nullptr;
  float4 vals[MAX_CHUNKS], w[MAX_CHUNKS];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAX_CHUNKS; ++j) {
    const int c = idx + LANES * j;
    vals[j] = c < chunks ? *reinterpret_cast<const float4*>(x + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (d) {
#pragma unroll
    for (int j = 0; j < MAX_CHUNKS; ++j) {
      const int c = idx + LANES * j;
      if (c < chunks) {
        const float4 e = load4_as_float<T>(d + 4 * c);
        vals[j].x += e.x;
        vals[j].y += e.y;
        vals[j].z += e.z;
        vals[j].w += e.w;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < MAX_CHUNKS; ++j) {
    const int c = idx + LANES * j;
    w[j] = c < chunks ? __ldg(reinterpret_cast<const float4*>(weight + 4 * c)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int j = 0; j < MAX_CHUNKS; ++j)
    ss += vals[j].x * vals[j].x + vals[j].y * vals[j].y + vals[j].z * vals[j].z + vals[j].w * vals[j].w;
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) warp_sums[warp] = ss;
  __syncthreads();
  if (!live) return;
  // The same terms in the same order in every warp of the row.
  ss = 0.f;
#pragma unroll
  for (int i = 0; i < WPR; ++i) ss += warp_sums[(warp / WPR) * WPR + i];
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* y = out + (size_t)o * hidden;
#pragma unroll
  for (int j = 0; j < MAX_CHUNKS; ++j) {
    const int c = idx + LANES * j;
    if (c < chunks) {
      const float4 v = vals[j];
      if (write_resid && d) *reinterpret_cast<float4*>(x + 4 * c) = v;
      store4_from_float<T>(y + 4 * c, make_float4(v.x * inv * w[j].x, v.y * inv * w[j].y, v.z * inv * w[j].z,
                                                   v.w * inv * w[j].w));
    }
  }
}

template <typename T, int MAX_CHUNKS, int WPR>
static void launch_rmsnorm_warp(float* resid, const void* delta, const float* weight, float eps, void* out,
                                const int* rows, int num_rows, int hidden, int write_resid, cudaStream_t stream) {
  const int rows_per_block = 8 / WPR;  // eight warps
  launch_pdl(add_rmsnorm_warp_kernel<T, MAX_CHUNKS, WPR>, dim3((num_rows + rows_per_block - 1) / rows_per_block),
             dim3(256), 0, stream, resid, (const T*)delta, weight, eps, (T*)out, rows, hidden, write_resid,
             num_rows);
}

VX_API int vx_add_rmsnorm(float* resid, const void* delta, const float* weight, float eps,
                          void* out, int dtype, const int* rows, int num_out_rows, int hidden,
                          int write_resid, cudaStream_t stream) {
  if (num_out_rows <= 0) return 0;
  const bool aligned = (reinterpret_cast<uintptr_t>(resid) & 15) == 0 && (reinterpret_cast<uintptr_t>(weight) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (reinterpret_cast<uintptr_t>(delta) & 15) == 0;
  // Many rows: a few warps per row (rows of up to 4,096 elements, whole chunks of four).  Not in
  // the float32 path: there a row's sum of squares is added up in the same order whatever the
  // step, so that results do not depend on how the work was cut.
  if (aligned && dtype == VX_DTYPE_BF16 && num_out_rows >= 256 && hidden % 4 == 0 && hidden <= 4096) {
    // Four warps a row (measured in a prefill of the 1.5B sizes: 9.1 us a launch at 2,048 rows
    // with one warp a row, 7.9 with two, 6.8 with four, 7.3 with eight; 8.5 -> 3.1 us at 512 rows).
    if (hidden <= 2048) launch_rmsnorm_warp<__nv_bfloat16, 4, 4>(resid, delta, weight, eps, out, rows, num_out_rows, hidden, write_resid, stream);
    else launch_rmsnorm_warp<__nv_bfloat16, 8, 4>(resid, delta, weight, eps, out, rows, num_out_rows, hidden, write_resid, stream);
    return (int)cudaGetLastError();
  }
  if (aligned && hidden % 4 == 0 && hidden / 4 <= 1024 * NORM_VEC_CHUNKS) {
    // One chunk of four per thread, two for rows of more than 4,096 elements.
    const int chunks = hidden / 4;
    int block = chunks <= 1024 ? chunks : (chunks + 1) / 2;
    block = (block + 31) / 32 * 32;
    if (block < 64) block = 64;
    if (dtype == VX_DTYPE_F32)
      launch_pdl(add_rmsnorm_vec_kernel<float>, dim3(num_out_rows), dim3(block), 0, stream, resid,
                 (const float*)delta, weight, eps, (float*)out, rows, hidden, write_resid);
    else
      launch_pdl(add_rmsnorm_vec_kernel<__nv_bfloat16>, dim3(num_out_rows), dim3(block), 0, stream, resid,
                 (const __nv_bfloat16*)delta, weight, eps, (__nv_bfloat16*)out, rows, hidden, write_resid);
    return (int)cudaGetLastError();
  }
  // About four elements per thread: enough loads in flight per row without starving the sum.
  int threads = ((hidden + 3) / 4 + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
  if (dtype == VX_DTYPE_F32)
    launch_pdl(add_rmsnorm_kernel<float>, dim3(num_out_rows), dim3(threads), 0, stream, 
        resid, (const float*)delta, weight, eps, (float*)out, rows, hidden, write_resid);
  else
    launch_pdl(add_rmsnorm_kernel<__nv_bfloat16>, dim3(num_out_rows), dim3(threads), 0, stream, 
        resid, (const __nv_bfloat16*)delta, weight, eps, (__nv_bfloat16*)out, rows, hidden,
        write_resid);
  return (int)cudaGetLastError();
}

VX_API int vx_rope_cache_write(void* qkv, int dtype, const int* positions, const float* cos_t,
                               const float* sin_t, const int* slots, void* k_cache,
                               void* v_cache, int num_tokens, int H, int G, int D, int rot,
                               int max_pos, long long num_slots, int write_cache, int* status,
                               cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int vec = dtype == VX_DTYPE_F32 ? 4 : 8;
  const bool aligned = (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0;
  // The whole head rotates and a half is whole vectors (of angles too): pairs of chunks.
  if (aligned && rot == D && (D / 2) % vec == 0 && (D / 2) % 4 == 0 &&
      (reinterpret_cast<uintptr_t>(cos_t) & 15) == 0 && (reinterpret_cast<uintptr_t>(sin_t) & 15) == 0) {
    const long long total = (long long)num_tokens * (H + 2 * G) * (D / 2 / vec);
    const int block = 256;
    long long blocks = (total + block - 1) / block;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == VX_DTYPE_F32)
      launch_pdl(rope_cache_write_pair_kernel<float>, dim3((int)blocks), dim3(block), 0, stream, (float*)qkv, positions,
                 cos_t, sin_t, slots, (float*)k_cache, (float*)v_cache, H, G, D, max_pos, num_slots, write_cache,
                 num_tokens, status);
    else
      launch_pdl(rope_cache_write_pair_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(block), 0, stream,
                 (__nv_bfloat16*)qkv, positions, cos_t, sin_t, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                 H, G, D, max_pos, num_slots, write_cache, num_tokens, status);
    return (int)cudaGetLastError();
  }
  if (aligned && D % vec == 0 && (rot / 2) % vec == 0) {
    const int work = (H + 2 * G) * (D / vec);
    const int block = work >= 256 ? 256 : (work + 31) / 32 * 32;
    if (dtype == VX_DTYPE_F32)
      launch_pdl(rope_cache_write_vec_kernel<float>, dim3(num_tokens), dim3(block), 0, stream,
                 (float*)qkv, positions, cos_t, sin_t, slots, (float*)k_cache, (float*)v_cache, H, G,
                 D, rot, max_pos, num_slots, write_cache, status);
    else
      launch_pdl(rope_cache_write_vec_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(block), 0,
                 stream, (__nv_bfloat16*)qkv, positions, cos_t, sin_t, slots,
                 (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, H, G, D, rot, max_pos, num_slots,
                 write_cache, status);
    return (int)cudaGetLastError();
  }
  const int threads = D >= 128 ? 64 : 32;
  const dim3 grid(num_tokens, H + 2 * G);
  if (dtype == VX_DTYPE_F32)
    launch_pdl(rope_cache_write_kernel<float>, dim3(grid), dim3(threads), 0, stream, 
        (float*)qkv, positions, cos_t, sin_t, slots, (float*)k_cache, (float*)v_cache, H, G, D,
        rot, max_pos, num_slots, write_cache, status);
  else
    launch_pdl(rope_cache_write_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, 
        (__nv_bfloat16*)qkv, positions, cos_t, sin_t, slots, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache, H, G, D, rot, max_pos, num_slots, write_cache, status);
  return (int)cudaGetLastError();
}

VX_API int vx_swiglu(const void* gate_up, void* out, int dtype, int num_tokens, int inter,
                     cudaStream_t stream) {
  const long long total = (long long)num_tokens * inter;
  if (total <= 0) return 0;
  const int vec = dtype == VX_DTYPE_F32 ? 4 : 8;
  if (inter % vec == 0 && (reinterpret_cast<uintptr_t>(gate_up) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0 && num_tokens <= 65535) {
    const int threads = 128;
    const dim3 grid((inter / vec + threads * SWIGLU_PER_THREAD - 1) / (threads * SWIGLU_PER_THREAD), num_tokens);
    if (dtype == VX_DTYPE_F32)
      launch_pdl(swiglu_vec_kernel<float>, grid, dim3(threads), 0, stream, (const float*)gate_up,
                 (float*)out, inter);
    else
      launch_pdl(swiglu_vec_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream,
                 (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter);
    return (int)cudaGetLastError();
  }
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == VX_DTYPE_F32)
    launch_pdl(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out,
                                                              total, inter);
  else
    launch_pdl(swiglu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, 
        (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, total, inter);
  return (int)cudaGetLastError();
}

VX_API int vx_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N,
                       int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
  launch_pdl(gemm_f32_kernel, dim3(grid), dim3(256), 0, stream, A, W, bias, C, M, N, K);
  return (int)cudaGetLastError();
}

VX_API int vx_cast_bf16_to_f32(const void* in, float* out, long long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_pdl(cast_bf16_to_f32_kernel, dim3((int)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)in, out, total);
  return (int)cudaGetLastError();
}

// Test entry: see bounded_wait_selftest_kernel.  `returned` (one int on the device) becomes 1
// when the wait gave up as it must, 2 if the barrier flipped.  limit_cycles is capped at the
// limit of the ordinary waits.
VX_API int vx_selftest_bounded_wait(int* status, long long limit_cycles, int* returned, cudaStream_t stream) {
  if (status == nullptr || returned == nullptr || limit_cycles <= 0) return (int)cudaErrorInvalidValue;
  unsigned long long limit = (unsigned long long)limit_cycles;
  if (limit > VX_WAIT_CYCLES) limit = VX_WAIT_CYCLES;
  bounded_wait_selftest_kernel<<<1, 64, 0, stream>>>(status, limit, returned);
  return (int)cudaGetLastError();
}
