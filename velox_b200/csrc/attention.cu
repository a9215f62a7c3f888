// Attention over the paged KV cache, for prefill portions and decode tokens alike.
//
// Compiled once per head size: -DVX_HEAD_DIM=<D>, D a multiple of 16 up to 256.
//
// What is computed follows the reference's two Triton kernels (paths inside that project):
//   src/attention_prefill.py:62-139 and src/decode_attention.py:64-131: scores (q.k) * scale in
//   float32, -inf where the key is after the query, online softmax over key tiles, p rounded to
//   the cache dtype before the PV product, o = acc / l;
//   src/decode_attention.py:132-153,188-211: a split of the key range writes o and
//   lse = m + log l, and the merge weights the splits by exp(lse - max lse).
// How the work is cut differs.  The host lays out *work items*; every item is one tile of rows
// of one sequence against a range of keys.  A row is a (query token, query head of the group)
// pair: row = token_in_portion * group + head_in_group, so the query heads that share a KV head
// share every K/V tile they read, in prefill and in decode.  A decode token is a portion of
// length 1.  When a key range is split, every split writes normalised partial rows and their
// log-sum-exp to scratch and a merge kernel combines them.
//
// Item layout, int32[8]:
//   {seq, row_begin, row_count, kv_begin, kv_end, partial_base, merge_index, num_splits}.
//   seq < 0: the item is padding and does nothing.
//   partial_base < 0: the item covers every key its rows may see and writes the output itself.
//   otherwise partial rows go to partial_base + kv_head * row_count + r, and merge_index names
//   the merge item that lists all splits of the same rows.
// Visibility of key n to a row whose token is at absolute position pos:
//   kv_begin <= n < kv_end, n <= pos, and n > pos - window when window > 0.
// Key tiles start at multiples of the tile width from position 0, whatever kv_begin is, so the
// float32 result of an unsplit row does not depend on how the prompt was cut into portions.
//
// Kernel families (the `kind` of a launch):
//   0  attn_f32_kernel      float32, FFMA, 16 rows x 32 keys; its splits are merged by
//                           attn_merge_kernel
//   1  attn_wide_kernel     bf16, mma.sync, 64 rows: prompt portions of head sizes without a
//                           tensor-memory kernel
//   2  attn_narrow_kernel   bf16, mma.sync with keys on the M side, up to 16 rows: decode tokens
//                           and short portions; producer warp, mbarrier ring, clusters
//   3  attn_tc_kernel       bf16, tcgen05.mma with S and O in tensor memory, 128 rows: prompt
//                           portions at head size 128
// The bf16 families merge split key ranges themselves (the last CTA of an item to finish).
#include <cuda.h>

#include "common.cuh"

#include <math_constants.h>
#include <string.h>

#include <map>
#include <mutex>
#include <tuple>

#ifndef VX_HEAD_DIM
#error "compile with -DVX_HEAD_DIM=<head size>"
#endif
#if (VX_HEAD_DIM % 16) != 0 || VX_HEAD_DIM < 16 || VX_HEAD_DIM > 256
#error "head size must be a multiple of 16 between 16 and 256"
#endif

namespace vx {

constexpr int D = VX_HEAD_DIM;
// A key range is cut into at most this many splits (the merge kernel keeps their weights in
// shared memory).
constexpr int ATTN_MAX_SPLITS = 64;

struct AttnArgs {
  // Tensor maps of the K and V caches viewed as [tokens = pages * page_size, G, D], boxes of
  // [min(page_size, 64) tokens, one KV head, 64 dims], 128-byte swizzle (TMA_KV kernels only).
  CUtensorMap map_k, map_v;
  const void* q;            // [tokens, q_stride]; head h at h * D
  void* out;                // [tokens, out_stride]; head h at h * D
  const void* k_cache;      // [pages, page_size, G, D]
  const void* v_cache;
  const int* block_tables;  // [S, table_stride]
  const int* q_start;       // [S] first batch row of the sequence's portion
  const int* q_len;         // [S] tokens of the portion
  const int* kv_len;        // [S] keys in the cache once this step's tokens are written
  const int* items;         // [n, 8]
  int* status;              // device status word (bounded waits report here)
  float* partial_o;         // [rows, D]
  float* partial_lse;       // [rows], log2 units
  // Rows that partial_o / partial_lse hold when the launcher knows it (the scratch inside the
  // library); a split item whose rows would lie beyond is skipped and flagged.  0: not checked.
  int partial_capacity;
  // Fused merge (bf16 families): when a split item is done it bumps the counter of its
  // (merge item, KV head); the CTA that brings it to the number of splits merges them all.
  const int* merge_items;   // [m, 8] or null
  int* split_counters;      // [m * G], zero between steps; null: a separate kernel merges
  int q_stride, out_stride, table_stride;
  int num_kv_heads, group, page_size, window;
  // Narrow bf16 family: CTAs of a thread-block cluster that share one work item (1, 2, 4, 8).
  int cluster;
  float scale_log2;  // softmax scale * log2(e)
};

__device__ __forceinline__ bool key_visible(int n, int pos, int kv_begin, int kv_end, int window) {
  return n >= kv_begin && n < kv_end && n <= pos && (window <= 0 || n > pos - window);
}

// =============================================================================================
// float32 family: FP32 pipes only.  4 warps x 4 rows, 32 keys per tile, one key per lane.
// =============================================================================================
constexpr int F_ROWS = 16, F_RPW = 4, F_BN = 32;
constexpr int F_DV = (D + 31) / 32;  // output dims per lane

__global__ void __launch_bounds__(128) attn_f32_kernel(AttnArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  float(*q_s)[D] = reinterpret_cast<float(*)[D]>(smem_raw);
  float(*k_s)[D + 1] = reinterpret_cast<float(*)[D + 1]>(smem_raw + sizeof(float) * F_ROWS * D);
  float(*v_s)[D + 1] = k_s + F_BN;
  __shared__ const float* krow_ptr[F_BN];
  __shared__ const float* vrow_ptr[F_BN];

  allow_dependents();
  grid_dependency_wait();
  const int* item = a.items + (size_t)blockIdx.x * 8;
  const int seq = item[0];
  if (seq < 0) return;
  const int row_begin = item[1], row_count = item[2];
  const int kv_begin = item[3], kv_end = item[4], partial_base = item[5];
  const int kvh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  const int q_start = a.q_start[seq], q_len = a.q_len[seq], kv_len = a.kv_len[seq];
  const int ctx = kv_len - q_len;
  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  const float* qbase = (const float*)a.q;
  const float* kc = (const float*)a.k_cache;
  const float* vc = (const float*)a.v_cache;

  for (int idx = tid; idx < F_ROWS * D; idx += 128) {
    const int r = idx / D, d = idx - r * D;
    float v = 0.f;
    if (r < row_count) {
      const int row = row_begin + r;
      const int tok = row / a.group, hg = row - tok * a.group;
      v = qbase[(size_t)(q_start + tok) * a.q_stride + (size_t)(kvh * a.group + hg) * D + d];
    }
    q_s[r][d] = v;
  }

  float m[F_RPW], l[F_RPW], acc[F_RPW][F_DV];
  int pos[F_RPW];
#pragma unroll
  for (int i = 0; i < F_RPW; ++i) {
    m[i] = -CUDART_INF_F;
    l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < F_DV; ++j) acc[i][j] = 0.f;
    const int r = warp * F_RPW + i;
    pos[i] = r < row_count ? ctx + (row_begin + r) / a.group : -1;
  }

  for (int n0 = (kv_begin / F_BN) * F_BN; n0 < kv_end; n0 += F_BN) {
    __syncthreads();
    if (tid < F_BN) {
      const int n = n0 + tid;
      const float* kp = nullptr;
      const float* vp = nullptr;
      if (n < kv_end) {
        const int page = table[n / a.page_size];
        const size_t slot = (size_t)page * a.page_size + (n % a.page_size);
        kp = kc + (slot * a.num_kv_heads + kvh) * D;
        vp = vc + (slot * a.num_kv_heads + kvh) * D;
      }
      krow_ptr[tid] = kp;
      vrow_ptr[tid] = vp;
    }
    __syncthreads();
    for (int idx = tid; idx < F_BN * D; idx += 128) {
      const int j = idx / D, d = idx - j * D;
      k_s[j][d] = krow_ptr[j] ? krow_ptr[j][d] : 0.f;
      v_s[j][d] = vrow_ptr[j] ? vrow_ptr[j][d] : 0.f;
    }
    __syncthreads();

#pragma unroll
    for (int i = 0; i < F_RPW; ++i) {
      const int r = warp * F_RPW + i;
      if (pos[i] < 0) continue;
      float s = 0.f;
      for (int d = 0; d < D; ++d) s = fmaf(q_s[r][d], k_s[lane][d], s);
      s *= a.scale_log2;
      const int n = n0 + lane;
      if (!key_visible(n, pos[i], kv_begin, kv_end, a.window)) s = -CUDART_INF_F;
      const float m_new = fmaxf(m[i], warp_max(s));
      const float m_safe = m_new == -CUDART_INF_F ? 0.f : m_new;
      const float p = exp2f(s - m_safe);
      const float alpha = exp2f(m[i] - m_safe);
      l[i] = l[i] * alpha + warp_sum(p);
#pragma unroll
      for (int j = 0; j < F_DV; ++j) acc[i][j] *= alpha;
      for (int kk = 0; kk < F_BN; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, p, kk);
#pragma unroll
        for (int j = 0; j < F_DV; ++j) {
          const int d = lane + 32 * j;
          if (d < D) acc[i][j] = fmaf(pk, v_s[kk][d], acc[i][j]);
        }
      }
      m[i] = m_new;
    }
  }

#pragma unroll
  for (int i = 0; i < F_RPW; ++i) {
    const int r = warp * F_RPW + i;
    if (r >= row_count) continue;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
    if (partial_base < 0) {
      const int row = row_begin + r;
      const int tok = row / a.group, hg = row - tok * a.group;
      float* o = (float*)a.out + (size_t)(q_start + tok) * a.out_stride +
                 (size_t)(kvh * a.group + hg) * D;
#pragma unroll
      for (int j = 0; j < F_DV; ++j) {
        const int d = lane + 32 * j;
        if (d < D) o[d] = acc[i][j] * inv;
      }
    } else {
      const size_t prow = (size_t)partial_base + (size_t)kvh * row_count + r;
#pragma unroll
      for (int j = 0; j < F_DV; ++j) {
        const int d = lane + 32 * j;
        if (d < D) a.partial_o[prow * D + d] = acc[i][j] * inv;
      }
      if (lane == 0) a.partial_lse[prow] = l[i] > 0.f ? m[i] + log2f(l[i]) : -CUDART_INF_F;
    }
  }
}

// =============================================================================================
// bfloat16 family: mma.sync m16n8k16 tensor-core tiles, float32 softmax and accumulators.
//   WIDE  : 64 rows per item; each of 4 warps owns 16 rows and sees all 64 keys of a tile.
//   NARROW: 16 rows per item; each of 4 warps owns 16 keys of every 64-key tile and the warps
//           merge at the end (decode tokens and short portions; this is what gets split).
// K/V tiles arrive by bulk copies (cp.async.bulk, one per key row, completion on an mbarrier)
// into a ring of shared-memory stages, gathered row by row through the block table.
// =============================================================================================
constexpr int B_BN = 64;
constexpr int B_BN_ = 64;
constexpr int B_LD = D + 8;  // row pitch in elements: 16-byte aligned, conflict-free ldmatrix
// Head sizes that are multiples of 64 get their K/V tiles by tensor-map TMA: a tile is then D / 64
// panels of [64 keys x 128 bytes], each 128-byte swizzled (16-byte chunk c of key row r sits at
// chunk c ^ (r & 7)), which ldmatrix reads without bank conflicts and without padding.
constexpr bool TMA_KV = (D % 64) == 0;
constexpr int KV_TILE_ELEMS = TMA_KV ? B_BN_ * D : B_BN_ * (D + 8);
// Row pitch (floats) of the narrow family's cross-warp merge buffer, and its size (eight
// consumer warps).
constexpr int NARROW_MERGE_LD = D + 8;
#ifndef VX_NARROW_GROUPS
#define VX_NARROW_GROUPS 1
#endif
#ifndef VX_NARROW_SMEM_KB
#define VX_NARROW_SMEM_KB 110
#endif
constexpr size_t NARROW_MERGE_BYTES = (size_t)(VX_NARROW_GROUPS * 4 * 16 * NARROW_MERGE_LD + 2 * VX_NARROW_GROUPS * 4 * 16) * sizeof(float);
// Where the CTAs of a cluster deposit the rows this CTA owns: [16 rows][D] floats and their
// log-sum-exps, in memory nothing else uses while the kernel runs.
constexpr size_t NARROW_RECV_BYTES = (size_t)16 * D * sizeof(float) + 64;
// Dynamic shared memory of a bf16 kernel past its 1024-byte alignment: the K/V stages and the Q
// tile, which the end of the kernel reuses (cross-warp merge, merge of the splits), and for the
// narrow family the cluster's receive buffer after them.
__host__ __device__ constexpr size_t attn_tiles_bytes(bool narrow, int stages) {
  const size_t tiles = ((size_t)(narrow ? 16 : 64) * (D + 8) + (size_t)2 * stages * KV_TILE_ELEMS) *
                       sizeof(__nv_bfloat16);
  return narrow && NARROW_MERGE_BYTES > tiles ? NARROW_MERGE_BYTES : tiles;
}
__host__ __device__ constexpr size_t attn_smem_bytes(bool narrow, int stages) {
  return attn_tiles_bytes(narrow, stages) + (narrow ? NARROW_RECV_BYTES : 0);
}
// Both families keep two CTAs on an SM.  The narrow family has one group of four consumer warps
// and as many stages as fit in half an SM's shared memory (three at head size 128): a decode
// step of 8 sequences x 2 KV heads then runs as 16 clusters of 8 CTAs on 128 SMs, where one CTA
// per SM with two groups and twice the stages fitted only 15 such clusters on the GPU (a
// cluster lives inside one GPC) and streamed from 64 SMs (measured: 1.73 -> 1.66 ms per step).
// VX_NARROW_GROUPS / VX_NARROW_SMEM_KB are the two knobs.
constexpr int WIDE_STAGES = 2;
constexpr int narrow_stages() {
  const size_t stage = (size_t)2 * KV_TILE_ELEMS * sizeof(__nv_bfloat16);
  const size_t budget = (size_t)VX_NARROW_SMEM_KB * 1024 - (size_t)16 * (D + 8) * sizeof(__nv_bfloat16) - NARROW_RECV_BYTES;
  const size_t n = budget / stage;
  return n > 8 ? 8 : (n < 2 ? 2 : (int)n);
}
constexpr int NARROW_STAGES = narrow_stages();

// Address of the 16-byte chunk holding dims [d, d + 8) of key row r in a K or V tile.
__device__ __forceinline__ const __nv_bfloat16* kv_chunk(const __nv_bfloat16* tile, int r, int d) {
  if (TMA_KV) {
    const int panel = d >> 6, chunk = (d & 63) >> 3;
    return tile + panel * (B_BN_ * 64) + r * 64 + ((chunk ^ (r & 7)) << 3);
  }
  return tile + r * (D + 8) + d;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Called by `threads` threads numbered tid = 0 .. threads - 1.
template <int ROWS>
__device__ __forceinline__ void load_q_tile(const AttnArgs& a, __nv_bfloat16* q_s, int q_start,
                                            int row_begin, int row_count, int kvh, int tid,
                                            int threads) {
  constexpr int CH = D / 8;
  const __nv_bfloat16* qbase = (const __nv_bfloat16*)a.q;
  for (int idx = tid; idx < ROWS * CH; idx += threads) {
    const int r = idx / CH, c = idx - r * CH;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < row_count) {
      const int row = row_begin + r;
      const int tok = row / a.group, hg = row - tok * a.group;
      v = *reinterpret_cast<const uint4*>(qbase + (size_t)(q_start + tok) * a.q_stride +
                                          (size_t)(kvh * a.group + hg) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(q_s + r * B_LD + c * 8) = v;
  }
}

// Block-table entries of an item's key range are copied to shared memory once, so that the
// loads of a tile do not wait for a table lookup first.
constexpr int TABLE_CAP = 1024;

// Requests keys [n0, n0 + 64) of one KV head into k_s / v_s: thread j < 64 asks the copy engine
// for key row j (a row of one KV head is D * 2 contiguous bytes in the cache; one bulk copy for
// K and one for V) and arrives on the stage's mbarrier with the bytes it expects; a row at or
// past kv_end is zeroed by the thread itself.  The barrier (64 arrivals) flips when all rows
// are in.  Called by every thread; threads 64.. do nothing.
__device__ __forceinline__ void request_kv_tile(const AttnArgs& a, __nv_bfloat16* k_s,
                                                __nv_bfloat16* v_s, uint32_t bar, const int* table,
                                                const int* table_s, int first_block, int n0,
                                                int kv_end, int kvh) {
  constexpr uint32_t ROW_BYTES = D * 2;
  const int j = threadIdx.x;
  if (j >= B_BN) return;
  const int n = n0 + j;
  __nv_bfloat16* kd = k_s + j * B_LD;
  __nv_bfloat16* vd = v_s + j * B_LD;
  if (n < kv_end) {
    const int block = n / a.page_size;
    const int local = block - first_block;
    const int page = local < TABLE_CAP ? table_s[local] : table[block];
    const size_t off =
        (((size_t)page * a.page_size + (n - block * a.page_size)) * a.num_kv_heads + kvh) * D;
    // The stage was read through ldmatrix before: order those reads before the engine's writes.
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_expect_tx(bar, 2 * ROW_BYTES);
    bulk_copy_g2s(smem_u32(kd), (const __nv_bfloat16*)a.k_cache + off, ROW_BYTES, bar);
    bulk_copy_g2s(smem_u32(vd), (const __nv_bfloat16*)a.v_cache + off, ROW_BYTES, bar);
  } else {
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
      *reinterpret_cast<uint4*>(kd + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(vd + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    mbar_arrive(bar);
  }
}

// The same tile by tensor-map TMA (TMA_KV head sizes): one thread asks for every page of the
// tile, per panel of 64 dims, for K and for V: boxes of [page rows x 128 bytes].  Rows past the
// sequence come from whatever page the table names there (the reserved zero page beyond the
// sequence's own pages); they are masked in the softmax.  The barrier takes one arrival.
__device__ __forceinline__ void request_kv_tile_tma(const AttnArgs& a, __nv_bfloat16* k_s,
                                                    __nv_bfloat16* v_s, uint32_t bar,
                                                    const int* table, const int* table_s,
                                                    int first_block, int last_block, int n0,
                                                    int kvh) {
  if (threadIdx.x != 0) return;
  const int box_rows = a.page_size < B_BN ? a.page_size : B_BN;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  mbar_expect_tx(bar, 2u * B_BN * D * 2u);
  for (int r = 0; r < B_BN; r += box_rows) {
    const int n = n0 + r;
    const int block = n / a.page_size;
    int page = 0;  // past the sequence: the reserved page
    if (block <= last_block) {
      const int local = block - first_block;
      page = local < TABLE_CAP ? table_s[local] : table[block];
    }
    const int token = page * a.page_size + (n - block * a.page_size);
#pragma unroll
    for (int panel = 0; panel < D / 64; ++panel) {
      const uint32_t k_dst = smem_u32(k_s + panel * (B_BN * 64) + r * 64);
      const uint32_t v_dst = smem_u32(v_s + panel * (B_BN * 64) + r * 64);
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
          "[%0], [%1, {%2, %3, %4}], [%5];"
          ::"r"(k_dst), "l"(reinterpret_cast<uint64_t>(&a.map_k)), "r"(panel * 64), "r"(kvh),
            "r"(token), "r"(bar)
          : "memory");
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
          "[%0], [%1, {%2, %3, %4}], [%5];"
          ::"r"(v_dst), "l"(reinterpret_cast<uint64_t>(&a.map_v)), "r"(panel * 64), "r"(kvh),
            "r"(token), "r"(bar)
          : "memory");
    }
  }
}

// One warp: S[16 rows x NT*8 keys] = Q[16 x D] * K^T, keys key0.. of the tile in smem.
template <int NT>
__device__ __forceinline__ void warp_qk(float (&s)[NT][4], const __nv_bfloat16* q_rows,
                                        const __nv_bfloat16* k_s, int key0, int lane) {
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t qa[4];
    ldmatrix_x4(qa, q_rows + (lane & 15) * B_LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      uint32_t kb[4];
      const int jm = lane >> 3;
      ldmatrix_x4(kb, kv_chunk(k_s, key0 + j * 8 + (jm >> 1) * 8 + (lane & 7),
                               kk * 16 + (jm & 1) * 8));
      mma_bf16(s[j], qa, kb[0], kb[1]);
      mma_bf16(s[j + 1], qa, kb[2], kb[3]);
    }
  }
}

// One warp: O[16 x D] += P[16 x NT*8] * V[NT*8 x D]; P comes from the score registers.
template <int NT>
__device__ __forceinline__ void warp_pv(float (&o)[D / 8][4], const float (&p)[NT][4],
                                        const __nv_bfloat16* v_s, int key0, int lane) {
#pragma unroll
  for (int ks = 0; ks < NT / 2; ++ks) {
    uint32_t pa[4];
    pa[0] = pack_bf16(p[2 * ks][0], p[2 * ks][1]);
    pa[1] = pack_bf16(p[2 * ks][2], p[2 * ks][3]);
    pa[2] = pack_bf16(p[2 * ks + 1][0], p[2 * ks + 1][1]);
    pa[3] = pack_bf16(p[2 * ks + 1][2], p[2 * ks + 1][3]);
#pragma unroll
    for (int jd = 0; jd < D / 8; jd += 2) {
      uint32_t vb[4];
      const int jm = lane >> 3;
      ldmatrix_x4_trans(vb, kv_chunk(v_s, key0 + ks * 16 + (jm & 1) * 8 + (lane & 7),
                                     jd * 8 + (jm >> 1) * 8));
      mma_bf16(o[jd], pa, vb[0], vb[1]);
      mma_bf16(o[jd + 1], pa, vb[2], vb[3]);
    }
  }
}

// Masks, online softmax and rescale for the two rows (g, g + 8) a thread holds.
template <int NT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&o)[D / 8][4],
                                             float (&m)[2], float (&l)[2], const int (&pos)[2],
                                             int nbase, int kv_begin, int kv_end, int window,
                                             float scale_log2, int lane) {
  float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int n = nbase + j * 8 + 2 * (lane & 3) + (e & 1);
      const int h = e >> 1;
      float v = s[j][e] * scale_log2;
      if (pos[h] < 0 || !key_visible(n, pos[h], kv_begin, kv_end, window)) v = -CUDART_INF_F;
      s[j][e] = v;
      mx[h] = fmaxf(mx[h], v);
    }
  float alpha[2], m_safe[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    const float m_new = fmaxf(m[h], mx[h]);
    m_safe[h] = m_new == -CUDART_INF_F ? 0.f : m_new;
    alpha[h] = exp2f(m[h] - m_safe[h]);
    m[h] = m_new;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int h = e >> 1;
      const float p = exp2f(s[j][e] - m_safe[h]);
      s[j][e] = p;
      sum[h] += p;
    }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
    sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
    l[h] = l[h] * alpha[h] + sum[h];
  }
#pragma unroll
  for (int jd = 0; jd < D / 8; ++jd) {
    o[jd][0] *= alpha[0];
    o[jd][1] *= alpha[0];
    o[jd][2] *= alpha[1];
    o[jd][3] *= alpha[1];
  }
}

// Writes the two rows a thread holds, to the output (bf16) or to the partial scratch (f32).
__device__ __forceinline__ void store_rows(const AttnArgs& a, const float (&o)[D / 8][4],
                                           const float (&m)[2], const float (&l)[2], int r0,
                                           int row_begin, int row_count, int q_start, int kvh,
                                           int partial_base, int lane) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = r0 + (lane >> 2) + 8 * h;
    if (r >= row_count) continue;
    const float inv = l[h] > 0.f ? 1.0f / l[h] : 0.f;
    if (partial_base < 0) {
      const int row = row_begin + r;
      const int tok = row / a.group, hg = row - tok * a.group;
      __nv_bfloat16* dst = (__nv_bfloat16*)a.out + (size_t)(q_start + tok) * a.out_stride +
                           (size_t)(kvh * a.group + hg) * D;
#pragma unroll
      for (int jd = 0; jd < D / 8; ++jd)
        *reinterpret_cast<__nv_bfloat162*>(dst + jd * 8 + 2 * (lane & 3)) =
            __floats2bfloat162_rn(o[jd][2 * h] * inv, o[jd][2 * h + 1] * inv);
    } else {
      const size_t prow = (size_t)partial_base + (size_t)kvh * row_count + r;
      float* dst = a.partial_o + prow * D;
#pragma unroll
      for (int jd = 0; jd < D / 8; ++jd)
        *reinterpret_cast<float2*>(dst + jd * 8 + 2 * (lane & 3)) =
            make_float2(o[jd][2 * h] * inv, o[jd][2 * h + 1] * inv);
      if ((lane & 3) == 0)
        a.partial_lse[prow] = l[h] > 0.f ? m[h] + log2f(l[h]) : -CUDART_INF_F;
    }
  }
}

// =============================================================================================
// Merge of split key ranges.  Merge item, int32[8]:
//   {seq, row_begin, row_count, first_partial_base, num_splits, split_stride, -, -}
// split s of the item wrote its rows at first_partial_base + s * split_stride.
// merge_row is called by all threads of a block for one row r of an item.
// =============================================================================================
template <typename T>
__device__ __forceinline__ void merge_row(const AttnArgs& a, const int* item, int kvh, int r,
                                          float* weight_s, float* denom_s) {
  const int seq = item[0], row_begin = item[1], row_count = item[2], first = item[3],
            splits = item[4], stride = item[5];
  const size_t base = (size_t)first + (size_t)kvh * row_count + r;
  // Weights of the splits from their log-sum-exps (warp 0), then every thread sums its dims.
  if (threadIdx.x < 32) {
    float mt = -CUDART_INF_F;
    for (int s = threadIdx.x; s < splits; s += 32)
      mt = fmaxf(mt, __ldcg(&a.partial_lse[base + (size_t)s * stride]));
    mt = warp_max(mt);
    const float m_safe = mt == -CUDART_INF_F ? 0.f : mt;
    float den = 0.f;
    for (int s = threadIdx.x; s < splits; s += 32) {
      const float lse = __ldcg(&a.partial_lse[base + (size_t)s * stride]);
      const float w = lse == -CUDART_INF_F ? 0.f : exp2f(lse - m_safe);
      weight_s[s] = w;
      den += w;
    }
    den = warp_sum(den);
    if (threadIdx.x == 0) *denom_s = den;
  }
  __syncthreads();
  const float den = *denom_s;
  const int row = row_begin + r;
  const int tok = row / a.group, hg = row - tok * a.group;
  T* dst = (T*)a.out + (size_t)(a.q_start[seq] + tok) * a.out_stride +
           (size_t)(kvh * a.group + hg) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
      const float o0 = __ldcg(&a.partial_o[(base + (size_t)s * stride) * D + d]);
      const float o1 = __ldcg(&a.partial_o[(base + (size_t)(s + 1) * stride) * D + d]);
      const float o2 = __ldcg(&a.partial_o[(base + (size_t)(s + 2) * stride) * D + d]);
      const float o3 = __ldcg(&a.partial_o[(base + (size_t)(s + 3) * stride) * D + d]);
      acc += weight_s[s] * o0;
      acc += weight_s[s + 1] * o1;
      acc += weight_s[s + 2] * o2;
      acc += weight_s[s + 3] * o3;
    }
    for (; s < splits; ++s)
      acc += weight_s[s] * __ldcg(&a.partial_o[(base + (size_t)s * stride) * D + d]);
    dst[d] = from_float<T>(den > 0.f ? acc / den : 0.f);
  }
  __syncthreads();  // weight_s is reused for the next row
}

template <typename T>
__global__ void attn_merge_kernel(AttnArgs a, const int* __restrict__ merge_items) {
  __shared__ float weight_s[ATTN_MAX_SPLITS];
  __shared__ float denom_s;
  VX_TRACE_SCOPE(22);
  allow_dependents();
  grid_dependency_wait();
  const int* item = merge_items + (size_t)blockIdx.x * 8;
  if (item[0] < 0) return;
  const int r = blockIdx.z;  // one block per row of the tile
  if (r >= item[2]) return;
  merge_row<T>(a, item, blockIdx.y, r, weight_s, &denom_s);
}

// All threads of a CTA (128) merge one (merge item, KV head), sixteen rows at a time.  What
// bounds the merge is the latency of reading what other SMs have just written (about 2 us a
// round trip), so everything is asked for at once: the partial rows of as many splits as fit
// come into shared memory by bulk copies (a split's rows are contiguous), the splits' weights
// are computed from the log-sum-exps meanwhile (a warp per row), and the sum runs from shared
// memory.  `scratch`: SMEM_BYTES of shared memory nobody else uses any more; `bar`: an
// initialised mbarrier (count 1) in phase 0 that only the merge uses.  Called by every thread
// of the CTA; threads past the first 128 only keep the barriers company.
struct MergeItem {
  int row_begin, rows, first, splits, stride, q_start;
};

// The same for taller tiles (up to 128 rows): sixteen rows a round would be eight round trips one
// after the other, so here every thread reads the splits' rows straight from memory, many
// 16-byte loads in flight at a time; only the weights go through shared memory.
// `scratch` holds at least rows * splits floats.
__device__ __forceinline__ void merge_tall_item_by_cta(const AttnArgs& a, const MergeItem& item, int kvh,
                                                       float* scratch) {
  const int row_begin = item.row_begin, rows = item.rows, splits = item.splits, stride = item.stride;
  const size_t base0 = (size_t)item.first + (size_t)kvh * rows;
  constexpr int VEC = D / 4;
  float* weights = scratch;  // [rows][splits]
  __syncthreads();           // nobody uses the scratch for anything else any more
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    float mt = -CUDART_INF_F;
    for (int s = 0; s < splits; ++s) mt = fmaxf(mt, __ldcg(&a.partial_lse[base0 + r + (size_t)s * stride]));
    const float m_safe = mt == -CUDART_INF_F ? 0.f : mt;
    float den = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float lse = __ldcg(&a.partial_lse[base0 + r + (size_t)s * stride]);
      const float w = lse == -CUDART_INF_F ? 0.f : exp2f(lse - m_safe);
      weights[r * splits + s] = w;
      den += w;
    }
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    for (int s = 0; s < splits; ++s) weights[r * splits + s] *= inv;
  }
  __syncthreads();
  constexpr int UNROLL = 4;
  const int total = rows * VEC;
  for (int idx0 = threadIdx.x; idx0 < total; idx0 += blockDim.x * UNROLL) {
    float4 acc[UNROLL];
    int row_of[UNROLL], col_of[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int idx = idx0 + u * blockDim.x;
      acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      row_of[u] = idx < total ? idx / VEC : -1;
      col_of[u] = idx - (idx / VEC) * VEC;
    }
    for (int s = 0; s < splits; ++s) {
      float4 v[UNROLL];
      float w[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const bool on = row_of[u] >= 0;
        v[u] = on ? __ldcg(reinterpret_cast<const float4*>(
                        a.partial_o + (base0 + row_of[u] + (size_t)s * stride) * D + 4 * col_of[u]))
                  : make_float4(0.f, 0.f, 0.f, 0.f);
        w[u] = on ? weights[row_of[u] * splits + s] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        acc[u].x += w[u] * v[u].x;
        acc[u].y += w[u] * v[u].y;
        acc[u].z += w[u] * v[u].z;
        acc[u].w += w[u] * v[u].w;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (row_of[u] < 0) continue;
      const int row = row_begin + row_of[u];
      const int tok = row / a.group, hg = row - tok * a.group;
      __nv_bfloat16* dst = (__nv_bfloat16*)a.out + (size_t)(item.q_start + tok) * a.out_stride +
                           (size_t)(kvh * a.group + hg) * D + 4 * col_of[u];
      *reinterpret_cast<uint2*>(dst) =
          make_uint2(pack_bf16(acc[u].x, acc[u].y), pack_bf16(acc[u].z, acc[u].w));
    }
  }
}

template <int SMEM_BYTES>
__device__ __forceinline__ void merge_item_by_cta(const AttnArgs& a, const MergeItem& item, int kvh,
                                                  float* scratch, uint64_t* bar) {
  static_assert(SMEM_BYTES >= 4096 + 16 * D * 4, "no room for one split's rows");
  constexpr int STAGE_BYTES = SMEM_BYTES - 4096;
  const int row_begin = item.row_begin, rows = item.rows, first = item.first,
            splits = item.splits, stride = item.stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int VEC = D / 4;                  // float4 columns of a row
  constexpr int E = (16 * VEC + 127) / 128;   // columns a thread owns per pass
  float* weights = scratch;                   // [16][64]
  float* stage = scratch + 1024;              // [splits of a round][nrows][D]
  const int q_start = item.q_start;
  uint32_t parity = 0;
  for (int r0 = 0; r0 < rows; r0 += 16) {
    const int nrows = min(16, rows - r0);
    const size_t base0 = (size_t)first + (size_t)kvh * rows + r0;
    const uint32_t split_bytes = (uint32_t)nrows * D * 4;
    const int per_round = min(splits, STAGE_BYTES / (int)split_bytes);
    const int total = nrows * VEC;
    float4 acc[E];
    int row_of[E], col_of[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const int idx = (int)threadIdx.x + 128 * e;
      acc[e] = make_float4(0.f, 0.f, 0.f, 0.f);
      row_of[e] = idx < total && threadIdx.x < 128 ? idx / VEC : -1;
      col_of[e] = idx - (idx / VEC) * VEC;
    }
    for (int s0 = 0; s0 < splits; s0 += per_round) {
      const int ns = min(per_round, splits - s0);
      __syncthreads();  // nobody reads the staging area (or the weights) of the round before
      if (warp == 0) {
        // The rows were written through the generic proxy, here and by other CTAs.
        asm volatile("fence.proxy.async;" ::: "memory");
        if (lane == 0) mbar_expect_tx(smem_u32(bar), (uint32_t)ns * split_bytes);
        __syncwarp();
        for (int i = lane; i < ns; i += 32)
          bulk_copy_g2s(smem_u32(stage + (size_t)i * nrows * D),
                        a.partial_o + (base0 + (size_t)(s0 + i) * stride) * D, split_bytes,
                        smem_u32(bar));
      }
      if (s0 == 0) {
        float lse0[4], lse1[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = warp + 4 * j;
          const bool valid = r < nrows && warp < 4;
          lse0[j] = valid && lane < splits
                        ? __ldcg(&a.partial_lse[base0 + r + (size_t)lane * stride])
                        : -CUDART_INF_F;
          lse1[j] = valid && lane + 32 < splits
                        ? __ldcg(&a.partial_lse[base0 + r + (size_t)(lane + 32) * stride])
                        : -CUDART_INF_F;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = warp + 4 * j;
          const float mt = warp_max(fmaxf(lse0[j], lse1[j]));
          const float m_safe = mt == -CUDART_INF_F ? 0.f : mt;
          const float w0 = lse0[j] == -CUDART_INF_F ? 0.f : exp2f(lse0[j] - m_safe);
          const float w1 = lse1[j] == -CUDART_INF_F ? 0.f : exp2f(lse1[j] - m_safe);
          const float den = warp_sum(w0 + w1);
          const float inv = den > 0.f ? 1.0f / den : 0.f;
          if (r < nrows && warp < 4) {
            weights[r * 64 + lane] = w0 * inv;
            weights[r * 64 + lane + 32] = w1 * inv;
          }
        }
        __syncthreads();
      }
      mbar_wait(smem_u32(bar), parity, a.status);  // on a timeout the status word says so
      parity ^= 1u;
      const int split_floats = nrows * D;
#pragma unroll 2
      for (int i = 0; i < ns; ++i) {
        float4 v[E];
        float w[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const bool on = row_of[e] >= 0;
          v[e] = on ? *reinterpret_cast<const float4*>(stage + (size_t)i * split_floats +
                                                       (size_t)row_of[e] * D + 4 * col_of[e])
                    : make_float4(0.f, 0.f, 0.f, 0.f);
          w[e] = on ? weights[row_of[e] * 64 + s0 + i] : 0.f;
        }
#pragma unroll
        for (int e = 0; e < E; ++e) {
          acc[e].x += w[e] * v[e].x;
          acc[e].y += w[e] * v[e].y;
          acc[e].z += w[e] * v[e].z;
          acc[e].w += w[e] * v[e].w;
        }
      }
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      if (row_of[e] < 0) continue;
      const int row = row_begin + r0 + row_of[e];
      const int tok = row / a.group, hg = row - tok * a.group;
      __nv_bfloat16* dst = (__nv_bfloat16*)a.out + (size_t)(q_start + tok) * a.out_stride +
                           (size_t)(kvh * a.group + hg) * D + 4 * col_of[e];
      *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc[e].x, acc[e].y);
      *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc[e].z, acc[e].w);
    }
  }
}

// Called by every thread of a CTA after it has written the partial rows of a split item.
// The CTA that completes the splits of its (merge item, KV head) merges them.
template <int SMEM_BYTES>
__device__ __forceinline__ void finish_split(const AttnArgs& a, int merge_index, int num_splits,
                                             const MergeItem& item, int kvh, float* scratch,
                                             uint64_t* bar) {
  __shared__ int last_s;
  __threadfence();  // this thread's partial rows are visible before the counter moves
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = a.split_counters + (size_t)merge_index * a.num_kv_heads + kvh;
    const int seen = atomicAdd(counter, 1);
    last_s = seen == num_splits - 1;
    if (last_s) *counter = 0;  // ready for the next step
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  if (item.rows > 16 && (size_t)item.rows * item.splits * 4 <= (size_t)SMEM_BYTES)
    merge_tall_item_by_cta(a, item, kvh, scratch);
  else
    merge_item_by_cta<SMEM_BYTES>(a, item, kvh, scratch, bar);
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
// Address, in the shared window of the cluster, of this CTA's `local` in the CTA of `rank`.
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
// Stores into a peer's shared memory that count their bytes on the peer's mbarrier `bar`.
__device__ __forceinline__ void send_cluster_f2(uint32_t addr, float2 v, uint32_t bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];"
               ::"r"(addr), "f"(v.x), "f"(v.y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void send_cluster_f1(uint32_t addr, float v, uint32_t bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];"
               ::"r"(addr), "f"(v), "r"(bar)
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// Wide family: 64 rows; every warp owns 16 rows and all 64 keys of a tile.  STAGES K/V tiles are
// in shared memory at a time: STAGES - 1 in flight while one is multiplied.
// ---------------------------------------------------------------------------------------------
template <int STAGES>
__global__ void __launch_bounds__(128) attn_wide_kernel(const __grid_constant__ AttnArgs a) {
  constexpr int NT = 8;
  constexpr int TILE = KV_TILE_ELEMS;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int table_s[TABLE_CAP];
  __shared__ __align__(8) uint64_t kv_full[STAGES];
  __shared__ __align__(8) uint64_t merge_bar;
  // K/V stages first (swizzled panels want 1024-byte alignment), the Q tile after them.
  unsigned char* smem_al = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __nv_bfloat16* kv_s = reinterpret_cast<__nv_bfloat16*>(smem_al);  // stage st: K at st*2*TILE, V after
  __nv_bfloat16* q_s = kv_s + STAGES * 2 * TILE;

  VX_TRACE_SCOPE(20);
  allow_dependents();
  // Before the dependency wait: only what no kernel of this step writes.  The work items, the
  // lengths and the block tables were copied in before the step's first kernel, and keys below
  // ctx (the sequence's length before this step) were written by earlier steps.
  const int* item = a.items + (size_t)blockIdx.x * 8;
  const int seq = item[0];
  if (seq < 0) return;
  const int row_begin = item[1], row_count = item[2];
  const int kv_begin = item[3], kv_end = item[4], partial_base = item[5];
  const int merge_index = item[6], num_splits = item[7];
  const bool fused_merge = partial_base >= 0 && a.split_counters != nullptr;
  const int kvh = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q_start = a.q_start[seq], q_len = a.q_len[seq], kv_len = a.kv_len[seq];
  const int ctx = kv_len - q_len;
  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  // What the merge of the splits needs is read now: a round trip to memory at the end of the
  // last CTA's life is time nothing hides.
  MergeItem merge_item = {row_begin, row_count, 0, num_splits, 0, q_start};
  if (fused_merge) {
    const int* mi = a.merge_items + (size_t)merge_index * 8;
    merge_item.first = mi[3];
    merge_item.stride = mi[5];
  }

  // Keys past the last row's position are hidden from every row of the item.
  const int last_pos = ctx + (row_begin + row_count - 1) / a.group;
  const int tile_end = min(kv_end, last_pos + 1);
  const int n_first = (kv_begin / B_BN) * B_BN;
  const int first_block = n_first / a.page_size;
  const int last_block = tile_end > 0 ? (tile_end - 1) / a.page_size : 0;
  if (n_first < tile_end) {
    const int blocks = min(TABLE_CAP, (tile_end - 1) / a.page_size - first_block + 1);
    for (int i = threadIdx.x; i < blocks; i += blockDim.x) table_s[i] = table[first_block + i];
  }
  if (threadIdx.x == 0) {
#pragma unroll
    for (int st = 0; st < STAGES; ++st) mbar_init(smem_u32(&kv_full[st]), TMA_KV ? 1 : B_BN);
    mbar_init(smem_u32(&merge_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  auto request = [&](int st, int n) {
    if (TMA_KV)
      request_kv_tile_tma(a, kv_s + st * 2 * TILE, kv_s + st * 2 * TILE + TILE,
                          smem_u32(&kv_full[st]), table, table_s, first_block, last_block, n, kvh);
    else
      request_kv_tile(a, kv_s + st * 2 * TILE, kv_s + st * 2 * TILE + TILE,
                      smem_u32(&kv_full[st]), table, table_s, first_block, n, kv_end, kvh);
  };
  // Tiles of old keys only are asked for at once, the others after the wait.
  int early = 0;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    const int n = n_first + st * B_BN;
    if (n < tile_end && n + B_BN <= ctx && early == st) {
      request(st, n);
      early = st + 1;
    }
  }
  grid_dependency_wait();
  VX_TRACE_MARK(0);
  load_q_tile<64>(a, q_s, q_start, row_begin, row_count, kvh, (int)threadIdx.x, 128);
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    const int n = n_first + st * B_BN;
    if (st >= early && n < tile_end) request(st, n);
  }
  __syncthreads();
  VX_TRACE_MARK(1);

  float o[D / 8][4];
#pragma unroll
  for (int jd = 0; jd < D / 8; ++jd)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[jd][e] = 0.f;
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
  const int row0 = warp * 16;  // first row this warp works on
  int pos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row0 + (lane >> 2) + 8 * h;
    pos[h] = r < row_count ? ctx + (row_begin + r) / a.group : -1;
  }

  int stage = 0, fill = STAGES - 1;
  uint32_t parity = 0;  // bit st: the phase of kv_full[st] that the next wait looks for
  bool alive = true;
  for (int n0 = n_first; n0 < tile_end; n0 += B_BN) {
    const int ahead = n0 + (STAGES - 1) * B_BN;
    if (ahead < tile_end) request(fill, ahead);
    if (alive) alive = mbar_wait(smem_u32(&kv_full[stage]), (parity >> stage) & 1u, a.status);
    parity ^= 1u << stage;
    if (n0 == n_first) VX_TRACE_MARK(2);
    if (alive) {
      const __nv_bfloat16* k_s = kv_s + stage * 2 * TILE;
      const __nv_bfloat16* v_s = k_s + TILE;
      float s[NT][4];
      warp_qk<NT>(s, q_s + row0 * B_LD, k_s, 0, lane);
      softmax_step<NT>(s, o, m, l, pos, n0, kv_begin, kv_end, a.window, a.scale_log2, lane);
      warp_pv<NT>(o, s, v_s, 0, lane);
    }
    __syncthreads();  // everyone is done with this stage before it is refilled
    stage = stage + 1 == STAGES ? 0 : stage + 1;
    fill = fill + 1 == STAGES ? 0 : fill + 1;
  }

  VX_TRACE_MARK(3);
  store_rows(a, o, m, l, row0, row_begin, row_count, q_start, kvh, partial_base, lane);
  if (fused_merge)
    finish_split<(int)attn_smem_bytes(false, STAGES)>(a, merge_index, num_splits, merge_item, kvh,
                                                      reinterpret_cast<float*>(smem_al), &merge_bar);
}

// ---------------------------------------------------------------------------------------------
// Narrow family: 16 rows (single decoded tokens, short portions); this is what streams the
// cache in a decode step.  Consumer warps in NARROW_GROUPS groups of four and one producer warp.
// The producer asks the copy engines for K/V tiles into a ring of STAGES stages and never
// computes; a group takes every NARROW_GROUPS-th tile, its four warps 16 keys of the tile each,
// and hands the stage back through an mbarrier when its warps have read it - there is no
// block-wide barrier in the loop.  At the end the consumer warps merge through shared memory.
// A cluster of 2, 4 or 8 such CTAs may share one work item: CTA `rank` takes a run of the
// item's key tiles, and the CTAs merge through distributed shared memory by rows.
// ---------------------------------------------------------------------------------------------
// 8x8 transpose of 16-bit elements across a warp: a thread that held (row lane / 4, columns
// 2 * (lane % 4) + {0, 1}) gets (row' = lane / 4 of the transposed matrix, columns' likewise).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}

// The tile loop of one consumer warp of the narrow family, keys on the M side of the tensor
// cores: S^T[16 keys x 8 NR rows] = K Q^T and O^T[D x 8 NR rows] += V^T P^T.  Few rows are what
// a decode step has (the query heads of one KV group), and with them on the N side eight rows
// cost one n-tile instead of a 16-row m-tile that is half padding: NR = 1 does half the
// tensor-core work of the rows-on-M form, which is what bounds this kernel on the legacy mma
// path.  Thread (g = lane / 4, q = lane % 4) holds, of an accumulator tile, keys (or dims)
// g and g + 8 of rows 8 j + 2 q + {0, 1}.
// Afterwards the warp's sums, maxima and denominators are in registers; write_rows() puts them
// into the cross-warp merge buffer.
constexpr float NARROW_RESCALE_AT = 8.0f;  // log2 units

// 2^x by the special-function unit alone: -inf gives 0.
__device__ __forceinline__ float narrow_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int NR>
struct NarrowWarp {
  float o[D / 16][NR][4];
  float m[NR][2], l[NR][2];
  int pos[NR][2];
  uint32_t qb[D / 16][2 * NR];

  __device__ __forceinline__ void init(const __nv_bfloat16* q_s, int row_begin, int row_count,
                                       int ctx, int group, int lane) {
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt)
#pragma unroll
      for (int j = 0; j < NR; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[mt][j][e] = 0.f;
#pragma unroll
    for (int j = 0; j < NR; ++j)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        m[j][i] = -CUDART_INF_F;
        l[j][i] = 0.f;
        const int r = 8 * j + 2 * (lane & 3) + i;
        pos[j][i] = r < row_count ? ctx + (row_begin + r) / group : -1;
      }
    // Q as the B operand, kept for the whole item: matrices (rows 0-7, dims lo), (rows 0-7,
    // dims hi), (rows 8-15, dims lo), (rows 8-15, dims hi) of every 16-dim step.
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t q4[4];
      ldmatrix_x4(q4, q_s + ((lane & 7) + (lane >> 4) * 8) * B_LD + kk * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int x = 0; x < 2 * NR; ++x) qb[kk][x] = q4[x];
    }
  }

  // Keys [n0 + key0, n0 + key0 + 16) of the tile in k_s / v_s.
  __device__ __forceinline__ void tile(const __nv_bfloat16* k_s, const __nv_bfloat16* v_s, int key0,
                                       int nbase, int kv_begin, int kv_end, int window,
                                       float scale_log2, int lane) {
    float s[NR][4];
#pragma unroll
    for (int j = 0; j < NR; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t ka[4];
      ldmatrix_x4(ka, kv_chunk(k_s, key0 + (lane & 15), kk * 16 + (lane >> 4) * 8));
#pragma unroll
      for (int j = 0; j < NR; ++j) mma_bf16(s[j], ka, qb[kk][2 * j], qb[kk][2 * j + 1]);
    }
    // The rows this thread holds (two per n-tile) have their keys in this thread's two halves
    // and in the eight lanes with the same lane % 4.  Most tiles lie wholly inside what every
    // row may see and need no masks (rows past the item's last are never read back: they count
    // as seeing everything).  The scores stay unscaled; the scale goes into the exponent's
    // multiply-add.  m is the maximum the exponentials refer to: it follows the true maximum
    // only when that has grown by more than 2^8 since (P then stays below 2^8, which bf16
    // holds as well as 1), so that most tiles rescale nothing.  l is this thread's share of
    // the row's sum; the lanes' shares are added up once, in write_rows().
    const int g = lane >> 2;
    bool sees_all = true;
#pragma unroll
    for (int j = 0; j < NR; ++j)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int p = pos[j][i];
        if (p >= 0)
          sees_all = sees_all && nbase >= kv_begin && nbase + 16 <= kv_end && nbase + 15 <= p &&
                     (window <= 0 || nbase > p - window);
      }
    if (!__all_sync(0xffffffffu, sees_all)) {
#pragma unroll
      for (int j = 0; j < NR; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int p = pos[j][e & 1];
          if (p >= 0 && !key_visible(nbase + g + 8 * (e >> 1), p, kv_begin, kv_end, window))
            s[j][e] = -CUDART_INF_F;
        }
    }
    float mx[NR][2];
    bool move = false;
#pragma unroll
    for (int j = 0; j < NR; ++j)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float v = fmaxf(s[j][i], s[j][i + 2]);
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
        mx[j][i] = v * scale_log2;  // the scale is positive
        move = move || mx[j][i] > m[j][i] + NARROW_RESCALE_AT ||
               (m[j][i] == -CUDART_INF_F && mx[j][i] > -CUDART_INF_F);
      }
    if (__any_sync(0xffffffffu, move)) {
      float alpha[NR][2];
#pragma unroll
      for (int j = 0; j < NR; ++j)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const bool mine = mx[j][i] > m[j][i] + NARROW_RESCALE_AT ||
                            (m[j][i] == -CUDART_INF_F && mx[j][i] > -CUDART_INF_F);
          const float m_new = mine ? mx[j][i] : m[j][i];
          alpha[j][i] = m[j][i] == -CUDART_INF_F ? 0.f : exp2f(m[j][i] - m_new);
          l[j][i] *= alpha[j][i];
          m[j][i] = m_new;
        }
#pragma unroll
      for (int mt = 0; mt < D / 16; ++mt)
#pragma unroll
        for (int j = 0; j < NR; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) o[mt][j][e] *= alpha[j][e & 1];
    }
#pragma unroll
    for (int j = 0; j < NR; ++j) {
      const float neg_m[2] = {m[j][0] == -CUDART_INF_F ? 0.f : -m[j][0],
                              m[j][1] == -CUDART_INF_F ? 0.f : -m[j][1]};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = narrow_exp2(fmaf(s[j][e], scale_log2, neg_m[e & 1]));
        s[j][e] = p;
        l[j][e & 1] += p;
      }
    }
    // P^T as the B operand: the accumulator layout, transposed eight by eight.
    uint32_t pb[NR][2];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
      pb[j][0] = movmatrix_trans(pack_bf16(s[j][0], s[j][1]));
      pb[j][1] = movmatrix_trans(pack_bf16(s[j][2], s[j][3]));
    }
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) {
      uint32_t va[4];
      ldmatrix_x4_trans(va, kv_chunk(v_s, key0 + (lane & 7) + (lane >> 4) * 8,
                                     mt * 16 + ((lane >> 3) & 1) * 8));
#pragma unroll
      for (int j = 0; j < NR; ++j) mma_bf16(o[mt][j], va, pb[j][0], pb[j][1]);
    }
  }

  // mo [16 rows][ld] sums, mm / ml [16] maxima and denominators of this warp.
  __device__ __forceinline__ void write_rows(float* mo, float* mm, float* ml, int ld, int lane) const {
    const int g = lane >> 2, q = lane & 3;
#pragma unroll
    for (int j = 0; j < NR; ++j)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = 8 * j + 2 * q + i;
        float* dst = mo + (size_t)r * ld + g;
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt) {
          dst[mt * 16] = o[mt][j][i];
          dst[mt * 16 + 8] = o[mt][j][i + 2];
        }
        float total = l[j][i];
        total += __shfl_xor_sync(0xffffffffu, total, 4);
        total += __shfl_xor_sync(0xffffffffu, total, 8);
        total += __shfl_xor_sync(0xffffffffu, total, 16);
        if (g == 0) {
          mm[r] = m[j][i];
          ml[r] = total;
        }
      }
  }
};

constexpr int NARROW_GROUPS = VX_NARROW_GROUPS;
constexpr int NARROW_TABLE_CAP = 256;  // block-table entries kept in shared memory
constexpr int NARROW_CONSUMERS = NARROW_GROUPS * 4 * 32;
constexpr int NARROW_THREADS = NARROW_CONSUMERS + 32;

// The producer warp's share of a tile: lanes issue the copies side by side.
__device__ __forceinline__ void produce_kv_tile(const AttnArgs& a, __nv_bfloat16* k_s,
                                                __nv_bfloat16* v_s, uint32_t bar, const int* table,
                                                const int* table_s, int first_block,
                                                int last_block, int n0, int kv_end, int kvh,
                                                int lane) {
  // The stage was read through ldmatrix before: order those reads before the engines' writes.
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (TMA_KV) {
    const int box_rows = a.page_size < B_BN ? a.page_size : B_BN;
    const int pages = B_BN / box_rows;
    constexpr int PANELS = D / 64 > 0 ? D / 64 : 1;
    if (lane == 0) mbar_expect_tx(bar, 2u * B_BN * D * 2u);
    __syncwarp();
    // One copy per (page, panel, K or V): lanes take them in turn.
    for (int op = lane; op < pages * PANELS * 2; op += 32) {
      const int which = op & 1, panel = (op >> 1) % PANELS, pg = (op >> 1) / PANELS;
      const int r = pg * box_rows;
      const int n = n0 + r;
      const int block = n / a.page_size;
      int page = 0;  // past the sequence: the reserved page
      if (block <= last_block) {
        const int local = block - first_block;
        page = local < NARROW_TABLE_CAP ? table_s[local] : table[block];
      }
      const int token = page * a.page_size + (n - block * a.page_size);
      const uint32_t dst = smem_u32((which ? v_s : k_s) + panel * (B_BN * 64) + r * 64);
      const CUtensorMap* map = which ? &a.map_v : &a.map_k;
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
          "[%0], [%1, {%2, %3, %4}], [%5];"
          ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(panel * 64), "r"(kvh), "r"(token),
            "r"(bar)
          : "memory");
    }
  } else {
    constexpr uint32_t ROW_BYTES = D * 2;
    // One arrival per key row (the barrier counts 64): a row in the cache comes by two bulk
    // copies, a row past the range is zeroed here.
    for (int j = lane; j < B_BN; j += 32) {
      const int n = n0 + j;
      __nv_bfloat16* kd = k_s + j * B_LD;
      __nv_bfloat16* vd = v_s + j * B_LD;
      if (n < kv_end) {
        const int block = n / a.page_size;
        const int local = block - first_block;
        const int page = local < NARROW_TABLE_CAP ? table_s[local] : table[block];
        const size_t off =
            (((size_t)page * a.page_size + (n - block * a.page_size)) * a.num_kv_heads + kvh) * D;
        mbar_expect_tx(bar, 2 * ROW_BYTES);
        bulk_copy_g2s(smem_u32(kd), (const __nv_bfloat16*)a.k_cache + off, ROW_BYTES, bar);
        bulk_copy_g2s(smem_u32(vd), (const __nv_bfloat16*)a.v_cache + off, ROW_BYTES, bar);
      } else {
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          *reinterpret_cast<uint4*>(kd + c * 8) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(vd + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
        mbar_arrive(bar);
      }
    }
  }
}

template <int STAGES>
__global__ void __launch_bounds__(NARROW_THREADS) attn_narrow_kernel(const __grid_constant__ AttnArgs a) {
  constexpr int TILE = KV_TILE_ELEMS;
  constexpr int WARPS = NARROW_GROUPS * 4;  // consumer warps
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int table_s[NARROW_TABLE_CAP];
  __shared__ __align__(8) uint64_t kv_full[STAGES];
  __shared__ __align__(8) uint64_t kv_empty[STAGES];
  __shared__ __align__(8) uint64_t merge_bar;
  __shared__ __align__(8) uint64_t recv_bar;  // cluster: the ranks' shares of this CTA's rows have arrived
  unsigned char* smem_al = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __nv_bfloat16* kv_s = reinterpret_cast<__nv_bfloat16*>(smem_al);  // stage st: K at st*2*TILE, V after
  __nv_bfloat16* q_s = kv_s + STAGES * 2 * TILE;

  VX_TRACE_SCOPE(21);
  allow_dependents();
  // Before the dependency wait: only what no kernel of this step writes (see the wide family).
  const int cluster = a.cluster;
  const int* item = a.items + (size_t)(cluster > 1 ? blockIdx.x / cluster : blockIdx.x) * 8;
  const int seq = item[0];
  if (seq < 0) return;  // padding: every CTA of the cluster leaves here
  const int row_begin = item[1], row_count = item[2];
  int kv_begin = item[3], kv_end = item[4];
  const int partial_base = item[5];
  const int merge_index = item[6], num_splits = item[7];
  const bool fused_merge = partial_base >= 0 && a.split_counters != nullptr;
  const int kvh = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q_start = a.q_start[seq], q_len = a.q_len[seq], kv_len = a.kv_len[seq];
  const int ctx = kv_len - q_len;
  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  MergeItem merge_item = {row_begin, row_count, 0, num_splits, 0, q_start};
  if (fused_merge) {
    const int* mi = a.merge_items + (size_t)merge_index * 8;
    merge_item.first = mi[3];
    merge_item.stride = mi[5];
  }

  // Keys past the last row's position are hidden from every row of the item.
  const int last_pos = ctx + (row_begin + row_count - 1) / a.group;
  if (cluster > 1) {
    // The item's key tiles, dealt out in runs: rank r gets tiles [r * per, (r + 1) * per).
    const int visible_end = min(kv_end, last_pos + 1);
    const int tile0 = kv_begin / B_BN;
    const int tiles = visible_end > kv_begin ? (visible_end + B_BN - 1) / B_BN - tile0 : 0;
    const int per = (tiles + cluster - 1) / cluster;
    const int rank = (int)cluster_rank();
    const int begin = max(kv_begin, (tile0 + rank * per) * B_BN);
    const int end = min(visible_end, (tile0 + (rank + 1) * per) * B_BN);
    kv_begin = begin;
    kv_end = max(end, begin);  // possibly empty: the CTA then contributes nothing to the merge
  }
  const int tile_end = min(kv_end, last_pos + 1);
  const int n_first = (kv_begin / B_BN) * B_BN;
  const int num_tiles = n_first < tile_end ? (tile_end - n_first + B_BN - 1) / B_BN : 0;
  const int first_block = n_first / a.page_size;
  const int last_block = tile_end > 0 ? (tile_end - 1) / a.page_size : 0;
  if (num_tiles > 0) {
    const int blocks = min(NARROW_TABLE_CAP, (tile_end - 1) / a.page_size - first_block + 1);
    for (int i = threadIdx.x; i < blocks; i += blockDim.x) table_s[i] = table[first_block + i];
  }
  if (threadIdx.x == 0) {
#pragma unroll
    for (int st = 0; st < STAGES; ++st) {
      mbar_init(smem_u32(&kv_full[st]), TMA_KV ? 1 : B_BN);
      mbar_init(smem_u32(&kv_empty[st]), 4);  // the four warps of the group that read it
    }
    mbar_init(smem_u32(&merge_bar), 1);
    mbar_init(smem_u32(&recv_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (cluster > 1) {
      // Every rank sends each row this CTA owns (rows rank, rank + cluster, ...): D floats and
      // the log-sum-exp.
      const int rank = (int)cluster_rank();
      const int owned = row_count > rank ? (row_count - rank + cluster - 1) / cluster : 0;
      mbar_expect_tx(smem_u32(&recv_bar), (uint32_t)(cluster * owned * (D * 4 + 4)));
    }
  }
  __syncthreads();
  // The one barrier of the whole cluster: "every CTA runs and its receive barrier is armed"
  // (nobody may write into a peer before).  Arrive now; the wait comes right before the first
  // remote store and costs nothing by then.
  if (cluster > 1) cluster_arrive();

  if (warp == WARPS) {
    // ------------------------------------------------------------------------------ producer
    // Tiles of old keys are asked for at once; the first tile that may hold one of this
    // step's keys waits for the kernel that writes them.
    bool waited = false, alive = true;
    int st = 0, round = 0;
    for (int t = 0; t < num_tiles; ++t) {
      const int n0 = n_first + t * B_BN;
      if (!waited && n0 + B_BN > ctx) {
        grid_dependency_wait();
        waited = true;
      }
      if (round > 0 && alive)
        alive = mbar_wait(smem_u32(&kv_empty[st]), (uint32_t)(round - 1) & 1u, a.status);
      produce_kv_tile(a, kv_s + st * 2 * TILE, kv_s + st * 2 * TILE + TILE, smem_u32(&kv_full[st]),
                      table, table_s, first_block, last_block, n0, kv_end, kvh, lane);
      if (++st == STAGES) {
        st = 0;
        ++round;
      }
    }
  } else {
    // ----------------------------------------------------------------------------- consumers
    grid_dependency_wait();
    VX_TRACE_MARK(0);
    load_q_tile<16>(a, q_s, q_start, row_begin, row_count, kvh, (int)threadIdx.x, NARROW_CONSUMERS);
    asm volatile("bar.sync 1, %0;" ::"n"(NARROW_CONSUMERS) : "memory");
    VX_TRACE_MARK(1);
  }
  // The merge buffer lies over the stages: [WARPS][16][MD] sums, then maxima and denominators.
  // Rows of up to eight (a decode token's heads of one KV group) take the form with one n-tile.
  constexpr int MD = NARROW_MERGE_LD;
  float* mo = reinterpret_cast<float*>(smem_al);  // [WARPS][16][MD]
  float* mm = mo + WARPS * 16 * MD;                 // [WARPS][16]
  float* ml = mm + WARPS * 16;                      // [WARPS][16]
  auto consume = [&](auto& state) {
    if (warp < WARPS) {
      state.init(q_s, row_begin, row_count, ctx, a.group, lane);
      const int group = warp >> 2;
      const int key0 = (warp & 3) * 16;  // the keys of a tile this warp works on
      bool alive = true;
      for (int t = group; t < num_tiles; t += NARROW_GROUPS) {
        const int st = t % STAGES, round = t / STAGES;
        const int n0 = n_first + t * B_BN;
        if (alive) alive = mbar_wait(smem_u32(&kv_full[st]), (uint32_t)round & 1u, a.status);
        if (t == group) VX_TRACE_MARK(2);
        if (alive) {
          const __nv_bfloat16* k_s = kv_s + st * 2 * TILE;
          state.tile(k_s, k_s + TILE, key0, n0 + key0, kv_begin, kv_end, a.window, a.scale_log2, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&kv_empty[st]));  // this warp has read the stage
      }
      VX_TRACE_MARK(3);
    }
    // No copy is writing the stages any more: every tile asked for has been waited for.
    __syncthreads();
    if (warp < WARPS) state.write_rows(mo + (size_t)warp * 16 * MD, mm + warp * 16, ml + warp * 16, MD, lane);
    __syncthreads();
  };
  if (row_count <= 8) {
    NarrowWarp<1> state;
    consume(state);
  } else {
    NarrowWarp<2> state;
    consume(state);
  }
  // Eight threads per row (threads 0..127); a thread takes dims 2 * seg + 16 * i, so the eight
  // cover 64 consecutive bytes of the row at a time.
  int r = threadIdx.x >> 3;
  const int seg = threadIdx.x & 7;
  bool valid = r < row_count && threadIdx.x < 128;
  float2 val[D / 16];
  float lse = -CUDART_INF_F;
  if (valid) {
    float mt = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mt = fmaxf(mt, mm[w * 16 + r]);
    const float m_safe = mt == -CUDART_INF_F ? 0.f : mt;
    float wgt[WARPS], lt = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      wgt[w] = exp2f(mm[w * 16 + r] - m_safe);
      lt += ml[w * 16 + r] * wgt[w];
    }
    const float inv = lt > 0.f ? 1.0f / lt : 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) wgt[w] *= inv;
    const float* src = mo + (size_t)r * MD + 2 * seg;
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      float2 acc = make_float2(0.f, 0.f);
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float2 v = *reinterpret_cast<const float2*>(src + (size_t)w * 16 * MD + 16 * i);
        acc.x += v.x * wgt[w];
        acc.y += v.y * wgt[w];
      }
      val[i] = acc;
    }
    lse = lt > 0.f ? mt + log2f(lt) : -CUDART_INF_F;
  }

  if (cluster > 1) {
    // Rows are dealt out to the CTAs of the cluster (row r belongs to rank r % cluster, as its
    // slot r / cluster).  Every CTA sends each of its rows to the owner; when the owner's own
    // barrier has counted all their bytes it weighs what the ranks sent by their log-sum-exps,
    // in rank order.
    const int slots = 16 / cluster;
    const uint32_t rank = cluster_rank();
    float* recv = reinterpret_cast<float*>(smem_al + attn_tiles_bytes(true, STAGES));  // [cluster][slots][D]
    float* recv_lse = recv + 16 * D;                                                    // [cluster][slots]
    cluster_wait();
    if (valid) {
      const uint32_t owner = (uint32_t)(r & (cluster - 1));
      const int slot = r / cluster;
      const uint32_t base = cluster_map(smem_u32(recv), owner);
      const uint32_t bar = cluster_map(smem_u32(&recv_bar), owner);
      const uint32_t at = base + (uint32_t)((((int)rank * slots + slot) * D + 2 * seg) * 4);
#pragma unroll
      for (int i = 0; i < D / 16; ++i) send_cluster_f2(at + 64u * i, val[i], bar);
      if (seg == 0) send_cluster_f1(base + (uint32_t)((16 * D + (int)rank * slots + slot) * 4), lse, bar);
    }
    // The owner learns from its own barrier that every rank's rows have arrived: no second
    // barrier of the whole cluster, and a CTA may end while its stores are still on their way
    // to owners that wait for them.
    mbar_wait(smem_u32(&recv_bar), 0u, a.status);
    const int slot = threadIdx.x >> 3;
    r = slot * cluster + (int)rank;
    valid = slot < slots && r < row_count;
    if (valid) {
      if constexpr (D <= 128) {
        // All loads are asked for at once (a loop over the ranks with its loads and exponentials
        // one after the other took 1.2 us here): eight slots, those past the cluster's size empty.
        constexpr int MAX_CLUSTER = 8;
        float lj[MAX_CLUSTER], w[MAX_CLUSTER];
#pragma unroll
        for (int j = 0; j < MAX_CLUSTER; ++j) lj[j] = j < cluster ? recv_lse[j * slots + slot] : -CUDART_INF_F;
        float2 part[MAX_CLUSTER][D / 16];
#pragma unroll
        for (int j = 0; j < MAX_CLUSTER; ++j) {
          const float* src = recv + (size_t)(j * slots + slot) * D + 2 * seg;
#pragma unroll
          for (int i = 0; i < D / 16; ++i)
            part[j][i] = j < cluster ? *reinterpret_cast<const float2*>(src + 16 * i) : make_float2(0.f, 0.f);
        }
        float mt = -CUDART_INF_F;
#pragma unroll
        for (int j = 0; j < MAX_CLUSTER; ++j) mt = fmaxf(mt, lj[j]);
        const float m_safe = mt == -CUDART_INF_F ? 0.f : mt;
        float den = 0.f;
#pragma unroll
        for (int j = 0; j < MAX_CLUSTER; ++j) {
          w[j] = lj[j] == -CUDART_INF_F ? 0.f : exp2f(lj[j] - m_safe);
          den += w[j];
        }
        const float inv = den > 0.f ? 1.0f / den : 0.f;
#pragma unroll
        for (int i = 0; i < D / 16; ++i) val[i] = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < MAX_CLUSTER; ++j) {
          const float wj = w[j] * inv;
#pragma unroll
          for (int i = 0; i < D / 16; ++i) {
            val[i].x += wj * part[j][i].x;
            val[i].y += wj * part[j][i].y;
          }
        }
        lse = den > 0.f ? mt + log2f(den) : -CUDART_INF_F;
      } else {
        // Heads too wide to hold every rank's share in registers: rank after rank.
        float mt = -CUDART_INF_F;
        for (int j = 0; j < cluster; ++j) mt = fmaxf(mt, recv_lse[j * slots + slot]);
        const float m_safe = mt == -CUDART_INF_F ? 0.f : mt;
        float den = 0.f;
        for (int j = 0; j < cluster; ++j) {
          const float lj = recv_lse[j * slots + slot];
          den += lj == -CUDART_INF_F ? 0.f : exp2f(lj - m_safe);
        }
        const float inv = den > 0.f ? 1.0f / den : 0.f;
#pragma unroll
        for (int i = 0; i < D / 16; ++i) val[i] = make_float2(0.f, 0.f);
        for (int j = 0; j < cluster; ++j) {
          const float lj = recv_lse[j * slots + slot];
          const float w = lj == -CUDART_INF_F ? 0.f : exp2f(lj - m_safe) * inv;
          const float* src = recv + (size_t)(j * slots + slot) * D + 2 * seg;
#pragma unroll
          for (int i = 0; i < D / 16; ++i) {
            const float2 v = *reinterpret_cast<const float2*>(src + 16 * i);
            val[i].x += w * v.x;
            val[i].y += w * v.y;
          }
        }
        lse = den > 0.f ? mt + log2f(den) : -CUDART_INF_F;
      }
    }
  }

  if (valid) {
    if (partial_base < 0) {
      const int row = row_begin + r;
      const int tok = row / a.group, hg = row - tok * a.group;
      __nv_bfloat16* dst = (__nv_bfloat16*)a.out + (size_t)(q_start + tok) * a.out_stride +
                           (size_t)(kvh * a.group + hg) * D + 2 * seg;
#pragma unroll
      for (int i = 0; i < D / 16; ++i)
        *reinterpret_cast<__nv_bfloat162*>(dst + 16 * i) = __floats2bfloat162_rn(val[i].x, val[i].y);
    } else {
      const size_t prow = (size_t)partial_base + (size_t)kvh * row_count + r;
      if (a.partial_capacity > 0 && prow >= (size_t)a.partial_capacity) {
        // The caller's count of partial rows was too small for its items: write nothing there.
        if (seg == 0) atomicOr(a.status, VX_STATUS_BAD_PARTIAL_ROW);
      } else {
        float* dst = a.partial_o + prow * D + 2 * seg;
#pragma unroll
        for (int i = 0; i < D / 16; ++i) *reinterpret_cast<float2*>(dst + 16 * i) = val[i];
        if (seg == 0) a.partial_lse[prow] = lse;
      }
    }
  }
  if (fused_merge)
    finish_split<(int)attn_smem_bytes(true, STAGES)>(a, merge_index, num_splits * cluster, merge_item,
                                                     kvh, reinterpret_cast<float*>(smem_al), &merge_bar);
}


#if VX_HEAD_DIM == 128 || VX_HEAD_DIM == 64
#define VX_HAS_TC_ATTENTION 1
// ---------------------------------------------------------------------------------------------
// Tensor-memory family (head sizes 128 and 64): prompt portions on the 5th-generation tensor cores.
// A CTA owns 128 rows (thread r of the four softmax warps owns row r, which is TMEM lane r) and
// walks the key tiles of 64:
//   S[128 x 64]   = Q K^T      tcgen05.mma, A = Q (shared, K-major, 128-byte swizzle), B = the
//                              K tile as the tensor-map copy left it; accumulator in TMEM
//   softmax       each thread reads its row of S from TMEM (no shuffles: the row is in one
//                 thread), masks, keeps the running maximum and sum, writes P as bf16 into
//                 shared memory - over the K tile, which the first product has finished with
//   O[128 x D] += P V          A = P (K-major), B = the V tile taken MN-major (keys x dims as
//                              stored); accumulator in TMEM for the whole item
// The maximum that the exponentials refer to only moves when the true maximum has grown by
// more than 2^8 since; O and the sum are then rescaled (TMEM load, multiply, store).  Between
// such moves P may reach 2^8, which bf16 holds as well as it holds 1.
// Warps 0-3 softmax and epilogue, warp 4 lane 0 the K/V producer, warp 5 lane 0 the MMA issuer
// (warp 5 owns the tensor memory).  Two CTAs fit on an SM (96 KB at head size 128 and 256 TMEM columns each), so
// one CTA's products run under the other's exponentials.
// ---------------------------------------------------------------------------------------------
constexpr int TC_ROWS = 128;
constexpr int TC_THREADS = 192;
constexpr uint32_t TC_Q_BYTES = TC_ROWS * D * 2;          // two panels of [128 rows x 128 bytes]
constexpr uint32_t TC_KV_BYTES = B_BN * D * 2;            // a K or V tile
constexpr uint32_t TC_P_BYTES = TC_ROWS * B_BN * 2;       // a P tile where it lies over the K tile
// The K tile's place in a stage also holds P (the form with P in shared memory): the larger of the two.
constexpr uint32_t TC_KP_BYTES = TC_KV_BYTES > TC_P_BYTES ? TC_KV_BYTES : TC_P_BYTES;
constexpr uint32_t TC_STAGE_BYTES = TC_KP_BYTES + TC_KV_BYTES;
__host__ __device__ constexpr size_t tc_smem_bytes(int stages) { return TC_Q_BYTES + (size_t)stages * TC_STAGE_BYTES; }
constexpr uint32_t TC_TMEM_COLS = 256;                    // S in columns 0..63, O behind it (D columns), then P
constexpr float TC_RESCALE_AT = 8.0f;                     // log2 units

__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  desc |= (uint64_t)((lbo_bytes & 0x3FFFFu) >> 4) << 16;
  desc |= (uint64_t)((sbo_bytes & 0x3FFFFu) >> 4) << 32;
  desc |= (uint64_t)1 << 46;  // descriptor version of sm_100
  desc |= (uint64_t)2 << 61;  // 128-byte swizzle
  return desc;
}

// kind::f16 instruction descriptor: D f32, A and B bf16, M = 128, N = n; b_mn: B is MN-major.
__host__ __device__ constexpr uint32_t tc_idesc(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same product with A read from tensor memory: row r of A in lane r, two bf16 to a column.
__device__ __forceinline__ void tc_mma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void tc_load32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tc_store32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
        "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
        "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
        "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
        "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
        "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Sixteen 32-bit words of this thread's lane into sixteen columns (no wait: see tc_store_wait).
__device__ __forceinline__ void tc_store16_words(uint32_t taddr, const uint32_t (&w)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]),
        "r"(w[8]), "r"(w[9]), "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15])
      : "memory");
}
__device__ __forceinline__ void tc_store_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// The K tile or the V tile (`which` 0 or 1) of keys n0 .. n0 + 63 into `dst`, by tensor-map
// copies that complete on `bar`: one per (page, panel of 64 dims), the lanes taking them in turn.
__device__ __forceinline__ void produce_tc_half(const AttnArgs& a, __nv_bfloat16* dst_s, uint32_t bar, int which,
                                                const int* table, const int* table_s, int first_block,
                                                int last_block, int n0, int kvh, int lane) {
  const int box_rows = a.page_size < B_BN ? a.page_size : B_BN;
  const int pages = B_BN / box_rows;
  constexpr int PANELS = D / 64 > 0 ? D / 64 : 1;
  if (lane == 0) mbar_expect_tx(bar, (uint32_t)B_BN * D * 2u);
  __syncwarp();
  const CUtensorMap* map = which ? &a.map_v : &a.map_k;
  for (int op = lane; op < pages * PANELS; op += 32) {
    const int panel = op % PANELS, pg = op / PANELS;
    const int r = pg * box_rows;
    const int n = n0 + r;
    const int block = n / a.page_size;
    int page = 0;  // past the sequence: the reserved page
    if (block <= last_block) {
      const int local = block - first_block;
      page = local < NARROW_TABLE_CAP ? table_s[local] : table[block];
    }
    const int token = page * a.page_size + (n - block * a.page_size);
    const uint32_t dst = smem_u32(dst_s + panel * (B_BN * 64) + r * 64);
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(panel * 64), "r"(kvh), "r"(token), "r"(bar)
        : "memory");
  }
}

// 2^x by the special-function unit alone: -inf gives 0, and the arguments here never exceed 8.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two multiply-adds, or two additions, in one instruction (the packed float32 forms of sm_100):
// the softmax threads are bound by the instructions they issue, not by a pipe.
__device__ __forceinline__ void fma_pair(float& x0, float& x1, float a0, float a1, float b, float c) {
  asm("{\n"
      ".reg .b64 ra, rb, rc, rd;\n"
      "mov.b64 ra, {%2, %3};\n"
      "mov.b64 rb, {%4, %4};\n"
      "mov.b64 rc, {%5, %5};\n"
      "fma.rn.f32x2 rd, ra, rb, rc;\n"
      "mov.b64 {%0, %1}, rd;\n"
      "}"
      : "=f"(x0), "=f"(x1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add_pair(float& s0, float& s1, float a0, float a1) {
  asm("{\n"
      ".reg .b64 ra, rs;\n"
      "mov.b64 ra, {%2, %3};\n"
      "mov.b64 rs, {%0, %1};\n"
      "add.rn.f32x2 rs, rs, ra;\n"
      "mov.b64 {%0, %1}, rs;\n"
      "}"
      : "+f"(s0), "+f"(s1)
      : "f"(a0), "f"(a1));
}

// TC_STAGES = 2: two CTAs per SM, for grids of several waves; 4: one CTA per SM with a deeper
// K/V ring, for grids where an SM gets one CTA anyway and nothing else hides the copies' latency.
// P_TMEM: the probabilities go back to tensor memory (two buffers of 32 columns, two bf16 to a
// column) and the second product reads them there; the K tile of a stage is then free as soon as
// its scores are made and the V tile as soon as its product is, each with a barrier of its own,
// so that with two stages both are asked for a tile earlier.  Without it P lies over the K tile
// in shared memory and a stage is one unit.
template <int TC_STAGES, bool P_TMEM>
__global__ void __launch_bounds__(TC_THREADS, TC_STAGES == 2 ? 2 : 1) attn_tc_kernel(const __grid_constant__ AttnArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int table_s[NARROW_TABLE_CAP];
  // kv_*: the K tile's barriers with P_TMEM, the stage's without; v_*: the V tile's (P_TMEM only).
  __shared__ __align__(8) uint64_t kv_full[TC_STAGES], kv_empty[TC_STAGES], v_full[TC_STAGES], v_empty[TC_STAGES];
  __shared__ __align__(8) uint64_t q_ready, s_ready, s_free, p_ready, pv_done, merge_bar;
  __shared__ uint32_t tmem_slot;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_addr = smem_base;
  const uint32_t stage_addr = smem_base + TC_Q_BYTES;  // stage st: K at + st * TC_STAGE_BYTES, V after
#ifdef VX_TRACE
  // Cycles of the MMA issuer: 0 waiting on barriers, 1 issuing first products, 2 second products, 3 commits.
  __shared__ long long mma_cycles[4];
  long long mma_tick = 0;
#define TC_MMA_WAIT(call) [&] { const long long from = clock64(); const bool got = (call); mma_cycles[0] += clock64() - from; return got; }()
#define TC_MMA_TICK() { mma_tick = clock64(); }
#define TC_MMA_TOCK(i) { const long long now = clock64(); mma_cycles[i] += now - mma_tick; mma_tick = now; }
#else
#define TC_MMA_WAIT(call) (call)
#define TC_MMA_TICK()
#define TC_MMA_TOCK(i)
#endif

  VX_TRACE_SCOPE(23);
  allow_dependents();
  const int* item = a.items + (size_t)blockIdx.x * 8;
  const int seq = item[0];
  if (seq < 0) return;
  const int row_begin = item[1], row_count = item[2];
  const int kv_begin = item[3], kv_end = item[4], partial_base = item[5];
  const int merge_index = item[6], num_splits = item[7];
  const bool fused_merge = partial_base >= 0 && a.split_counters != nullptr;
  const int kvh = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q_start = a.q_start[seq], q_len = a.q_len[seq], kv_len = a.kv_len[seq];
  const int ctx = kv_len - q_len;
  const int* table = a.block_tables + (size_t)seq * a.table_stride;
  MergeItem merge_item = {row_begin, row_count, 0, num_splits, 0, q_start};
  if (fused_merge) {
    const int* mi = a.merge_items + (size_t)merge_index * 8;
    merge_item.first = mi[3];
    merge_item.stride = mi[5];
  }
  const int last_pos = ctx + (row_begin + row_count - 1) / a.group;
  const int tile_end = min(kv_end, last_pos + 1);
  const int n_first = (kv_begin / B_BN) * B_BN;
  const int num_tiles = n_first < tile_end ? (tile_end - n_first + B_BN - 1) / B_BN : 0;
  const int first_block = n_first / a.page_size;
  const int last_block = tile_end > 0 ? (tile_end - 1) / a.page_size : 0;
  if (num_tiles > 0) {
    const int blocks = min(NARROW_TABLE_CAP, (tile_end - 1) / a.page_size - first_block + 1);
    for (int i = threadIdx.x; i < blocks; i += blockDim.x) table_s[i] = table[first_block + i];
  }
  if (threadIdx.x == 0) {
    for (int st = 0; st < TC_STAGES; ++st) {
      mbar_init(smem_u32(&kv_full[st]), 1);
      mbar_init(smem_u32(&kv_empty[st]), 1);
      mbar_init(smem_u32(&v_full[st]), 1);
      mbar_init(smem_u32(&v_empty[st]), 1);
    }
    mbar_init(smem_u32(&q_ready), 4);
    mbar_init(smem_u32(&s_ready), 1);
    mbar_init(smem_u32(&s_free), 4);
    mbar_init(smem_u32(&p_ready), 4);
    mbar_init(smem_u32(&pv_done), 1);
    mbar_init(smem_u32(&merge_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#ifdef VX_TRACE
    for (int i = 0; i < 4; ++i) mma_cycles[i] = 0;
#endif
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(TC_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_s = tmem_slot;         // S: 64 columns
  const uint32_t tmem_o = tmem_slot + 64u;   // O: D columns
  const uint32_t tmem_p = tmem_slot + 64u + (uint32_t)D;  // P (P_TMEM): two buffers of 32 columns
  static_assert(64 + D + 64 <= (int)TC_TMEM_COLS, "S, O and two P buffers do not fit the allocation");

  // Row state of the softmax threads (valid for warps 0-3).
  const int r = (int)threadIdx.x;  // row of the tile, TMEM lane
  float m_ref = -CUDART_INF_F, m_true = -CUDART_INF_F, l = 0.f;
  bool failed = false;

  if (warp == 4) {
    // ------------------------------------------------------------------------- K/V producer
    bool waited = false, alive = true;
    for (int t = 0; t < num_tiles; ++t) {
      const int st = t % TC_STAGES, round = t / TC_STAGES;
      const int n0 = n_first + t * B_BN;
      if (!waited && n0 + B_BN > ctx) {
        grid_dependency_wait();
        waited = true;
      }
      if (round > 0 && alive)
        alive = mbar_wait(smem_u32(&kv_empty[st]), (uint32_t)(round - 1) & 1u, a.status);
      __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_al + TC_Q_BYTES + st * TC_STAGE_BYTES);
      if (P_TMEM) {
        produce_tc_half(a, k_s, smem_u32(&kv_full[st]), 0, table, table_s, first_block, last_block, n0, kvh, lane);
        if (round > 0 && alive)
          alive = mbar_wait(smem_u32(&v_empty[st]), (uint32_t)(round - 1) & 1u, a.status);
        produce_tc_half(a, k_s + TC_KP_BYTES / 2, smem_u32(&v_full[st]), 1, table, table_s, first_block, last_block, n0,
                        kvh, lane);
      } else {
        produce_kv_tile(a, k_s, k_s + TC_KP_BYTES / 2, smem_u32(&kv_full[st]), table, table_s, first_block, last_block,
                        n0, kv_end, kvh, lane);
      }
    }
  } else if (warp == 5) {
    // --------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(smem_u32(&q_ready), 0u, a.status);
      constexpr uint32_t idesc_qk = tc_idesc(B_BN, false);
      constexpr uint32_t idesc_pv = tc_idesc(D, true);
      // S = Q K^T of tile t: eight steps of 16 dims; a panel holds 64 dims (four steps of 32 bytes).
      auto first_product = [&](int t) -> bool {
        const int st = t % TC_STAGES, round = t / TC_STAGES;
        const uint32_t k_addr = stage_addr + st * TC_STAGE_BYTES;
        if (!TC_MMA_WAIT(mbar_wait(smem_u32(&kv_full[st]), (uint32_t)round & 1u, a.status))) return false;
        // The softmax threads have S of the tile before in registers.
        if (t > 0 && !TC_MMA_WAIT(mbar_wait(smem_u32(&s_free), (uint32_t)(t - 1) & 1u, a.status))) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        TC_MMA_TICK();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t qa = q_addr + (kk >> 2) * (TC_ROWS * 128) + (kk & 3) * 32;
          const uint32_t kb = k_addr + (kk >> 2) * (B_BN * 128) + (kk & 3) * 32;
          tc_mma(tmem_s, tc_desc(qa, 0, 1024), tc_desc(kb, 0, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        TC_MMA_TOCK(1);
        tc_commit(smem_u32(&s_ready));
        if (P_TMEM) tc_commit(smem_u32(&kv_empty[st]));  // nothing else reads the K tile
        TC_MMA_TOCK(3);
        return true;
      };
      if (ok && num_tiles > 0) ok = first_product(0);
      for (int t = 0; t < num_tiles && ok; ++t) {
        const int st = t % TC_STAGES;
        const uint32_t k_addr = stage_addr + st * TC_STAGE_BYTES, v_addr = k_addr + TC_KP_BYTES;
        // The next tile's scores are made while this tile's exponentials run.
        if (t + 1 < num_tiles) ok = first_product(t + 1);
        if (!ok) break;
        ok = TC_MMA_WAIT(mbar_wait(smem_u32(&p_ready), (uint32_t)t & 1u, a.status));
        if (!ok) break;
        if (P_TMEM) {
          ok = TC_MMA_WAIT(mbar_wait(smem_u32(&v_full[st]), (uint32_t)(t / TC_STAGES) & 1u, a.status));
          if (!ok) break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        TC_MMA_TICK();
        // O += P V: four steps of 16 keys.  P lies over the K tile (one panel of [128 x 128 B])
        // or in tensor memory (eight columns a step); V is [64 keys x 128 dims]: MN-major B, 16
        // keys are two groups of eight rows (2 KB), the second 64 dims are the next panel (8 KB on).
#pragma unroll
        for (int ks = 0; ks < B_BN / 16; ++ks) {
          const uint32_t pa = k_addr + ks * 32;
          const uint32_t vb = v_addr + ks * 2048;
          if (P_TMEM)
            tc_mma_a_tmem(tmem_o, tmem_p + (uint32_t)(t & 1) * 32u + (uint32_t)ks * 8u,
                          tc_desc(vb, B_BN * 128, 1024), idesc_pv, (t > 0 || ks > 0) ? 1u : 0u);
          else
            tc_mma(tmem_o, tc_desc(pa, 0, 1024), tc_desc(vb, B_BN * 128, 1024), idesc_pv,
                   (t > 0 || ks > 0) ? 1u : 0u);
        }
        TC_MMA_TOCK(2);
        tc_commit(smem_u32(P_TMEM ? &v_empty[st] : &kv_empty[st]));
        tc_commit(smem_u32(&pv_done));
        TC_MMA_TOCK(3);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax (warps 0-3)
    grid_dependency_wait();
    // Q rows into shared memory, K-major, 128-byte swizzled: chunk c of row r at c ^ (r & 7).
    {
      const bool on = r < row_count;
      const int row = row_begin + r;
      const int tok = row / a.group, hg = row - tok * a.group;
      const __nv_bfloat16* src = (const __nv_bfloat16*)a.q + (size_t)(q_start + tok) * a.q_stride +
                                 (size_t)(kvh * a.group + hg) * D;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        const uint4 v = on ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0u, 0u, 0u, 0u);
        unsigned char* dst = smem_al + (c >> 3) * (TC_ROWS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = v;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&q_ready));
    }
    const int pos = r < row_count ? ctx + (row_begin + r) / a.group : -1;
    // The keys this row sees are vis_lo <= n < vis_lo + vis_span (none for a row past the end).
    const int vis_lo = max(kv_begin, a.window > 0 ? pos - a.window + 1 : 0);
    const unsigned vis_span = pos < 0 ? 0u : (unsigned)max(0, min(kv_end, pos + 1) - vis_lo);
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
#ifdef VX_TRACE
    // Cycles of the softmax threads' four phases, summed over the tiles (thread 0 reports them
    // in the low words of the event's marks; the high words are the MMA issuer's).
    long long phase_cycles[4] = {0, 0, 0, 0};
    long long tick = clock64();
#define TC_PHASE(i) { const long long now = clock64(); phase_cycles[i] += now - tick; tick = now; }
#else
#define TC_PHASE(i)
#endif
    for (int t = 0; t < num_tiles; ++t) {
      const int st = t % TC_STAGES;
      const int n0 = n_first + t * B_BN;
      if (!failed) failed = !mbar_wait(smem_u32(&s_ready), (uint32_t)t & 1u, a.status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      TC_PHASE(0);  // waiting for the scores
      float s[B_BN];
      {
        float half[32];
        tc_load32(tmem_s + lane_base, half);
#pragma unroll
        for (int i = 0; i < 32; ++i) s[i] = half[i];
        tc_load32(tmem_s + lane_base + 32u, half);
#pragma unroll
        for (int i = 0; i < 32; ++i) s[32 + i] = half[i];
      }
      // S is in registers: the next tile's first product may overwrite it.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_free));
      TC_PHASE(1);  // the scores into registers
      // Most tiles lie wholly inside what every row of the warp may see: no masks then.  The
      // scores stay unscaled; the scale goes into the exponent's multiply-add.
      const bool row_sees_all = pos >= 0 && n0 >= kv_begin && n0 + B_BN <= kv_end && n0 + B_BN - 1 <= pos &&
                                (a.window <= 0 || n0 > pos - a.window);
      if (!__all_sync(0xffffffffu, row_sees_all)) {
        const int rel = n0 - vis_lo;  // one unsigned compare per key: rel + i in [0, vis_span)
#pragma unroll
        for (int i = 0; i < B_BN; ++i)
          if ((unsigned)(rel + i) >= vis_span) s[i] = -CUDART_INF_F;
      }
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int i = 0; i < B_BN; i += 4) {
        mx4[0] = fmaxf(mx4[0], s[i]);
        mx4[1] = fmaxf(mx4[1], s[i + 1]);
        mx4[2] = fmaxf(mx4[2], s[i + 2]);
        mx4[3] = fmaxf(mx4[3], s[i + 3]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;  // the scale is positive
      m_true = fmaxf(m_true, mx);
      // The second product of the tile before is observed once per tile, always before this
      // thread allows the next one (the barrier's phases are then never two ahead of the
      // parity asked for): early if O has to be rescaled, else after the exponentials, by when
      // it has long finished.
      bool observed = t == 0;
      const bool move = m_true > m_ref + TC_RESCALE_AT || (m_ref == -CUDART_INF_F && m_true > -CUDART_INF_F);
      if (__any_sync(0xffffffffu, move)) {
        const float m_new = move ? m_true : m_ref;
        const float alpha = (m_ref == -CUDART_INF_F) ? 0.f : exp2f(m_ref - m_new);  // 1 if not moved
        if (t > 0) {
          // O is rescaled between two of its products: the one of the tile before is done,
          // the one of this tile waits for this thread's P.
          if (!failed) failed = !mbar_wait(smem_u32(&pv_done), (uint32_t)(t - 1) & 1u, a.status);
          observed = true;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            float o[32];
            tc_load32(tmem_o + lane_base + (uint32_t)c0, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tc_store32(tmem_o + lane_base + (uint32_t)c0, o);
          }
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        l *= alpha;
        m_ref = m_new;
      }
      const float neg_m = m_ref == -CUDART_INF_F ? 0.f : -m_ref;
      TC_PHASE(2);  // masks, maximum, rescaling
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      if (P_TMEM) {
        // This tile's buffer was last read by the product of two tiles ago, which was observed
        // (through pv_done) before this thread let the tile before go on.
        const uint32_t p_at = tmem_p + (uint32_t)(t & 1) * 32u + lane_base;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t words[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x0, x1;
            fma_pair(x0, x1, s[half * 32 + 2 * i], s[half * 32 + 2 * i + 1], a.scale_log2, neg_m);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            add_pair(sum4[2 * (i & 1)], sum4[2 * (i & 1) + 1], p0, p1);
            words[i] = pack_bf16(p0, p1);
          }
          tc_store16_words(p_at + (uint32_t)half * 16u, words);
        }
        tc_store_wait();
      } else {
        unsigned char* p_row = smem_al + TC_Q_BYTES + st * TC_STAGE_BYTES + r * 128;
#pragma unroll
        for (int c = 0; c < B_BN / 8; ++c) {
          float p[8];
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            float x0, x1;
            fma_pair(x0, x1, s[c * 8 + i], s[c * 8 + i + 1], a.scale_log2, neg_m);
            p[i] = fast_exp2(x0);
            p[i + 1] = fast_exp2(x1);
            add_pair(sum4[i & 2], sum4[(i & 2) + 1], p[i], p[i + 1]);
          }
          const uint4 packed = make_uint4(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]), pack_bf16(p[4], p[5]),
                                          pack_bf16(p[6], p[7]));
          *reinterpret_cast<uint4*>(p_row + ((c ^ (r & 7)) << 4)) = packed;
        }
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l += sum;
      if (!observed && !failed) failed = !mbar_wait(smem_u32(&pv_done), (uint32_t)(t - 1) & 1u, a.status);
      if (!P_TMEM) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_ready));
      TC_PHASE(3);  // exponentials, P stored and announced
    }
#ifdef VX_TRACE
    for (int i = 0; i < 4; ++i) VX_TRACE_SET(i, (unsigned long long)phase_cycles[i] & 0xffffffffull);
#endif
    // Epilogue: O / l to the output, or to the partial rows of a split.
    if (num_tiles > 0 && !failed) failed = !mbar_wait(smem_u32(&pv_done), (uint32_t)(num_tiles - 1) & 1u, a.status);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    const bool on = r < row_count;
    const int row = row_begin + r;
    const int tok = row / a.group, hg = row - tok * a.group;
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
      float o[32];
      if (num_tiles > 0) {
        tc_load32(tmem_o + lane_base + (uint32_t)c0, o);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0.f;
      }
      if (!on) continue;
      if (partial_base < 0) {
        __nv_bfloat16* dst = (__nv_bfloat16*)a.out + (size_t)(q_start + tok) * a.out_stride +
                             (size_t)(kvh * a.group + hg) * D + c0;
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          *reinterpret_cast<uint4*>(dst + i) =
              make_uint4(pack_bf16(o[i] * inv, o[i + 1] * inv), pack_bf16(o[i + 2] * inv, o[i + 3] * inv),
                         pack_bf16(o[i + 4] * inv, o[i + 5] * inv), pack_bf16(o[i + 6] * inv, o[i + 7] * inv));
      } else {
        float* dst = a.partial_o + ((size_t)partial_base + (size_t)kvh * row_count + r) * D + c0;
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(dst + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
      }
    }
    if (on && partial_base >= 0)
      a.partial_lse[(size_t)partial_base + (size_t)kvh * row_count + r] =
          l > 0.f ? m_ref + log2f(l) : -CUDART_INF_F;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
#ifdef VX_TRACE
  if (threadIdx.x == 0)
    for (int i = 0; i < 4; ++i)
      VX_TRACE_SET(i, vx_trace_scope_.marks[i] | ((unsigned long long)mma_cycles[i] << 32));
#endif
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(TC_TMEM_COLS)
                 : "memory");
  }
  if (fused_merge)
    finish_split<(int)tc_smem_bytes(TC_STAGES)>(a, merge_index, num_splits, merge_item, kvh,
                                     reinterpret_cast<float*>(smem_al), &merge_bar);
}
#endif  // VX_HEAD_DIM == 128 || VX_HEAD_DIM == 64

}  // namespace vx

using namespace vx;

VX_TRACE_API(vx_attn)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map of a bf16 cache [pages, page_size, G, D] as [tokens, G, D] with boxes of
// [box_rows tokens, 1 head, 64 dims], 128-byte swizzled.  Cached by (pointer, shape).
static bool cache_tensor_map(CUtensorMap* map, const void* base, long long tokens, int heads,
                             int box_rows) {
  static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> cache;
  static std::mutex lock;
  static EncodeTiledFn encode = nullptr;
  std::lock_guard<std::mutex> guard(lock);
  const auto key = std::make_tuple(base, tokens, heads, box_rows);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *map = it->second;
    return true;
  }
  if (encode == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) !=
            cudaSuccess || result != cudaDriverEntryPointSuccess)
      return false;
    encode = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)tokens};
  const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)heads * D * 2};
  const cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
  const cuuint32_t elem[3] = {1, 1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
             box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache[key] = *map;
  return true;
}

static AttnArgs make_args(const void* q, void* out, const void* k_cache, const void* v_cache,
                          const int* block_tables, const int* q_start, const int* q_len,
                          const int* kv_len, const int* items, int* status, float* partial_o,
                          float* partial_lse, const int* merge_items, int* split_counters,
                          int q_stride, int out_stride, int table_stride,
                          int num_kv_heads, int group, int page_size, int window,
                          float softmax_scale) {
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.q = q;
  a.out = out;
  a.k_cache = k_cache;
  a.v_cache = v_cache;
  a.block_tables = block_tables;
  a.q_start = q_start;
  a.q_len = q_len;
  a.kv_len = kv_len;
  a.items = items;
  a.status = status;
  a.partial_o = partial_o;
  a.partial_lse = partial_lse;
  a.partial_capacity = 0;
  a.merge_items = merge_items;
  a.split_counters = split_counters;
  a.q_stride = q_stride;
  a.out_stride = out_stride;
  a.table_stride = table_stride;
  a.num_kv_heads = num_kv_heads;
  a.group = group;
  a.page_size = page_size;
  a.window = window;
  a.cluster = 1;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  return a;
}

VX_API int vx_attn_head_dim() { return D; }

// Rows per item that each family expects: kind 0 = float32, 1 = bf16 wide, 2 = bf16 narrow.
VX_API int vx_attn_tile_rows(int kind) { return kind == 3 ? 128 : (kind == 1 ? 64 : 16); }

// Whether this head size has the tensor-memory family (kind 3, 128-row tiles).
VX_API int vx_attn_has_tc() {
#ifdef VX_HAS_TC_ATTENTION
  return 1;
#else
  return 0;
#endif
}

// kind: 0 = float32, 1 = bf16 wide (64 rows), 2 = bf16 narrow (16 rows).
VX_API int vx_attention(int kind, const void* q, void* out, const void* k_cache,
                        const void* v_cache, const int* block_tables, const int* q_start,
                        const int* q_len, const int* kv_len, const int* items, int num_items,
                        int* status, float* partial_o, float* partial_lse, const int* merge_items,
                        int* split_counters, int q_stride, int out_stride, int table_stride,
                        int num_kv_heads, int group, int page_size, long long num_pages,
                        int window, float softmax_scale, int cluster, cudaStream_t stream) {
  if (num_items <= 0) return 0;
  // Only the narrow bf16 family shares an item among the CTAs of a cluster; for the
  // tensor-memory family 2 means "two CTAs on an SM" (see its launch below).
  if (cluster != 1 && !(kind == 3 && cluster == 2) &&
      (kind != 2 || (cluster != 2 && cluster != 4 && cluster != 8)))
    return (int)cudaErrorInvalidValue;
  // The float32 family leaves merging to the merge kernel.
  if (kind == 0) split_counters = nullptr;
  AttnArgs a = make_args(q, out, k_cache, v_cache, block_tables, q_start, q_len, kv_len,
                               items, status, partial_o, partial_lse, merge_items, split_counters,
                               q_stride, out_stride, table_stride,
                               num_kv_heads, group, page_size, window, softmax_scale);
  if (kind != 0 && TMA_KV) {
    // Page sizes are powers of two: a 64-key tile is whole pages, or lies inside one page.
    if (page_size <= 0 || (page_size & (page_size - 1)) != 0) return -1;
    const int box_rows = page_size < B_BN ? page_size : B_BN;
    const long long tokens = num_pages * page_size;
    if (!cache_tensor_map(&a.map_k, k_cache, tokens, num_kv_heads, box_rows) ||
        !cache_tensor_map(&a.map_v, v_cache, tokens, num_kv_heads, box_rows))
      return -1;
  }
  const dim3 grid(num_items, num_kv_heads);
  if (kind == 0) {
    const size_t smem = sizeof(float) * (size_t)(F_ROWS * D + 2 * F_BN * (D + 1));
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_f32_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    launch_pdl(attn_f32_kernel, dim3(grid), dim3(128), smem, stream, a);
  } else if (kind == 1) {
    const size_t smem = attn_smem_bytes(false, WIDE_STAGES) + 1024;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_wide_kernel<WIDE_STAGES>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    launch_pdl(attn_wide_kernel<WIDE_STAGES>, dim3(grid), dim3(128), smem, stream, a);
  } else if (kind == 2) {
    const size_t smem = attn_smem_bytes(true, NARROW_STAGES) + 1024;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_narrow_kernel<NARROW_STAGES>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    if (cluster == 1) {
      launch_pdl(attn_narrow_kernel<NARROW_STAGES>, dim3(grid), dim3(NARROW_THREADS), smem, stream, a);
    } else {
      a.cluster = cluster;
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3((unsigned)num_items * (unsigned)cluster, (unsigned)num_kv_heads);
      config.blockDim = dim3(NARROW_THREADS);
      config.dynamicSmemBytes = smem;
      config.stream = stream;
      cudaLaunchAttribute attributes[2];
      int count = 0;
      const char* serialised = getenv("VELOX_B200_NO_PDL");
      if (serialised == nullptr || serialised[0] != '1') {
        attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
      }
      attributes[count].id = cudaLaunchAttributeClusterDimension;
      attributes[count].val.clusterDim.x = (unsigned)cluster;
      attributes[count].val.clusterDim.y = 1;
      attributes[count].val.clusterDim.z = 1;
      ++count;
      config.attrs = attributes;
      config.numAttrs = count;
      cudaError_t e = cudaLaunchKernelEx(&config, attn_narrow_kernel<NARROW_STAGES>, a);
      if (e != cudaSuccess) return (int)e;
    }
#ifdef VX_HAS_TC_ATTENTION
  } else if (kind == 3) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaSuccess;
      const void* kernels_of[3] = {(const void*)attn_tc_kernel<2, true>, (const void*)attn_tc_kernel<2, false>,
                                   (const void*)attn_tc_kernel<4, false>};
      for (int i = 0; i < 3 && e == cudaSuccess; ++i)
        e = cudaFuncSetAttribute(kernels_of[i], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)tc_smem_bytes(i < 2 ? 2 : 4) + 1024);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    // VELOX_B200_TC_P_IN_SMEM=1 keeps the probabilities in shared memory with two CTAs per SM
    // too, VELOX_B200_TC_CTAS_PER_SM=1|2 forces the number of CTAs per SM (for A/B runs).
    static const bool p_tmem = [] {
      const char* value = getenv("VELOX_B200_TC_P_IN_SMEM");
      return !(value != nullptr && value[0] == '1');
    }();
    static int sms = 0;
    if (sms == 0) {
      int device = 0;
      if (cudaGetDevice(&device) != cudaSuccess ||
          cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
        sms = 148;
    }
    static const int forced = [] {
      const char* value = getenv("VELOX_B200_TC_CTAS_PER_SM");
      return value != nullptr ? atoi(value) : 0;
    }();
    // Two CTAs per SM (probabilities in tensor memory, K and V asked for a tile earlier) where
    // the grid is more than two CTAs per SM anyway, or where the caller says that the items'
    // key ranges are long (`cluster` = 2): a CTA alone on its SM walks a tile in 0.84 us, two
    // side by side in 1.46 us each, so two pay where the SM's work, not one CTA's chain, decides.
    const bool one_per_sm = forced == 1 || (forced != 2 && cluster < 2 &&
                                            (long long)num_items * num_kv_heads <= 2LL * sms);
    if (one_per_sm)
      launch_pdl(attn_tc_kernel<4, false>, dim3(grid), dim3(TC_THREADS), tc_smem_bytes(4) + 1024, stream, a);
    else if (p_tmem)
      launch_pdl(attn_tc_kernel<2, true>, dim3(grid), dim3(TC_THREADS), tc_smem_bytes(2) + 1024, stream, a);
    else
      launch_pdl(attn_tc_kernel<2, false>, dim3(grid), dim3(TC_THREADS), tc_smem_bytes(2) + 1024, stream, a);
#endif
  } else {
    return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

// What the planner needs to know about the narrow family: how many of its CTAs an SM holds
// (by shared memory), and the largest cluster that may share a work item.
VX_API int vx_attn_narrow_ctas_per_sm() {
  const size_t smem = attn_smem_bytes(true, NARROW_STAGES) + 1024 + 3 * 1024;  // + static, reserved
  const size_t per_sm = (size_t)228 * 1024;
  const int n = (int)(per_sm / smem);
  return n < 1 ? 1 : (n > 8 ? 8 : n);
}
VX_API int vx_attn_max_cluster() { return 8; }

// How many clusters of `cluster` CTAs of the narrow family the device holds at a time (a
// cluster lives inside one GPC, so this is less than the SM count suggests), or a negative
// cudaError_t.  A launch of more clusters than this runs in waves.
VX_API int vx_attn_narrow_max_active_clusters(int cluster) {
  if (cluster != 2 && cluster != 4 && cluster != 8) return -(int)cudaErrorInvalidValue;
  static int cached[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (cached[cluster] > 0) return cached[cluster];
  const size_t smem = attn_smem_bytes(true, NARROW_STAGES) + 1024;
  cudaError_t e = cudaFuncSetAttribute(attn_narrow_kernel<NARROW_STAGES>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return -(int)e;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)cluster * 64u, 1, 1);
  config.blockDim = dim3(NARROW_THREADS);
  config.dynamicSmemBytes = smem;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = (unsigned)cluster;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  int clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&clusters, attn_narrow_kernel<NARROW_STAGES>, &config);
  if (e != cudaSuccess) return -(int)e;
  cached[cluster] = clusters;
  return clusters;
}

// max_rows: the most rows a merge item has (the height of the tiles that were split).
VX_API int vx_attention_merge(int dtype, void* out, const int* q_start, const int* merge_items,
                              int num_items, int max_rows, const float* partial_o,
                              const float* partial_lse, int out_stride, int num_kv_heads,
                              int group, cudaStream_t stream) {
  if (num_items <= 0 || max_rows <= 0) return 0;
  AttnArgs a = make_args(nullptr, out, nullptr, nullptr, nullptr, q_start, nullptr, nullptr,
                         nullptr, nullptr, const_cast<float*>(partial_o), const_cast<float*>(partial_lse),
                         merge_items, nullptr, 0, out_stride, 0, num_kv_heads, group, 1, 0, 1.0f);
  const dim3 grid(num_items, num_kv_heads, max_rows);
  const int threads = D >= 128 ? 128 : (D >= 64 ? 64 : 32);
  if (dtype == VX_DTYPE_F32)
    launch_pdl(attn_merge_kernel<float>, dim3(grid), dim3(threads), 0, stream, a, merge_items);
  else
    launch_pdl(attn_merge_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, a, merge_items);
  return (int)cudaGetLastError();
}

// =============================================================================================
// vx_attention_decode_static: the 16-row bfloat16 family with its scratch inside the library.
// Declared and described in attention_static.h.  Nothing here allocates: no device allocation,
// no host container; the tensor maps are encoded into the kernel's arguments on every call.
// =============================================================================================
#include "attention_static.h"

#include <stdarg.h>
#include <stdio.h>

namespace {
constexpr size_t STATIC_O_BYTES = (size_t)VX_ATTENTION_STATIC_MAX_PARTIAL_ROWS * D * sizeof(float);
constexpr size_t STATIC_LSE_BYTES = (size_t)VX_ATTENTION_STATIC_MAX_PARTIAL_ROWS * sizeof(float);
constexpr size_t STATIC_COUNTER_BYTES = (size_t)VX_ATTENTION_STATIC_MAX_COUNTERS * sizeof(int);
constexpr int STATIC_MAX_DEVICES = 64;
}  // namespace

// [partial_o | partial_lse | counters]; every part starts on a 256-byte boundary.
static __device__ __align__(256) unsigned char
    g_static_scratch[STATIC_O_BYTES + STATIC_LSE_BYTES + STATIC_COUNTER_BYTES];

static int static_fail(char* error, int capacity, int code, const char* format, ...) {
  if (error != nullptr && capacity > 0) {
    va_list args;
    va_start(args, format);
    vsnprintf(error, (size_t)capacity, format, args);
    va_end(args);
  }
  return code;
}

// Tensor map of a bf16 cache as cache_tensor_map() makes it, written straight into `map`.
static bool encode_cache_map(EncodeTiledFn encode, CUtensorMap* map, const void* base,
                             long long tokens, int heads, int box_rows) {
  const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)tokens};
  const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)heads * D * 2};
  const cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
  const cuuint32_t elem[3] = {1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
         CUDA_SUCCESS;
}

int vx_attention_decode_static(const void* q, void* out, const void* k_cache, const void* v_cache,
                               const int* block_tables, const int* q_start, const int* q_len,
                               const int* kv_len, const int* items, int num_items,
                               const int* merge_items, int num_merges, int partial_rows,
                               int* status, int q_stride, int out_stride, int table_stride,
                               int num_kv_heads, int group, int page_size, long long num_pages,
                               int window, float softmax_scale, cudaStream_t stream, char* error,
                               int error_capacity) {
  if (error != nullptr && error_capacity > 0) error[0] = 0;
  if (num_items < 0 || num_merges < 0 || partial_rows < 0 || num_kv_heads <= 0 || group <= 0)
    return static_fail(error, error_capacity, VX_ATTENTION_STATIC_BAD_ARGUMENT,
                       "vx_attention_decode_static: negative count or no heads (items %d, merges "
                       "%d, partial rows %d, KV heads %d, group %d)",
                       num_items, num_merges, partial_rows, num_kv_heads, group);
  if (partial_rows > VX_ATTENTION_STATIC_MAX_PARTIAL_ROWS)
    return static_fail(error, error_capacity, VX_ATTENTION_STATIC_TOO_LARGE,
                       "vx_attention_decode_static: the split key ranges need %d partial rows, the "
                       "library's scratch holds %d (head size %d); use fewer splits or "
                       "vx_attention with scratch of your own",
                       partial_rows, VX_ATTENTION_STATIC_MAX_PARTIAL_ROWS, D);
  const long long counters = (long long)num_merges * num_kv_heads;
  if (counters > VX_ATTENTION_STATIC_MAX_COUNTERS)
    return static_fail(error, error_capacity, VX_ATTENTION_STATIC_TOO_LARGE,
                       "vx_attention_decode_static: %d merge items on %d KV heads need %lld "
                       "counters, the library's scratch holds %d",
                       num_merges, num_kv_heads, counters, VX_ATTENTION_STATIC_MAX_COUNTERS);
  if ((num_merges > 0 && merge_items == nullptr) || (partial_rows > 0 && num_merges == 0))
    return static_fail(error, error_capacity, VX_ATTENTION_STATIC_BAD_ARGUMENT,
                       "vx_attention_decode_static: split items need their merge items");
  if (page_size <= 0 || (page_size & (page_size - 1)) != 0)
    return static_fail(error, error_capacity, VX_ATTENTION_STATIC_BAD_ARGUMENT,
                       "vx_attention_decode_static: page size %d is not a power of two", page_size);
  if (num_items == 0) return 0;

  const size_t smem = attn_smem_bytes(true, NARROW_STAGES) + 1024;

  // Set-up, once per device.
  static std::mutex lock;
  static unsigned char* scratch_of[STATIC_MAX_DEVICES] = {};
  static EncodeTiledFn encode = nullptr;
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess)
    return static_fail(error, error_capacity, (int)e, "vx_attention_decode_static: cudaGetDevice: %s",
                       cudaGetErrorString(e));
  if (device < 0 || device >= STATIC_MAX_DEVICES)
    return static_fail(error, error_capacity, VX_ATTENTION_STATIC_BAD_ARGUMENT,
                       "vx_attention_decode_static: device %d is beyond the %d this library keeps "
                       "scratch addresses for", device, STATIC_MAX_DEVICES);
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> guard(lock);
    if (scratch_of[device] == nullptr) {
      void* address = nullptr;
      e = cudaGetSymbolAddress(&address, g_static_scratch);
      if (e != cudaSuccess || address == nullptr)
        return static_fail(error, error_capacity, e != cudaSuccess ? (int)e : (int)cudaErrorInvalidSymbol,
                           "vx_attention_decode_static: cudaGetSymbolAddress of the scratch array: %s",
                           cudaGetErrorString(e));
      e = cudaFuncSetAttribute(attn_narrow_kernel<NARROW_STAGES>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess)
        e = cudaMemset((unsigned char*)address + STATIC_O_BYTES + STATIC_LSE_BYTES, 0,
                       STATIC_COUNTER_BYTES);
      if (e != cudaSuccess)
        return static_fail(error, error_capacity, (int)e, "vx_attention_decode_static: set-up: %s",
                           cudaGetErrorString(e));
      if (TMA_KV && encode == nullptr) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result);
        if (e != cudaSuccess || result != cudaDriverEntryPointSuccess || entry == nullptr)
          return static_fail(error, error_capacity, e != cudaSuccess ? (int)e : (int)cudaErrorNotSupported,
                             "vx_attention_decode_static: the driver has no cuTensorMapEncodeTiled");
        encode = reinterpret_cast<EncodeTiledFn>(entry);
      }
      scratch_of[device] = (unsigned char*)address;
    }
    scratch = scratch_of[device];
  }
  float* partial_o = reinterpret_cast<float*>(scratch);
  float* partial_lse = reinterpret_cast<float*>(scratch + STATIC_O_BYTES);
  int* split_counters = reinterpret_cast<int*>(scratch + STATIC_O_BYTES + STATIC_LSE_BYTES);

  AttnArgs a = make_args(q, out, k_cache, v_cache, block_tables, q_start, q_len, kv_len, items,
                         status, partial_o, partial_lse, merge_items,
                         num_merges > 0 ? split_counters : nullptr, q_stride, out_stride,
                         table_stride, num_kv_heads, group, page_size, window, softmax_scale);
  // The items live on the device and are not read here, so partial_rows is the caller's word;
  // the kernel holds every partial row against the array's real size.
  a.partial_capacity = VX_ATTENTION_STATIC_MAX_PARTIAL_ROWS;
  if (TMA_KV) {
    const int box_rows = page_size < B_BN ? page_size : B_BN;
    const long long tokens = num_pages * page_size;
    if (!encode_cache_map(encode, &a.map_k, k_cache, tokens, num_kv_heads, box_rows) ||
        !encode_cache_map(encode, &a.map_v, v_cache, tokens, num_kv_heads, box_rows))
      return static_fail(error, error_capacity, VX_ATTENTION_STATIC_BAD_ARGUMENT,
                         "vx_attention_decode_static: the cache (%lld pages of %d, %d KV heads) "
                         "cannot be described by a tensor map; is it 16-byte aligned?",
                         num_pages, page_size, num_kv_heads);
  }
  if (counters > 0) {
    e = cudaMemsetAsync(split_counters, 0, (size_t)counters * sizeof(int), stream);
    if (e != cudaSuccess)
      return static_fail(error, error_capacity, (int)e, "vx_attention_decode_static: clearing the counters: %s",
                         cudaGetErrorString(e));
  }
  const dim3 grid(num_items, num_kv_heads);
  e = launch_pdl(attn_narrow_kernel<NARROW_STAGES>, dim3(grid), dim3(NARROW_THREADS), smem, stream, a);
  if (e != cudaSuccess)
    return static_fail(error, error_capacity, (int)e, "vx_attention_decode_static: launch: %s",
                       cudaGetErrorString(e));
  return 0;
}
