// bfloat16 projections on the 5th-generation tensor cores: Y[T, N] = X[T, K] * W[N, K]^T.
//
// The weight is the M operand of the MMA: a CTA owns 128 rows of W (128 output features) and
// BN tokens, D^T[128, BN] = W_tile[128, K] * X_tile[BN, K]^T, accumulated in tensor memory.
// With few tokens (decode) the tensor-core tile is still full, because its 128-row side is made
// of weight rows; the kernel then streams W once at memory speed.  A projection with few output
// tiles is split along K over a thread-block cluster (2, 4 or 8 CTAs): every CTA accumulates its
// share of K in its own tensor memory and sends every row (output feature) of its partial tile
// to the CTA that owns that row, by st.async stores into the owner's shared memory (distributed
// shared memory) that count their bytes on the owner's own mbarrier; when all its bytes are in,
// each CTA sums what the ranks sent, in rank order, and writes its rows out.  The one barrier
// of the whole cluster is at the start ("everybody runs").  No partial product touches global
// memory and the order of the sums is fixed.
//
//   warp 0, one lane : TMA producer.  cp.async.bulk.tensor 2-D tiles of W [128 x 64] and
//                      X [BN x 64] into a ring of 128-byte-swizzled shared-memory stages.
//   warp 1, one lane : tcgen05.mma issuer (kind::f16, bf16 x bf16 -> f32 in TMEM), four
//                      K=16 instructions per stage; tcgen05.commit frees the stage and, after
//                      the last stage, signals the epilogue.  The warp owns the TMEM allocation.
//   warps 2..5       : epilogue.  tcgen05.ld 32 lanes x 32 columns; a thread holds one output
//                      feature for 32 tokens, so for a fixed token a warp writes 32 consecutive
//                      features (one coalesced segment).
//
// Fused input norm (GemmArgs::resid): the X operand is made on the spot.  While the weight tiles
// stream in, the epilogue warps read the float32 residual rows of the CTA's tokens, multiply by
// the norm weight, round to bf16 and store the [BN x 64] tile of every K block of the CTA into
// shared memory of their own (after the stages), in the 128-byte-swizzled layout the tensor map
// would have produced (16-byte chunk c of row r at chunk c ^ (r & 7)); they also sum the
// squares.  They work in batches of a few K blocks, all loads of a batch in flight at once, and
// signal every batch on an mbarrier the MMA issuer waits for.  y = rstd[t] * (W (w_norm x)) + b:
// the row scale is applied in the epilogue; with split K the CTAs of a cluster add up their
// sums of squares through the same exchange that carries the partial tiles.
//
// Epilogue modes:
//   0  out bf16  [T, ldy] = acc + bias
//   1  out f32   [T, ldy] = acc + bias          (logits)
//   2  out f32   [T, ldy] += acc                (projection added straight into the float32
//                                                residual stream; one CTA owns each element;
//                                                optionally the sums go to a second buffer too)
//   3  out bf16  [T, ldy] = silu(gate) * up     W rows are [64 gate | 64 up] per CTA (the host
//                                                passes two tensor maps of the same matrix)
//   4  QKV of heads of 128 dims, split K only: a CTA's 128 rows are one head; acc + bias is
//      rotated by the token's position (rotate-half over the whole head, float32 tables) for
//      query and key heads; query heads go to out bf16 [T, ldy], key and value heads straight
//      into the paged cache at the token's slot.  The rows of a tile are dealt to the cluster's
//      CTAs in pairs (d, d + 64), so the owner of a pair rotates it without another exchange.
//
// Every wait on an mbarrier is bounded: when the bound is hit the thread sets a status bit,
// stops issuing work, and the CTA still frees its tensor memory and returns.
// The reference engine leaves these products to cuBLAS (nn.Linear; src/self_attention.py:32-33,
// src/mlp.py:9-15, src/transformer.py:60 of that project).
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace vx {

constexpr int GB_BM = 128;
constexpr int GB_BK = 64;
constexpr int GB_THREADS = 192;
constexpr uint32_t GB_A_BYTES = GB_BM * GB_BK * 2;

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows at a 128-byte pitch,
// groups of eight rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, bits 0-13
  desc |= (uint64_t)0 << 16;                         // leading byte offset (unused here)
  desc |= (uint64_t)(1024u >> 4) << 32;              // stride byte offset, bits 32-45
  desc |= (uint64_t)1 << 46;                         // descriptor version of sm_100
  desc |= (uint64_t)2 << 61;                         // 128-byte swizzle
  return desc;
}

// Instruction descriptor of kind::f16: D f32, A and B bf16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(GB_BM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float (&v)[32]) {
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

__device__ __forceinline__ void tmem_load_16(uint32_t taddr, float (&v)[32]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

struct GemmArgs {
  const float* bias;  // [N] or null
  void* out;
  int* status;
  long long ldy;         // row pitch of out, in elements
  int T, N, K;
  int mode;
  int kb_per_split;      // 64-wide K blocks per split
  int splits;            // CTAs of the cluster that share one output tile (1: no cluster)
  // Fused RMSNorm of the input (token tiles up to 64): x is not read; the epilogue warps make
  // the X tiles themselves as bf16(resid[t, k] * norm_w[k]) from the float32 residual stream,
  // and the row's 1 / rms is applied to the accumulator, where it commutes with the product.
  const float* resid;    // [T, resid_ld] float32, or null: plain input through the tensor map
  const float* norm_w;   // [K]
  long long resid_ld;
  float eps;
  // X tiles of the fused norm that shared memory holds at a time (a multiple of the batch in
  // which they are made).  At least the CTA's K blocks: every tile has a place of its own.
  // Fewer: the places are a ring, and a batch is written when the products that read the
  // batch before it in its place have finished.
  int x_slots;
  // Mode 4.
  const int* positions;  // [T]
  const float* cos_t;    // [max_pos, 64]
  const float* sin_t;
  const int* slots;      // [T] cache slot of the token (page * page_size + offset), < 0: none
  void* k_cache;         // [slots, kv_heads, 128] bf16, or null: nothing is written to a cache
  void* v_cache;
  int heads, kv_heads, max_pos;
  long long num_slots;
  // Mode 2 with split K only: the sums out + acc are also written to out2 [T, ld2] float32, a
  // copy of the rows that stays as it is while a later kernel adds to `out` again.
  float* out2;
  long long ld2;
};

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

// Stores four floats into a peer CTA's shared memory, at the same offset as `local_addr` here,
// and counts their 16 bytes on the peer's mbarrier at the offset of `local_bar`: the peer
// learns from its own barrier that what it waits for has arrived, without a barrier of the
// whole cluster.
__device__ __forceinline__ void send_peer_shared4(uint32_t local_addr, uint32_t local_bar, uint32_t rank,
                                                  float a, float b, float c, float d) {
  uint32_t remote, remote_bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(local_bar), "r"(rank));
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(remote), "f"(a), "f"(b), "f"(c), "f"(d), "r"(remote_bar)
               : "memory");
}

__device__ __forceinline__ void send_peer_shared1(uint32_t local_addr, uint32_t local_bar, uint32_t rank,
                                                  float a) {
  uint32_t remote, remote_bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(local_bar), "r"(rank));
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];"
               ::"r"(remote), "f"(a), "r"(remote_bar)
               : "memory");
}

// One element of the output in the epilogue mode of the launch (modes 0, 1, 2).
__device__ __forceinline__ void store_output(const GemmArgs& g, size_t index, float value) {
  if (g.mode == 0)
    ((__nv_bfloat16*)g.out)[index] = __float2bfloat16_rn(value);
  else if (g.mode == 1)
    ((float*)g.out)[index] = value;
  else
    // Nobody else adds to this element during the launch, so the sum is the same as with a load
    // and a store; as a reduction at the L2 it needs no round trip and threads do not wait for it.
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"((float*)g.out + index), "f"(value) : "memory");
}

constexpr int GB_MAX_SPLITS = 8;  // CTAs of a cluster (a portable one; the device holds too few clusters of sixteen)

template <int BN, int STAGES_>
struct GemmShape {
  static constexpr uint32_t B_BYTES = BN * GB_BK * 2;
  static constexpr uint32_t STAGE_BYTES = GB_A_BYTES + B_BYTES;
  // Four stages: 64 KB of weight tiles in flight per CTA, and with few tokens two CTAs fit on
  // an SM, so the next projection's CTAs can move in and prefetch while this one drains.
  // Eight stages (narrow token tiles only): 128 KB in flight for a grid that gives every SM one
  // CTA at most, which is what keeps HBM busy at its loaded latency.
  static constexpr int STAGES = STAGES_;
  static constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  // Where the peers of a cluster deposit their shares of this CTA's output slice:
  // [splits][128 / splits rows][BN tokens] floats, then [8][BN] sums of squares of the fused
  // norm (token tiles up to 64 only).  The SwiGLU epilogue, which is never clustered, uses the
  // same place for the exchange between its gate and up rows (64 x 33 floats).
  // A row of the receive area is four floats longer than its BN tokens, so that the rows that
  // the 32 lanes of a warp write or read at a time fall on different banks.
  static constexpr uint32_t RECV_ROW = BN + 4;
  static constexpr uint32_t RECV_BYTES = BN <= 64 ? ((GB_BM * RECV_ROW * 4 + GB_MAX_SPLITS * BN * 4 + 1023) / 1024) * 1024 : 9216;
  // Fused norm: K blocks whose X tiles one batch of loads makes, and the most batches.
  static constexpr int NORM_BATCH = BN <= 16 ? 6 : (BN <= 32 ? 4 : 2);
  static constexpr int NORM_MAX_BATCHES = 32;
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + RECV_BYTES + 1024;
};

template <int BN, int STAGES_>
__global__ void __launch_bounds__(GB_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                 const __grid_constant__ CUtensorMap map_x, GemmArgs g) {
  using S = GemmShape<BN, STAGES_>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[S::STAGES];
  __shared__ __align__(8) uint64_t empty_bar[S::STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ __align__(8) uint64_t recv_bar;  // split K: the peers' shares of this CTA's rows have arrived
  __shared__ uint32_t tmem_slot;
  __shared__ int epilogue_failed;
  __shared__ float ssq_s[64];  // fused norm: this CTA's sums of squares, then 1 / rms, per token
  __shared__ __align__(8) uint64_t x_bar[S::NORM_MAX_BATCHES];   // fused norm: a batch of X tiles is ready
  __shared__ __align__(8) uint64_t x_free[S::NORM_MAX_BATCHES];  // ... and its place may be written again

  VX_TRACE_SCOPE(10 + g.mode);
  allow_dependents();
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  float* swap_buf = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)) + S::STAGES * S::STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * (g.mode == 3 ? 64 : GB_BM);
  const int t0 = blockIdx.y * BN;
  const int split = blockIdx.z;
  const int num_kb_total = (g.K + GB_BK - 1) / GB_BK;
  const int kb_begin = split * g.kb_per_split;
  const int kb_end = min(num_kb_total, kb_begin + g.kb_per_split);
  const int num_kb = max(0, kb_end - kb_begin);
  const bool clustered = g.splits > 1;
  const bool normed = BN <= 64 && g.resid != nullptr;

  if (threadIdx.x == 0) {
    epilogue_failed = 0;
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    if (normed)
      for (int b = 0; b < S::NORM_MAX_BATCHES; ++b) {
        mbar_init(smem_u32(&x_bar[b]), 1);
        mbar_init(smem_u32(&x_free[b]), 1);
      }
    mbar_init(smem_u32(&acc_bar), 1);
    mbar_init(smem_u32(&recv_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // What the cluster will send here: every rank's share of this CTA's 128 / splits rows (its
    // own included), BN floats a row, and with the fused norm every rank's sums of squares.
    if (clustered) mbar_expect_tx(smem_u32(&recv_bar), (uint32_t)(GB_BM * BN * 4 + (normed ? g.splits * BN * 4 : 0)));
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(S::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_slot;
  // The one barrier of the whole cluster: "every CTA runs and its receive barrier is armed"
  // (nobody may write into a peer before).  Arrive now; the wait comes right before the first
  // remote store and costs nothing by then.
  if (clustered) cluster_arrive();

  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- TMA producer
    // The weight does not depend on the kernel before this one: its tiles for the first
    // round of stages are requested at once, the activations after the dependency wait.
    const int first_round = min(num_kb, S::STAGES);
    auto load_w = [&](int i) {
      const int stage = i % S::STAGES;
      const uint32_t full = smem_u32(&full_bar[stage]);
      const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
      const int kx = (kb_begin + i) * GB_BK;
      mbar_expect_tx(full, normed ? GB_A_BYTES : S::STAGE_BYTES);
      if (g.mode == 3) {
        // 64 gate rows then 64 up rows: two boxes of 64 rows each.
        tma_load_2d(a_dst, &map_w, kx, n0, full);
        tma_load_2d(a_dst + GB_A_BYTES / 2, &map_w2, kx, n0, full);
      } else {
        tma_load_2d(a_dst, &map_w, kx, n0, full);
      }
    };
    auto load_x = [&](int i) {
      const int stage = i % S::STAGES;
      const uint32_t b_dst = smem_base + stage * S::STAGE_BYTES + GB_A_BYTES;
      tma_load_2d(b_dst, &map_x, (kb_begin + i) * GB_BK, t0, smem_u32(&full_bar[stage]));
    };
    for (int i = 0; i < first_round; ++i) load_w(i);
    grid_dependency_wait();
    VX_TRACE_MARK(0);
    if (!normed)
      for (int i = 0; i < first_round; ++i) load_x(i);
    for (int i = first_round; i < num_kb; ++i) {
      const int stage = i % S::STAGES;
      const uint32_t phase = (uint32_t)(i / S::STAGES) & 1u;
      if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, g.status)) break;
      load_w(i);
      if (!normed) load_x(i);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = umma_instr_desc(BN);
    bool ok = true;
    for (int i = 0; i < num_kb && ok; ++i) {
      const int stage = i % S::STAGES;
      const uint32_t phase = (uint32_t)(i / S::STAGES) & 1u;
      ok = mbar_wait(smem_u32(&full_bar[stage]), phase, g.status);
      // Batch b of X tiles lies in place b % ring_batches; its barrier has been used b / ring_batches times.
      const int batch = i / S::NORM_BATCH, ring_batches = normed ? g.x_slots / S::NORM_BATCH : 1;
      if (ok && normed && i % S::NORM_BATCH == 0)
        ok = mbar_wait(smem_u32(&x_bar[batch % ring_batches]), (uint32_t)(batch / ring_batches) & 1u, g.status);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = smem_base + stage * S::STAGE_BYTES;
      const uint32_t b_addr = normed ? smem_base + S::STAGES * S::STAGE_BYTES + S::RECV_BYTES +
                                           (uint32_t)(i % g.x_slots) * S::B_BYTES
                                     : a_addr + GB_A_BYTES;
#pragma unroll
      for (int k = 0; k < GB_BK / 16; ++k) {
        umma_bf16(tmem_acc, umma_smem_desc(a_addr + k * 32), umma_smem_desc(b_addr + k * 32),
                  idesc, (i > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(smem_u32(&empty_bar[stage]));
      // The last product of a batch: when it has finished, the batch's place is free again.
      if (normed && (i % S::NORM_BATCH == S::NORM_BATCH - 1 || i == num_kb - 1))
        umma_commit(smem_u32(&x_free[batch % ring_batches]));
    }
    // Arrives when every MMA above has finished (or at once if there were none).
    umma_commit(smem_u32(&acc_bar));
  } else if (warp >= 2) {
    // ---------------------------------------------------------------- epilogue
    grid_dependency_wait();
    if (BN <= 64 && normed) {
      // The X tiles of the fused norm.  Thread q of the 128 takes 16-byte chunks q, q + 128, ...
      // of a tile: token q / 8 (+ 16 per further chunk), dims 8 * (q % 8) .. + 7 of the K block.
      constexpr int CPT = BN <= 64 ? (BN * 8 + 127) / 128 : 1;  // chunks per thread and K block
      constexpr int NB = S::NORM_BATCH;
      const int q = (int)threadIdx.x - 64;
      const int c = q & 7;
      float ssq[CPT];
#pragma unroll
      for (int u = 0; u < CPT; ++u) ssq[u] = 0.f;
      unsigned char* x_tiles = smem_raw + (smem_base - smem_u32(smem_raw)) + S::STAGES * S::STAGE_BYTES + S::RECV_BYTES;
      const int ring_batches = g.x_slots / NB;
      bool x_alive = true;
      for (int i0 = 0; i0 < num_kb; i0 += NB) {
        float4 xa[NB][CPT], xb[NB][CPT], wa[NB], wb[NB];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          const int k = (kb_begin + i0 + j) * GB_BK + c * 8;
          const bool in_k = i0 + j < num_kb && k < g.K;  // K is a multiple of 8: a chunk is inside or outside
          wa[j] = in_k ? __ldg(reinterpret_cast<const float4*>(g.norm_w + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
          wb[j] = in_k ? __ldg(reinterpret_cast<const float4*>(g.norm_w + k + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < CPT; ++u) {
            const int r = (q >> 3) + 16 * u;
            const int t = t0 + r;
            const bool on = in_k && t < g.T && r < BN;
            const float* src = g.resid + (size_t)t * g.resid_ld + k;
            xa[j][u] = on ? *reinterpret_cast<const float4*>(src) : make_float4(0.f, 0.f, 0.f, 0.f);
            xb[j][u] = on ? *reinterpret_cast<const float4*>(src + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        // The place of this batch: free from the start the first time round, afterwards when
        // the products of the batch that lay there have finished (the loads above are under way
        // meanwhile).
        const int batch = i0 / NB;
        if (batch >= ring_batches && x_alive)
          x_alive = mbar_wait(smem_u32(&x_free[batch % ring_batches]), (uint32_t)(batch / ring_batches - 1) & 1u, g.status);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          if (i0 + j >= num_kb) break;
          unsigned char* tile = x_tiles + (size_t)((i0 + j) % g.x_slots) * S::B_BYTES;
#pragma unroll
          for (int u = 0; u < CPT; ++u) {
            const float4 a4 = xa[j][u], b4 = xb[j][u];
            ssq[u] += a4.x * a4.x + a4.y * a4.y + a4.z * a4.z + a4.w * a4.w +
                      b4.x * b4.x + b4.y * b4.y + b4.z * b4.z + b4.w * b4.w;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(a4.x * wa[j].x, a4.y * wa[j].y);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(a4.z * wa[j].z, a4.w * wa[j].w);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(b4.x * wb[j].x, b4.y * wb[j].y);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(b4.z * wb[j].z, b4.w * wb[j].w);
            const int r = (q >> 3) + 16 * u;
            if (r < BN)
              *reinterpret_cast<uint4*>(tile + r * 128 + ((c ^ (r & 7)) << 4)) =
                  make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                             *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
          }
        }
        // The tensor core reads the tiles through the async proxy.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (q == 0) mbar_arrive(smem_u32(&x_bar[batch % ring_batches]));
      }
      // The eight threads of a token sit in consecutive lanes.
#pragma unroll
      for (int u = 0; u < CPT; ++u) {
        float v = ssq[u];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        const int r = (q >> 3) + 16 * u;
        if (c == 0 && r < BN) ssq_s[r] = v;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!clustered) {
        // This CTA saw all of K: its sums are the rows' sums.
        if (q < BN) ssq_s[q] = rsqrtf(ssq_s[q] / (float)g.K + g.eps);
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    }
    const int quarter = warp & 3;  // TMEM lanes 32 * quarter .. + 31 belong to this warp
    if (!mbar_wait(smem_u32(&acc_bar), 0u, g.status)) epilogue_failed = 1;
    // All four epilogue warps take the same path below (mode 3 has barriers among them).
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool ready = epilogue_failed == 0 && num_kb > 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = quarter * 32 + lane;  // row of the CTA's W tile
    constexpr int cols = BN >= 32 ? 32 : 16;
    const uint32_t lane_base = tmem_acc + ((uint32_t)(quarter * 32) << 16);
    if (clustered) {
      // Every CTA of the cluster owns 128 / splits rows (output features) of the tile.  Send this
      // thread's row of the partial tile to its owner, into slot [this rank][row in slice][token]
      // of the owner's receive area: BN contiguous floats, four per store.
      cluster_wait();
      const int rows_per_cta = GB_BM / g.splits;
      const uint32_t rank = cluster_rank();
      // Mode 4 deals rows in pairs (d, d + 64): a CTA owns 64 / splits dims and their partners.
      const int pairs_per_cta = rows_per_cta / 2;
      const uint32_t owner = g.mode == 4 ? (uint32_t)((row & 63) / pairs_per_cta) : (uint32_t)(row / rows_per_cta);
      const uint32_t slot_row = g.mode == 4 ? (uint32_t)((row >> 6) * pairs_per_cta + (row & 63) % pairs_per_cta)
                                            : (uint32_t)(row % rows_per_cta);
      const uint32_t recv = smem_base + S::STAGES * S::STAGE_BYTES +
                            ((rank * (uint32_t)rows_per_cta + slot_row) * S::RECV_ROW) * 4u;
      if (normed && row < BN) {
        // This CTA's share of the sums of squares goes to every CTA of the cluster.
        const uint32_t at = smem_base + S::STAGES * S::STAGE_BYTES + (uint32_t)(GB_BM * S::RECV_ROW) * 4u +
                            (rank * (uint32_t)BN + (uint32_t)row) * 4u;
        for (uint32_t peer = 0; peer < (uint32_t)g.splits; ++peer)
          send_peer_shared1(at, smem_u32(&recv_bar), peer, ssq_s[row]);
      }
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        if (ready) {
          if (BN >= 32) tmem_load_32(lane_base + c0, v); else tmem_load_16(lane_base + c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < cols; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < cols; j += 4)
          send_peer_shared4(recv + (uint32_t)(c0 + j) * 4u, smem_u32(&recv_bar), owner, v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
    } else if (ready) {
      if (g.mode == 3) {
        // rows 0..63 gate, 64..127 up of the same 64 output features
        const int n = n0 + (row & 63);
        __nv_bfloat16* out = (__nv_bfloat16*)g.out;
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          if (BN >= 32) tmem_load_32(lane_base + c0, v); else tmem_load_16(lane_base + c0, v);
          // up rows hand their values to the gate rows through shared memory
          if (row >= 64) {
            for (int j = 0; j < cols; ++j) swap_buf[(row - 64) * 33 + j] = v[j];
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (row < 64 && n < g.N) {
            for (int j = 0; j < cols; ++j) {
              const int t = t0 + c0 + j;
              if (t < g.T) {
                const float scale = normed ? ssq_s[c0 + j] : 1.0f;
                const float gate = v[j] * scale, up = swap_buf[row * 33 + j] * scale;
                out[(size_t)t * g.ldy + n] = __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      } else {
        const int n = n0 + row;
        const float b = (g.bias != nullptr && n < g.N) ? g.bias[n] : 0.f;
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          if (BN >= 32) tmem_load_32(lane_base + c0, v); else tmem_load_16(lane_base + c0, v);
          if (n < g.N) {
            for (int j = 0; j < cols; ++j) {
              const int t = t0 + c0 + j;
              if (t < g.T) store_output(g, (size_t)t * g.ldy + n, v[j] * (normed ? ssq_s[c0 + j] : 1.0f) + b);
            }
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  // Warps 0 and 1 have not waited on the first cluster phase yet (the epilogue warps did).
  if (clustered && warp < 2) {
    __syncwarp();  // lane 0 ran a role loop; the barrier instruction wants the whole warp
    cluster_wait();
  }
  __syncthreads();
  VX_TRACE_MARK(1);
  if (clustered) {
    // Every rank's stores into this CTA's receive area have arrived (and nobody writes here
    // after that, so this CTA may end while its own stores are still on their way to peers that
    // wait for them).
    // With a second output the old values of this thread's elements are asked for now, so
    // that they are here when the shares are.
    constexpr int MIRROR_SLOTS = 8;
    float old_out[MIRROR_SLOTS];
    if (g.out2 != nullptr && warp >= 2) {
      const int rows_per_cta = GB_BM / g.splits;
      const int rank = (int)cluster_rank();
#pragma unroll
      for (int u = 0; u < MIRROR_SLOTS; ++u) {
        const int e = (warp - 2) * 32 + lane + 128 * u;
        const int j = e / rows_per_cta, rl = e - j * rows_per_cta;
        const int t = t0 + j, n = n0 + rank * rows_per_cta + rl;
        old_out[u] = (e < rows_per_cta * BN && t < g.T && n < g.N) ? __ldcg((const float*)g.out + (size_t)t * g.ldy + n) : 0.f;
      }
    }
    mbar_wait(smem_u32(&recv_bar), 0u, g.status);
    VX_TRACE_MARK(2);
    if (warp >= 2) {
      // Sum the shares of this CTA's rows in rank order and write them; consecutive threads take
      // consecutive features of one token.
      const int rows_per_cta = GB_BM / g.splits;
      const int rank = (int)cluster_rank();
      const float* recv = reinterpret_cast<const float*>(
          smem_raw + (smem_base - smem_u32(smem_raw)) + S::STAGES * S::STAGE_BYTES);
      if (normed) {
        const int j = (int)threadIdx.x - 64;
        if (j < BN) {
          float total = 0.f;
          for (int peer = 0; peer < g.splits; ++peer) total += recv[GB_BM * S::RECV_ROW + peer * BN + j];
          ssq_s[j] = rsqrtf(total / (float)g.K + g.eps);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (g.mode == 4) {
        // This CTA's pairs (d, d + 64) of one head: sum, scale, bias, rotate, store.
        const int pairs = rows_per_cta / 2;
        const int head = blockIdx.x;
        const bool is_q = head < g.heads, is_k = !is_q && head < g.heads + g.kv_heads;
        for (int e = (warp - 2) * 32 + lane; e < pairs * BN; e += 128) {
          const int j = e / pairs, pl = e - j * pairs;
          const int t = t0 + j;
          if (t >= g.T) continue;
          const int d = rank * pairs + pl;
          float lo = 0.f, hi = 0.f;
          for (int peer = 0; peer < g.splits; ++peer) {
            lo += recv[((size_t)peer * rows_per_cta + pl) * S::RECV_ROW + j];
            hi += recv[((size_t)peer * rows_per_cta + pairs + pl) * S::RECV_ROW + j];
          }
          if (normed) {
            lo *= ssq_s[j];
            hi *= ssq_s[j];
          }
          if (g.bias != nullptr) {
            lo += g.bias[n0 + d];
            hi += g.bias[n0 + d + 64];
          }
          if (is_q || is_k) {
            int pos = g.positions[t];
            if (pos < 0 || pos >= g.max_pos) {
              atomicOr(g.status, VX_STATUS_BAD_POSITION);
              pos = 0;
            }
            const float cs = g.cos_t[(size_t)pos * 64 + d], sn = g.sin_t[(size_t)pos * 64 + d];
            const float r_lo = lo * cs - hi * sn, r_hi = lo * sn + hi * cs;
            lo = r_lo;
            hi = r_hi;
          }
          __nv_bfloat16* dst;
          if (is_q) {
            dst = (__nv_bfloat16*)g.out + (size_t)t * g.ldy + n0 + d;
          } else {
            if (g.k_cache == nullptr) continue;
            const int slot = g.slots[t];
            if (slot < 0) continue;
            if ((long long)slot >= g.num_slots) {
              atomicOr(g.status, VX_STATUS_BAD_SLOT);
              continue;
            }
            const int kvh = is_k ? head - g.heads : head - g.heads - g.kv_heads;
            dst = (__nv_bfloat16*)(is_k ? g.k_cache : g.v_cache) + ((size_t)slot * g.kv_heads + kvh) * 128 + d;
          }
          dst[0] = __float2bfloat16_rn(lo);
          dst[64] = __float2bfloat16_rn(hi);
        }
      } else
      if (g.out2 != nullptr) {
#pragma unroll
        for (int u = 0; u < MIRROR_SLOTS; ++u) {
          const int e = (warp - 2) * 32 + lane + 128 * u;
          if (e >= rows_per_cta * BN) break;
          const int j = e / rows_per_cta, rl = e - j * rows_per_cta;
          const int t = t0 + j, n = n0 + rank * rows_per_cta + rl;
          if (t >= g.T || n >= g.N) continue;
          float acc = 0.f;
          for (int peer = 0; peer < g.splits; ++peer)
            acc += recv[((size_t)peer * rows_per_cta + rl) * S::RECV_ROW + j];
          if (normed) acc *= ssq_s[j];
          const float sum = old_out[u] + (acc + (g.bias != nullptr ? g.bias[n] : 0.f));
          ((float*)g.out)[(size_t)t * g.ldy + n] = sum;
          g.out2[(size_t)t * g.ld2 + n] = sum;
        }
      } else
      for (int e = (warp - 2) * 32 + lane; e < rows_per_cta * BN; e += 128) {
        const int j = e / rows_per_cta, rl = e - j * rows_per_cta;
        const int t = t0 + j, n = n0 + rank * rows_per_cta + rl;
        if (t >= g.T || n >= g.N) continue;
        float acc = 0.f;
        for (int peer = 0; peer < g.splits; ++peer)
          acc += recv[((size_t)peer * rows_per_cta + rl) * S::RECV_ROW + j];
        if (normed) acc *= ssq_s[j];
        store_output(g, (size_t)t * g.ldy + n, acc + (g.bias != nullptr ? g.bias[n] : 0.f));
      }
    }
    VX_TRACE_MARK(3);
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc),
                 "r"(S::TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// Host side: tensor maps (cached) and the launcher.
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) ==
            cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// A [rows, K] row-major bf16 matrix cut into boxes of [box_rows, 64], 128-byte swizzled.
static bool tensor_map_2d(CUtensorMap* map, const void* base, long long rows, long long K,
                          int box_rows) {
  static std::map<std::tuple<const void*, long long, long long, int>, CUtensorMap> cache;
  static std::mutex lock;
  const auto key = std::make_tuple(base, rows, K, box_rows);
  std::lock_guard<std::mutex> guard(lock);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *map = it->second;
    return true;
  }
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)GB_BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                            dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache[key] = *map;
  return true;
}

// Dynamic shared memory of a CTA that leaves room for a second one on its SM.
constexpr int TWO_PER_SM_BYTES = 113 * 1024;

// SMs of the current device (asked once).
static int device_sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0, value = 0;
    if (cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && value > 0)
      count = value;
    else
      count = 148;
  }
  return count;
}

// `one_wave`: launch only if all the grid's clusters are resident at once with this variant's
// shared memory (-2 otherwise: the caller takes the variant of which an SM holds two CTAs).
template <int BN, int STAGES_>
static int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx,
                       const GemmArgs& g, dim3 grid, cudaStream_t stream, bool one_wave = false) {
  using S = GemmShape<BN, STAGES_>;
  // The most dynamic shared memory a CTA may have beside the kernel's static arrays.
  static int dynamic_limit = 0;
  if (dynamic_limit == 0) {
    cudaFuncAttributes attributes_of;
    cudaError_t e = cudaFuncGetAttributes(&attributes_of, gemm_bf16_kernel<BN, STAGES_>);
    if (e != cudaSuccess) return (int)e;
    const int limit = 227 * 1024 - (int)attributes_of.sharedSizeBytes;
    e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES_>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             limit);
    if (e != cudaSuccess) return (int)e;
    dynamic_limit = limit;
  }
  // With the fused norm the X tiles follow the stages: all of the CTA's K blocks if they fit
  // (beside a second CTA on the SM when the grid has more CTAs than the device has SMs), else a
  // ring of at least two batches.
  size_t smem = S::SMEM_BYTES;
  GemmArgs launched = g;
  if (g.resid != nullptr) {
    if (BN > 64) return -2;
    const int batches = (g.kb_per_split + S::NORM_BATCH - 1) / S::NORM_BATCH;
    const size_t batch_bytes = (size_t)S::NORM_BATCH * S::B_BYTES;
    const bool shares_sm = (long long)grid.x * grid.y * grid.z > (long long)device_sm_count();
    // A grid of more CTAs than SMs runs in one wave only with two CTAs on an SM: the X tiles
    // then have to fit beside that (measured at the 7B sizes, 32 tokens: the gate|up projection
    // with a ring that filled the SM took 84 us, norm and projection as two kernels 61).
    const size_t budget = shares_sm ? (size_t)TWO_PER_SM_BYTES : (size_t)dynamic_limit;
    const size_t all_resident = S::SMEM_BYTES + (size_t)g.kb_per_split * S::B_BYTES;
    int ring;
    if (all_resident <= budget) {
      ring = batches;  // every tile in a place of its own
    } else if (BN <= 16 && S::SMEM_BYTES + 2 * batch_bytes <= budget) {
      // A ring, for the narrowest token tile only: every CTA reads the rows again, and at 64
      // tokens those are as many bytes as its weights.  Then the step is faster with the norm
      // as a kernel of its own (measured: 1.5B sizes, 64 tokens, 3.03 ms a step against 3.56;
      // 14B sizes, 32 tokens, QKV 41 us against 7 + 31).
      ring = (int)((budget - S::SMEM_BYTES) / batch_bytes);
      if (ring > S::NORM_MAX_BATCHES) ring = S::NORM_MAX_BATCHES;
      if (ring >= batches) ring = batches;
    } else if (all_resident <= (size_t)dynamic_limit && batches <= S::NORM_MAX_BATCHES) {
      ring = batches;  // fits, at the price of the SM to itself
    } else {
      return -2;
    }
    launched.x_slots = ring * S::NORM_BATCH;
    // All resident: exactly the CTA's K blocks (the last batch may be a short one); every
    // kilobyte counts where two CTAs are to share an SM.
    smem += ring == batches ? (size_t)g.kb_per_split * S::B_BYTES : (size_t)ring * batch_bytes;
  } else {
    launched.x_slots = S::NORM_BATCH;
    // Nothing is exchanged through shared memory without a cluster, a SwiGLU epilogue or the
    // norm: the launch leaves the receive area out, and with token tiles of 64 two CTAs then
    // fit on an SM, one loading while the other stores (the LM head at 64 rows: 1,187 CTAs).
    if (g.splits <= 1 && g.mode != 3) smem -= S::RECV_BYTES;
  }
  if (smem > (size_t)dynamic_limit) return -2;
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(GB_THREADS);
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
  if (g.splits > 1) {
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = 1;
    attributes[count].val.clusterDim.y = 1;
    attributes[count].val.clusterDim.z = (unsigned)g.splits;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  if (one_wave && g.splits > 1) {
    // Clusters of this size and shared memory that the device holds at a time (asked once).
    static std::map<std::pair<size_t, int>, int> held;
    static std::mutex held_lock;
    int active = 0;
    {
      std::lock_guard<std::mutex> guard(held_lock);
      const auto key = std::make_pair(smem, g.splits);
      auto it = held.find(key);
      if (it == held.end()) {
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_bf16_kernel<BN, STAGES_>, &config) != cudaSuccess) {
          (void)cudaGetLastError();
          clusters = 0;
        }
        it = held.emplace(key, clusters).first;
      }
      active = it->second;
    }
    const long long clusters_wanted = (long long)grid.x * grid.y;
    if (active > 0 && clusters_wanted > active) return -2;
  }
  return (int)cudaLaunchKernelEx(&config, gemm_bf16_kernel<BN, STAGES_>, mw, mw2, mx, launched);
}


// ---------------------------------------------------------------------------------------------
// The gated feed-forward of a small step (at most 32 tokens: a tile of 16 or of 32) in one kernel:
//   resid_out[t, :] += W_down * (silu(W_gate x_t) * (W_up x_t)),  x_t = rmsnorm(resid_in[t, :]) * w_norm.
// CTA j owns 64 features of the inner width: it streams their 64 gate rows and 64 up rows of
// [2 I, E] (as the SwiGLU mode above, the input norm made on the spot), turns the accumulator
// into the [tokens x 64 features] bf16 activation tile in shared memory, and goes straight
// on, with the same ring of stages, to the 64 columns of W_down [E, I] that belong to these
// features: E / 128 tiles of [128 rows x 64], each one product with the activation tile, each
// with one tile width of tensor-memory columns of its own.  What comes out is this CTA's share of the sum
// over the inner width; the shares meet in the float32 residual stream by reductions at the
// L2 (red.global.add.f32), so their order, and with it the last bits of the sum, is not fixed.
// The activations never leave the SM, the W_down tiles are already on their way while the
// activation is computed, and a layer has one kernel boundary less.
// resid_in must not be resid_out: other CTAs add to resid_out while this one still reads its
// input rows.
// ---------------------------------------------------------------------------------------------
struct MlpArgs {
  const float* resid_in;  // [T, resid_in_ld] float32; nobody writes it during the launch
  const float* norm_w;    // [E]
  float* resid_out;       // [T, resid_out_ld] float32
  long long resid_in_ld, resid_out_ld;
  int* status;
  float eps;
  int T, E, I;
  int tmem_cols;          // tile width x (1 + E / 128), rounded up to a power of two (at least 32)
};

constexpr int MF_MAX_BN = 32;
constexpr int MF_MAX_BATCHES = 32;
constexpr int MF_MAX_TILES = 31;  // row tiles of W_down: MF_BN columns of tensor memory each, after the first MF_BN

// MF_BN: tokens of the tile (16 or 32).  MF_STAGES: stages of 16 KB, as many as fit beside the X tiles.
template <int MF_BN, int MF_STAGES>
__global__ void __launch_bounds__(GB_THREADS, 1)
mlp_fused_kernel(const __grid_constant__ CUtensorMap map_gate, const __grid_constant__ CUtensorMap map_up,
                 const __grid_constant__ CUtensorMap map_down, MlpArgs m) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[MF_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MF_STAGES];
  __shared__ __align__(8) uint64_t acc1_bar, act_bar;
  __shared__ __align__(8) uint64_t tile_bar[MF_MAX_TILES];  // row tile i of the second part is in tensor memory
  __shared__ __align__(8) uint64_t x_bar[MF_MAX_BATCHES];
  __shared__ uint32_t tmem_slot;
  __shared__ int epilogue_failed;
  __shared__ float rstd_s[MF_BN];
  __shared__ float swap_buf[64 * (MF_BN + 1)];
  constexpr uint32_t MF_X_BYTES = MF_BN * GB_BK * 2;
  constexpr int MF_NORM_BATCH = MF_BN == 16 ? 6 : 3;

  VX_TRACE_SCOPE(15);
  allow_dependents();
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  // stages | activation tile | X tiles of the E / 64 blocks of the first product
  const uint32_t act_addr = smem_base + MF_STAGES * GB_A_BYTES;
  const uint32_t x_addr = act_addr + MF_X_BYTES;
  unsigned char* act_tile = smem_al + MF_STAGES * GB_A_BYTES;
  unsigned char* x_tiles = act_tile + MF_X_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 64;    // first of this CTA's features of the inner width
  const int kb1 = m.E / GB_BK;       // blocks of K of the first product
  const int tiles2 = m.E / GB_BM;    // row tiles of W_down
  const int total = kb1 + tiles2;

  if (threadIdx.x == 0) {
    epilogue_failed = 0;
    for (int s = 0; s < MF_STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < MF_MAX_BATCHES; ++b) mbar_init(smem_u32(&x_bar[b]), 1);
    mbar_init(smem_u32(&acc1_bar), 1);
    for (int i = 0; i < MF_MAX_TILES; ++i) mbar_init(smem_u32(&tile_bar[i]), 1);
    mbar_init(smem_u32(&act_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(m.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_slot;  // columns 0..MF_BN-1: gate|up; MF_BN (1 + i) ..: row tile i of W_down

  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- TMA producer
    // Weights only: nothing here depends on the kernel before this one.
    auto load = [&](int i) {
      const int stage = i % MF_STAGES;
      const uint32_t full = smem_u32(&full_bar[stage]);
      const uint32_t dst = smem_base + stage * GB_A_BYTES;
      mbar_expect_tx(full, GB_A_BYTES);
      if (i < kb1) {
        tma_load_2d(dst, &map_gate, i * GB_BK, n0, full);
        tma_load_2d(dst + GB_A_BYTES / 2, &map_up, i * GB_BK, n0, full);
      } else {
        tma_load_2d(dst, &map_down, n0, (i - kb1) * GB_BM, full);
      }
    };
    const int first_round = min(total, MF_STAGES);
    for (int i = 0; i < first_round; ++i) load(i);
    for (int i = first_round; i < total; ++i) {
      const int stage = i % MF_STAGES;
      const uint32_t phase = (uint32_t)(i / MF_STAGES) & 1u;
      if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, m.status)) break;
      load(i);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = umma_instr_desc(MF_BN);
    bool ok = true;
    for (int i = 0; i < kb1 && ok; ++i) {
      const int stage = i % MF_STAGES;
      const uint32_t phase = (uint32_t)(i / MF_STAGES) & 1u;
      ok = mbar_wait(smem_u32(&full_bar[stage]), phase, m.status);
      if (ok && i % MF_NORM_BATCH == 0) ok = mbar_wait(smem_u32(&x_bar[i / MF_NORM_BATCH]), 0u, m.status);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = smem_base + stage * GB_A_BYTES;
      const uint32_t b_addr = x_addr + i * MF_X_BYTES;
#pragma unroll
      for (int k = 0; k < GB_BK / 16; ++k)
        umma_bf16(tmem_acc, umma_smem_desc(a_addr + k * 32), umma_smem_desc(b_addr + k * 32), idesc,
                  (i > 0 || k > 0) ? 1u : 0u);
      umma_commit(smem_u32(&empty_bar[stage]));
    }
    umma_commit(smem_u32(&acc1_bar));
    // The activation tile is the B operand of every product of the second part.
    if (ok) ok = mbar_wait(smem_u32(&act_bar), 0u, m.status);
    for (int t2 = 0; t2 < tiles2 && ok; ++t2) {
      const int i = kb1 + t2;
      const int stage = i % MF_STAGES;
      const uint32_t phase = (uint32_t)(i / MF_STAGES) & 1u;
      ok = mbar_wait(smem_u32(&full_bar[stage]), phase, m.status);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = smem_base + stage * GB_A_BYTES;
#pragma unroll
      for (int k = 0; k < GB_BK / 16; ++k)
        umma_bf16(tmem_acc + (uint32_t)MF_BN * (1u + (uint32_t)t2), umma_smem_desc(a_addr + k * 32),
                  umma_smem_desc(act_addr + k * 32), idesc, k > 0 ? 1u : 0u);
      umma_commit(smem_u32(&empty_bar[stage]));
      umma_commit(smem_u32(&tile_bar[t2]));
    }
  } else if (warp >= 2) {
    // ---------------------------------------------------------------- norm, activation, output
    grid_dependency_wait();
    const int q = (int)threadIdx.x - 64;
    {
      // X tiles: thread q takes the 16-byte chunk q % 8 of tokens q / 8 (+ 16) in every K block.
      constexpr int NB = MF_NORM_BATCH;
      constexpr int CPT = MF_BN / 16;  // chunks (tokens) per thread and K block
      const int c = q & 7;
      float ssq[CPT];
#pragma unroll
      for (int u = 0; u < CPT; ++u) ssq[u] = 0.f;
      for (int i0 = 0; i0 < kb1; i0 += NB) {
        float4 xa[NB][CPT], xb[NB][CPT], wa[NB], wb[NB];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          const int k = (i0 + j) * GB_BK + c * 8;
          const bool in_k = i0 + j < kb1;
          wa[j] = in_k ? __ldg(reinterpret_cast<const float4*>(m.norm_w + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
          wb[j] = in_k ? __ldg(reinterpret_cast<const float4*>(m.norm_w + k + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < CPT; ++u) {
            const int r = (q >> 3) + 16 * u;
            const bool on = in_k && r < m.T;
            const float* src = m.resid_in + (size_t)r * m.resid_in_ld + k;
            xa[j][u] = on ? *reinterpret_cast<const float4*>(src) : make_float4(0.f, 0.f, 0.f, 0.f);
            xb[j][u] = on ? *reinterpret_cast<const float4*>(src + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          if (i0 + j >= kb1) break;
#pragma unroll
          for (int u = 0; u < CPT; ++u) {
            const int r = (q >> 3) + 16 * u;
            const float4 a4 = xa[j][u], b4 = xb[j][u];
            ssq[u] += a4.x * a4.x + a4.y * a4.y + a4.z * a4.z + a4.w * a4.w +
                      b4.x * b4.x + b4.y * b4.y + b4.z * b4.z + b4.w * b4.w;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(a4.x * wa[j].x, a4.y * wa[j].y);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(a4.z * wa[j].z, a4.w * wa[j].w);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(b4.x * wb[j].x, b4.y * wb[j].y);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(b4.z * wb[j].z, b4.w * wb[j].w);
            *reinterpret_cast<uint4*>(x_tiles + (size_t)(i0 + j) * MF_X_BYTES + r * 128 + ((c ^ (r & 7)) << 4)) =
                make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                           *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (q == 0) mbar_arrive(smem_u32(&x_bar[i0 / NB]));
      }
      // The eight threads of a token sit in consecutive lanes.
#pragma unroll
      for (int u = 0; u < CPT; ++u) {
        float v = ssq[u];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if (c == 0) rstd_s[(q >> 3) + 16 * u] = rsqrtf(v / (float)m.E + m.eps);
      }
    }
    const int quarter = warp & 3;  // TMEM lanes 32 * quarter .. + 31 belong to this warp
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem_acc + ((uint32_t)(quarter * 32) << 16);
    if (!mbar_wait(smem_u32(&acc1_bar), 0u, m.status)) epilogue_failed = 1;
    asm volatile("bar.sync 1, 128;" ::: "memory");  // also: rstd_s is written
    bool ready = epilogue_failed == 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    float v[32];
    if (ready) {
      if (MF_BN == 32) tmem_load_32(lane_base, v); else tmem_load_16(lane_base, v);
    } else {
#pragma unroll
      for (int j = 0; j < MF_BN; ++j) v[j] = 0.f;
    }
    // Rows 0..63 are gate, 64..127 up of the same 64 features: up rows hand their values over.
    if (row >= 64) {
#pragma unroll
      for (int j = 0; j < MF_BN; ++j) swap_buf[(row - 64) * (MF_BN + 1) + j] = v[j];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (row < 64) {
      // Activation tile [MF_BN tokens x 64 features] bf16, K-major, 128-byte swizzled: feature f
      // of token t in chunk (f / 8) ^ (t & 7) of row t.
#pragma unroll
      for (int j = 0; j < MF_BN; ++j) {
        const float scale = rstd_s[j];
        const float gate = v[j] * scale, up = swap_buf[row * (MF_BN + 1) + j] * scale;
        const float a = j < m.T ? gate / (1.0f + __expf(-gate)) * up : 0.f;
        *reinterpret_cast<__nv_bfloat16*>(act_tile + j * 128 + ((((row >> 3) ^ (j & 7))) << 4) + (row & 7) * 2) =
            __float2bfloat16_rn(a);
      }
    }
    // The tensor core reads the tile through the async proxy.
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (q == 0) mbar_arrive(smem_u32(&act_bar));

    // Row tiles are written out as they finish, the last ones while their weights still arrive.
    if (ready) {
      for (int t2 = 0; t2 < tiles2; ++t2) {
        if (!mbar_wait(smem_u32(&tile_bar[t2]), 0u, m.status)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t at = lane_base + (uint32_t)MF_BN * (1u + (uint32_t)t2);
        if (MF_BN == 32) tmem_load_32(at, v); else tmem_load_16(at, v);
        float* dst = m.resid_out + (size_t)t2 * GB_BM + row;
#pragma unroll
        for (int j = 0; j < MF_BN; ++j)
          if (j < m.T)
            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + (size_t)j * m.resid_out_ld), "f"(v[j]) : "memory");
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(m.tmem_cols)
                 : "memory");
  }
}

}  // namespace vx

using namespace vx;

VX_TRACE_API(vx_gemm)

// Token-tile widths the kernel is built for.
VX_API int vx_gemm_bf16_token_tile(int num_tokens) {
  if (num_tokens <= 16) return 16;
  if (num_tokens <= 32) return 32;
  if (num_tokens <= 64) return 64;
  if (num_tokens <= 128) return 128;
  return 256;
}

static int sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0, value = 0;
    if (cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && value > 0)
      count = value;
    else
      count = 148;
  }
  return count;
}

// Largest power of two <= value, at most `most`.
static int floor_pow2(int value, int most) {
  int p = 1;
  while (p * 2 <= value && p * 2 <= most) p *= 2;
  return p;
}

// x [T, K] bf16, w [N, K] bf16 (mode 3: w [2 * N, K], gate rows then up rows).
// x_rows is the number of rows the x buffer really has (>= T); rows T.. are read but their
// results are never written.  `splits` (rounded down to 1, 2, 4 or 8 and to what K and the
// token tile allow) CTAs share each output tile as a cluster.
// With resid != null the input is rmsnorm(resid) * norm_w instead of x (see the head of the
// file); x is then not read and T must be at most 64.
// Returns 0 on launch, a cudaError_t on failure, -1 if the sizes are refused (K not a multiple
// of 8, unaligned pointers, no driver entry point), or -2 if the fused norm's tiles do not fit
// in shared memory (the caller then runs the norm by itself).
struct RopeArgs {
  const int* positions;
  const float* cos_t;
  const float* sin_t;
  const int* slots;
  void* k_cache;
  void* v_cache;
  int heads, kv_heads, max_pos;
  long long num_slots;
};

static int gemm_bf16(const void* x, int x_rows, const float* resid, long long resid_ld,
                     const float* norm_w, float eps, const void* w, const float* bias, void* out,
                     int mode, int T, int N, int K, long long ldy, int splits, int* status,
                     cudaStream_t stream, const RopeArgs* rope = nullptr, float* out2 = nullptr,
                     long long ld2 = 0, int chunks = 1) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) != 0) return -1;
  const bool normed = resid != nullptr;
  if (reinterpret_cast<uintptr_t>(w) & 15) return -1;
  if (!normed && (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  if (normed && (T > 64 || norm_w == nullptr || (resid_ld % 4) != 0 ||
                 (reinterpret_cast<uintptr_t>(resid) & 15) || (reinterpret_cast<uintptr_t>(norm_w) & 15)))
    return -1;
  if (mode < 0 || mode > 4 || (mode == 4) != (rope != nullptr)) return -1;
  const int bn = vx_gemm_bf16_token_tile(T);
  const int num_kb = (K + GB_BK - 1) / GB_BK;
  if (splits < 1 || mode == 3 || bn > 64) splits = 1;
  splits = floor_pow2(splits < num_kb ? splits : num_kb, GB_MAX_SPLITS);
  if (splits > bn) splits = bn;
  if (normed && bn <= 64) {
    // With the norm made in the kernel the X tiles lie in shared memory beside the stages.  A
    // grid of more CTAs than SMs needs two CTAs on an SM to run in one wave; where the tiles
    // (or a ring of two batches of them, narrowest token tile only) do not leave room for
    // that, fewer and longer splits do better.
    const long long tiles = (long long)((N + (mode == 3 ? 64 : GB_BM) - 1) / (mode == 3 ? 64 : GB_BM)) * ((T + bn - 1) / bn);
    const size_t b_bytes = (size_t)bn * GB_BK * 2;
    const size_t recv = ((size_t)GB_BM * (bn + 4) * 4 + GB_MAX_SPLITS * bn * 4 + 1023) / 1024 * 1024;
    const size_t base = 4 * (GB_A_BYTES + b_bytes) + recv + 1024;
    const size_t batch = (size_t)(bn <= 16 ? 6 : (bn <= 32 ? 4 : 2)) * b_bytes;
    while (splits > (mode == 4 ? 2 : 1) && tiles * splits > (long long)sm_count()) {
      const size_t kb = (size_t)(num_kb + splits - 1) / splits;
      if (base + kb * b_bytes <= (size_t)TWO_PER_SM_BYTES || (bn <= 16 && base + 2 * batch <= (size_t)TWO_PER_SM_BYTES)) break;
      splits /= 2;
    }
  }
  if (mode == 4) {
    // Heads of 128 dims, rotated in the cluster exchange's final sum: split K only.
    if (splits < 2 || rope->heads <= 0 || rope->kv_heads <= 0 ||
        N != (rope->heads + 2 * rope->kv_heads) * 128)
      return -2;
  }
  GemmArgs g;
  g.bias = bias;
  g.out = out;
  g.status = status;
  g.ldy = ldy;
  g.T = T;
  g.N = N;
  g.K = K;
  g.mode = mode;
  g.kb_per_split = (num_kb + splits - 1) / splits;
  g.splits = splits;
  // K in chunks of independent CTAs (mode 2 only): every CTA adds its partial tile to the output
  // by reductions at the L2, so no cluster and any number of chunks; the order of the additions
  // is then not fixed.
  if (chunks > 1) {
    if (mode != 2 || normed || bias != nullptr || out2 != nullptr || rope != nullptr) return -1;
    if (chunks > num_kb) chunks = num_kb;
    g.splits = 1;
    g.kb_per_split = (num_kb + chunks - 1) / chunks;
    chunks = (num_kb + g.kb_per_split - 1) / g.kb_per_split;  // no empty chunk
  } else {
    chunks = 1;
  }
  g.resid = resid;
  g.norm_w = norm_w;
  g.resid_ld = resid_ld;
  g.eps = eps;
  g.positions = nullptr;
  g.cos_t = g.sin_t = nullptr;
  g.slots = nullptr;
  g.k_cache = g.v_cache = nullptr;
  g.heads = g.kv_heads = g.max_pos = 0;
  g.num_slots = 0;
  g.out2 = out2;
  g.ld2 = ld2;
  // The second output: mode 2, split K, at most eight elements per thread of the final sum.
  if (out2 != nullptr && (mode != 2 || splits < 2 || (GB_BM / splits) * bn > 8 * 128)) return -4;
  if (rope != nullptr) {
    g.positions = rope->positions;
    g.cos_t = rope->cos_t;
    g.sin_t = rope->sin_t;
    g.slots = rope->slots;
    g.k_cache = rope->k_cache;
    g.v_cache = rope->v_cache;
    g.heads = rope->heads;
    g.kv_heads = rope->kv_heads;
    g.max_pos = rope->max_pos;
    g.num_slots = rope->num_slots;
  }

  CUtensorMap mw, mw2, mx;
  if (mode == 3) {
    if (!tensor_map_2d(&mw, w, N, K, 64)) return -1;
    if (!tensor_map_2d(&mw2, (const __nv_bfloat16*)w + (size_t)N * K, N, K, 64)) return -1;
  } else {
    if (!tensor_map_2d(&mw, w, N, K, GB_BM)) return -1;
    mw2 = mw;
  }
  if (normed) {
    mx = mw;  // not used
  } else {
    if (x_rows < T) return -1;
    if (!tensor_map_2d(&mx, x, x_rows, K, bn)) return -1;
  }
  const int n_tile = mode == 3 ? 64 : GB_BM;
  const dim3 grid((N + n_tile - 1) / n_tile, (T + bn - 1) / bn, chunks > 1 ? chunks : splits);
  // A grid that gives an SM one CTA at most keeps more tiles in flight per CTA instead.
  const bool deep = bn <= 32 && g.kb_per_split > 4 &&
                    (long long)grid.x * grid.y * grid.z <= (long long)sm_count();
  switch (bn) {
    case 16: {
      const int code = deep ? launch_gemm<16, 8>(mw, mw2, mx, g, grid, stream, true) : -2;
      return code != -2 ? code : launch_gemm<16, 4>(mw, mw2, mx, g, grid, stream);
    }
    case 32: {
      const int code = deep ? launch_gemm<32, 8>(mw, mw2, mx, g, grid, stream, true) : -2;
      return code != -2 ? code : launch_gemm<32, 4>(mw, mw2, mx, g, grid, stream);
    }
    // A short K chunk needs no deep ring, and with two stages two CTAs share an SM: sixteen
    // clusters of eight then run in one wave (one CTA per SM fits fifteen of them on this GPU).
    case 64: return g.kb_per_split <= 4 ? launch_gemm<64, 2>(mw, mw2, mx, g, grid, stream)
                                        : launch_gemm<64, 4>(mw, mw2, mx, g, grid, stream);
    case 128: return launch_gemm<128, 4>(mw, mw2, mx, g, grid, stream);
    default: return launch_gemm<256, 4>(mw, mw2, mx, g, grid, stream);
  }
}

VX_API int vx_gemm_bf16(const void* x, const void* w, const float* bias, void* out, int mode,
                        int T, int x_rows, int N, int K, long long ldy, int splits,
                        int* status, cudaStream_t stream) {
  return gemm_bf16(x, x_rows, nullptr, 0, nullptr, 0.f, w, bias, out, mode, T, N, K, ldy, splits,
                   status, stream);
}

// Mode 2 (out += x w^T, float32) that also writes the sums to out2 [T, ld2]: a copy of the rows
// for a later kernel that reads them while others already add to `out` again.  -4 (nothing
// launched) where the launch would not split K or a thread would own more than eight sums.
VX_API int vx_gemm_bf16_add_mirrored(const void* x, const void* w, float* out, float* out2, int T,
                                     int x_rows, int N, int K, long long ldy, long long ld2, int splits,
                                     int* status, cudaStream_t stream) {
  if (out2 == nullptr) return -1;
  return gemm_bf16(x, x_rows, nullptr, 0, nullptr, 0.f, w, nullptr, out, 2, T, N, K, ldy, splits, status,
                   stream, nullptr, out2, ld2);
}

// Mode 2 (out += x w^T, float32) with K cut into `chunks` ranges that independent CTAs take:
// each adds its partial tile to `out` by float32 reductions at the L2.  Fills the GPU whatever
// the number of output tiles (a cluster holds eight CTAs at most and wants a power of two);
// the order of the additions, and with it the last bits of the sums, is not fixed.
VX_API int vx_gemm_bf16_add_chunked(const void* x, const void* w, float* out, int T, int x_rows, int N, int K,
                                    long long ldy, int chunks, int* status, cudaStream_t stream) {
  return gemm_bf16(x, x_rows, nullptr, 0, nullptr, 0.f, w, nullptr, out, 2, T, N, K, ldy, 1, status, stream,
                   nullptr, nullptr, 0, chunks < 1 ? 1 : chunks);
}

// The same product on rmsnorm(resid) * norm_w: resid [T, resid_ld] float32, norm_w [K] float32.
VX_API int vx_gemm_bf16_normed(const float* resid, long long resid_ld, const float* norm_w,
                               float eps, const void* w, const float* bias, void* out, int mode,
                               int T, int N, int K, long long ldy, int splits, int* status,
                               cudaStream_t stream) {
  if (resid == nullptr) return -1;
  return gemm_bf16(nullptr, 0, resid, resid_ld, norm_w, eps, w, bias, out, mode, T, N, K, ldy,
                   splits, status, stream);
}

// The QKV projection of heads of 128 dims with the rotation and the cache write in its
// epilogue (mode 4): w [(heads + 2 kv_heads) * 128, K]; query heads go to out bf16 [T, ldy]
// rotated, key heads rotated and value heads as they are into k_cache / v_cache [num_slots,
// kv_heads, 128] at slots[t] (null caches: nothing is written).  The input is x, or
// rmsnorm(resid) * norm_w when resid is given.  -2: this shape is not taken (no split K, other
// head sizes, too many tokens); the caller runs the projection and the rotation separately.
VX_API int vx_gemm_bf16_qkv_rope(const void* x, int x_rows, const float* resid, long long resid_ld,
                                 const float* norm_w, float eps, const void* w, const float* bias,
                                 void* out, int T, int K, long long ldy, int splits,
                                 const int* positions, const float* cos_t, const float* sin_t,
                                 int max_pos, const int* slots, void* k_cache, void* v_cache,
                                 long long num_slots, int heads, int kv_heads, int* status,
                                 cudaStream_t stream) {
  if (T > 64) return -2;
  RopeArgs rope = {positions, cos_t, sin_t, slots, k_cache, v_cache, heads, kv_heads, max_pos, num_slots};
  return gemm_bf16(x, x_rows, resid, resid_ld, norm_w, eps, w, bias, out, 4, T,
                   (heads + 2 * kv_heads) * 128, K, ldy, splits, status, stream, &rope);
}

// One instantiation of the fused feed-forward: the most dynamic shared memory a CTA of it may
// have (set once; minus a cudaError_t on failure) and its launch.
template <int BN, int STAGES>
struct MlpFusedVariant {
  static int limit() {
    static int value = 0;
    if (value == 0) {
      cudaFuncAttributes attributes_of;
      cudaError_t e = cudaFuncGetAttributes(&attributes_of, mlp_fused_kernel<BN, STAGES>);
      if (e != cudaSuccess) return -(int)e;
      const int most = 227 * 1024 - (int)attributes_of.sharedSizeBytes;
      e = cudaFuncSetAttribute(mlp_fused_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
      if (e != cudaSuccess) return -(int)e;
      value = most;
    }
    return value;
  }
  // 0 launched, a cudaError_t, or -2 if `tiles_bytes` beside the stages do not fit.
  static int launch(cudaLaunchConfig_t& config, size_t tiles_bytes, const CUtensorMap& mg, const CUtensorMap& mu,
                    const CUtensorMap& md, const MlpArgs& m) {
    const int most = limit();
    if (most < 0) return -most;
    const size_t smem = (size_t)STAGES * GB_A_BYTES + tiles_bytes;
    if (smem > (size_t)most) return -2;
    config.dynamicSmemBytes = smem;
    return (int)cudaLaunchKernelEx(&config, mlp_fused_kernel<BN, STAGES>, mg, mu, md, m);
  }
};

// The gated feed-forward of at most 32 tokens in one kernel (see mlp_fused_kernel):
// resid_out += W_down (silu(W_gate x) * (W_up x)), x = rmsnorm(resid_in) * norm_w, with
// w_gate_up [2 I, E] (gate rows, then up rows) and w_down [E, I] bf16.  Returns 0 on launch, a
// cudaError_t on failure, -1 if the arguments are refused (more than 32 tokens, E no multiple
// of 128, I no multiple of 64, unaligned pointers, resid_in == resid_out), -2 if a row this wide
// does not fit in shared or tensor memory (the caller then uses the separate projections).
VX_API int vx_mlp_fused(const float* resid_in, long long resid_in_ld, const float* norm_w, float eps,
                        const void* w_gate_up, const void* w_down, float* resid_out,
                        long long resid_out_ld, int T, int E, int I, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (T > MF_MAX_BN || E <= 0 || I <= 0 || (E % GB_BM) != 0 || (I % 64) != 0) return -1;
  if (resid_in == nullptr || resid_out == nullptr || norm_w == nullptr || (const float*)resid_out == resid_in) return -1;
  if ((reinterpret_cast<uintptr_t>(resid_in) & 15) || (reinterpret_cast<uintptr_t>(norm_w) & 15) ||
      (reinterpret_cast<uintptr_t>(w_gate_up) & 15) || (reinterpret_cast<uintptr_t>(w_down) & 15) ||
      (resid_in_ld % 4) != 0)
    return -1;
  const int bn = T <= 16 ? 16 : 32;
  const int norm_batch = bn == 16 ? 6 : 3;
  const int kb1 = E / GB_BK, tiles2 = E / GB_BM;
  if ((kb1 + norm_batch - 1) / norm_batch > MF_MAX_BATCHES || tiles2 > MF_MAX_TILES) return -2;
  int cols = 32;
  while (cols < bn * (1 + tiles2)) cols *= 2;
  if (cols > 512) return -2;
  // The activation tile and the X tiles of the first product's K blocks, and the alignment.
  const size_t tiles_bytes = (size_t)(1 + kb1) * bn * GB_BK * 2 + 1024;
  CUtensorMap mg, mu, md;
  if (!tensor_map_2d(&mg, w_gate_up, I, E, 64)) return -1;
  if (!tensor_map_2d(&mu, (const __nv_bfloat16*)w_gate_up + (size_t)I * E, I, E, 64)) return -1;
  if (!tensor_map_2d(&md, w_down, E, I, GB_BM)) return -1;
  MlpArgs m;
  m.resid_in = resid_in;
  m.norm_w = norm_w;
  m.resid_out = resid_out;
  m.resid_in_ld = resid_in_ld;
  m.resid_out_ld = resid_out_ld;
  m.status = status;
  m.eps = eps;
  m.T = T;
  m.E = E;
  m.I = I;
  m.tmem_cols = cols;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(I / 64);
  config.blockDim = dim3(GB_THREADS);
  config.stream = stream;
  cudaLaunchAttribute attributes[1];
  int count = 0;
  const char* serialised = getenv("VELOX_B200_NO_PDL");
  if (serialised == nullptr || serialised[0] != '1') {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  // As many stages as fit beside the tiles.
  int code;
  if (bn == 16) {
    code = MlpFusedVariant<16, 10>::launch(config, tiles_bytes, mg, mu, md, m);
    if (code == -2) code = MlpFusedVariant<16, 8>::launch(config, tiles_bytes, mg, mu, md, m);
    if (code == -2) code = MlpFusedVariant<16, 4>::launch(config, tiles_bytes, mg, mu, md, m);
  } else {
    code = MlpFusedVariant<32, 7>::launch(config, tiles_bytes, mg, mu, md, m);
    if (code == -2) code = MlpFusedVariant<32, 4>::launch(config, tiles_bytes, mg, mu, md, m);
  }
  return code;
}
