// On-device sampling over float32 logits [R, V]: greedy, temperature, top-k, top-p, and the
// repetition / presence / frequency penalties.
//
// What is sampled follows the reference's sampler (engine/sampler.py:131-258 in that project):
//   penalties   logit[v] -= frequency * count(v); then logit[v] = logit[v] > 0 ? logit[v] / rep
//               : logit[v] * rep; then logit[v] -= presence, for every token v in the request's
//               prompt and output so far (sampler.py:169-189);
//   greedy      argmax, first index on ties (sampler.py:155-156);
//   otherwise   scaled = logit / max(temperature, 1e-5); candidates are the k most probable
//               tokens and the smallest most-probable set whose mass reaches top_p
//               (sampler.py:216-228); the draw is the exponential race
//               argmax(p / noise), noise ~ Exp(1) clamped at 1e-10 (sampler.py:230-258).
// How it is done differs: the race runs over the whole vocabulary as argmax(scaled - log noise)
// (the same draw, since log is monotone and the normaliser is a constant), the candidate set is
// found as a value threshold, digit by digit of its bit pattern, instead of by a sort, and the noise comes from a
// counter-based generator (Philox4x32-10) keyed by the request's seed and counted by
// (index of the output token, vocabulary index), so a request's draws do not depend on what
// else is in the batch.  Bit-equality with torch's generator stream is not a goal.
#include "common.cuh"

#include <math_constants.h>

namespace vx {

// ---------------------------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// Uniform in (0, 1) from 32 random bits.
__device__ __forceinline__ float uniform_open(uint32_t bits) {
  return ((float)(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

// Order-preserving map float -> uint32 (larger float, larger key).
__device__ __forceinline__ uint32_t float_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  const uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(b);
}

struct Best {
  float score;
  int index;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  // Larger score wins; on equal scores the lower index (torch.argmax returns the first maximum).
  if (b.index < 0) return a;
  if (a.index < 0) return b;
  if (b.score > a.score || (b.score == a.score && b.index < a.index)) return b;
  return a;
}

__device__ __forceinline__ Best block_best(Best v, Best* scratch /* 32 */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int num_warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    Best o;
    o.score = __shfl_xor_sync(0xffffffffu, v.score, offset);
    o.index = __shfl_xor_sync(0xffffffffu, v.index, offset);
    v = better(v, o);
  }
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    Best w;
    w.score = 0.f;
    w.index = -1;
    if (lane < num_warps) w = scratch[lane];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      Best o;
      o.score = __shfl_xor_sync(0xffffffffu, w.score, offset);
      o.index = __shfl_xor_sync(0xffffffffu, w.index, offset);
      w = better(w, o);
    }
    if (lane == 0) scratch[0] = w;
  }
  __syncthreads();
  const Best out = scratch[0];
  __syncthreads();
  return out;
}

// ---------------------------------------------------------------------------------------------
// One token per row.  temperature[r] == 0: argmax.  Otherwise the exponential race over the
// entries with logit / T >= threshold[r] (threshold may be null: no filter).
//
// A row is cut into gridDim.y segments (multiples of four entries, so that the generator's
// counter, the index of a group of four, means the same for every cut).  Every block leaves its
// best entry in `partial`; the block that arrives last at the row's counter takes the best of
// all of them (`better` is associative and commutative, ties included, so the result does not
// depend on the cut or on the order of arrival), writes the token and puts the counter back to
// zero for the next launch.
// ---------------------------------------------------------------------------------------------
constexpr int SAMPLE_THREADS = 256;
constexpr int SAMPLE_MAX_SEGMENTS = 64;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
              const float* __restrict__ temperature, const unsigned long long* __restrict__ seeds,
              const int* __restrict__ draw_index, const float* __restrict__ threshold,
              int* __restrict__ out, int* __restrict__ history, long long history_stride,
              const int* __restrict__ history_slots, const int* __restrict__ history_lengths,
              int segment_len, Best* __restrict__ partial, unsigned int* __restrict__ counters,
              const int* __restrict__ status_word) {
  __shared__ Best scratch[32];
  __shared__ bool is_last;
  allow_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int segments = (int)gridDim.y;
  const int begin = blockIdx.y * segment_len;
  const int end = min(vocab, begin + segment_len);
  const float* row = logits + (size_t)r * row_stride;
  const float temp = temperature ? temperature[r] : 0.f;
  // Groups of four entries by one 16-byte load where the row allows it.
  const bool vec = (row_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  Best best;
  best.score = 0.f;
  best.index = -1;

  if (temp == 0.f) {
    for (int base = begin + threadIdx.x * 4; base < end; base += SAMPLE_THREADS * 4) {
      float v[4];
      if (vec && base + 4 <= vocab) {
        const float4 q = *reinterpret_cast<const float4*>(row + base);
        v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = base + j < vocab ? row[base + j] : CUDART_NAN_F;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        Best c;
        c.score = v[j];
        c.index = base + j;
        if (c.score == c.score) best = better(best, c);
      }
    }
  } else {
    const float inv_t = 1.0f / fmaxf(temp, 1e-5f);
    const float cut = threshold ? threshold[r] : -CUDART_INF_F;
    const unsigned long long seed = seeds[r];
    const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
    const uint32_t draw = (uint32_t)draw_index[r];
    for (int base = begin + threadIdx.x * 4; base < end; base += SAMPLE_THREADS * 4) {
      float v[4];
      if (vec && base + 4 <= vocab) {
        const float4 q = *reinterpret_cast<const float4*>(row + base);
        v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = base + j < vocab ? row[base + j] : CUDART_NAN_F;
      }
      const uint4 bits = philox4x32_10(make_uint4((uint32_t)(base >> 2), draw, 0u, 0u), key);
      const uint32_t b[4] = {bits.x, bits.y, bits.z, bits.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float scaled = v[j] * inv_t;
        if (!(scaled >= cut)) continue;  // also what lies past the row's end (NaN)
        const float noise = fmaxf(-logf(uniform_open(b[j])), 1e-10f);
        Best c;
        c.score = scaled - logf(noise);
        c.index = base + j;
        best = better(best, c);
      }
    }
  }
  best = block_best(best, scratch);
  if (segments > 1) {
    if (threadIdx.x == 0) {
      partial[(size_t)r * segments + blockIdx.y] = best;
      __threadfence();
      is_last = atomicAdd(&counters[r], 1u) == (unsigned int)segments - 1u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    best.score = 0.f;
    best.index = -1;
    if ((int)threadIdx.x < segments) {
      const volatile Best* p = partial + (size_t)r * segments + threadIdx.x;
      best.score = p->score;
      best.index = p->index;
    }
    best = block_best(best, scratch);
    if (threadIdx.x == 0) counters[r] = 0u;
  }
  if (threadIdx.x == 0) {
    const int token = best.index < 0 ? 0 : best.index;
    out[r] = token;
    // The device status word rides behind the tokens, so the host's one read-back of the step
    // also tells it whether a kernel of the step refused an access or gave up a wait.
    if (status_word != nullptr && r == 0) out[gridDim.x] = *reinterpret_cast<const volatile int*>(status_word);
    // Append to the request's token history (kept for the penalties) when there is one.
    if (history != nullptr) {
      const int n = history_lengths[r];
      if (n >= 0 && n < history_stride) history[(size_t)history_slots[r] * history_stride + n] = token;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Candidate threshold for top-k / top-p.  For a value x let count(x) be the number of entries
// with scaled > x and mass(x) their softmax probability.  An entry is a candidate iff
// count(scaled_i) < k (when k > 0) and mass(scaled_i) < top_p: it is among the k largest, and
// the entries before it do not already reach top_p.  Both are monotone in x, so the candidates
// are the entries >= a threshold: the smallest x with count(x) < k and mass(x) < top_p.
//
// The threshold is found digit by digit over the ordered bit patterns of float (11 + 11 + 10
// bits): a sweep over the row builds, in shared memory, the histogram of the next digit among
// the entries that share the digits found so far (how many, and their mass); the digit is the
// smallest one above which count and mass still pass.  Four sweeps over the row in all (maximum,
// three digits; the first digit's histogram also gives the normaliser) where a bisection over
// the patterns took up to 34.  Masses are summed as 2^-40 fixed-point
// integers, so the histogram, and with it the threshold, does not depend on the order in which
// threads add.
// ---------------------------------------------------------------------------------------------
constexpr int FILTER_THREADS = 1024;
constexpr int FILTER_BINS = 2048;
// Copies of the histogram for the first digit.  That digit is sign, exponent and two bits of
// the mantissa, so a row's entries share a few dozen of its values and their atomics queue up
// on those bins; with a copy per four warps the queues are an eighth as long.  The copies are
// added up before the digit is chosen (integer sums: the result does not depend on the copies).
constexpr int FILTER_COPIES = 8;
constexpr size_t FILTER_SMEM_BYTES = (size_t)FILTER_COPIES * FILTER_BINS * (sizeof(unsigned int) + sizeof(unsigned long long));
constexpr float FILTER_MASS_SCALE = 1099511627776.0f;  // 2^40

__device__ __forceinline__ unsigned long long fixed_mass(float e) {
  return (unsigned long long)(e * FILTER_MASS_SCALE);
}

// For this thread's values c and m: their sums over the block's threads with a larger index.
__device__ __forceinline__ void suffix_sums(unsigned int c, unsigned long long m, unsigned int* sc /* 32 */,
                                            unsigned long long* sm /* 32 */, unsigned int& c_above,
                                            unsigned long long& m_above) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // inclusive suffix scan inside the warp
  unsigned int ci = c;
  unsigned long long mi = m;
#pragma unroll
  for (int offset = 1; offset < 32; offset <<= 1) {
    const unsigned int co = __shfl_down_sync(0xffffffffu, ci, offset);
    const unsigned long long mo = __shfl_down_sync(0xffffffffu, mi, offset);
    if (lane + offset < 32) {
      ci += co;
      mi += mo;
    }
  }
  if (lane == 0) {
    sc[warp] = ci;
    sm[warp] = mi;
  }
  __syncthreads();
  unsigned int cw = 0;
  unsigned long long mw = 0;
  const int warps = (int)(blockDim.x >> 5);
  for (int w = warp + 1; w < warps; ++w) {
    cw += sc[w];
    mw += sm[w];
  }
  c_above = cw + ci - c;
  m_above = mw + mi - m;
  __syncthreads();
}

// What the digit search carries from one digit to the next: how many entries, and how much
// mass, lie above the digits found so far, and the mass that top_p allows.
struct DigitSearch {
  unsigned int above_count;
  unsigned long long above_mass, mass_limit;
};

struct DigitChoice {
  unsigned int digit, count;
  unsigned long long mass, total;
};

// The next digit from the row's histogram of it, by a block of 1,024 threads: thread t brings
// the bins of digits 2t and 2t + 1.  A digit d passes if what lies above it (the larger digits,
// and everything above the digits found before) is fewer than k entries and less than top_p of
// the mass; passing is monotone in the digit, and the digit chosen is the smallest that passes.
// The first digit's histogram holds every entry of the row, so its masses add up to the
// normaliser: the sums that are compared are sums of the same integers.
__device__ __forceinline__ unsigned int choose_digit(unsigned int c0, unsigned int c1, unsigned long long m0,
                                                     unsigned long long m1, bool first, bool use_k, int k, bool use_p,
                                                     float p, DigitSearch& search, unsigned int* sc,
                                                     unsigned long long* sm, DigitChoice* choice) {
  unsigned int c_above;
  unsigned long long m_above;
  suffix_sums(c0 + c1, m0 + m1, sc, sm, c_above, m_above);
  if (first) {
    if (threadIdx.x == 0) choice->total = m_above + m0 + m1;
    __syncthreads();
    search.mass_limit = (unsigned long long)((double)p * (double)choice->total);
  }
  const unsigned int c_hi = search.above_count + c_above, c_lo = c_hi + c1;  // above digit 2t + 1, above 2t
  const unsigned long long m_hi = search.above_mass + m_above, m_lo = m_hi + m1;
  const bool pass_hi = (!use_k || c_hi < (unsigned int)k) && (!use_p || m_hi < search.mass_limit);
  const bool pass_lo = (!use_k || c_lo < (unsigned int)k) && (!use_p || m_lo < search.mass_limit);
  // The smallest passing digit is the one whose lower neighbour fails (or digit 0).
  if (pass_hi && !pass_lo) {
    choice->digit = 2u * threadIdx.x + 1u;
    choice->count = c_hi;
    choice->mass = m_hi;
  }
  if (pass_lo) {
    // The digit below 2t is 2t - 1 (thread t - 1's); what lies above it is also digit 2t.
    bool below_fails = threadIdx.x == 0;
    if (!below_fails) {
      const unsigned int cb = c_lo + c0;
      const unsigned long long mb = m_lo + m0;
      below_fails = !((!use_k || cb < (unsigned int)k) && (!use_p || mb < search.mass_limit));
    }
    if (below_fails) {
      choice->digit = 2u * threadIdx.x;
      choice->count = c_lo;
      choice->mass = m_lo;
    }
  }
  __syncthreads();
  search.above_count = choice->count;
  search.above_mass = choice->mass;
  return choice->digit;
}

// Calls f(value) for every entry of a row, the block's threads side by side.  With a row that
// starts on a 16-byte boundary a thread asks for four vectors of four entries before it looks
// at the first: sixteen loads' worth under way per thread instead of one (a sweep with one was
// bound by the latency of its loads, about 15 GB/s a block).  The order in which entries are
// seen differs from a plain loop; every use below (maximum, integer sums, histograms) is
// independent of it.
template <typename F>
__device__ __forceinline__ void sweep_row(const float* __restrict__ row, int vocab, bool vectors, F&& f) {
  const int step = (int)blockDim.x;
  if (vectors) {
    const int n4 = vocab >> 2;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    int i = (int)threadIdx.x;
    for (; i + 3 * step < n4; i += 4 * step) {
      const float4 a = row4[i], b = row4[i + step], c = row4[i + 2 * step], d = row4[i + 3 * step];
      f(a.x), f(a.y), f(a.z), f(a.w);
      f(b.x), f(b.y), f(b.z), f(b.w);
      f(c.x), f(c.y), f(c.z), f(c.w);
      f(d.x), f(d.y), f(d.z), f(d.w);
    }
    for (; i < n4; i += step) {
      const float4 a = row4[i];
      f(a.x), f(a.y), f(a.z), f(a.w);
    }
    for (int j = (n4 << 2) + (int)threadIdx.x; j < vocab; j += step) f(row[j]);
  } else {
    for (int i = (int)threadIdx.x; i < vocab; i += step) f(row[i]);
  }
}

__global__ void __launch_bounds__(FILTER_THREADS)
filter_threshold_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                        const float* __restrict__ temperature, const int* __restrict__ top_k,
                        const float* __restrict__ top_p, float* __restrict__ threshold) {
  __shared__ float scratch[32];
  __shared__ unsigned int sc[32];
  __shared__ unsigned long long sm[32];
  extern __shared__ __align__(16) unsigned char filter_smem[];
  unsigned long long* hist_mass = reinterpret_cast<unsigned long long*>(filter_smem);          // [COPIES][BINS]
  unsigned int* hist_count = reinterpret_cast<unsigned int*>(hist_mass + FILTER_COPIES * FILTER_BINS);  // [COPIES][BINS]
  __shared__ DigitChoice choice;
  allow_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const float temp = temperature[r];
  const int k = top_k[r];
  const float p = top_p[r];
  const bool use_k = k > 0 && k < vocab;
  const bool use_p = p < 1.0f;
  if (temp == 0.f || (!use_k && !use_p)) {
    if (threadIdx.x == 0) threshold[r] = -CUDART_INF_F;
    return;
  }
  const float* row = logits + (size_t)r * row_stride;
  const float inv_t = 1.0f / fmaxf(temp, 1e-5f);

  const bool vectors = (reinterpret_cast<uintptr_t>(row) & 15) == 0;

  float m = -CUDART_INF_F;
  sweep_row(row, vocab, vectors, [&](float x) { m = fmaxf(m, __fmul_rn(x, inv_t)); });
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float w = threadIdx.x < ((blockDim.x + 31) >> 5) ? scratch[threadIdx.x] : -CUDART_INF_F;
    w = warp_max(w);
    if (threadIdx.x == 0) scratch[0] = w;
  }
  __syncthreads();
  m = scratch[0];
  __syncthreads();

  // Digits of the threshold's pattern, most significant first.
  uint32_t prefix = 0u;
  DigitSearch search = {0u, 0ull, 0ull};
  const int shifts[3] = {21, 10, 0};
  const int bits[3] = {11, 11, 10};
  for (int level = 0; level < 3; ++level) {
    const int shift = shifts[level];
    const uint32_t digit_mask = (1u << bits[level]) - 1u;
    const int copies = level == 0 ? FILTER_COPIES : 1;
    for (int b = threadIdx.x; b < copies * FILTER_BINS; b += blockDim.x) {
      hist_count[b] = 0u;
      hist_mass[b] = 0ull;
    }
    __syncthreads();
    unsigned int* my_count = hist_count + (level == 0 ? ((threadIdx.x >> 7) % FILTER_COPIES) * FILTER_BINS : 0);
    unsigned long long* my_mass = hist_mass + (level == 0 ? ((threadIdx.x >> 7) % FILTER_COPIES) * FILTER_BINS : 0);
    const float top = m;
    const uint32_t above = prefix;
    const int level_bits = bits[level];
    sweep_row(row, vocab, vectors, [&](float x) {
      // The rounded product, never folded into the subtraction below: the scaled value is the
      // same number wherever it is looked at (here, in the cluster kernel, in the sampler).
      const float s = __fmul_rn(x, inv_t);
      if (!(s == s)) return;  // NaN is never a candidate
      const uint32_t key = float_key(s);
      if (level > 0 && (key >> (shift + level_bits)) != above) return;
      const uint32_t digit = (key >> shift) & digit_mask;
      // What the filter in force does not look at is not counted.
      if (use_k) atomicAdd(&my_count[digit], 1u);
      if (use_p) atomicAdd(&my_mass[digit], fixed_mass(expf(s - top)));
    });
    __syncthreads();
    unsigned int c[2] = {0u, 0u};
    unsigned long long w[2] = {0ull, 0ull};
    for (int copy = 0; copy < copies; ++copy)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        c[i] += hist_count[copy * FILTER_BINS + 2 * threadIdx.x + i];
        w[i] += hist_mass[copy * FILTER_BINS + 2 * threadIdx.x + i];
      }
    const unsigned int digit = choose_digit(c[0], c[1], w[0], w[1], level == 0, use_k, k, use_p, p, search, sc, sm, &choice);
    prefix = (prefix << bits[level]) | digit;
    __syncthreads();
  }
  if (threadIdx.x == 0) threshold[r] = key_float(prefix);
}

// ---------------------------------------------------------------------------------------------
// The same threshold by a cluster of eight CTAs per row, for rows of up to 196,608 entries.  Each
// CTA reads an eighth of the row once and keeps it in registers (24 entries a thread); what the
// kernel above does in five sweeps over memory happens here over registers.  Every CTA builds
// the histogram of its share in its own shared memory and adds the bins that are not empty into
// the row's histogram, which lies in the shared memory of the cluster's first CTA; that CTA
// chooses the digit (with the same code as above) and writes it into its peers' shared memory.
// The normaliser is the sum of the first histogram's masses: all sums are of the same integers
// as above, so both kernels give the same threshold bit for bit.
//
// A 64-bit sum in shared memory is a compare-and-swap loop; the masses (41 bits at most) are
// therefore added as two 32-bit words, the low word's carry found from the value it held before.
// ---------------------------------------------------------------------------------------------
constexpr int FC_CLUSTER = 8;
constexpr int FC_PER_THREAD = 24;
constexpr int FC_COPIES = 4;
constexpr int FC_MAX_VOCAB = FC_CLUSTER * FILTER_THREADS * FC_PER_THREAD;
constexpr size_t FC_SMEM_BYTES = (size_t)FILTER_BINS * (sizeof(unsigned long long) + sizeof(unsigned int)) +
                                 (size_t)FC_COPIES * FILTER_BINS * 3 * sizeof(unsigned int);

__device__ __forceinline__ void add_mass_words(unsigned int* lo, unsigned int* hi, uint32_t bin, unsigned long long w) {
  const unsigned int wl = (unsigned int)w;
  unsigned int wh = (unsigned int)(w >> 32);
  if (wl != 0u) {
    const unsigned int before = atomicAdd(&lo[bin], wl);
    if (before + wl < before) ++wh;  // the low word wrapped
  }
  if (wh != 0u) atomicAdd(&hi[bin], wh);
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The address, in this CTA's window onto the cluster's shared memory, of `local` in CTA `rank`.
template <typename T>
__device__ __forceinline__ T* cluster_peer(T* local, unsigned int rank) {
  uint64_t out;
  asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"(reinterpret_cast<uint64_t>(local)), "r"(rank));
  return reinterpret_cast<T*>(out);
}

__global__ void __launch_bounds__(FILTER_THREADS, 1)
filter_threshold_cluster_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                                const float* __restrict__ temperature, const int* __restrict__ top_k,
                                const float* __restrict__ top_p, float* __restrict__ threshold) {
  __shared__ float scratch[32];
  __shared__ unsigned int sc[32];
  __shared__ unsigned long long sm[32];
  __shared__ float peer_max[FC_CLUSTER];
  __shared__ unsigned int chosen_digit;
  __shared__ DigitChoice choice;
  extern __shared__ __align__(16) unsigned char filter_smem[];
  unsigned long long* row_mass = reinterpret_cast<unsigned long long*>(filter_smem);   // [BINS], used in CTA 0
  unsigned int* row_count = reinterpret_cast<unsigned int*>(row_mass + FILTER_BINS);    // [BINS], used in CTA 0
  unsigned int* own_count = row_count + FILTER_BINS;                                    // [COPIES][BINS]
  unsigned int* own_lo = own_count + FC_COPIES * FILTER_BINS;
  unsigned int* own_hi = own_lo + FC_COPIES * FILTER_BINS;
  allow_dependents();
  grid_dependency_wait();
  unsigned int rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int r = blockIdx.x / FC_CLUSTER;
  const int tid = (int)threadIdx.x;
  const float temp = temperature[r];
  const int k = top_k[r];
  const float p = top_p[r];
  const bool use_k = k > 0 && k < vocab;
  const bool use_p = p < 1.0f;
  // The same for every CTA of the cluster: none is left waiting at a barrier.
  if (temp == 0.f || (!use_k && !use_p)) {
    if (rank == 0u && tid == 0) threshold[r] = -CUDART_INF_F;
    return;
  }
  const float* row = logits + (size_t)r * row_stride;
  const float inv_t = 1.0f / fmaxf(temp, 1e-5f);
  const bool vectors = (reinterpret_cast<uintptr_t>(row) & 15) == 0;

  // This CTA's share in groups of four entries, the threads side by side; what lies past the
  // share or the row is NaN, which no step below counts.
  const int groups = (vocab + 3) >> 2;
  const int share = (groups + FC_CLUSTER - 1) / FC_CLUSTER;
  const int group_begin = (int)rank * share, group_end = min(groups, group_begin + share);
  float s[FC_PER_THREAD];
#pragma unroll
  for (int j = 0; j < FC_PER_THREAD / 4; ++j) {
    const int g = group_begin + j * FILTER_THREADS + tid;
    const int base = g << 2;
    if (g < group_end && vectors && base + 4 <= vocab) {
      const float4 q = reinterpret_cast<const float4*>(row)[g];
      s[4 * j] = __fmul_rn(q.x, inv_t), s[4 * j + 1] = __fmul_rn(q.y, inv_t), s[4 * j + 2] = __fmul_rn(q.z, inv_t),
      s[4 * j + 3] = __fmul_rn(q.w, inv_t);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) s[4 * j + i] = (g < group_end && base + i < vocab) ? __fmul_rn(row[base + i], inv_t) : CUDART_NAN_F;
    }
  }
  for (int b = tid; b < FILTER_BINS; b += FILTER_THREADS) {
    row_mass[b] = 0ull;
    row_count[b] = 0u;
  }
  for (int b = tid; b < FC_COPIES * FILTER_BINS; b += FILTER_THREADS) {
    own_count[b] = 0u;
    own_lo[b] = 0u;
    own_hi[b] = 0u;
  }
  float m = -CUDART_INF_F;
#pragma unroll
  for (int j = 0; j < FC_PER_THREAD; ++j) m = fmaxf(m, s[j]);  // fmaxf passes over NaN
  m = warp_max(m);
  if ((tid & 31) == 0) scratch[tid >> 5] = m;
  __syncthreads();
  if (tid < 32) {
    float w = scratch[tid];
    w = warp_max(w);
    if (tid < FC_CLUSTER) *cluster_peer(&peer_max[rank], (unsigned int)tid) = w;
  }
  // Every CTA's maximum is in every CTA, and CTA 0's row histogram is zero, before anyone adds.
  cluster_sync_all();
  m = peer_max[0];
#pragma unroll
  for (int c = 1; c < FC_CLUSTER; ++c) m = fmaxf(m, peer_max[c]);
  const float top = m;

  unsigned int* count0 = cluster_peer(row_count, 0u);
  unsigned long long* mass0 = cluster_peer(row_mass, 0u);
  uint32_t prefix = 0u;
  DigitSearch search = {0u, 0ull, 0ull};
  const int shifts[3] = {21, 10, 0};
  const int bits[3] = {11, 11, 10};
#pragma unroll
  for (int level = 0; level < 3; ++level) {
    const int shift = shifts[level], level_bits = bits[level];
    const uint32_t digit_mask = (1u << level_bits) - 1u;
    const int copies = level == 0 ? FC_COPIES : 1;
    const int copy = level == 0 ? ((tid >> 6) % FC_COPIES) * FILTER_BINS : 0;
#pragma unroll
    for (int j = 0; j < FC_PER_THREAD; ++j) {
      const float x = s[j];
      if (!(x == x)) continue;
      const uint32_t key = float_key(x);
      if (level > 0 && (key >> (shift + level_bits)) != prefix) continue;
      const uint32_t digit = (key >> shift) & digit_mask;
      if (use_k) atomicAdd(&own_count[copy + digit], 1u);
      if (use_p) add_mass_words(own_lo + copy, own_hi + copy, digit, fixed_mass(expf(x - top)));
    }
    __syncthreads();
    // This CTA's bins into the row's histogram; its own go back to zero for the next digit.
    for (int b = tid; b < FILTER_BINS; b += FILTER_THREADS) {
      unsigned int c = 0u;
      unsigned long long w = 0ull;
      for (int i = 0; i < copies; ++i) {
        const int at = i * FILTER_BINS + b;
        c += own_count[at];
        w += ((unsigned long long)own_hi[at] << 32) + own_lo[at];
        own_count[at] = 0u, own_lo[at] = 0u, own_hi[at] = 0u;
      }
      if (c != 0u) atomicAdd(&count0[b], c);
      if (w != 0ull) atomicAdd(&mass0[b], w);
    }
    cluster_sync_all();
    if (rank == 0u) {
      const unsigned int c0 = row_count[2 * tid], c1 = row_count[2 * tid + 1];
      const unsigned long long m0 = row_mass[2 * tid], m1 = row_mass[2 * tid + 1];
      row_count[2 * tid] = 0u, row_count[2 * tid + 1] = 0u;
      row_mass[2 * tid] = 0ull, row_mass[2 * tid + 1] = 0ull;
      const unsigned int digit = choose_digit(c0, c1, m0, m1, level == 0, use_k, k, use_p, p, search, sc, sm, &choice);
      if (tid < FC_CLUSTER) *cluster_peer(&chosen_digit, (unsigned int)tid) = digit;
    }
    cluster_sync_all();
    prefix = (prefix << level_bits) | chosen_digit;
  }
  if (rank == 0u && tid == 0) threshold[r] = key_float(prefix);
}

// ---------------------------------------------------------------------------------------------
// Penalties.  `history` holds each request's prompt and output tokens, one row per state slot.
// counts is scratch [R, V] int32, zeroed by the first kernel.
// ---------------------------------------------------------------------------------------------
__global__ void penalty_count_kernel(const int* __restrict__ history, long long history_stride,
                                     const int* __restrict__ slots,
                                     const int* __restrict__ lengths, int* __restrict__ counts,
                                     int vocab) {
  allow_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  int* c = counts + (size_t)r * vocab;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) c[i] = 0;
  __syncthreads();
  const int* h = history + (size_t)slots[r] * history_stride;
  const int n = lengths[r];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int v = h[i];
    if (v >= 0 && v < vocab) atomicAdd(&c[v], 1);
  }
}

__global__ void penalty_apply_kernel(float* __restrict__ logits, long long row_stride,
                                     const int* __restrict__ counts, int vocab,
                                     const float* __restrict__ repetition,
                                     const float* __restrict__ presence,
                                     const float* __restrict__ frequency) {
  allow_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  float* row = logits + (size_t)r * row_stride;
  const int* c = counts + (size_t)r * vocab;
  const float rep = repetition[r], pres = presence[r], freq = frequency[r];
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const int n = c[i];
    if (n == 0) continue;
    float x = row[i] - freq * (float)n;
    x = x > 0.f ? x / rep : x * rep;
    row[i] = x - pres;
  }
}

}  // namespace vx

using namespace vx;

// How many segments vx_sample cuts a row into, and with that the size of its scratch:
// `partial` holds num_rows * segments pairs (float, int), `counters` num_rows zeroed uint32
// (the kernel leaves them zero).  Both may be null when the answer is 1.
VX_API int vx_sample_segments(int num_rows, int vocab) {
  if (num_rows <= 0 || vocab < 8192) return 1;
  // About two blocks per SM, and no segment below 2,048 entries.
  int segments = (2 * 148 + num_rows - 1) / num_rows;
  const int most = vocab / 2048;
  if (segments > most) segments = most;
  if (segments > SAMPLE_MAX_SEGMENTS) segments = SAMPLE_MAX_SEGMENTS;
  return segments < 1 ? 1 : segments;
}

VX_API int vx_sample(const float* logits, int num_rows, int vocab, long long row_stride,
                     const float* temperature, const unsigned long long* seeds,
                     const int* draw_index, const float* threshold, int* out, int* history,
                     long long history_stride, const int* history_slots,
                     const int* history_lengths, void* partial, unsigned int* counters,
                     const int* status_word, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  int segments = vx_sample_segments(num_rows, vocab);
  if (partial == nullptr || counters == nullptr) segments = 1;
  // Segments are multiples of four entries.
  const int segment_len = (((vocab + segments - 1) / segments) + 3) / 4 * 4;
  segments = (vocab + segment_len - 1) / segment_len;
  launch_pdl(sample_kernel, dim3(num_rows, segments), dim3(SAMPLE_THREADS), 0, stream, logits, vocab,
             row_stride, temperature, seeds, draw_index, threshold, out, history, history_stride,
             history_slots, history_lengths, segment_len, (Best*)partial, counters, status_word);
  return (int)cudaGetLastError();
}

// kind 0: the cluster kernel where the row fits its registers, else one CTA a row; 1: one CTA a
// row; 2: the cluster kernel or an error.
VX_API int vx_filter_threshold(const float* logits, int num_rows, int vocab, long long row_stride,
                               const float* temperature, const int* top_k, const float* top_p,
                               float* threshold, int kind, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(filter_threshold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)FILTER_SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(filter_threshold_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)FC_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (kind == 2 && vocab > FC_MAX_VOCAB) return (int)cudaErrorInvalidValue;
  if (kind != 1 && vocab <= FC_MAX_VOCAB) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)num_rows * FC_CLUSTER);
    config.blockDim = dim3(FILTER_THREADS);
    config.dynamicSmemBytes = FC_SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    int count = 0;
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = FC_CLUSTER;
    attributes[count].val.clusterDim.y = 1;
    attributes[count].val.clusterDim.z = 1;
    ++count;
    const char* serialised = getenv("VELOX_B200_NO_PDL");
    if (serialised == nullptr || serialised[0] != '1') {
      attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attributes[count].val.programmaticStreamSerializationAllowed = 1;
      ++count;
    }
    config.attrs = attributes;
    config.numAttrs = count;
    return (int)cudaLaunchKernelEx(&config, filter_threshold_cluster_kernel, logits, vocab, row_stride, temperature,
                                   top_k, top_p, threshold);
  }
  launch_pdl(filter_threshold_kernel, dim3(num_rows), dim3(FILTER_THREADS), FILTER_SMEM_BYTES, stream, logits, vocab, row_stride,
                                                            temperature, top_k, top_p, threshold);
  return (int)cudaGetLastError();
}

VX_API int vx_apply_penalties(float* logits, int num_rows, int vocab, long long row_stride,
                              const int* history, long long history_stride, const int* slots,
                              const int* lengths, int* counts, const float* repetition,
                              const float* presence, const float* frequency,
                              cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  launch_pdl(penalty_count_kernel, dim3(num_rows), dim3(256), 0, stream, history, history_stride, slots, lengths,
                                                     counts, vocab);
  launch_pdl(penalty_apply_kernel, dim3(num_rows), dim3(256), 0, stream, logits, row_stride, counts, vocab,
                                                     repetition, presence, frequency);
  return (int)cudaGetLastError();
}
