// Per-group min / max, per-sample sensitivities and the greedy bit allocation.
#include <math.h>

#include "quant_math.cuh"

namespace actnn {
namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------- minimax
// cols == 256: a warp takes kMinimaxRows consecutive rows (as many independent vector loads
// per lane), reduces each with one redux.sync.min/max.f32, and the first lanes write the
// results.  FULL tasks (all rows present) carry no per-row predicate, so the loads sit in one
// basic block and are issued back to back.
constexpr int kMinimaxRows = 8;

template <typename T, bool FULL>
ACTNN_DEV void minimax256_task(const T* __restrict__ data, T* __restrict__ mn, T* __restrict__ mx, int64_t rows,
                               int64_t r0, int lane) {
  const int cnt = FULL ? kMinimaxRows : (int)min((int64_t)kMinimaxRows, rows - r0);
  Oct<T> x[kMinimaxRows];
#pragma unroll
  for (int i = 0; i < kMinimaxRows; ++i)
    x[i] = (FULL || i < cnt) ? load_oct<T>(data + (r0 + i) * kGroup + lane * kOct) : zero_oct<T>();
  float my_mn = 0.f, my_mx = 0.f;
#pragma unroll
  for (int i = 0; i < kMinimaxRows; ++i) {
    float lo, hi;
    oct_minmax<T>(x[i], lo, hi);
    lo = warp_min(lo);
    hi = warp_max(hi);
    if (lane == i) { my_mn = lo; my_mx = hi; }
  }
  if (lane < cnt) {
    store_scalar<T>(mn, r0 + lane, my_mn);
    store_scalar<T>(mx, r0 + lane, my_mx);
  }
}

// `reverse`: walk the rows from the last to the first, so that the head of the tensor is what
// the L2 holds when a second pass (the pack) starts reading it from the front.
// `clear_word` (optional) is set to zero: the ticket of the kernel that follows in the stream.
template <typename T>
__global__ void __launch_bounds__(kThreads)
minimax256_kernel(const T* __restrict__ data, T* __restrict__ mn, T* __restrict__ mx, int64_t rows, int reverse,
                  unsigned* __restrict__ clear_word) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t total = (rows + kMinimaxRows - 1) / kMinimaxRows;
  const int64_t whole = rows / kMinimaxRows;
  if (clear_word && blockIdx.x == 0 && threadIdx.x == 0) *clear_word = 0u;
  for (int64_t t = warp; t < total; t += nwarps) {
    const int64_t task = reverse ? total - 1 - t : t;
    if (task < whole) minimax256_task<T, true>(data, mn, mx, rows, task * kMinimaxRows, lane);
    else minimax256_task<T, false>(data, mn, mx, rows, task * kMinimaxRows, lane);
  }
}

// Any cols that is a multiple of 32: one warp per row, scalar loads.
template <typename T>
__global__ void __launch_bounds__(kThreads)
minimax_generic_kernel(const T* __restrict__ data, T* __restrict__ mn, T* __restrict__ mx, int64_t rows,
                       int64_t cols) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  for (int64_t r = warp; r < rows; r += nwarps) {
    float lo = INFINITY, hi = -INFINITY;
    for (int64_t c = lane; c < cols; c += 32) {
      const float v = load_scalar<T>(data, r * cols + c);
      lo = fminf(lo, v);
      hi = fmaxf(hi, v);
    }
    lo = warp_min(lo);
    hi = warp_max(hi);
    if (lane == 0) {
      store_scalar<T>(mn, r, lo);
      store_scalar<T>(mx, r, hi);
    }
  }
}

template <typename T>
int launch_minimax(const void* data, void* mn, void* mx, int64_t rows, int64_t cols, cudaStream_t s,
                   int reverse = 0, unsigned* clear_word = nullptr) {
  const int64_t cap = (int64_t)device_info().sm_count * 8;
  if (cols == kGroup) {
    const int64_t tasks = (rows + kMinimaxRows - 1) / kMinimaxRows;
    const int grid = (int)max((int64_t)1, min((tasks + 7) / 8, cap));
    minimax256_kernel<T><<<grid, kThreads, 0, s>>>((const T*)data, (T*)mn, (T*)mx, rows, reverse, clear_word);
  } else {
    if (clear_word && cudaMemsetAsync(clear_word, 0, sizeof(unsigned), s) != cudaSuccess) return ACTNN_ERR_LAUNCH;
    const int grid = (int)max((int64_t)1, min((rows + 7) / 8, cap));
    minimax_generic_kernel<T><<<grid, kThreads, 0, s>>>((const T*)data, (T*)mn, (T*)mx, rows, cols);
  }
  return check_launch();
}

// ---------------------------------------------------------------------------- range_sqr
// One block per sample; fixed-shape tree reduction, hence deterministic.
// Every kThreads threads of the block take one sample (a block of THREADS threads takes
// THREADS / kThreads consecutive samples); the order of the additions of a sample does not
// depend on the block width, so every caller gets the same sums.
template <typename ST, int THREADS>
ACTNN_DEV void range_sqr_block(const ST* __restrict__ mn, const ST* __restrict__ mx, int64_t first_sample, int64_t N,
                               int64_t G, float range_factor, float coeff, const float* __restrict__ grad_scale,
                               float* __restrict__ C) {
  constexpr int SUBS = THREADS / kThreads;
  __shared__ float partial[SUBS][kThreads / 32];
  const int sub = threadIdx.x / kThreads, t = threadIdx.x % kThreads;
  const int64_t n = first_sample + sub;
  if (n < N) {
    float acc = 0.f;
    // four groups per trip so that their loads travel together; a group past the end adds
    // fma(0, 0, acc) = acc, and the order of the additions stays g ascending
    for (int64_t g0 = t; g0 < G; g0 += 4 * kThreads) {
      float d[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t g = g0 + u * kThreads;
        d[u] = g < G ? round_to<ST>(__fsub_rn(load_scalar<ST>(mx, n * G + g), load_scalar<ST>(mn, n * G + g))) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) acc = __fmaf_rn(d[u], d[u], acc);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(kFull, acc, s);
    if ((t & 31) == 0) partial[sub][t >> 5] = acc;
  }
  __syncthreads();
  if (t == 0 && n < N) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) tot += partial[sub][i];
    const float r = round_to<ST>(sqrtf(tot));                  // torch.norm returns the stats' dtype
    float c = __fmul_rn(__fmul_rn(r, r), range_factor);        // .float().square() * (gs / num_pixels)
    c = __fmul_rn(coeff, c);
    if (grad_scale) c = __fmul_rn(c, __ldg(grad_scale));
    C[n] = c;
  }
}

template <typename ST>
__global__ void __launch_bounds__(kThreads)
range_sqr_kernel(const ST* __restrict__ mn, const ST* __restrict__ mx, int64_t G, float range_factor,
                 float coeff, const float* __restrict__ grad_scale, float* __restrict__ C) {
  range_sqr_block<ST, kThreads>(mn, mx, blockIdx.x, gridDim.x, G, range_factor, coeff, grad_scale, C);
}

// ---------------------------------------------------------------------------- sample_sumsq
// Per-sample sum of squares of a gradient [N, F] in float32 (QScheme.set_scale,
// actnn/actnn/qscheme.py:47-55: grad.view(N, -1).float().norm(dim=1).square()).  One block per
// sample, vector loads, fixed reduction tree: one read of the gradient, deterministic.
template <typename T>
__global__ void __launch_bounds__(512)
sample_sumsq_kernel(const T* __restrict__ x, float* __restrict__ out, int64_t F, int vector_ok) {
  __shared__ float partial[16];
  const T* row = x + (int64_t)blockIdx.x * F;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int64_t octs = vector_ok ? F / kOct : 0;
  int64_t o = threadIdx.x;
  for (; o + 3 * 512 < octs; o += 4 * 512) {                    // four independent loads in flight
    Oct<T> v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = load_oct<T>(row + (o + k * 512) * kOct);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const T* e = reinterpret_cast<const T*>(&v[k]);
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float f = (float)e[j]; acc[k] = __fmaf_rn(f, f, acc[k]); }
    }
  }
  for (; o < octs; o += 512) {
    const Oct<T> v = load_oct<T>(row + o * kOct);
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float f = (float)e[j]; acc[0] = __fmaf_rn(f, f, acc[0]); }
  }
  for (int64_t i = octs * kOct + threadIdx.x; i < F; i += 512) {  // tail, or everything if unaligned
    const float f = load_scalar<T>(row, i);
    acc[1] = __fmaf_rn(f, f, acc[1]);
  }
  float v = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(kFull, v, s);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) tot += partial[i];
    out[blockIdx.x] = tot;
  }
}

// ---------------------------------------------------------------------------- greedy
// The reference pops a max-heap of (float priority, index) pairs, one bit at a time,
// until sum(b * w) <= target.  Sample i at width b offers the decrement with priority
//     float( double(C_i) * (1/(2^b-1)^2 - 1/(2^(b-1)-1)^2) / w_i ),
// and its decrements come out in order b = initial, initial-1, ..., 2 because the
// priority falls with b.  So the pop sequence is the list of all (i, b) candidates sorted
// by (priority desc, index desc, b desc), cut at the first prefix whose weight reaches
// need = sum(initial * w) - target.  That cut is a weighted selection problem: find the
// smallest 64-bit key T with weight({key >= T}) >= need; every candidate with key >= T is
// taken.  T is found four bits per block-wide counting pass; keys are unique, so ties need
// no special handling.
struct GreedyCoef { double c[16]; };

ACTNN_DEV uint64_t candidate_key(float C, int w, int b, int64_t i, const GreedyCoef& coef) {
  float p = (float)((double)C * coef.c[b] / (double)w);
  if (p == 0.f) p = 0.f;                                        // -0.0 and +0.0 compare equal
  uint32_t u = __float_as_uint(p);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);               // order-preserving
  return ((uint64_t)u << 32) | ((uint64_t)i << 5) | (uint64_t)b;
}

constexpr int kGreedyThreads = 1024;
constexpr int kCache = 8;             // candidate keys a thread keeps in registers

template <bool WEIGHTED>
__global__ void __launch_bounds__(kGreedyThreads)
greedy_kernel(const float* __restrict__ C, const int32_t* __restrict__ w, int64_t N, int initial_bits,
              double target, GreedyCoef coef, int32_t* __restrict__ b_out, int64_t* __restrict__ word_offsets,
              int64_t words_per_bit) {
  __shared__ unsigned long long part[2][32];
  __shared__ long long scan_sums[32];
  __shared__ long long carry;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int per = initial_bits - 1;                               // candidates per sample
  const int64_t total = N * per;
  const bool cached = total <= (int64_t)kGreedyThreads * kCache;

  auto block_sum = [&](unsigned long long v, int buf) -> unsigned long long {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(kFull, v, s);
    if (lane == 0) part[buf][wid] = v;
    __syncthreads();
    unsigned long long t = part[buf][lane];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) t += __shfl_xor_sync(kFull, t, s);
    return t;                                                    // every thread has the total
  };

  // total starting weight
  unsigned long long wsum = 0;
  for (int64_t i = tid; i < N; i += kGreedyThreads) wsum += WEIGHTED ? (unsigned long long)w[i] : 1ull;
  const unsigned long long b_sum0 = block_sum(wsum, 0) * (unsigned long long)initial_bits;
  const double deficit = (double)b_sum0 - target;
  // pops continue while b_sum > target: the removed weight must reach ceil(deficit)
  const unsigned long long need = deficit > 0.0 ? (unsigned long long)ceil(deficit) : 0ull;

  uint64_t keys[kCache];
  uint32_t wts[kCache];
  if (cached) {
#pragma unroll
    for (int k = 0; k < kCache; ++k) {
      const int64_t cidx = (int64_t)tid + (int64_t)k * kGreedyThreads;
      keys[k] = 0; wts[k] = 0;
      if (cidx < total) {
        const int64_t i = cidx / per;
        const int b = initial_bits - (int)(cidx - i * per);
        const int wi = WEIGHTED ? w[i] : 1;
        keys[k] = candidate_key(C[i], wi, b, i, coef);
        wts[k] = (uint32_t)wi;
      }
    }
  }

  // Largest T with weight({key >= T}) >= need; if even T = 0 falls short every candidate
  // is taken (the reference's heap would run empty there).  Four key bits per block-wide
  // pass: the weights at or above the 15 trial thresholds T | (j << shift) are summed at
  // once.  Bits of the low word above those an (index, width) pair can set are skipped.
  int low_bits = 5;
  while (((int64_t)1 << (low_bits - 5)) < N) ++low_bits;
  low_bits = (low_bits + 3) & ~3;
  __shared__ unsigned long long part15[2][32][15];
  uint64_t T = 0;
  if (need == 0) {
    T = ~0ull;                                                    // nothing is taken (keys < 2^64 - 1)
  } else {
    int buf = 0;
    for (int shift = 60; shift >= 0; shift -= 4) {
      if (shift < 32 && shift >= low_bits) continue;
      unsigned long long sum[15];
#pragma unroll
      for (int j = 0; j < 15; ++j) sum[j] = 0;
      if (cached) {
#pragma unroll
        for (int k = 0; k < kCache; ++k) {
#pragma unroll
          for (int j = 0; j < 15; ++j) sum[j] += keys[k] >= (T | ((uint64_t)(j + 1) << shift)) ? wts[k] : 0u;
        }
      } else {
        for (int64_t i = tid; i < N; i += kGreedyThreads) {
          const int wi = WEIGHTED ? w[i] : 1;
          const float c = C[i];
          for (int b = initial_bits; b >= 2; --b) {
            const uint64_t key = candidate_key(c, wi, b, i, coef);
#pragma unroll
            for (int j = 0; j < 15; ++j) sum[j] += key >= (T | ((uint64_t)(j + 1) << shift)) ? (unsigned long long)wi : 0ull;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 15; ++j) {
#pragma unroll
        for (int s2 = 16; s2 > 0; s2 >>= 1) sum[j] += __shfl_xor_sync(kFull, sum[j], s2);
      }
      if (lane < 15) {
        unsigned long long mine = 0;
#pragma unroll
        for (int j = 0; j < 15; ++j) mine = lane == j ? sum[j] : mine;
        part15[buf][wid][lane] = mine;
      }
      __syncthreads();
      int digit = 0;
#pragma unroll
      for (int j = 0; j < 15; ++j) {
        unsigned long long tot = 0;
        for (int w2 = 0; w2 < kGreedyThreads / 32; ++w2) tot += part15[buf][w2][j];
        if (tot >= need) digit = j + 1;                            // sums fall as j grows
      }
      T |= (uint64_t)digit << shift;
      buf ^= 1;
    }
  }
  __syncthreads();

  // final widths and (optionally) the word offsets of the mixed-precision stream
  if (tid == 0) carry = 0;
  __syncthreads();
  for (int64_t start = 0; start < N; start += kGreedyThreads) {
    const int64_t i = start + tid;
    int b = 0;
    if (i < N) {
      const int wi = WEIGHTED ? w[i] : 1;
      const float c = C[i];
      b = initial_bits;
      for (int bb = initial_bits; bb >= 2; --bb) b -= candidate_key(c, wi, bb, i, coef) >= T ? 1 : 0;
      b_out[i] = b;
    }
    if (word_offsets) {
      long long incl = b;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const long long t = __shfl_up_sync(kFull, incl, s);
        if (lane >= s) incl += t;
      }
      if (lane == 31) scan_sums[wid] = incl;
      __syncthreads();
      if (wid == 0) {
        const long long ws = scan_sums[lane];
        long long wincl = ws;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
          const long long t = __shfl_up_sync(kFull, wincl, s);
          if (lane >= s) wincl += t;
        }
        scan_sums[lane] = wincl - ws;
      }
      __syncthreads();
      const long long excl = carry + scan_sums[wid] + incl - b;
      if (i < N) word_offsets[i] = excl * words_per_bit;
      __syncthreads();
      if (tid == kGreedyThreads - 1) carry = excl + b;
      __syncthreads();
    }
  }
  if (word_offsets && tid == 0) word_offsets[N] = carry * words_per_bit;
}

// Fast path for unit weights and at most THREADS samples (the per-layer call of every
// training step): thread i owns sample i and keeps its initial_bits - 1 candidate keys in
// registers, so nothing is recomputed and nothing but C is read.  The K-th largest key is
// found by radix selection, eight bits per pass over a 256-bin histogram in shared memory:
// the bits all keys have in common are skipped first (one block-wide min / max), so that the
// first digit already mixes exponent and mantissa bits and the histogram's atomics spread
// over many bins.  The priority word is selected first; the (index, width) word is searched
// only when several candidates share the boundary priority.  All THREADS threads of the block
// must call it.
template <int THREADS>
ACTNN_DEV void greedy_block(float c_mine, int N, int initial_bits, double target, const GreedyCoef& coef,
                            int32_t* __restrict__ b_out, int64_t* __restrict__ word_offsets,
                            int64_t words_per_bit) {
  constexpr int WARPS = THREADS / 32;
  constexpr int KEYS = 8;                                      // widths initial_bits .. 2, initial_bits <= 9
  __shared__ uint32_t hist[256];
  __shared__ uint32_t sel[3];                                  // digit, remaining, size of the digit's bin
  __shared__ uint32_t ext[2][WARPS];
  __shared__ int scan_sums[WARPS];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int per = initial_bits - 1;
  const int total = N * per;
  const double deficit = (double)N * (double)initial_bits - target;
  const int64_t need64 = deficit > 0.0 ? (int64_t)ceil(deficit) : 0;
  const int need = (int)min(need64, (int64_t)total + 1);

  uint32_t key_hi[KEYS], key_lo[KEYS];                         // priority word; (index << 4) | width
#pragma unroll
  for (int k = 0; k < KEYS; ++k) { key_hi[k] = 0; key_lo[k] = 0; }
  const bool have = tid < N;
  if (have) {
    const double c = (double)c_mine;
#pragma unroll
    for (int k = 0; k < KEYS; ++k) {
      const int b = initial_bits - k;
      if (k < per) {
        float p = (float)(c * coef.c[b]);
        if (p == 0.f) p = 0.f;
        const uint32_t u = __float_as_uint(p);
        key_hi[k] = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        key_lo[k] = ((uint32_t)tid << 4) | (uint32_t)b;
      }
    }
  }

  // One selection pass over the digit of `width` <= 8 bits at `shift` of `word[k]`, among the
  // keys whose bits above the digit equal `prefix` (and that pass `live[k]`).  Returns the digit
  // of the `remaining`-th largest such key and updates `remaining` to its rank inside that
  // digit's bin.
  uint32_t bin_size = 0;
  auto pass = [&](const uint32_t (&word)[KEYS], const bool (&live)[KEYS], uint32_t prefix, int shift, int width,
                  uint32_t& remaining) -> uint32_t {
    for (int i = tid; i < 256; i += THREADS) hist[i] = 0;
    __syncthreads();
    const uint32_t above_mask = shift + width >= 32 ? 0u : ~0u << (shift + width);
    const uint32_t digit_mask = (1u << width) - 1u;
#pragma unroll
    for (int k = 0; k < KEYS; ++k)
      if (live[k] && (word[k] & above_mask) == prefix) atomicAdd(&hist[(word[k] >> shift) & digit_mask], 1u);
    __syncthreads();
    if (wid == 0) {
      uint32_t h[8], s = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { h[j] = hist[8 * lane + j]; s += h[j]; }
      uint32_t suffix = s;                                     // keys in the bins of lanes >= this one
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t t = __shfl_down_sync(kFull, suffix, d);
        if (lane + d < 32) suffix += t;
      }
      uint32_t acc = suffix - s;                               // keys in higher bins
      if (acc < remaining && remaining <= suffix) {            // exactly one lane
#pragma unroll
        for (int j = 7; j >= 0; --j) {
          if (acc < remaining && remaining <= acc + h[j]) {
            sel[0] = 8u * lane + j;
            sel[1] = remaining - acc;
            sel[2] = h[j];
          }
          acc += h[j];
        }
      }
    }
    __syncthreads();
    remaining = sel[1];
    bin_size = sel[2];
    return sel[0];
  };

  uint32_t T_hi = 0, T_lo = 0;
  if (need == 0) {
    T_hi = ~0u; T_lo = ~0u;                                     // nothing is taken
  } else if (need >= total) {
    T_hi = 0; T_lo = 1;                                         // every candidate is taken
  } else {
    bool live[KEYS];
#pragma unroll
    for (int k = 0; k < KEYS; ++k) live[k] = have && k < per;
    // bits shared by every key: nothing to select there
    uint32_t lo_key = ~0u, hi_key = 0u;
#pragma unroll
    for (int k = 0; k < KEYS; ++k)
      if (live[k]) { lo_key = min(lo_key, key_hi[k]); hi_key = max(hi_key, key_hi[k]); }
    lo_key = __reduce_min_sync(kFull, lo_key);
    hi_key = __reduce_max_sync(kFull, hi_key);
    if (lane == 0) { ext[0][wid] = lo_key; ext[1][wid] = hi_key; }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < WARPS; ++w) { lo_key = min(lo_key, ext[0][w]); hi_key = max(hi_key, ext[1][w]); }
    const int varying = 32 - __clz((int)(lo_key ^ hi_key));      // low bits in which keys differ (0..32)
    uint32_t remaining = (uint32_t)need;
    uint32_t prefix = varying >= 32 ? 0u : (hi_key >> varying) << varying;
    for (int top = varying; top > 0; top -= 8) {
      const int width = top >= 8 ? 8 : top, shift = top - width;
      prefix |= pass(key_hi, live, prefix, shift, width, remaining) << shift;
    }
    if (varying == 0) bin_size = (uint32_t)total;               // every key has the same priority
    T_hi = prefix;
    if (remaining >= bin_size) {
      T_lo = 0;                                                 // the whole tie is taken
    } else {
      bool tied[KEYS];
#pragma unroll
      for (int k = 0; k < KEYS; ++k) tied[k] = live[k] && key_hi[k] == T_hi;
      const uint32_t d1 = pass(key_lo, tied, 0u, 8, 8, remaining);      // (index << 4 | width) < 2^14
      const uint32_t d0 = pass(key_lo, tied, d1 << 8, 0, 8, remaining);
      T_lo = (d1 << 8) | d0;
    }
  }

  int b = 0;
  if (have) {
    b = initial_bits;
#pragma unroll
    for (int k = 0; k < KEYS; ++k)
      b -= (k < per && (key_hi[k] > T_hi || (key_hi[k] == T_hi && key_lo[k] >= T_lo))) ? 1 : 0;
    b_out[tid] = b;
  }
  if (word_offsets) {
    int incl = b;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int t = __shfl_up_sync(kFull, incl, s);
      if (lane >= s) incl += t;
    }
    __syncthreads();
    if (lane == 31) scan_sums[wid] = incl;
    __syncthreads();
    int before = 0, block_total = 0;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const int v = scan_sums[w];
      before += w < wid ? v : 0;
      block_total += v;
    }
    if (have) word_offsets[tid] = (int64_t)(before + incl - b) * words_per_bit;
    if (tid == 0) word_offsets[N] = (int64_t)block_total * words_per_bit;
  }
}

template <int THREADS>
__global__ void __launch_bounds__(THREADS)
greedy_sample_kernel(const float* __restrict__ C, int N, int initial_bits, double target, GreedyCoef coef,
                     int32_t* __restrict__ b_out, int64_t* __restrict__ word_offsets, int64_t words_per_bit) {
  const float c = (int)threadIdx.x < N ? C[threadIdx.x] : 0.f;
  greedy_block<THREADS>(c, N, initial_bits, target, coef, b_out, word_offsets, words_per_bit);
}

// Sensitivities and bit allocation of one layer in ONE launch: a block computes C[n] of
// THREADS / 256 consecutive samples (so that all blocks are resident at once); the
// block that takes the last ticket (no block waits for another) then runs the greedy over all
// N sensitivities and leaves the ticket at zero for the next call on the same workspace.
template <typename ST, int THREADS>
__global__ void __launch_bounds__(THREADS)
range_greedy_kernel(const ST* __restrict__ mn, const ST* __restrict__ mx, int64_t G, float range_factor,
                    float coeff, const float* __restrict__ grad_scale, float* __restrict__ C, unsigned* ticket,
                    int N, int initial_bits, double target, GreedyCoef coef, int32_t* __restrict__ b_out,
                    int64_t* __restrict__ word_offsets, int64_t words_per_bit) {
  static_assert(THREADS % kThreads == 0, "whole samples per block");
  __shared__ bool last;
  range_sqr_block<ST, THREADS>(mn, mx, (int64_t)blockIdx.x * (THREADS / kThreads), N, G, range_factor, coeff,
                               grad_scale, C);
  __syncthreads();                                             // every C[n] of this block is written
  if (threadIdx.x == 0) {
    __threadfence();                                           // ... and visible before the ticket
    last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  const float c = (int)threadIdx.x < N ? __ldcg(C + threadIdx.x) : 0.f;
  if (threadIdx.x == 0) *ticket = 0u;
  greedy_block<THREADS>(c, N, initial_bits, target, coef, b_out, word_offsets, words_per_bit);
}

// Large or weighted problems (the once-per-step allocation over layers x samples) with a
// caller workspace: the same 4-bits-per-pass selection, but every pass is one launch over
// many blocks.  Blocks add their 15 partial sums to global counters; the block that takes
// the last ticket of a pass picks the digit and clears the counters for the next pass, so
// no block ever waits for another.
struct GreedyState {
  unsigned long long sums[15];
  unsigned long long T;
  unsigned long long need;
  unsigned long long total_weight;
  unsigned int ticket;
  unsigned int pad;
};
constexpr int kWsThreads = 256;

__global__ void __launch_bounds__(1024)
greedy_ws_init_kernel(const int32_t* __restrict__ w, int64_t N, int initial_bits, double target, GreedyState* st) {
  __shared__ unsigned long long part[32];
  unsigned long long s = 0;
  for (int64_t i = threadIdx.x; i < N; i += 1024) s += w ? (unsigned long long)w[i] : 1ull;
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) s += __shfl_xor_sync(kFull, s, k);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long tot = 0;
    for (int k = 0; k < 32; ++k) tot += part[k];
    const double deficit = (double)(tot * (unsigned long long)initial_bits) - target;
    for (int j = 0; j < 15; ++j) st->sums[j] = 0;
    st->total_weight = tot * (unsigned long long)(initial_bits - 1);
    st->need = deficit > 0.0 ? (unsigned long long)ceil(deficit) : 0ull;
    st->T = deficit > 0.0 ? 0ull : ~0ull;                        // nothing to take: threshold above every key
    st->ticket = 0;
  }
}

__global__ void __launch_bounds__(kWsThreads)
greedy_ws_pass_kernel(const float* __restrict__ C, const int32_t* __restrict__ w, int64_t N, int initial_bits,
                      GreedyCoef coef, int shift, GreedyState* st) {
  __shared__ unsigned long long part[kWsThreads / 32][15];
  __shared__ bool last;
  const unsigned long long T = st->T, need = st->need;
  if (need == 0 || need >= st->total_weight) return;              // uniform over the grid: nothing to search
  unsigned long long sum[15];
#pragma unroll
  for (int j = 0; j < 15; ++j) sum[j] = 0;
  for (int64_t i = (int64_t)blockIdx.x * kWsThreads + threadIdx.x; i < N; i += (int64_t)gridDim.x * kWsThreads) {
    const int wi = w ? w[i] : 1;
    const float c = C[i];
    for (int b = initial_bits; b >= 2; --b) {
      const uint64_t key = candidate_key(c, wi, b, i, coef);
#pragma unroll
      for (int j = 0; j < 15; ++j) sum[j] += key >= (T | ((uint64_t)(j + 1) << shift)) ? (unsigned long long)wi : 0ull;
    }
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 15; ++j) {
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) sum[j] += __shfl_xor_sync(kFull, sum[j], k);
    if (lane == 0) part[wid][j] = sum[j];
  }
  __syncthreads();
  if (threadIdx.x < 15) {
    unsigned long long tot = 0;
    for (int k = 0; k < kWsThreads / 32; ++k) tot += part[k][threadIdx.x];
    if (tot) atomicAdd(&st->sums[threadIdx.x], tot);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&st->ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    int digit = 0;
    for (int j = 0; j < 15; ++j) {
      const unsigned long long v = atomicAdd(&st->sums[j], 0ull);
      if (v >= need) digit = j + 1;                                // sums fall as j grows
      st->sums[j] = 0;
    }
    st->T = T | ((uint64_t)digit << shift);
    st->ticket = 0;
  }
}

__global__ void __launch_bounds__(kWsThreads)
greedy_ws_finish_kernel(const float* __restrict__ C, const int32_t* __restrict__ w, int64_t N, int initial_bits,
                        GreedyCoef coef, const GreedyState* st, int32_t* __restrict__ b_out) {
  unsigned long long T = st->T;
  if (st->need != 0 && st->need >= st->total_weight) T = 1;        // every candidate is taken
  for (int64_t i = (int64_t)blockIdx.x * kWsThreads + threadIdx.x; i < N; i += (int64_t)gridDim.x * kWsThreads) {
    const int wi = w ? w[i] : 1;
    const float c = C[i];
    int b = initial_bits;
    for (int bb = initial_bits; bb >= 2; --bb) b -= candidate_key(c, wi, bb, i, coef) >= T ? 1 : 0;
    b_out[i] = b;
  }
}

}  // namespace
}  // namespace actnn

using namespace actnn;

static GreedyCoef make_greedy_coef() {
  GreedyCoef coef;
  for (int b = 0; b < 16; ++b) {
    if (b < 2) { coef.c[b] = 0.0; continue; }
    // the reference's get_obj (calc_precision.cc:24-28), in integers wide enough not to wrap
    const int64_t c1 = (((int64_t)1 << b) - 1) * (((int64_t)1 << b) - 1);
    const int64_t c2 = (((int64_t)1 << (b - 1)) - 1) * (((int64_t)1 << (b - 1)) - 1);
    coef.c[b] = 1.0 / (double)c1 - 1.0 / (double)c2;
  }
  return coef;
}

namespace actnn {
int minimax_impl(const void* data, void* mn, void* mx, int64_t rows, int64_t cols, int dtype, int reverse,
                 unsigned* clear_word, cudaStream_t s) {
  if (rows < 0 || cols <= 32 || cols % 32 != 0) return ACTNN_ERR_SHAPE;    // minimax_cuda_kernel.cu:80
  if (rows > ((int64_t)1 << 52) / cols) return ACTNN_ERR_SHAPE;
  if (rows == 0) return ACTNN_OK;
  if (!data || !mn || !mx) return ACTNN_ERR_NULL;
  if (cols == kGroup && !aligned(data, dtype == ACTNN_F32 ? 32 : 16)) return ACTNN_ERR_ALIGN;
  switch (dtype) {
    case ACTNN_F32: return launch_minimax<float>(data, mn, mx, rows, cols, s, reverse, clear_word);
    case ACTNN_F16: return launch_minimax<__half>(data, mn, mx, rows, cols, s, reverse, clear_word);
    case ACTNN_BF16: return launch_minimax<__nv_bfloat16>(data, mn, mx, rows, cols, s, reverse, clear_word);
    default: return ACTNN_ERR_DTYPE;
  }
}

bool range_greedy_supported(int64_t N, int initial_bits) { return N >= 1 && N <= 1024 && initial_bits >= 1 && initial_bits <= 9; }

int range_greedy_impl(const void* mn, const void* mx, int64_t N, int64_t G, int stat_dtype, float range_factor,
                      float coeff, const float* grad_scale, float* C, unsigned* ticket, int initial_bits,
                      double target, int32_t* b_out, int64_t* word_offsets, int64_t group_size, cudaStream_t s) {
  if (!range_greedy_supported(N, initial_bits)) return ACTNN_ERR_SHAPE;
  if (!mn || !mx || !C || !ticket || !b_out || !word_offsets) return ACTNN_ERR_NULL;
  if (!(target == target)) return ACTNN_ERR_ARG;
  const GreedyCoef coef = make_greedy_coef();
  const int64_t wpb = G * group_size / 32;
  const int n = (int)N;
#define ACTNN_RG(ST, T)                                                                                     \
  range_greedy_kernel<ST, T><<<(n + T / 256 - 1) / (T / 256), T, 0, s>>>((const ST*)mn, (const ST*)mx, G, range_factor, coeff, grad_scale, C, \
                                             ticket, n, initial_bits, target, coef, b_out, word_offsets, wpb)
#define ACTNN_RG_N(ST)                                     \
  if (n <= 256) ACTNN_RG(ST, 256);                         \
  else if (n <= 512) ACTNN_RG(ST, 512);                    \
  else ACTNN_RG(ST, 1024)
  switch (stat_dtype) {
    case ACTNN_F32: ACTNN_RG_N(float); break;
    case ACTNN_F16: ACTNN_RG_N(__half); break;
    case ACTNN_BF16: ACTNN_RG_N(__nv_bfloat16); break;
    default: return ACTNN_ERR_DTYPE;
  }
#undef ACTNN_RG_N
#undef ACTNN_RG
  return check_launch();
}
}  // namespace actnn

extern "C" int actnn_minimax(const void* data, void* mn, void* mx, int64_t rows, int64_t cols, int dtype,
                             actnn_stream_t stream) {
  return minimax_impl(data, mn, mx, rows, cols, dtype, 0, nullptr, (cudaStream_t)stream);
}

extern "C" int actnn_range_sqr(const void* mn, const void* mx, int64_t N, int64_t G, int stat_dtype,
                               float range_factor, float coeff, const float* grad_scale, float* C,
                               actnn_stream_t stream) {
  if (N < 0 || G < 0 || N > 0x7fffffff) return ACTNN_ERR_SHAPE;
  if (N == 0) return ACTNN_OK;
  if (!mn || !mx || !C) return ACTNN_ERR_NULL;
  cudaStream_t s = (cudaStream_t)stream;
  switch (stat_dtype) {
    case ACTNN_F32:
      range_sqr_kernel<float><<<(int)N, kThreads, 0, s>>>((const float*)mn, (const float*)mx, G, range_factor,
                                                          coeff, grad_scale, C);
      break;
    case ACTNN_F16:
      range_sqr_kernel<__half><<<(int)N, kThreads, 0, s>>>((const __half*)mn, (const __half*)mx, G,
                                                           range_factor, coeff, grad_scale, C);
      break;
    case ACTNN_BF16:
      range_sqr_kernel<__nv_bfloat16><<<(int)N, kThreads, 0, s>>>((const __nv_bfloat16*)mn,
                                                                  (const __nv_bfloat16*)mx, G, range_factor,
                                                                  coeff, grad_scale, C);
      break;
    default: return ACTNN_ERR_DTYPE;
  }
  return check_launch();
}

extern "C" int64_t actnn_calc_precision_workspace(void) { return 256; }

extern "C" int actnn_calc_precision(const float* C, const int32_t* w, int64_t N, int initial_bits, double target,
                                    int32_t* b_out, int64_t* word_offsets, int64_t G, int64_t group_size,
                                    void* workspace, int64_t workspace_bytes, actnn_stream_t stream) {
  if (initial_bits < 1 || initial_bits > 15) return ACTNN_ERR_BITS;   // 1: nothing to remove, all ones
  if (N < 0 || N > (1 << 20)) return ACTNN_ERR_SHAPE;
  if (word_offsets && (G < 0 || group_size <= 0 || group_size % 32 != 0)) return ACTNN_ERR_SHAPE;
  if (!(target == target)) return ACTNN_ERR_ARG;
  if (N == 0) {
    if (word_offsets) return cudaMemsetAsync(word_offsets, 0, sizeof(int64_t), (cudaStream_t)stream) == cudaSuccess
                                 ? ACTNN_OK : ACTNN_ERR_LAUNCH;
    return ACTNN_OK;
  }
  if (!C || !b_out) return ACTNN_ERR_NULL;
  const GreedyCoef coef = make_greedy_coef();
  const int64_t wpb = word_offsets ? G * group_size / 32 : 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t candidates = N * (initial_bits - 1);
  static_assert(sizeof(GreedyState) <= 256, "workspace size");
  if (workspace && workspace_bytes >= 256 && aligned(workspace, 8) && !word_offsets &&
      (w || candidates > 1024 * 8)) {
    // multi-block selection, one launch per four key bits
    GreedyState* st = (GreedyState*)workspace;
    int low_bits = 5;
    while (((int64_t)1 << (low_bits - 5)) < N) ++low_bits;
    low_bits = (low_bits + 3) & ~3;
    const int grid = (int)max((int64_t)1, min((N + kWsThreads - 1) / kWsThreads, (int64_t)device_info().sm_count * 4));
    greedy_ws_init_kernel<<<1, 1024, 0, s>>>(w, N, initial_bits, target, st);
    for (int shift = 60; shift >= 0; shift -= 4) {
      if (shift < 32 && shift >= low_bits) continue;
      greedy_ws_pass_kernel<<<grid, kWsThreads, 0, s>>>(C, w, N, initial_bits, coef, shift, st);
    }
    greedy_ws_finish_kernel<<<grid, kWsThreads, 0, s>>>(C, w, N, initial_bits, coef, st, b_out);
    return check_launch();
  }
  if (!w && N <= 1024 && initial_bits <= 9) {
    const int n = (int)N;
#define ACTNN_GREEDY_SAMPLE(T) \
  greedy_sample_kernel<T><<<1, T, 0, s>>>(C, n, initial_bits, target, coef, b_out, word_offsets, wpb)
    if (n <= 32) ACTNN_GREEDY_SAMPLE(32);
    else if (n <= 64) ACTNN_GREEDY_SAMPLE(64);
    else if (n <= 128) ACTNN_GREEDY_SAMPLE(128);
    else if (n <= 256) ACTNN_GREEDY_SAMPLE(256);
    else if (n <= 512) ACTNN_GREEDY_SAMPLE(512);
    else ACTNN_GREEDY_SAMPLE(1024);
#undef ACTNN_GREEDY_SAMPLE
    return check_launch();
  }
  if (w) greedy_kernel<true><<<1, kGreedyThreads, 0, s>>>(C, w, N, initial_bits, target, coef, b_out, word_offsets, wpb);
  else greedy_kernel<false><<<1, kGreedyThreads, 0, s>>>(C, w, N, initial_bits, target, coef, b_out, word_offsets, wpb);
  return check_launch();
}

extern "C" int actnn_sample_sumsq(const void* grad, float* out, int64_t N, int64_t F, int dtype,
                                  actnn_stream_t stream) {
  if (N < 0 || F < 0 || N > 0x7fffffff) return ACTNN_ERR_SHAPE;
  if (N == 0) return ACTNN_OK;
  if (!grad || !out) return ACTNN_ERR_NULL;
  if (dtype < ACTNN_F32 || dtype > ACTNN_BF16) return ACTNN_ERR_DTYPE;
  const size_t al = dtype == ACTNN_F32 ? 32 : 16;
  const int vector_ok = aligned(grad, al) && (F * dtype_size(dtype)) % al == 0;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case ACTNN_F32: sample_sumsq_kernel<float><<<(int)N, 512, 0, s>>>((const float*)grad, out, F, vector_ok); break;
    case ACTNN_F16: sample_sumsq_kernel<__half><<<(int)N, 512, 0, s>>>((const __half*)grad, out, F, vector_ok); break;
    default:
      sample_sumsq_kernel<__nv_bfloat16><<<(int)N, 512, 0, s>>>((const __nv_bfloat16*)grad, out, F, vector_ok);
  }
  return check_launch();
}
