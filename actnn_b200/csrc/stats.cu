// Per-group min / max, per-sample sensitivities and the greedy bit allocation.
#include <math.h>

#include "quant_math.cuh"

namespace actnn {
namespace {

constexpr int kThreads = 256;
constexpr int kBundle = 4;

// ---------------------------------------------------------------------------- minimax
// cols == 256: a warp takes four consecutive rows (four independent vector loads per
// lane), reduces each with one redux.sync.min/max.f32, and lanes 0..3 write the results.
template <typename T>
__global__ void __launch_bounds__(kThreads)
minimax256_kernel(const T* __restrict__ data, T* __restrict__ mn, T* __restrict__ mx, int64_t rows) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t total = (rows + kBundle - 1) / kBundle;
  for (int64_t task = warp; task < total; task += nwarps) {
    const int64_t r0 = task * kBundle;
    const int cnt = (int)min((int64_t)kBundle, rows - r0);
    Oct<T> x[kBundle];
#pragma unroll
    for (int i = 0; i < kBundle; ++i)
      x[i] = i < cnt ? load_oct<T>(data + (r0 + i) * kGroup + lane * kOct) : zero_oct<T>();
    float my_mn = 0.f, my_mx = 0.f;
#pragma unroll
    for (int i = 0; i < kBundle; ++i) {
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
int launch_minimax(const void* data, void* mn, void* mx, int64_t rows, int64_t cols, cudaStream_t s) {
  const int64_t cap = (int64_t)device_info().sm_count * 8;
  if (cols == kGroup) {
    const int64_t tasks = (rows + kBundle - 1) / kBundle;
    const int grid = (int)max((int64_t)1, min((tasks + 7) / 8, cap));
    minimax256_kernel<T><<<grid, kThreads, 0, s>>>((const T*)data, (T*)mn, (T*)mx, rows);
  } else {
    const int grid = (int)max((int64_t)1, min((rows + 7) / 8, cap));
    minimax_generic_kernel<T><<<grid, kThreads, 0, s>>>((const T*)data, (T*)mn, (T*)mx, rows, cols);
  }
  return check_launch();
}

// ---------------------------------------------------------------------------- range_sqr
// One block per sample; fixed-shape tree reduction, hence deterministic.
template <typename ST>
__global__ void __launch_bounds__(kThreads)
range_sqr_kernel(const ST* __restrict__ mn, const ST* __restrict__ mx, int64_t G, float range_factor,
                 float coeff, const float* __restrict__ grad_scale, float* __restrict__ C) {
  __shared__ float partial[kThreads / 32];
  const int64_t n = blockIdx.x;
  float acc = 0.f;
  for (int64_t g = threadIdx.x; g < G; g += kThreads) {
    const float d = round_to<ST>(__fsub_rn(load_scalar<ST>(mx, n * G + g), load_scalar<ST>(mn, n * G + g)));
    acc = __fmaf_rn(d, d, acc);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(kFull, acc, s);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) tot += partial[i];
    const float r = round_to<ST>(sqrtf(tot));                  // torch.norm returns the stats' dtype
    float c = __fmul_rn(__fmul_rn(r, r), range_factor);        // .float().square() * (gs / num_pixels)
    c = __fmul_rn(coeff, c);
    if (grad_scale) c = __fmul_rn(c, __ldg(grad_scale));
    C[n] = c;
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
// taken.  T is found bit by bit (64 block-wide counting passes); keys are unique, so ties
// need no special handling.
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

  auto weight_at_least = [&](uint64_t thr) -> unsigned long long {
    unsigned long long s = 0;
    if (cached) {
#pragma unroll
      for (int k = 0; k < kCache; ++k) s += keys[k] >= thr ? wts[k] : 0u;
    } else {
      for (int64_t i = tid; i < N; i += kGreedyThreads) {
        const int wi = WEIGHTED ? w[i] : 1;
        const float c = C[i];
        for (int b = initial_bits; b >= 2; --b)
          s += candidate_key(c, wi, b, i, coef) >= thr ? (unsigned long long)wi : 0ull;
      }
    }
    return s;
  };

  // Largest T with weight({key >= T}) >= need; if even T = 0 falls short every candidate
  // is taken (the reference's heap would run empty there).
  uint64_t T = 0;
  if (need == 0) {
    T = ~0ull;                                                    // nothing is taken (keys < 2^64 - 1)
  } else {
    int buf = 1;
    for (int bit = 63; bit >= 0; --bit) {
      const uint64_t trial = T | (1ull << bit);
      const unsigned long long got = block_sum(weight_at_least(trial), buf);
      buf ^= 1;
      if (got >= need) T = trial;
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

// Fast path for unit weights and few candidates (the per-layer call of every training step):
// every thread keeps its candidate keys in registers and the threshold is found four bits
// per block-wide pass (15 trial thresholds at once) instead of one, skipping the bits of
// the key that are zero for every candidate.  THREADS * kCache keys at most.
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
greedy_small_kernel(const float* __restrict__ C, int64_t N, int initial_bits, double target, GreedyCoef coef,
                    int32_t* __restrict__ b_out, int64_t* __restrict__ word_offsets, int64_t words_per_bit) {
  constexpr int WARPS = THREADS / 32;
  __shared__ uint32_t part[2][WARPS][8];                       // 15 counts, two per word
  __shared__ int scan_sums[WARPS];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int per = initial_bits - 1;
  const int64_t total = N * per;
  const int64_t b_sum0 = N * initial_bits;
  const double deficit = (double)b_sum0 - target;
  const int64_t need = deficit > 0.0 ? (int64_t)ceil(deficit) : 0;

  uint64_t keys[kCache];
#pragma unroll
  for (int k = 0; k < kCache; ++k) {
    const int64_t cidx = (int64_t)tid + (int64_t)k * THREADS;
    keys[k] = 0;                                               // below every real key (b >= 2)
    if (cidx < total) {
      const int64_t i = cidx / per;
      keys[k] = candidate_key(C[i], 1, initial_bits - (int)(cidx - i * per), i, coef);
    }
  }
  // bits of the low word that can be set: (i << 5) | b with i < N
  int low_bits = 5;
  while (((int64_t)1 << (low_bits - 5)) < N) ++low_bits;
  low_bits = (low_bits + 3) & ~3;

  uint64_t T = 0;
  if (need == 0) {
    T = ~0ull;
  } else if (need >= total) {
    T = 1;                                                     // every candidate is taken
  } else {
    int buf = 0;
    for (int shift = 60; shift >= 0; shift -= 4) {
      if (shift < 32 && shift >= low_bits) continue;           // always-zero key bits
      uint32_t cnt[8];
#pragma unroll
      for (int w = 0; w < 8; ++w) cnt[w] = 0;
#pragma unroll
      for (int j = 1; j < 16; ++j) {
        const uint64_t trial = T | ((uint64_t)j << shift);
        uint32_t c = 0;
#pragma unroll
        for (int k = 0; k < kCache; ++k) c += keys[k] >= trial ? 1u : 0u;
        cnt[j >> 1] += c << (16 * (j & 1));
      }
#pragma unroll
      for (int w = 0; w < 8; ++w) cnt[w] = __reduce_add_sync(kFull, cnt[w]);
      if (lane < 8) part[buf][wid][lane] = cnt[lane];
      __syncthreads();
      int digit = 0;
#pragma unroll
      for (int j = 1; j < 16; ++j) {
        uint32_t tot = 0;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) tot += (part[buf][w][j >> 1] >> (16 * (j & 1))) & 0xffffu;
        if ((int64_t)tot >= need) digit = j;                   // counts fall as j grows
      }
      T |= (uint64_t)digit << shift;
      buf ^= 1;
    }
  }
  // widths and word offsets (N <= THREADS * kCache / per, one or more rounds of THREADS)
  int carry = 0;
  for (int64_t start = 0; start < N; start += THREADS) {
    const int64_t i = start + tid;
    int b = 0;
    if (i < N) {
      const float c = C[i];
      b = initial_bits;
      for (int bb = initial_bits; bb >= 2; --bb) b -= candidate_key(c, 1, bb, i, coef) >= T ? 1 : 0;
      b_out[i] = b;
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
      if (i < N) word_offsets[i] = (int64_t)(carry + before + incl - b) * words_per_bit;
      carry += block_total;
    }
  }
  if (word_offsets && tid == 0) word_offsets[N] = (int64_t)carry * words_per_bit;
}

}  // namespace
}  // namespace actnn

using namespace actnn;

extern "C" int actnn_minimax(const void* data, void* mn, void* mx, int64_t rows, int64_t cols, int dtype,
                             actnn_stream_t stream) {
  if (rows < 0 || cols <= 32 || cols % 32 != 0) return ACTNN_ERR_SHAPE;    // minimax_cuda_kernel.cu:80
  if (rows > ((int64_t)1 << 52) / cols) return ACTNN_ERR_SHAPE;
  if (rows == 0) return ACTNN_OK;
  if (!data || !mn || !mx) return ACTNN_ERR_NULL;
  if (cols == kGroup && !aligned(data, dtype == ACTNN_F32 ? 32 : 16)) return ACTNN_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case ACTNN_F32: return launch_minimax<float>(data, mn, mx, rows, cols, s);
    case ACTNN_F16: return launch_minimax<__half>(data, mn, mx, rows, cols, s);
    case ACTNN_BF16: return launch_minimax<__nv_bfloat16>(data, mn, mx, rows, cols, s);
    default: return ACTNN_ERR_DTYPE;
  }
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

extern "C" int actnn_calc_precision(const float* C, const int32_t* w, int64_t N, int initial_bits, double target,
                                    int32_t* b_out, int64_t* word_offsets, int64_t G, int64_t group_size,
                                    actnn_stream_t stream) {
  if (initial_bits < 2 || initial_bits > 15) return ACTNN_ERR_BITS;
  if (N < 0 || N > (1 << 20)) return ACTNN_ERR_SHAPE;
  if (word_offsets && (G < 0 || group_size <= 0 || group_size % 32 != 0)) return ACTNN_ERR_SHAPE;
  if (!(target == target)) return ACTNN_ERR_ARG;
  if (N == 0) {
    if (word_offsets) return cudaMemsetAsync(word_offsets, 0, sizeof(int64_t), (cudaStream_t)stream) == cudaSuccess
                                 ? ACTNN_OK : ACTNN_ERR_LAUNCH;
    return ACTNN_OK;
  }
  if (!C || !b_out) return ACTNN_ERR_NULL;
  GreedyCoef coef;
  for (int b = 0; b < 16; ++b) {
    if (b < 2) { coef.c[b] = 0.0; continue; }
    // the reference's get_obj (calc_precision.cc:24-28), in integers wide enough not to wrap
    const int64_t c1 = (((int64_t)1 << b) - 1) * (((int64_t)1 << b) - 1);
    const int64_t c2 = (((int64_t)1 << (b - 1)) - 1) * (((int64_t)1 << (b - 1)) - 1);
    coef.c[b] = 1.0 / (double)c1 - 1.0 / (double)c2;
  }
  const int64_t wpb = word_offsets ? G * group_size / 32 : 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t candidates = N * (initial_bits - 1);
  if (w) greedy_kernel<true><<<1, kGreedyThreads, 0, s>>>(C, w, N, initial_bits, target, coef, b_out, word_offsets, wpb);
  else if (candidates <= 256 * kCache)
    greedy_small_kernel<256><<<1, 256, 0, s>>>(C, N, initial_bits, target, coef, b_out, word_offsets, wpb);
  else if (candidates <= 1024 * kCache)
    greedy_small_kernel<1024><<<1, 1024, 0, s>>>(C, N, initial_bits, target, coef, b_out, word_offsets, wpb);
  else greedy_kernel<false><<<1, kGreedyThreads, 0, s>>>(C, w, N, initial_bits, target, coef, b_out, word_offsets, wpb);
  return check_launch();
}
