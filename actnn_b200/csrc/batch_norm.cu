// Training-mode batch normalisation over NCHW tensors, forward and backward.
//
// The reference routes this step to cuDNN (actnn/actnn/cpp_extension/backward_func.cc:87-88,
// called from actnn/actnn/ops.py:456-458 and :490-493).  cuDNN's spatial kernels give one
// block to a channel, which leaves most of a 148-SM part idle for the 64..256-channel layers
// of a ResNet, so the step is rebuilt here as two bandwidth-bound passes each way:
//
//   forward   reduce  : per channel sum and sum of squares of (x - shift)      reads x
//             apply   : y = (x - mean) * (invstd * w) + b                       reads x, writes y
//   backward  reduce  : per channel sum(dy) and sum(dy * (x - mean))           reads x, dy
//             apply   : dx = a * (dy - mean_dy - (x - mean) * q)                reads x, dy, writes dx
//
// A channel is split over S blocks (S chosen so that C * S is a few blocks per SM); each
// block writes its partial sums, and the block that takes the channel's last ticket adds
// the S partials in index order, so the result does not depend on block scheduling.  No
// block waits for another.  `shift` is the channel's first element: sums of shifted data
// keep the variance accurate in float32 when |mean| is large against the deviation.
//
// Elements are read VEC at a time (16 bytes when the plane size allows it); a flat index
// is split into (plane, offset) by a multiply-high division.
#include "quant_math.cuh"

namespace actnn {
namespace {

constexpr int kBnThreads = 256;
constexpr int kBnUnroll = 4;
constexpr int kBnReduceUnroll = 8;     // the forward reduce has one input stream: twice the loads in flight

// n / d for n < 2^31 by multiply-high: q = (umulhi(n, m) + n) >> s.
struct FastDiv {
  uint32_t d, m, s;
};
FastDiv make_fastdiv(uint32_t d) {
  FastDiv f{d, 0, 0};
  if (d <= 1) return f;
  uint32_t s = 0;
  while (((uint64_t)1 << s) < d) ++s;
  f.m = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << s) - d)) / d + 1);
  f.s = s;
  return f;
}
ACTNN_DEV uint32_t fdiv(uint32_t n, const FastDiv& f) { return (__umulhi(n, f.m) + n) >> f.s; }

template <int BYTES> struct RawOf;
template <> struct RawOf<16> { using type = uint4; };
template <> struct RawOf<8> { using type = uint2; };
template <> struct RawOf<4> { using type = uint32_t; };
template <> struct RawOf<2> { using type = uint16_t; };

template <typename T> ACTNN_DEV float to_float(T v);
template <> ACTNN_DEV float to_float<float>(float v) { return v; }
template <> ACTNN_DEV float to_float<__half>(__half v) { return __half2float(v); }
template <> ACTNN_DEV float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> ACTNN_DEV T from_float(float v);
template <> ACTNN_DEV float from_float<float>(float v) { return v; }
template <> ACTNN_DEV __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> ACTNN_DEV __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T, int VEC>
struct Vec {
  using raw_t = typename RawOf<VEC * sizeof(T)>::type;
  raw_t raw;
  ACTNN_DEV void load(const T* p) { raw = *reinterpret_cast<const raw_t*>(p); }
  ACTNN_DEV void store(T* p) const { *reinterpret_cast<raw_t*>(p) = raw; }
  ACTNN_DEV float get(int i) const { return to_float<T>(reinterpret_cast<const T*>(&raw)[i]); }
  ACTNN_DEV void set(int i, float v) { reinterpret_cast<T*>(&raw)[i] = from_float<T>(v); }
};

struct BnShape {
  int N, C, HW, S, planes_per_split;
  FastDiv vecs_per_plane;                                    // HW / VEC
};

// Sums (a, b) over the block in a fixed order; the result is valid in thread 0.
ACTNN_DEV float2 block_sum2(float a, float b) {
  __shared__ float2 warp_part[kBnThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(kFull, a, o);
    b += __shfl_xor_sync(kFull, b, o);
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) warp_part[wid] = make_float2(a, b);
  __syncthreads();
  float2 r = make_float2(0.f, 0.f);
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 0; w < kBnThreads / 32; ++w) { r.x += warp_part[w].x; r.y += warp_part[w].y; }
  }
  return r;
}

// Publishes this block's partial and tells whether it was the channel's last; if so, warp 0
// of the block returns (in lane 0) the sums over the S partials in index order.
ACTNN_DEV bool publish_and_collect(float2 mine, float2* partial, unsigned* tickets, int c, int s, int S,
                                   float2* total) {
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    partial[(int64_t)c * S + s] = mine;
    __threadfence();
    is_last = atomicAdd(&tickets[c], 1u) == (unsigned)(S - 1);
  }
  __syncthreads();
  if (!is_last || threadIdx.x >= 32) return false;
  __threadfence();
  float a = 0.f, b = 0.f;
  for (int i = threadIdx.x; i < S; i += 32) {
    const float2 p = __ldcg(&partial[(int64_t)c * S + i]);
    a += p.x; b += p.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(kFull, a, o);
    b += __shfl_xor_sync(kFull, b, o);
  }
  *total = make_float2(a, b);
  if (threadIdx.x == 0) tickets[c] = 0;                       // ready for the next call
  return threadIdx.x == 0;
}

// coef[c] for the forward apply pass: (mean, invstd * weight, bias, unused)
template <typename T, int VEC>
__global__ void __launch_bounds__(kBnThreads)
bn_forward_reduce_kernel(const T* __restrict__ x, BnShape sh, float2* __restrict__ partial,
                         unsigned* __restrict__ tickets, const float* __restrict__ weight,
                         const float* __restrict__ bias, float* __restrict__ running_mean,
                         float* __restrict__ running_var, float* __restrict__ save_mean,
                         float* __restrict__ save_invstd, float4* __restrict__ coef, float momentum, float eps) {
  const int c = blockIdx.x, s = blockIdx.y;
  const int n0 = s * sh.planes_per_split, n1 = min(sh.N, n0 + sh.planes_per_split);
  const uint32_t vpp = sh.vecs_per_plane.d, total = (uint32_t)(n1 - n0) * vpp;
  const int64_t plane_stride = (int64_t)sh.C * sh.HW;
  const float shift = to_float<T>(x[(int64_t)c * sh.HW]);
  const T* base = x + ((int64_t)n0 * sh.C + c) * sh.HW;
  float sum = 0.f, sq = 0.f;
  for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kBnThreads * kBnReduceUnroll) {
    Vec<T, VEC> v[kBnReduceUnroll];
#pragma unroll
    for (int u = 0; u < kBnReduceUnroll; ++u) {
      const uint32_t idx = i0 + u * kBnThreads;
      if (idx < total) {
        const uint32_t n = fdiv(idx, sh.vecs_per_plane), off = idx - n * vpp;
        v[u].load(base + n * plane_stride + (int64_t)off * VEC);
      }
    }
#pragma unroll
    for (int u = 0; u < kBnReduceUnroll; ++u) {
      if (i0 + u * kBnThreads < total) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float d = v[u].get(e) - shift;
          sum += d;
          sq = fmaf(d, d, sq);
        }
      }
    }
  }
  float2 tot;
  if (!publish_and_collect(block_sum2(sum, sq), partial, tickets, c, s, sh.S, &tot)) return;
  const float M = (float)sh.N * (float)sh.HW;
  const float m_s = tot.x / M;
  const float var = fmaxf(tot.y / M - m_s * m_s, 0.f);
  const float mean = shift + m_s;
  const float invstd = 1.0f / sqrtf(var + eps);
  save_mean[c] = mean;
  save_invstd[c] = invstd;
  if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mean;
  if (running_var) {
    const float unbiased = M > 1.f ? var * (M / (M - 1.f)) : var;
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * unbiased;
  }
  coef[c] = make_float4(mean, invstd * (weight ? weight[c] : 1.f), bias ? bias[c] : 0.f, 0.f);
}

template <typename T, int VEC>
__global__ void __launch_bounds__(kBnThreads)
bn_forward_apply_kernel(const T* __restrict__ x, T* __restrict__ y, const float4* __restrict__ coef,
                        uint32_t total_vecs, FastDiv vecs_per_plane, FastDiv channels) {
  const uint32_t step = gridDim.x * kBnThreads * kBnUnroll;
  for (uint32_t i0 = blockIdx.x * kBnThreads * kBnUnroll + threadIdx.x; i0 < total_vecs; i0 += step) {
    Vec<T, VEC> v[kBnUnroll];
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const uint32_t idx = i0 + u * kBnThreads;
      if (idx < total_vecs) v[u].load(x + (int64_t)idx * VEC);
    }
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const uint32_t idx = i0 + u * kBnThreads;
      if (idx < total_vecs) {
        const uint32_t plane = fdiv(idx, vecs_per_plane);
        const uint32_t c = plane - fdiv(plane, channels) * channels.d;
        const float4 k = __ldg(&coef[c]);
        Vec<T, VEC> o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) o.set(e, fmaf(v[u].get(e) - k.x, k.y, k.z));
        o.store(y + (int64_t)idx * VEC);
      }
    }
  }
}

// coef[c] for the backward apply pass: (mean, weight * invstd, sum_dy / M, sum_dy_xmu * invstd^2 / M)
template <typename T, int VEC>
__global__ void __launch_bounds__(kBnThreads)
bn_backward_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy, BnShape sh,
                          float2* __restrict__ partial, unsigned* __restrict__ tickets,
                          const float* __restrict__ weight, const float* __restrict__ save_mean,
                          const float* __restrict__ save_invstd, float* __restrict__ dweight,
                          float* __restrict__ dbias, float* __restrict__ sum_dy_xmu, float4* __restrict__ coef) {
  const int c = blockIdx.x, s = blockIdx.y;
  const int n0 = s * sh.planes_per_split, n1 = min(sh.N, n0 + sh.planes_per_split);
  const uint32_t vpp = sh.vecs_per_plane.d, total = (uint32_t)(n1 - n0) * vpp;
  const int64_t plane_stride = (int64_t)sh.C * sh.HW;
  const float mean = save_mean[c];
  const int64_t base = ((int64_t)n0 * sh.C + c) * sh.HW;
  float sdy = 0.f, sdyx = 0.f;
  for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kBnThreads * kBnUnroll) {
    Vec<T, VEC> vx[kBnUnroll], vg[kBnUnroll];
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const uint32_t idx = i0 + u * kBnThreads;
      if (idx < total) {
        const uint32_t n = fdiv(idx, sh.vecs_per_plane), off = idx - n * vpp;
        const int64_t at = base + n * plane_stride + (int64_t)off * VEC;
        vx[u].load(x + at);
        vg[u].load(dy + at);
      }
    }
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      if (i0 + u * kBnThreads < total) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float g = vg[u].get(e);
          sdy += g;
          sdyx = fmaf(g, vx[u].get(e) - mean, sdyx);
        }
      }
    }
  }
  float2 tot;
  if (!publish_and_collect(block_sum2(sdy, sdyx), partial, tickets, c, s, sh.S, &tot)) return;
  const float M = (float)sh.N * (float)sh.HW;
  const float invstd = save_invstd[c];
  if (dbias) dbias[c] = tot.x;
  if (dweight) dweight[c] = tot.y * invstd;
  if (sum_dy_xmu) sum_dy_xmu[c] = tot.y;
  coef[c] = make_float4(mean, (weight ? weight[c] : 1.f) * invstd, tot.x / M, tot.y * invstd * invstd / M);
}

template <typename T, int VEC>
__global__ void __launch_bounds__(kBnThreads)
bn_backward_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx,
                         const float4* __restrict__ coef, uint32_t total_vecs, FastDiv vecs_per_plane,
                         FastDiv channels) {
  const uint32_t step = gridDim.x * kBnThreads * kBnUnroll;
  for (uint32_t i0 = blockIdx.x * kBnThreads * kBnUnroll + threadIdx.x; i0 < total_vecs; i0 += step) {
    Vec<T, VEC> vx[kBnUnroll], vg[kBnUnroll];
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const uint32_t idx = i0 + u * kBnThreads;
      if (idx < total_vecs) {
        vx[u].load(x + (int64_t)idx * VEC);
        vg[u].load(dy + (int64_t)idx * VEC);
      }
    }
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const uint32_t idx = i0 + u * kBnThreads;
      if (idx < total_vecs) {
        const uint32_t plane = fdiv(idx, vecs_per_plane);
        const uint32_t c = plane - fdiv(plane, channels) * channels.d;
        const float4 k = __ldg(&coef[c]);
        Vec<T, VEC> o;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          o.set(e, k.y * (vg[u].get(e) - k.z - (vx[u].get(e) - k.x) * k.w));
        o.store(dx + (int64_t)idx * VEC);
      }
    }
  }
}

// Coefficients of the apply passes from statistics that were combined elsewhere (across
// ranks): the two halves of a synchronised batch norm.
__global__ void bn_forward_coef_kernel(const float* __restrict__ mean, const float* __restrict__ invstd,
                                       const float* __restrict__ weight, const float* __restrict__ bias,
                                       float4* __restrict__ coef, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < C) coef[c] = make_float4(mean[c], invstd[c] * (weight ? weight[c] : 1.f), bias ? bias[c] : 0.f, 0.f);
}
__global__ void bn_backward_coef_kernel(const float* __restrict__ mean, const float* __restrict__ invstd,
                                        const float* __restrict__ weight, const float* __restrict__ sum_dy,
                                        const float* __restrict__ sum_dy_xmu, const float* __restrict__ counts,
                                        int n_counts, float4* __restrict__ coef, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  float total = 0.f;                                           // elements per channel over all ranks
  for (int i = 0; i < n_counts; ++i) total += counts[i];
  const float inv_count = 1.f / total;
  if (c < C) {
    const float is = invstd[c];
    coef[c] = make_float4(mean[c], (weight ? weight[c] : 1.f) * is, sum_dy[c] * inv_count,
                          sum_dy_xmu[c] * is * is * inv_count);
  }
}

// ------------------------------------------------------------------ statistics + group min / max
// The batch-norm statistics AND the per-group min / max of the activation codec from ONE read
// of x (the reference reads x for the statistics, ops.py:456-458, and again for min / max,
// qbnscheme.py:21-52).  The pass is organised like the codec: a sample is [G, 256] rows, a warp
// task is R consecutive rows, lane t owns elements 8t..8t+7 of a row.  R * 256 <= HW, so a
// task touches at most two channels and every lane adds its eight (x - shift) and their
// squares to one of two slots; an octet never straddles channels because HW % 8 == 0.  A task
// writes its four partial sums; the sums of a channel are added up by a second, tiny kernel in
// a fixed order, so the statistics do not depend on scheduling.  `shift` is the channel's
// first element, as in the plain reduce kernel above.
struct StatMinimaxShape {
  int N, C, HW, G, R, T;            // T = tasks per sample = ceil(G / R)
  FastDiv hw;                       // element offset within a sample / HW = channel
};

template <typename T> ACTNN_DEV void oct_to_floats(const Oct<T>& o, float (&f)[8]);
template <> ACTNN_DEV void oct_to_floats<float>(const Oct<float>& o, float (&f)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = o.f[j];
}
template <> ACTNN_DEV void oct_to_floats<__half>(const Oct<__half>& o, float (&f)[8]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&o.r[k]));
    f[2 * k] = v.x; f[2 * k + 1] = v.y;
  }
}
template <> ACTNN_DEV void oct_to_floats<__nv_bfloat16>(const Oct<__nv_bfloat16>& o, float (&f)[8]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    f[2 * k] = __uint_as_float(o.r[k] << 16);
    f[2 * k + 1] = __uint_as_float(o.r[k] & 0xffff0000u);
  }
}

constexpr int kStatRowsMax = 8;

template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_stats_minimax_kernel(const T* __restrict__ x, StatMinimaxShape sh, T* __restrict__ mn, T* __restrict__ mx,
                        float4* __restrict__ partial) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kBnThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kBnThreads) >> 5;
  const int64_t total = (int64_t)sh.N * sh.T;
  for (int64_t task = warp; task < total; task += nwarps) {
    const int n = (int)(task / sh.T), j = (int)(task - (int64_t)n * sh.T);
    const int row0 = j * sh.R;
    const int rows = min(sh.R, sh.G - row0);
    const uint32_t e0 = (uint32_t)row0 * kGroup;                 // first element of the task within its sample
    const uint32_t c0 = fdiv(e0, sh.hw);
    const uint32_t boundary = (c0 + 1) * (uint32_t)sh.HW;        // first element of the next channel
    const float shift0 = to_float<T>(__ldg(x + (int64_t)c0 * sh.HW));
    const float shift1 = c0 + 1 < (uint32_t)sh.C ? to_float<T>(__ldg(x + (int64_t)(c0 + 1) * sh.HW)) : 0.f;
    const T* base = x + ((int64_t)n * sh.G + row0) * kGroup + lane * kOct;
    Oct<T> v[kStatRowsMax];
#pragma unroll
    for (int r = 0; r < kStatRowsMax; ++r) v[r] = r < rows ? load_oct<T>(base + r * kGroup) : zero_oct<T>();
    float s0 = 0.f, q0 = 0.f, s1 = 0.f, q1 = 0.f, my_mn = 0.f, my_mx = 0.f;
#pragma unroll
    for (int r = 0; r < kStatRowsMax; ++r) {
      if (r < rows) {                                              // warp-uniform
        float lo, hi;
        oct_minmax<T>(v[r], lo, hi);
        lo = warp_min(lo);
        hi = warp_max(hi);
        if (lane == r) { my_mn = lo; my_mx = hi; }
        const bool second = e0 + (uint32_t)(r * kGroup + lane * kOct) >= boundary;
        const float shift = second ? shift1 : shift0;
        float f[8], s = 0.f, q = 0.f;
        oct_to_floats<T>(v[r], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float d = f[e] - shift;
          s += d;
          q = fmaf(d, d, q);
        }
        s0 += second ? 0.f : s; q0 += second ? 0.f : q;
        s1 += second ? s : 0.f; q1 += second ? q : 0.f;
      }
    }
    if (lane < rows) {
      const int64_t g = (int64_t)n * sh.G + row0 + lane;
      mn[g] = from_float<T>(my_mn);
      mx[g] = from_float<T>(my_mx);
    }
    // four sums over the warp in 6 + 6 shuffle-adds: halves of the warp specialise on a slot,
    // then quarters on sum / sum of squares; lanes 0, 8, 16, 24 end with s0, q0, s1, q1
    {
      const bool hi16 = lane & 16;
      const float ks = hi16 ? s1 : s0, kq = hi16 ? q1 : q0;       // kept
      const float gs = hi16 ? s0 : s1, gq = hi16 ? q0 : q1;       // given to the other half
      float a = ks + __shfl_xor_sync(kFull, gs, 16);
      float b = kq + __shfl_xor_sync(kFull, gq, 16);
      const bool hi8 = lane & 8;
      float t = (hi8 ? b : a) + __shfl_xor_sync(kFull, hi8 ? a : b, 8);
      t += __shfl_xor_sync(kFull, t, 4);
      t += __shfl_xor_sync(kFull, t, 2);
      t += __shfl_xor_sync(kFull, t, 1);
      if ((lane & 7) == 0) reinterpret_cast<float*>(partial + task)[lane >> 3] = t;
    }
  }
}

// One block per channel: adds the partial sums of every task that touches the channel (sample
// after sample, task after task: a fixed order) and finishes like bn_forward_reduce_kernel.
__global__ void __launch_bounds__(kBnThreads)
bn_stats_finish_kernel(const float4* __restrict__ partial, StatMinimaxShape sh, const void* __restrict__ x, int dtype, const float* __restrict__ weight,
                       const float* __restrict__ bias, float* __restrict__ running_mean,
                       float* __restrict__ running_var, float* __restrict__ save_mean,
                       float* __restrict__ save_invstd, float4* __restrict__ coef, float momentum, float eps) {
  const int c = blockIdx.x;
  const uint32_t span = (uint32_t)sh.R * kGroup;
  const uint32_t first = (uint32_t)c * sh.HW, last = first + sh.HW - 1;
  const int j_lo = (int)(first / span), j_hi = min((int)(last / span), sh.T - 1);
  float sum = 0.f, sq = 0.f;
  for (int n = threadIdx.x; n < sh.N; n += kBnThreads) {
    for (int j = j_lo; j <= j_hi; ++j) {
      const uint32_t c0 = fdiv((uint32_t)j * span, sh.hw);
      const float4 p = __ldg(partial + (int64_t)n * sh.T + j);
      if (c0 == (uint32_t)c) { sum += p.x; sq += p.y; }
      else if (c0 + 1 == (uint32_t)c) { sum += p.z; sq += p.w; }
    }
  }
  const float2 tot = block_sum2(sum, sq);
  if (threadIdx.x != 0) return;
  float shift;
  if (dtype == ACTNN_F32) shift = reinterpret_cast<const float*>(x)[(int64_t)c * sh.HW];
  else if (dtype == ACTNN_F16) shift = __half2float(reinterpret_cast<const __half*>(x)[(int64_t)c * sh.HW]);
  else shift = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[(int64_t)c * sh.HW]);
  const float M = (float)sh.N * (float)sh.HW;
  const float m_s = tot.x / M;
  const float var = fmaxf(tot.y / M - m_s * m_s, 0.f);
  const float mean = shift + m_s;
  const float invstd = 1.0f / sqrtf(var + eps);
  save_mean[c] = mean;
  save_invstd[c] = invstd;
  if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mean;
  if (running_var) {
    const float unbiased = M > 1.f ? var * (M / (M - 1.f)) : var;
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * unbiased;
  }
  if (coef) coef[c] = make_float4(mean, invstd * (weight ? weight[c] : 1.f), bias ? bias[c] : 0.f, 0.f);
}

// ------------------------------------------------------------------ host side
// Upper bound of the splits per channel (sizes the workspace): about 8 blocks per SM.
int splits_for(int64_t N, int64_t C) {
  const int64_t want = ((int64_t)device_info().sm_count * 8 + C - 1) / C;
  int64_t S = max((int64_t)1, min(min(N, want), (int64_t)65535));
  const int64_t pps = (N + S - 1) / S;
  return (int)((N + pps - 1) / pps);
}
// Splits for one reduce kernel: C * S blocks should fill the blocks that kernel can keep
// resident but not spill into a second, mostly empty wave.
int splits_for_kernel(const void* kernel, int64_t N, int64_t C, int cap) {
  const int64_t resident = (int64_t)device_info().sm_count * cached_blocks_per_sm(kernel, kBnThreads, 0);
  int64_t S = max((int64_t)1, min((int64_t)cap, resident / max(C, (int64_t)1)));
  const int64_t pps = (N + S - 1) / S;
  return (int)((N + pps - 1) / pps);
}

struct Workspace {
  float4* coef;
  float2* partial;
  unsigned* tickets;
};
int64_t workspace_bytes_for(int64_t C, int S) {
  return ((16 * C + 8 * C * S + 4 * C) + 255) / 256 * 256;
}
Workspace carve(void* ws, int64_t C, int S) {
  char* p = (char*)ws;
  Workspace w;
  w.coef = (float4*)p;
  w.partial = (float2*)(p + 16 * C);
  w.tickets = (unsigned*)(p + 16 * C + 8 * C * S);
  return w;
}

int check_shape(int64_t N, int64_t C, int64_t HW) {
  if (N < 0 || C < 0 || HW < 0) return ACTNN_ERR_SHAPE;
  if (N > 0x7fffffff || C > 0x7fffffff || HW > 0x7fffffff) return ACTNN_ERR_SHAPE;
  if (N * C >= ((int64_t)1 << 31) || N * C * HW >= ((int64_t)1 << 40)) return ACTNN_ERR_SHAPE;
  return ACTNN_OK;
}

template <typename T>
int vec_width(int64_t HW, const void* a, const void* b, const void* c) {
  int vec = 16 / (int)sizeof(T);
  while (vec > 1 && (HW % vec != 0 || !aligned(a, vec * sizeof(T)) || (b && !aligned(b, vec * sizeof(T))) ||
                     (c && !aligned(c, vec * sizeof(T)))))
    vec >>= 1;
  return vec;
}

int apply_grid(int64_t total_vecs) {
  const int64_t per_block = (int64_t)kBnThreads * kBnUnroll;
  const int64_t needed = (total_vecs + per_block - 1) / per_block;
  return (int)max((int64_t)1, min(needed, (int64_t)device_info().sm_count * 8));
}

template <typename T, int VEC>
int forward_vec(const T* x, const float* weight, const float* bias, float* running_mean, float* running_var, T* y,
                float* save_mean, float* save_invstd, int64_t N, int64_t C, int64_t HW, float momentum, float eps,
                Workspace w, int cap, cudaStream_t s) {
  const int S = splits_for_kernel((const void*)bn_forward_reduce_kernel<T, VEC>, N, C, cap);
  BnShape sh{(int)N, (int)C, (int)HW, S, (int)((N + S - 1) / S), make_fastdiv((uint32_t)(HW / VEC))};
  bn_forward_reduce_kernel<T, VEC><<<dim3((unsigned)C, (unsigned)S), kBnThreads, 0, s>>>(
      x, sh, w.partial, w.tickets, weight, bias, running_mean, running_var, save_mean, save_invstd, w.coef,
      momentum, eps);
  if (int st = check_launch()) return st;
  if (!y) return ACTNN_OK;
  const int64_t total_vecs = N * C * (HW / VEC);
  if (total_vecs >= ((int64_t)1 << 31)) return ACTNN_ERR_SHAPE;
  bn_forward_apply_kernel<T, VEC><<<apply_grid(total_vecs), kBnThreads, 0, s>>>(
      x, y, w.coef, (uint32_t)total_vecs, sh.vecs_per_plane, make_fastdiv((uint32_t)C));
  return check_launch();
}

template <typename T>
int forward_typed(const void* x, const float* weight, const float* bias, float* rm, float* rv, void* y,
                  float* save_mean, float* save_invstd, int64_t N, int64_t C, int64_t HW, float momentum, float eps,
                  Workspace w, int S, cudaStream_t s) {
#define ACTNN_BN_FWD(V)                                                                                        \
  return forward_vec<T, V>((const T*)x, weight, bias, rm, rv, (T*)y, save_mean, save_invstd, N, C, HW, momentum, \
                           eps, w, S, s)
  switch (vec_width<T>(HW, x, y, nullptr)) {
    case 8: if constexpr (sizeof(T) == 2) { ACTNN_BN_FWD(8); }
    case 4: ACTNN_BN_FWD(4);
    case 2: ACTNN_BN_FWD(2);
    default: ACTNN_BN_FWD(1);
  }
#undef ACTNN_BN_FWD
}

template <typename T, int VEC>
int backward_vec(const T* x, const T* dy, const float* weight, const float* save_mean, const float* save_invstd,
                 T* dx, float* dweight, float* dbias, float* sum_dy_xmu, int64_t N, int64_t C, int64_t HW,
                 Workspace w, int cap, cudaStream_t s) {
  const int S = splits_for_kernel((const void*)bn_backward_reduce_kernel<T, VEC>, N, C, cap);
  BnShape sh{(int)N, (int)C, (int)HW, S, (int)((N + S - 1) / S), make_fastdiv((uint32_t)(HW / VEC))};
  bn_backward_reduce_kernel<T, VEC><<<dim3((unsigned)C, (unsigned)S), kBnThreads, 0, s>>>(
      x, dy, sh, w.partial, w.tickets, weight, save_mean, save_invstd, dweight, dbias, sum_dy_xmu, w.coef);
  if (int st = check_launch()) return st;
  if (!dx) return ACTNN_OK;
  const int64_t total_vecs = N * C * (HW / VEC);
  if (total_vecs >= ((int64_t)1 << 31)) return ACTNN_ERR_SHAPE;
  bn_backward_apply_kernel<T, VEC><<<apply_grid(total_vecs), kBnThreads, 0, s>>>(
      x, dy, dx, w.coef, (uint32_t)total_vecs, sh.vecs_per_plane, make_fastdiv((uint32_t)C));
  return check_launch();
}

template <typename T>
int backward_typed(const void* x, const void* dy, const float* weight, const float* save_mean,
                   const float* save_invstd, void* dx, float* dweight, float* dbias, float* sum_dy_xmu,
                   int64_t N, int64_t C, int64_t HW, Workspace w, int S, cudaStream_t s) {
#define ACTNN_BN_BWD(V)                                                                                      \
  return backward_vec<T, V>((const T*)x, (const T*)dy, weight, save_mean, save_invstd, (T*)dx, dweight, dbias, \
                            sum_dy_xmu, N, C, HW, w, S, s)
  switch (vec_width<T>(HW, x, dy, dx)) {
    case 8: if constexpr (sizeof(T) == 2) { ACTNN_BN_BWD(8); }
    case 4: ACTNN_BN_BWD(4);
    case 2: ACTNN_BN_BWD(2);
    default: ACTNN_BN_BWD(1);
  }
#undef ACTNN_BN_BWD
}

template <typename T>
int forward_apply_typed(const void* x, void* y, const float4* coef, int64_t N, int64_t C, int64_t HW,
                        cudaStream_t s) {
  const int vec = vec_width<T>(HW, x, y, nullptr);
  const int64_t total_vecs = N * C * (HW / vec);
  if (total_vecs >= ((int64_t)1 << 31)) return ACTNN_ERR_SHAPE;
  const FastDiv vpp = make_fastdiv((uint32_t)(HW / vec)), ch = make_fastdiv((uint32_t)C);
  const int grid = apply_grid(total_vecs);
#define ACTNN_BN_APPLY(V) \
  bn_forward_apply_kernel<T, V><<<grid, kBnThreads, 0, s>>>((const T*)x, (T*)y, coef, (uint32_t)total_vecs, vpp, ch)
  switch (vec) {
    case 8: if constexpr (sizeof(T) == 2) { ACTNN_BN_APPLY(8); } break;
    case 4: ACTNN_BN_APPLY(4); break;
    case 2: ACTNN_BN_APPLY(2); break;
    default: ACTNN_BN_APPLY(1); break;
  }
#undef ACTNN_BN_APPLY
  return check_launch();
}

template <typename T>
int backward_apply_typed(const void* x, const void* dy, void* dx, const float4* coef, int64_t N, int64_t C,
                         int64_t HW, cudaStream_t s) {
  const int vec = vec_width<T>(HW, x, dy, dx);
  const int64_t total_vecs = N * C * (HW / vec);
  if (total_vecs >= ((int64_t)1 << 31)) return ACTNN_ERR_SHAPE;
  const FastDiv vpp = make_fastdiv((uint32_t)(HW / vec)), ch = make_fastdiv((uint32_t)C);
  const int grid = apply_grid(total_vecs);
#define ACTNN_BN_APPLY(V)                                                                                  \
  bn_backward_apply_kernel<T, V><<<grid, kBnThreads, 0, s>>>((const T*)x, (const T*)dy, (T*)dx, coef,        \
                                                            (uint32_t)total_vecs, vpp, ch)
  switch (vec) {
    case 8: if constexpr (sizeof(T) == 2) { ACTNN_BN_APPLY(8); } break;
    case 4: ACTNN_BN_APPLY(4); break;
    case 2: ACTNN_BN_APPLY(2); break;
    default: ACTNN_BN_APPLY(1); break;
  }
#undef ACTNN_BN_APPLY
  return check_launch();
}

// Geometry the fused statistics + min / max pass covers: groups must not need padding, an octet
// must not straddle two channels and a row of 256 must not span more than two.
bool stats_minimax_supported(int64_t N, int64_t C, int64_t HW) {
  return N > 0 && C > 0 && HW >= kGroup && HW % 8 == 0 && (C * HW) % kGroup == 0 && check_shape(N, C, HW) == ACTNN_OK;
}
StatMinimaxShape stats_minimax_shape(int64_t N, int64_t C, int64_t HW) {
  StatMinimaxShape sh;
  sh.N = (int)N; sh.C = (int)C; sh.HW = (int)HW;
  sh.G = (int)(C * HW / kGroup);
  sh.R = (int)min((int64_t)kStatRowsMax, HW / kGroup);
  sh.T = (sh.G + sh.R - 1) / sh.R;
  sh.hw = make_fastdiv((uint32_t)HW);
  return sh;
}

}  // namespace
}  // namespace actnn

using namespace actnn;

extern "C" int64_t actnn_batch_norm_workspace(int64_t N, int64_t C, int64_t HW) {
  if (check_shape(N, C, HW) != ACTNN_OK || C == 0) return 0;
  return workspace_bytes_for(C, splits_for(max(N, (int64_t)1), C));
}

extern "C" int actnn_batch_norm_forward(const void* x, const float* weight, const float* bias, float* running_mean,
                                        float* running_var, void* y, float* save_mean, float* save_invstd,
                                        int64_t N, int64_t C, int64_t HW, double momentum, double eps, int dtype,
                                        void* workspace, int64_t workspace_bytes, actnn_stream_t stream) {
  if (int st = check_shape(N, C, HW)) return st;
  if (C == 0) return ACTNN_OK;
  if (N * HW == 0) return ACTNN_ERR_SHAPE;                     // statistics of an empty batch
  if (!x || !save_mean || !save_invstd || !workspace) return ACTNN_ERR_NULL;   // y NULL: statistics only
  const int S = splits_for(N, C);
  if (workspace_bytes < workspace_bytes_for(C, S) || !aligned(workspace, 16)) return ACTNN_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  Workspace w = carve(workspace, C, S);
  if (cudaMemsetAsync(w.tickets, 0, 4 * C, s) != cudaSuccess) return ACTNN_ERR_LAUNCH;
  switch (dtype) {
    case ACTNN_F32:
      return forward_typed<float>(x, weight, bias, running_mean, running_var, y, save_mean, save_invstd, N, C, HW,
                                  (float)momentum, (float)eps, w, S, s);
    case ACTNN_F16:
      return forward_typed<__half>(x, weight, bias, running_mean, running_var, y, save_mean, save_invstd, N, C, HW,
                                   (float)momentum, (float)eps, w, S, s);
    case ACTNN_BF16:
      return forward_typed<__nv_bfloat16>(x, weight, bias, running_mean, running_var, y, save_mean, save_invstd, N,
                                          C, HW, (float)momentum, (float)eps, w, S, s);
    default: return ACTNN_ERR_DTYPE;
  }
}

extern "C" int actnn_batch_norm_backward(const void* x, const void* grad_out, const float* weight,
                                         const float* save_mean, const float* save_invstd, void* grad_in,
                                         float* grad_weight, float* grad_bias, int64_t N, int64_t C, int64_t HW,
                                         int dtype, void* workspace, int64_t workspace_bytes,
                                         actnn_stream_t stream) {
  if (int st = check_shape(N, C, HW)) return st;
  if (C == 0) return ACTNN_OK;
  if (N * HW == 0) return ACTNN_ERR_SHAPE;
  if (!x || !grad_out || !save_mean || !save_invstd || !workspace) return ACTNN_ERR_NULL;
  const int S = splits_for(N, C);
  if (workspace_bytes < workspace_bytes_for(C, S) || !aligned(workspace, 16)) return ACTNN_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  Workspace w = carve(workspace, C, S);
  if (cudaMemsetAsync(w.tickets, 0, 4 * C, s) != cudaSuccess) return ACTNN_ERR_LAUNCH;
  switch (dtype) {
    case ACTNN_F32:
      return backward_typed<float>(x, grad_out, weight, save_mean, save_invstd, grad_in, grad_weight, grad_bias,
                                   nullptr, N, C, HW, w, S, s);
    case ACTNN_F16:
      return backward_typed<__half>(x, grad_out, weight, save_mean, save_invstd, grad_in, grad_weight, grad_bias,
                                    nullptr, N, C, HW, w, S, s);
    case ACTNN_BF16:
      return backward_typed<__nv_bfloat16>(x, grad_out, weight, save_mean, save_invstd, grad_in, grad_weight,
                                           grad_bias, nullptr, N, C, HW, w, S, s);
    default: return ACTNN_ERR_DTYPE;
  }
}

// ---- the four halves a synchronised batch norm is made of (statistics are combined across
// ranks between them)
extern "C" int actnn_batch_norm_stats(const void* x, float* mean, float* invstd, int64_t N, int64_t C, int64_t HW,
                                      double eps, int dtype, void* workspace, int64_t workspace_bytes,
                                      actnn_stream_t stream) {
  return actnn_batch_norm_forward(x, nullptr, nullptr, nullptr, nullptr, nullptr, mean, invstd, N, C, HW, 0.0, eps,
                                  dtype, workspace, workspace_bytes, stream);
}

extern "C" int actnn_batch_norm_elemt(const void* x, const float* weight, const float* bias, const float* mean,
                                      const float* invstd, void* y, int64_t N, int64_t C, int64_t HW, int dtype,
                                      void* workspace, int64_t workspace_bytes, actnn_stream_t stream) {
  if (int st = check_shape(N, C, HW)) return st;
  if (N * C * HW == 0) return ACTNN_OK;
  if (!x || !y || !mean || !invstd || !workspace) return ACTNN_ERR_NULL;
  if (workspace_bytes < 16 * C || !aligned(workspace, 16)) return ACTNN_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  float4* coef = (float4*)workspace;
  bn_forward_coef_kernel<<<(unsigned)((C + 255) / 256), 256, 0, s>>>(mean, invstd, weight, bias, coef, (int)C);
  switch (dtype) {
    case ACTNN_F32: return forward_apply_typed<float>(x, y, coef, N, C, HW, s);
    case ACTNN_F16: return forward_apply_typed<__half>(x, y, coef, N, C, HW, s);
    case ACTNN_BF16: return forward_apply_typed<__nv_bfloat16>(x, y, coef, N, C, HW, s);
    default: return ACTNN_ERR_DTYPE;
  }
}

extern "C" int actnn_batch_norm_backward_reduce(const void* x, const void* grad_out, const float* weight,
                                                const float* mean, const float* invstd, float* sum_dy,
                                                float* sum_dy_xmu, float* grad_weight, int64_t N, int64_t C,
                                                int64_t HW, int dtype, void* workspace, int64_t workspace_bytes,
                                                actnn_stream_t stream) {
  if (int st = check_shape(N, C, HW)) return st;
  if (C == 0) return ACTNN_OK;
  if (N * HW == 0) return ACTNN_ERR_SHAPE;
  if (!x || !grad_out || !mean || !invstd || !workspace) return ACTNN_ERR_NULL;
  const int S = splits_for(N, C);
  if (workspace_bytes < workspace_bytes_for(C, S) || !aligned(workspace, 16)) return ACTNN_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  Workspace w = carve(workspace, C, S);
  if (cudaMemsetAsync(w.tickets, 0, 4 * C, s) != cudaSuccess) return ACTNN_ERR_LAUNCH;
  switch (dtype) {
    case ACTNN_F32:
      return backward_typed<float>(x, grad_out, weight, mean, invstd, nullptr, grad_weight, sum_dy, sum_dy_xmu, N, C,
                                   HW, w, S, s);
    case ACTNN_F16:
      return backward_typed<__half>(x, grad_out, weight, mean, invstd, nullptr, grad_weight, sum_dy, sum_dy_xmu, N,
                                    C, HW, w, S, s);
    case ACTNN_BF16:
      return backward_typed<__nv_bfloat16>(x, grad_out, weight, mean, invstd, nullptr, grad_weight, sum_dy,
                                           sum_dy_xmu, N, C, HW, w, S, s);
    default: return ACTNN_ERR_DTYPE;
  }
}

extern "C" int actnn_batch_norm_backward_elemt(const void* x, const void* grad_out, const float* weight,
                                               const float* mean, const float* invstd, const float* sum_dy,
                                               const float* sum_dy_xmu, const float* counts, int64_t n_counts,
                                               void* grad_in,
                                               int64_t N, int64_t C, int64_t HW, int dtype, void* workspace,
                                               int64_t workspace_bytes, actnn_stream_t stream) {
  if (int st = check_shape(N, C, HW)) return st;
  if (N * C * HW == 0) return ACTNN_OK;
  if (n_counts <= 0 || n_counts > 65536) return ACTNN_ERR_ARG;
  if (!x || !grad_out || !grad_in || !mean || !invstd || !sum_dy || !sum_dy_xmu || !counts || !workspace)
    return ACTNN_ERR_NULL;
  if (workspace_bytes < 16 * C || !aligned(workspace, 16)) return ACTNN_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  float4* coef = (float4*)workspace;
  bn_backward_coef_kernel<<<(unsigned)((C + 255) / 256), 256, 0, s>>>(mean, invstd, weight, sum_dy, sum_dy_xmu,
                                                                       counts, (int)n_counts, coef, (int)C);
  switch (dtype) {
    case ACTNN_F32: return backward_apply_typed<float>(x, grad_out, grad_in, coef, N, C, HW, s);
    case ACTNN_F16: return backward_apply_typed<__half>(x, grad_out, grad_in, coef, N, C, HW, s);
    case ACTNN_BF16: return backward_apply_typed<__nv_bfloat16>(x, grad_out, grad_in, coef, N, C, HW, s);
    default: return ACTNN_ERR_DTYPE;
  }
}

extern "C" int64_t actnn_batch_norm_stats_minimax_workspace(int64_t N, int64_t C, int64_t HW) {
  if (!stats_minimax_supported(N, C, HW)) return -1;
  const StatMinimaxShape sh = stats_minimax_shape(N, C, HW);
  return ((int64_t)16 * N * sh.T + 16 * C + 255) / 256 * 256;
}

extern "C" int actnn_batch_norm_stats_minimax(const void* x, void* mn, void* mx, const float* weight,
                                              const float* bias, float* running_mean, float* running_var,
                                              float* save_mean, float* save_invstd, int64_t N, int64_t C, int64_t HW,
                                              double momentum, double eps, int dtype, void* workspace,
                                              int64_t workspace_bytes, actnn_stream_t stream) {
  if (dtype < ACTNN_F32 || dtype > ACTNN_BF16) return ACTNN_ERR_DTYPE;
  if (!stats_minimax_supported(N, C, HW)) return ACTNN_ERR_SHAPE;
  if (!x || !mn || !mx || !save_mean || !save_invstd || !workspace) return ACTNN_ERR_NULL;
  if (workspace_bytes < actnn_batch_norm_stats_minimax_workspace(N, C, HW)) return ACTNN_ERR_CAPACITY;
  if (!aligned(x, dtype == ACTNN_F32 ? 32 : 16) || !aligned(workspace, 16)) return ACTNN_ERR_ALIGN;
  const StatMinimaxShape sh = stats_minimax_shape(N, C, HW);
  float4* partial = (float4*)workspace;
  float4* coef = partial + (int64_t)N * sh.T;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t tasks = (int64_t)N * sh.T;
#define ACTNN_SM(T)                                                                                        \
  {                                                                                                        \
    auto kernel = bn_stats_minimax_kernel<T>;                                                              \
    kernel<<<persistent_grid(kernel, kBnThreads, tasks), kBnThreads, 0, s>>>((const T*)x, sh, (T*)mn, (T*)mx, \
                                                                             partial);                     \
  }
  switch (dtype) {
    case ACTNN_F32: ACTNN_SM(float) break;
    case ACTNN_F16: ACTNN_SM(__half) break;
    default: ACTNN_SM(__nv_bfloat16) break;
  }
#undef ACTNN_SM
  if (int st = check_launch()) return st;
  bn_stats_finish_kernel<<<(unsigned)C, kBnThreads, 0, s>>>(partial, sh, x, dtype, weight, bias, running_mean,
                                                           running_var, save_mean, save_invstd, coef,
                                                           (float)momentum, (float)eps);
  return check_launch();
}
