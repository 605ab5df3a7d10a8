// Mixed-precision stream: per-sample bit widths, int32 words.
//
// Layout (reference: quantization_cuda_kernel.cu:51-79).  For 256-element groups the
// reference formula "bit i of element d goes to word (d*b+i) % W, bit (d*b+i) / W,
// W = 8b" reads, with d = 8t + j:  word j*b + i, bit t.  Word w of a group is therefore
// the 32-lane ballot of bit w of each lane's "row" (its eight b-bit codes laid end to
// end), and a group's 8b words are the bit-matrix transpose of the 32 rows.
//
// A warp owns a bundle of four consecutive groups of one sample.  Each lane concatenates
// the rows of the four groups into a 32b-bit string S[0..b-1]; transposing word k of that
// string across the warp yields output words 32k .. 32k+31 of the bundle, lane w holding
// word 32k + w, so every store is one fully coalesced 128-byte line.  No shared memory,
// no atomics, no block-level synchronisation.
#include "quant_math.cuh"

namespace actnn {
namespace {

constexpr int kBundle = 4;            // groups per warp task
constexpr int kThreads = 256;

struct BundleCoord {
  int64_t n, q0;                      // sample, first flat group
  int g0, count;                      // first group within the sample, groups in this bundle
};

ACTNN_DEV BundleCoord bundle_coord(int64_t task, int64_t bundles_per_sample, int64_t G) {
  BundleCoord c;
  c.n = task / bundles_per_sample;
  c.g0 = (int)(task - c.n * bundles_per_sample) * kBundle;
  c.count = (int)min((int64_t)kBundle, G - c.g0);
  c.q0 = c.n * G + c.g0;
  return c;
}

// ---------------------------------------------------------------------------- pack
template <typename T, typename ST, int B>
ACTNN_DEV void pack_bundle(const Oct<T> (&x)[kBundle], const Oct<T> (&nz)[kBundle], const BundleCoord& c,
                           const T* __restrict__ mn, const T* __restrict__ mx, ST* __restrict__ scale,
                           ST* __restrict__ mn_out, int32_t* __restrict__ out, const TransposePlan& plan,
                           int lane) {
  // lanes 0..3 prepare one group each, then broadcast
  GroupParams mine = {0.f, 0.f};
  if (lane < c.count) {
    const float gmn = load_scalar<T>(mn, c.q0 + lane), gmx = load_scalar<T>(mx, c.q0 + lane);
    mine = prepare_group<T>(gmn, gmx, B);
    store_scalar<ST>(scale, c.q0 + lane, mine.scale);
    if (mn_out) store_scalar<ST>(mn_out, c.q0 + lane, gmn);
  }
  uint32_t S[B];
#pragma unroll
  for (int k = 0; k < B; ++k) S[k] = 0u;
#pragma unroll
  for (int gi = 0; gi < kBundle; ++gi) {
    GroupParams p;
    p.mn1 = __shfl_sync(kFull, mine.mn1, gi);
    p.scale = __shfl_sync(kFull, mine.scale, gi);
    if (gi < c.count) {
      uint32_t cp[4];
      quantize_oct<T>(x[gi], nz[gi], p, B, cp);
      if (gi == 0) put_codes<B, 0 * 8 * B>(S, cp);
      if (gi == 1) put_codes<B, 1 * 8 * B>(S, cp);
      if (gi == 2) put_codes<B, 2 * 8 * B>(S, cp);
      if (gi == 3) put_codes<B, 3 * 8 * B>(S, cp);
    }
  }
  const int words = c.count * 8 * B;
#pragma unroll
  for (int k = 0; k < B; ++k) {
    const uint32_t y = warp_transpose32(S[k], plan);
    const int o = k * 32 + lane;
    if (o < words) out[o] = (int32_t)y;
  }
}

template <typename T, typename ST>
__global__ void __launch_bounds__(kThreads)
pack_mixed_kernel(const T* __restrict__ data, const T* __restrict__ mn, const T* __restrict__ mx,
                  const int32_t* __restrict__ bits, const int64_t* __restrict__ word_offsets,
                  int32_t* __restrict__ packed, ST* __restrict__ scale, ST* __restrict__ mn_out,
                  int64_t N, int64_t G, const T* __restrict__ noise, int stochastic, NoiseKey key) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t bps = (G + kBundle - 1) / kBundle;
  const int64_t total = N * bps;
  const TransposePlan plan = make_transpose_plan(lane);
  NoiseGen<T> gen(key, lane);

  for (int64_t task = warp; task < total; task += nwarps) {
    const BundleCoord c = bundle_coord(task, bps, G);
    Oct<T> x[kBundle], nz[kBundle];
#pragma unroll
    for (int gi = 0; gi < kBundle; ++gi)
      x[gi] = gi < c.count ? load_oct<T>(data + (c.q0 + gi) * kGroup + lane * kOct) : zero_oct<T>();
    const int b = __ldg(bits + c.n);
    const int64_t base = __ldg(word_offsets + c.n) + (int64_t)c.g0 * 8 * b;
#pragma unroll
    for (int gi = 0; gi < kBundle; ++gi) {
      if (!stochastic || gi >= c.count) nz[gi] = zero_oct<T>();
      else if (noise) nz[gi] = load_oct<T>(noise + (c.q0 + gi) * kGroup + lane * kOct);
      else nz[gi] = gen.get((uint64_t)(c.q0 + gi));
    }
    int32_t* out = packed + base;
    switch (b) {
      case 1: pack_bundle<T, ST, 1>(x, nz, c, mn, mx, scale, mn_out, out, plan, lane); break;
      case 2: pack_bundle<T, ST, 2>(x, nz, c, mn, mx, scale, mn_out, out, plan, lane); break;
      case 3: pack_bundle<T, ST, 3>(x, nz, c, mn, mx, scale, mn_out, out, plan, lane); break;
      case 4: pack_bundle<T, ST, 4>(x, nz, c, mn, mx, scale, mn_out, out, plan, lane); break;
      case 5: pack_bundle<T, ST, 5>(x, nz, c, mn, mx, scale, mn_out, out, plan, lane); break;
      case 6: pack_bundle<T, ST, 6>(x, nz, c, mn, mx, scale, mn_out, out, plan, lane); break;
      case 7: pack_bundle<T, ST, 7>(x, nz, c, mn, mx, scale, mn_out, out, plan, lane); break;
      case 8: pack_bundle<T, ST, 8>(x, nz, c, mn, mx, scale, mn_out, out, plan, lane); break;
      default: break;     // widths outside 1..8 are skipped; the host documents the range
    }
  }
}

// ---------------------------------------------------------------------------- unpack
template <typename T, typename ST, int B>
ACTNN_DEV void unpack_bundle(const int32_t* __restrict__ in, const BundleCoord& c,
                             const ST* __restrict__ scale, const ST* __restrict__ mn, T* __restrict__ out,
                             const TransposePlan& plan, int lane) {
  float my_scale = 1.f, my_mn = 0.f;
  if (lane < c.count) {
    my_scale = load_scalar<ST>(scale, c.q0 + lane);
    my_mn = load_scalar<ST>(mn, c.q0 + lane);
  }
  const int words = c.count * 8 * B;
  uint32_t S[B];
#pragma unroll
  for (int k = 0; k < B; ++k) {
    const int o = k * 32 + lane;
    const uint32_t w = o < words ? (uint32_t)__ldg(in + o) : 0u;
    S[k] = warp_transpose32(w, plan);
  }
#pragma unroll
  for (int gi = 0; gi < kBundle; ++gi) {
    const float sc = __shfl_sync(kFull, my_scale, gi);
    const float m = __shfl_sync(kFull, my_mn, gi);
    uint32_t code[8];
    if (gi == 0) get_codes<B, 0 * 8 * B>(S, code);
    if (gi == 1) get_codes<B, 1 * 8 * B>(S, code);
    if (gi == 2) get_codes<B, 2 * 8 * B>(S, code);
    if (gi == 3) get_codes<B, 3 * 8 * B>(S, code);
    uint32_t v[8];
    if constexpr (B <= 5) {
      // 2^B distinct outputs per group: lane k computes the one for code k (one IEEE
      // division per lane instead of eight), elements fetch theirs with a shuffle
      const uint32_t entry = dequant_bits<T>((float)lane, sc, m);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __shfl_sync(kFull, entry, (int)code[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = dequant_bits<T>((float)code[j], sc, m);
    }
    if (gi < c.count) {
      Oct<T> o;
      if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int j = 0; j < 8; ++j) reinterpret_cast<uint32_t*>(&o)[j] = v[j];
      } else {
#pragma unroll
        for (int mth = 0; mth < 4; ++mth) reinterpret_cast<uint32_t*>(&o)[mth] = v[2 * mth] | (v[2 * mth + 1] << 16);
      }
      store_oct<T>(out + (c.q0 + gi) * kGroup + lane * kOct, o);
    }
  }
}

template <typename T, typename ST>
__global__ void __launch_bounds__(kThreads)
unpack_mixed_kernel(const int32_t* __restrict__ packed, const int32_t* __restrict__ bits,
                    const int64_t* __restrict__ word_offsets, const ST* __restrict__ scale,
                    const ST* __restrict__ mn, T* __restrict__ out, int64_t N, int64_t G) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t bps = (G + kBundle - 1) / kBundle;
  const int64_t total = N * bps;
  const TransposePlan plan = make_transpose_plan(lane);

  for (int64_t task = warp; task < total; task += nwarps) {
    const BundleCoord c = bundle_coord(task, bps, G);
    const int b = __ldg(bits + c.n);
    const int32_t* in = packed + __ldg(word_offsets + c.n) + (int64_t)c.g0 * 8 * b;
    switch (b) {
      case 1: unpack_bundle<T, ST, 1>(in, c, scale, mn, out, plan, lane); break;
      case 2: unpack_bundle<T, ST, 2>(in, c, scale, mn, out, plan, lane); break;
      case 3: unpack_bundle<T, ST, 3>(in, c, scale, mn, out, plan, lane); break;
      case 4: unpack_bundle<T, ST, 4>(in, c, scale, mn, out, plan, lane); break;
      case 5: unpack_bundle<T, ST, 5>(in, c, scale, mn, out, plan, lane); break;
      case 6: unpack_bundle<T, ST, 6>(in, c, scale, mn, out, plan, lane); break;
      case 7: unpack_bundle<T, ST, 7>(in, c, scale, mn, out, plan, lane); break;
      case 8: unpack_bundle<T, ST, 8>(in, c, scale, mn, out, plan, lane); break;
      default: break;
    }
  }
}

// ---------------------------------------------------------------------------- prefix
// word_offsets[n] = (G * gs / 32) * sum_{m < n} bits[m]; one block, chunked scan.
__global__ void __launch_bounds__(1024)
bits_prefix_kernel(const int32_t* __restrict__ bits, int64_t N, int64_t words_per_bit,
                   int64_t* __restrict__ word_offsets) {
  __shared__ int64_t warp_sums[32];
  __shared__ int64_t carry;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t start = 0; start < N; start += 1024) {
    const int64_t i = start + threadIdx.x;
    const int64_t v = i < N ? (int64_t)bits[i] : 0;
    int64_t incl = v;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int64_t t = __shfl_up_sync(kFull, incl, s);
      if (lane >= s) incl += t;
    }
    if (lane == 31) warp_sums[wid] = incl;
    __syncthreads();
    if (wid == 0) {
      int64_t ws = warp_sums[lane], wincl = ws;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const int64_t t = __shfl_up_sync(kFull, wincl, s);
        if (lane >= s) wincl += t;
      }
      warp_sums[lane] = wincl - ws;          // exclusive over warps
    }
    __syncthreads();
    const int64_t excl = carry + warp_sums[wid] + incl - v;
    if (i < N) word_offsets[i] = excl * words_per_bit;
    __syncthreads();
    if (threadIdx.x == 1023) carry = excl + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) word_offsets[N] = carry * words_per_bit;
}

int grid_for(int64_t warp_tasks) {
  const int64_t blocks = (warp_tasks + (kThreads / 32) - 1) / (kThreads / 32);
  const int64_t cap = (int64_t)device_info().sm_count * 8;      // 8 x 256 threads fill an SM
  return (int)max((int64_t)1, min(blocks, cap));
}

template <typename T, typename ST>
int launch_pack(const void* data, const void* mn, const void* mx, const int32_t* bits,
                const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out, int64_t N,
                int64_t G, int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                cudaStream_t stream) {
  const int64_t tasks = N * ((G + kBundle - 1) / kBundle);
  pack_mixed_kernel<T, ST><<<grid_for(tasks), kThreads, 0, stream>>>(
      (const T*)data, (const T*)mn, (const T*)mx, bits, word_offsets, packed, (ST*)scale, (ST*)mn_out, N, G,
      (const T*)noise, stochastic, make_noise_key(seed, offset));
  return check_launch();
}

template <typename T, typename ST>
int launch_unpack(const int32_t* packed, const int32_t* bits, const int64_t* word_offsets,
                  const void* scale, const void* mn, void* out, int64_t N, int64_t G, cudaStream_t stream) {
  const int64_t tasks = N * ((G + kBundle - 1) / kBundle);
  unpack_mixed_kernel<T, ST><<<grid_for(tasks), kThreads, 0, stream>>>(
      packed, bits, word_offsets, (const ST*)scale, (const ST*)mn, (T*)out, N, G);
  return check_launch();
}

int check_common(int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype) {
  if (N < 0 || G < 0) return ACTNN_ERR_SHAPE;
  if (group_size != kGroup) return ACTNN_ERR_SHAPE;
  if (dtype < ACTNN_F32 || dtype > ACTNN_BF16) return ACTNN_ERR_DTYPE;
  if (!(stat_dtype == dtype || (dtype == ACTNN_F32 && stat_dtype == ACTNN_BF16))) return ACTNN_ERR_DTYPE;
  if (N > (int64_t)1 << 40 || G > (int64_t)1 << 40 || (G && N > ((int64_t)1 << 52) / G)) return ACTNN_ERR_SHAPE;
  return ACTNN_OK;
}

}  // namespace
}  // namespace actnn

using namespace actnn;

extern "C" int actnn_bits_prefix(const int32_t* bits, int64_t N, int64_t G, int64_t group_size,
                                 int64_t* word_offsets, actnn_stream_t stream) {
  if (!word_offsets || (N > 0 && !bits)) return ACTNN_ERR_NULL;
  if (N < 0 || G < 0 || group_size <= 0 || group_size % 32 != 0 || N > (1 << 20)) return ACTNN_ERR_SHAPE;
  bits_prefix_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(bits, N, G * group_size / 32, word_offsets);
  return check_launch();
}

extern "C" int actnn_pack_mixed(const void* data, const void* mn, const void* mx, const int32_t* bits,
                                const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out,
                                int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype,
                                int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                                actnn_stream_t stream) {
  if (int st = check_common(N, G, group_size, dtype, stat_dtype)) return st;
  if (N == 0 || G == 0) return ACTNN_OK;
  if (!data || !mn || !mx || !bits || !word_offsets || !packed || !scale) return ACTNN_ERR_NULL;
  const size_t al = dtype == ACTNN_F32 ? 32 : 16;
  if (!aligned(data, al) || (noise && !aligned(noise, al)) || !aligned(packed, 4)) return ACTNN_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case ACTNN_F16:
      return launch_pack<__half, __half>(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G,
                                         stochastic, noise, seed, offset, s);
    case ACTNN_BF16:
      return launch_pack<__nv_bfloat16, __nv_bfloat16>(data, mn, mx, bits, word_offsets, packed, scale, mn_out,
                                                       N, G, stochastic, noise, seed, offset, s);
    default:
      if (stat_dtype == ACTNN_BF16)
        return launch_pack<float, __nv_bfloat16>(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G,
                                                 stochastic, noise, seed, offset, s);
      return launch_pack<float, float>(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G,
                                       stochastic, noise, seed, offset, s);
  }
}

extern "C" int actnn_unpack_mixed(const int32_t* packed, const int32_t* bits, const int64_t* word_offsets,
                                  const void* scale, const void* mn, void* out, int64_t N, int64_t G,
                                  int64_t group_size, int dtype, int stat_dtype, actnn_stream_t stream) {
  if (int st = check_common(N, G, group_size, dtype, stat_dtype)) return st;
  if (N == 0 || G == 0) return ACTNN_OK;
  if (!packed || !bits || !word_offsets || !scale || !mn || !out) return ACTNN_ERR_NULL;
  if (!aligned(out, dtype == ACTNN_F32 ? 32 : 16) || !aligned(packed, 4)) return ACTNN_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case ACTNN_F16: return launch_unpack<__half, __half>(packed, bits, word_offsets, scale, mn, out, N, G, s);
    case ACTNN_BF16:
      return launch_unpack<__nv_bfloat16, __nv_bfloat16>(packed, bits, word_offsets, scale, mn, out, N, G, s);
    default:
      if (stat_dtype == ACTNN_BF16)
        return launch_unpack<float, __nv_bfloat16>(packed, bits, word_offsets, scale, mn, out, N, G, s);
      return launch_unpack<float, float>(packed, bits, word_offsets, scale, mn, out, N, G, s);
  }
}
