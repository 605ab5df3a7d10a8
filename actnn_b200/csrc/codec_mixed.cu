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

// Walks the (sample, bundle-in-sample) pairs a warp owns without 64-bit divisions: the
// stride between a warp's tasks is split once into whole samples and a remainder.
struct BundleWalker {
  int64_t n, N, G;
  int r, bps, step_n, step_r, gpb;
  ACTNN_DEV BundleWalker(int64_t warp, int64_t nwarps, int64_t N_, int64_t G_, int gpb_ = kBundle)
      : N(N_), G(G_), gpb(gpb_) {
    bps = (int)((G_ + gpb - 1) / gpb);
    n = warp / bps;
    r = (int)(warp - n * bps);
    step_n = (int)(nwarps / bps);
    step_r = (int)(nwarps - (int64_t)step_n * bps);
  }
  ACTNN_DEV bool valid() const { return n < N; }
  ACTNN_DEV BundleCoord coord() const {
    BundleCoord c;
    c.n = n;
    c.g0 = r * gpb;
    c.count = (int)min((int64_t)gpb, G - c.g0);
    c.q0 = n * G + c.g0;
    return c;
  }
  ACTNN_DEV void next() {
    n += step_n;
    r += step_r;
    if (r >= bps) { r -= bps; ++n; }
  }
};

// ---------------------------------------------------------------------------- pack
// Groups per pack bundle: eight octets per lane for 16-bit types, four for float32.
template <typename T> struct PackShape { static constexpr int GPB = sizeof(T) == 2 ? 8 : 4; };

// PHILOX (whole bundles): the noise is known at compile time to come from the generator, so
// the body has no branch on `stochastic` / `noise` and the generator's dependent chain can be
// interleaved with the arithmetic of neighbouring groups.
template <typename T, typename ST, int B, bool FULL, bool PHILOX>
ACTNN_DEV void pack_bundle(const Oct<T> (&x)[PackShape<T>::GPB], const BundleCoord& c, const T* __restrict__ mn,
                           const T* __restrict__ mx, ST* __restrict__ scale, ST* __restrict__ mn_out,
                           int32_t* __restrict__ out, const T* __restrict__ noise, int stochastic,
                           NoiseGen<T>& gen, const TransposePlan& plan, int lane) {
  constexpr int GPB = PackShape<T>::GPB;
  constexpr int W = GPB * 8 * B / 32;                    // words per lane string = transposes
  const int count = FULL ? GPB : c.count;
  // lane g (< count) prepares group g, then ships (mn', scale) to everyone
  ParamWords mine = {0u, 0u};
  if (lane < count) {
    const float gmn = load_scalar<T>(mn, c.q0 + lane), gmx = load_scalar<T>(mx, c.q0 + lane);
    const GroupParams gp = prepare_group<T>(gmn, gmx, B);
    store_scalar<ST>(scale, c.q0 + lane, gp.scale);
    if (mn_out) store_scalar<ST>(mn_out, c.q0 + lane, gmn);
    mine = pack_params<T>(gp);
  }
  uint32_t S[W];
#pragma unroll
  for (int k = 0; k < W; ++k) S[k] = 0u;
  Oct<T> nzb[NoiseShape<T>::GPC];                     // one call's worth of noise octets
#pragma unroll
  for (int gi = 0; gi < GPB; ++gi) {
    const QP<T> qp = fetch_params<T>(mine, gi);
    if (FULL || gi < count) {
      Oct<T> nz;
      if constexpr (PHILOX) {
        if (gi % NoiseShape<T>::GPC == 0) noise_block<T>(gen.key, (uint64_t)(c.q0 + gi), lane, nzb);
        nz = nzb[gi % NoiseShape<T>::GPC];
      } else if (!stochastic) nz = zero_oct<T>();
      else if (noise) nz = load_oct<T>(noise + (c.q0 + gi) * kGroup + lane * kOct);
      else if (!FULL) nz = gen.get((uint64_t)(c.q0 + gi));
      else {                                          // FULL: q0 is a multiple of the groups per call
        if (gi % NoiseShape<T>::GPC == 0) noise_block<T>(gen.key, (uint64_t)(c.q0 + gi), lane, nzb);
        nz = nzb[gi % NoiseShape<T>::GPC];
      }
      uint32_t lo, hi;
      row_from_magic<T, B>(quantize_oct<T, true, B>(x[gi], nz, qp), lo, hi);
      if (gi == 0) put_row<B, 0 * 8 * B>(S, lo, hi);
      if (gi == 1) put_row<B, 1 * 8 * B>(S, lo, hi);
      if (gi == 2) put_row<B, 2 * 8 * B>(S, lo, hi);
      if (gi == 3) put_row<B, 3 * 8 * B>(S, lo, hi);
      if constexpr (GPB > 4) {
        if (gi == 4) put_row<B, 4 * 8 * B>(S, lo, hi);
        if (gi == 5) put_row<B, 5 * 8 * B>(S, lo, hi);
        if (gi == 6) put_row<B, 6 * 8 * B>(S, lo, hi);
        if (gi == 7) put_row<B, 7 * 8 * B>(S, lo, hi);
      }
    }
  }
  const int words = count * 8 * B;
#pragma unroll
  for (int k = 0; k < W; ++k) {
    const uint32_t y = warp_transpose32(S[k], plan);
    const int o = k * 32 + lane;
    if (FULL || o < words) out[o] = (int32_t)y;
  }
}

template <typename T, typename ST, bool FULL, bool PHILOX = false>
__global__ void __launch_bounds__(kThreads, (MagicInfo<T>::paired && !PHILOX) ? 3 : 2)
pack_mixed_kernel(const T* __restrict__ data, const T* __restrict__ mn, const T* __restrict__ mx,
                  const int32_t* __restrict__ bits, const int64_t* __restrict__ word_offsets,
                  int32_t* __restrict__ packed, ST* __restrict__ scale, ST* __restrict__ mn_out,
                  int64_t N, int64_t G, const T* __restrict__ noise, int stochastic, const NoiseKey key) {
  constexpr int GPB = PackShape<T>::GPB;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const TransposePlan plan = make_transpose_plan(lane);
  NoiseGen<T> gen(key, lane);

  for (BundleWalker walk(warp, nwarps, N, G, GPB); walk.valid(); walk.next()) {
    const BundleCoord c = walk.coord();
    Oct<T> x[GPB];
#pragma unroll
    for (int gi = 0; gi < GPB; ++gi)
      x[gi] = (FULL || gi < c.count) ? load_oct<T>(data + (c.q0 + gi) * kGroup + lane * kOct) : zero_oct<T>();
    const int b = __ldg(bits + c.n);
    int32_t* out = packed + (__ldg(word_offsets + c.n) + (int64_t)c.g0 * 8 * b);
#define ACTNN_CASE(B)                                                                                     \
    case B:                                                                                               \
      pack_bundle<T, ST, B, FULL, PHILOX>(x, c, mn, mx, scale, mn_out, out, noise, stochastic, gen, plan, lane); \
      break;
    switch (b) {
      ACTNN_CASE(1) ACTNN_CASE(2) ACTNN_CASE(3) ACTNN_CASE(4) ACTNN_CASE(5) ACTNN_CASE(6) ACTNN_CASE(7)
      ACTNN_CASE(8)
      default: break;     // widths outside 1..8 are skipped; the host documents the range
    }
#undef ACTNN_CASE
  }
}

// ---------------------------------------------------------------------------- unpack
// Decoding a group needs only 2^B distinct outputs, code / scale + min for code = 0..2^B-1.
// Lanes compute those once (one IEEE division per lane for up to four groups at a time)
// and the elements look theirs up: for 16-bit types and B <= 2 the table of a group fits
// two registers and a byte-permute picks two elements per instruction; otherwise a warp
// shuffle fetches the entry; from 6 bits on the division is done per element.
template <int B> ACTNN_DEV uint32_t spread_codes_to_bytes(uint32_t r) {   // four B-bit codes -> one per byte
  if constexpr (B == 2) {
    uint32_t t = (r | (r << 12)) & 0x000f000fu;
    return (t | (t << 6)) & 0x03030303u;
  } else {
    uint32_t t = (r | (r << 14)) & 0x00030003u;
    return (t | (t << 7)) & 0x01010101u;
  }
}

// `words[k]` is word 32k + lane of the bundle (zero past its end); lanes 0..count-1 hold the
// statistics of their group in (stat_scale, stat_mn).  Both were loaded ahead of time.
template <typename T, int B>
ACTNN_DEV void unpack_bundle(const uint32_t (&words)[8], float stat_scale, float stat_mn, const BundleCoord& c,
                             T* __restrict__ out, const TransposePlan& plan, int lane) {
  constexpr int E = 1 << (B < 6 ? B : 5);              // table entries per group
  constexpr int GPC = (32 / E) < kBundle ? (32 / E) : kBundle;   // groups served by one table computation
  uint32_t S[B];
#pragma unroll
  for (int k = 0; k < B; ++k) S[k] = warp_transpose32(words[k], plan);
  uint32_t entry = 0u, pairs = 0u;
#pragma unroll
  for (int gi = 0; gi < kBundle; ++gi) {
    if constexpr (B < 6) {
      if (gi % GPC == 0) {                               // (re)build the table for groups gi .. gi+GPC-1
        const int g = (gi + lane / E) & (kBundle - 1);
        const float sc = __shfl_sync(kFull, stat_scale, g), m = __shfl_sync(kFull, stat_mn, g);
        entry = dequant_bits<T>((float)(lane % E), sc, m);
        if constexpr (sizeof(T) == 2 && B <= 2)
          pairs = entry | (__shfl_down_sync(kFull, entry, 1) << 16);
      }
    }
    uint32_t lo = 0u, hi = 0u;                           // this group's row
    if (gi == 0) { lo = get_bits<0 * 8 * B, (8 * B < 32 ? 8 * B : 32)>(S); if constexpr (8 * B > 32) hi = get_bits<0 * 8 * B + 32, 8 * B - 32>(S); }
    if (gi == 1) { lo = get_bits<1 * 8 * B, (8 * B < 32 ? 8 * B : 32)>(S); if constexpr (8 * B > 32) hi = get_bits<1 * 8 * B + 32, 8 * B - 32>(S); }
    if (gi == 2) { lo = get_bits<2 * 8 * B, (8 * B < 32 ? 8 * B : 32)>(S); if constexpr (8 * B > 32) hi = get_bits<2 * 8 * B + 32, 8 * B - 32>(S); }
    if (gi == 3) { lo = get_bits<3 * 8 * B, (8 * B < 32 ? 8 * B : 32)>(S); if constexpr (8 * B > 32) hi = get_bits<3 * 8 * B + 32, 8 * B - 32>(S); }
    Oct<T> o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
    if constexpr (sizeof(T) == 2 && B <= 2) {
      const int base = (gi % GPC) * E;
      const uint32_t t01 = __shfl_sync(kFull, pairs, base);
      const uint32_t t23 = B == 2 ? __shfl_sync(kFull, pairs, base + 2) : t01;
#pragma unroll
      for (int h = 0; h < 2; ++h) {                      // four elements per step
        const uint32_t y = spread_codes_to_bytes<B>((lo >> (4 * B * h)) & ((1u << (4 * B)) - 1u));
        const uint32_t sel = y * 0x22u + 0x10101010u;    // byte pair (2c, 2c+1) per element
        ow[2 * h] = __byte_perm(t01, t23, sel);
        ow[2 * h + 1] = __byte_perm(t01, t23, sel >> 16);
      }
    } else {
      uint32_t v[8];
      const uint32_t S2[2] = {lo, hi};
      uint32_t code[8];
      get_codes<B, 0>(S2, code);
      if constexpr (B < 6) {
        const int base = (gi % GPC) * E;
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __shfl_sync(kFull, entry, base + (int)code[j]);
      } else {
        const float sc = __shfl_sync(kFull, stat_scale, gi), m = __shfl_sync(kFull, stat_mn, gi);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = dequant_bits<T>((float)code[j], sc, m);
      }
      if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ow[j] = v[j];
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) ow[k] = v[2 * k] | (v[2 * k + 1] << 16);
      }
    }
    if (gi < c.count) store_oct<T>(out + (c.q0 + gi) * kGroup + lane * kOct, o);
  }
}

template <typename T, typename ST>
__global__ void __launch_bounds__(kThreads, 4)
unpack_mixed_kernel(const int32_t* __restrict__ packed, const int32_t* __restrict__ bits,
                    const int64_t* __restrict__ word_offsets, const ST* __restrict__ scale,
                    const ST* __restrict__ mn, T* __restrict__ out, int64_t N, int64_t G) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const TransposePlan plan = make_transpose_plan(lane);

  // A bundle's input is only b * 128 bytes per warp: issue the loads of DEPTH bundles before
  // decoding the first, so that enough bytes are in flight to cover the memory latency.
  constexpr int DEPTH = 2;
  BundleWalker walk(warp, nwarps, N, G);
  while (walk.valid()) {
    BundleCoord t_c[DEPTH];
    int t_b[DEPTH];
    bool t_ok[DEPTH];
    uint32_t t_w[DEPTH][8];
    float t_sc[DEPTH], t_m[DEPTH];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      t_ok[d] = walk.valid();
      t_b[d] = 0;
      t_sc[d] = 1.f;
      t_m[d] = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) t_w[d][k] = 0u;
      if (t_ok[d]) {
        t_c[d] = walk.coord();
        const BundleCoord& c = t_c[d];
        const int b = __ldg(bits + c.n);
        t_b[d] = b;
        const int32_t* in = packed + (__ldg(word_offsets + c.n) + (int64_t)c.g0 * 8 * b);
        const int words = c.count * 8 * b;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (k < b && k * 32 + lane < words) t_w[d][k] = (uint32_t)__ldg(in + k * 32 + lane);
        if (lane < c.count) {
          t_sc[d] = load_scalar<ST>(scale, c.q0 + lane);
          t_m[d] = load_scalar<ST>(mn, c.q0 + lane);
        }
        walk.next();
      }
    }
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      if (!t_ok[d]) break;                                // warp-uniform
#define ACTNN_CASE(B) \
      case B: unpack_bundle<T, B>(t_w[d], t_sc[d], t_m[d], t_c[d], out, plan, lane); break;
      switch (t_b[d]) {
        ACTNN_CASE(1) ACTNN_CASE(2) ACTNN_CASE(3) ACTNN_CASE(4) ACTNN_CASE(5) ACTNN_CASE(6) ACTNN_CASE(7)
        ACTNN_CASE(8)
        default: break;
      }
#undef ACTNN_CASE
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

template <typename T, typename ST>
int launch_pack(const void* data, const void* mn, const void* mx, const int32_t* bits,
                const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out, int64_t N,
                int64_t G, int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                cudaStream_t stream) {
  constexpr int GPB = PackShape<T>::GPB;
  const int64_t tasks = N * ((G + GPB - 1) / GPB);
  const NoiseKey key = make_noise_key(seed, offset);
  if (G % GPB == 0 && stochastic && !noise)
    pack_mixed_kernel<T, ST, true, true><<<persistent_grid(pack_mixed_kernel<T, ST, true, true>, kThreads, tasks),
                                           kThreads, 0, stream>>>(
        (const T*)data, (const T*)mn, (const T*)mx, bits, word_offsets, packed, (ST*)scale, (ST*)mn_out, N, G,
        (const T*)noise, stochastic, key);
  else if (G % GPB == 0)
    pack_mixed_kernel<T, ST, true><<<persistent_grid(pack_mixed_kernel<T, ST, true>, kThreads, tasks), kThreads, 0,
                                     stream>>>(
        (const T*)data, (const T*)mn, (const T*)mx, bits, word_offsets, packed, (ST*)scale, (ST*)mn_out, N, G,
        (const T*)noise, stochastic, key);
  else
    pack_mixed_kernel<T, ST, false><<<persistent_grid(pack_mixed_kernel<T, ST, false>, kThreads, tasks), kThreads, 0,
                                      stream>>>(
        (const T*)data, (const T*)mn, (const T*)mx, bits, word_offsets, packed, (ST*)scale, (ST*)mn_out, N, G,
        (const T*)noise, stochastic, key);
  return check_launch();
}

template <typename T, typename ST>
int launch_unpack(const int32_t* packed, const int32_t* bits, const int64_t* word_offsets,
                  const void* scale, const void* mn, void* out, int64_t N, int64_t G, cudaStream_t stream) {
  const int64_t tasks = N * ((G + kBundle - 1) / kBundle);
  unpack_mixed_kernel<T, ST><<<persistent_grid(unpack_mixed_kernel<T, ST>, kThreads, tasks), kThreads, 0, stream>>>(
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
