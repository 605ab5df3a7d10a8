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

// Device counter of bundles whose width was outside 1..8 (nothing is written for them).
__device__ unsigned g_bad_width_bundles;

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
      default:            // widths outside 1..8: nothing is written, the bundle is counted
        if (lane == 0) atomicAdd(&g_bad_width_bundles, 1u);
        break;
    }
#undef ACTNN_CASE
  }
}

// ---------------------------------------------------------------------------- pack, flat tasks
// Fast path for G % 4 == 0 and G >= 32 (every layer of the usual networks).  A warp task is
// 32 consecutive groups of the flattened [N * G] list:
//   * lane l prepares group q0 + l: its sample, width and stream position, one coalesced load
//     of min / max, ONE division, coalesced stores of scale / min.  All 32 lanes work, so the
//     per-group cost is a quarter of what a four-group bundle with four active lanes pays;
//   * the task is then worked off as eight bundles of four groups (one generator call per
//     lane, `B` transposes, `B` coalesced 128-byte stores).  A bundle never straddles two
//     samples because G % 4 == 0, so its width is warp-uniform;
//   * the octets of the next bundle (also across the task boundary) are requested before the
//     current one is quantized: a warp always has loads in flight.
constexpr int kFlatGroups = 32;       // groups per task
constexpr int kFlatBundle = 4;        // groups per bundle
enum NoiseMode { kNoisePhilox = 0, kNoiseTensor = 1, kNoiseNone = 2 };
#ifndef ACTNN_FLAT_BLOCKS
#define ACTNN_FLAT_BLOCKS 2
#endif
#ifndef ACTNN_FLAT_UNPACK_BLOCKS
#define ACTNN_FLAT_UNPACK_BLOCKS 3   // 85 registers, nothing spilled: measured 3-4 % faster than 4 blocks (64 registers, spills)
#endif
constexpr int kFlatUnpackBlocks = ACTNN_FLAT_UNPACK_BLOCKS;
constexpr int kFlatBlocks16 = ACTNN_FLAT_BLOCKS;   // resident blocks per SM the flat kernels are compiled for (16-bit types)

// (mn', scale) of the lane's own group in the form the quantizer consumes.
template <typename T> struct LaneParams { uint32_t a, b; };
template <typename T> ACTNN_DEV LaneParams<T> lane_params(const GroupParams& gp) {
  LaneParams<T> p;
  if constexpr (sizeof(T) == 4) {
    p.a = __float_as_uint(gp.mn1);
    p.b = __float_as_uint(gp.scale);
  } else {
    p.a = bits_of<T>(gp.mn1) * 0x00010001u;
    p.b = bits_of<T>(gp.scale) * 0x00010001u;
  }
  return p;
}
template <typename T> ACTNN_DEV QP<T> fetch_lane_params(const LaneParams<T>& mine, int src_lane) {
  const uint32_t a = __shfl_sync(kFull, mine.a, src_lane), b = __shfl_sync(kFull, mine.b, src_lane);
  QP<T> q;
  if constexpr (sizeof(T) == 4) {
    q.mn1 = __uint_as_float(a);
    q.scale = __uint_as_float(b);
  } else {
    q.mn2 = *reinterpret_cast<const decltype(q.mn2)*>(&a);
    q.sc2 = *reinterpret_cast<const decltype(q.sc2)*>(&b);
  }
  return q;
}

template <typename T, int B, int MODE, bool CLAMP_LOW>
ACTNN_DEV void pack_flat_bundle(const Oct<T> (&x)[kFlatBundle], const LaneParams<T>& mine, int first_lane,
                                int64_t q, int32_t* __restrict__ out, const T* __restrict__ noise,
                                const NoiseKey& key, const TransposePlan& plan, int lane) {
  constexpr int GPC = NoiseShape<T>::GPC;
  uint32_t S[B];
#pragma unroll
  for (int k = 0; k < B; ++k) S[k] = 0u;
  Oct<T> nzb[GPC];
#pragma unroll
  for (int gi = 0; gi < kFlatBundle; ++gi) {
    const QP<T> qp = fetch_lane_params<T>(mine, first_lane + gi);
    Oct<T> nz;
    if constexpr (MODE == kNoisePhilox) {
      if (gi % GPC == 0) noise_block<T>(key, (uint64_t)(q + gi), lane, nzb);
      nz = nzb[gi % GPC];
    } else if constexpr (MODE == kNoiseTensor) {
      nz = load_oct<T>(noise + (q + gi) * kGroup + lane * kOct);
    } else {
      nz = zero_oct<T>();
    }
    uint32_t lo, hi;
    row_from_magic<T, B>(quantize_oct<T, CLAMP_LOW, B>(x[gi], nz, qp), lo, hi);
    if (gi == 0) put_row<B, 0 * 8 * B>(S, lo, hi);
    if (gi == 1) put_row<B, 1 * 8 * B>(S, lo, hi);
    if (gi == 2) put_row<B, 2 * 8 * B>(S, lo, hi);
    if (gi == 3) put_row<B, 3 * 8 * B>(S, lo, hi);
  }
#pragma unroll
  for (int k = 0; k < B; ++k) out[k * 32 + lane] = (int32_t)warp_transpose32(S[k], plan);
}

// A run: bundles k0 .. k1-1 of a task, all of the same width B (a run ends where the next
// sample has another width).  The width is a template argument here, so the loop over the
// bundles has no dispatch in it and the octets of bundle k+1 are requested before bundle k is
// quantized (two register buffers used alternately; nothing is copied).  `a` already holds the
// octets of bundle k0.
template <typename T, int B, int MODE, bool CLAMP_LOW, bool PREFETCH>
ACTNN_DEV void pack_flat_run(Oct<T> (&a)[kFlatBundle], Oct<T> (&b)[kFlatBundle], int k0, int k1, int64_t q0,
                             const T* __restrict__ data, const LaneParams<T>& mine, int32_t* __restrict__ out,
                             const T* __restrict__ noise, const NoiseKey& key, const TransposePlan& plan, int lane) {
  auto load = [&](Oct<T> (&dst)[kFlatBundle], int k) {
#pragma unroll
    for (int gi = 0; gi < kFlatBundle; ++gi)
      dst[gi] = load_oct<T>(data + (q0 + k * kFlatBundle + gi) * kGroup + lane * kOct);
  };
  if constexpr (!PREFETCH) {
    for (int k = k0; k < k1; ++k) {
      if (k > k0) load(a, k);
      pack_flat_bundle<T, B, MODE, CLAMP_LOW>(a, mine, k * kFlatBundle, q0 + k * kFlatBundle, out, noise, key, plan,
                                              lane);
      out += 32 * B;                                           // consecutive groups are consecutive in the stream
    }
  } else {
    for (int k = k0; k < k1; k += 2) {
      if (k + 1 < k1) load(b, k + 1);
      pack_flat_bundle<T, B, MODE, CLAMP_LOW>(a, mine, k * kFlatBundle, q0 + k * kFlatBundle, out, noise, key, plan,
                                              lane);
      out += 32 * B;
      if (k + 1 >= k1) break;
      if (k + 2 < k1) load(a, k + 2);
      pack_flat_bundle<T, B, MODE, CLAMP_LOW>(b, mine, (k + 1) * kFlatBundle, q0 + (k + 1) * kFlatBundle, out,
                                              noise, key, plan, lane);
      out += 32 * B;
    }
  }
}

template <typename T, typename ST, int MODE, bool CLAMP_LOW>
__global__ void __launch_bounds__(kThreads, sizeof(T) == 2 ? kFlatBlocks16 : 2)
pack_mixed_flat_kernel(const T* __restrict__ data, const T* __restrict__ mn, const T* __restrict__ mx,
                       const int32_t* __restrict__ bits, const int64_t* __restrict__ word_offsets,
                       int32_t* __restrict__ packed, ST* __restrict__ scale, ST* __restrict__ mn_out,
                       int64_t Q, int64_t G, const T* __restrict__ noise, const NoiseKey key) {
  constexpr bool PREFETCH = sizeof(T) == 2;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const TransposePlan plan = make_transpose_plan(lane);
  const int64_t tasks = (Q + kFlatGroups - 1) / kFlatGroups;
  if (warp >= tasks) return;

  // (sample, group) of the task's first group, advanced without divisions inside the loop
  int64_t q0 = warp * kFlatGroups;
  int64_t n0 = q0 / G;
  int64_t r0 = q0 - n0 * G;
  const int64_t stride = nwarps * kFlatGroups;
  const int64_t step_n = stride / G, step_r = stride - step_n * G;

  Oct<T> bufA[kFlatBundle], bufB[kFlatBundle];                  // bufB stays unused without PREFETCH
  for (; q0 < Q; q0 += stride) {
    // the octets of the task's first bundle are requested before anything else, so that they
    // travel while the lanes prepare their groups
#pragma unroll
    for (int gi = 0; gi < kFlatBundle; ++gi) bufA[gi] = load_oct<T>(data + (q0 + gi) * kGroup + lane * kOct);
    // ---- this lane's group
    const int64_t q = q0 + lane;
    int64_t n = n0, r = r0 + lane;
    if (r >= G) { r -= G; ++n; }                              // G >= 32: at most one wrap
    int b_l = -1;                                             // past the end of the activation
    int64_t off_l = 0;
    LaneParams<T> mine = {0u, 0u};
    if (q < Q) {
      b_l = __ldg(bits + n);
      if (b_l < 1 || b_l > 8) b_l = 0;                        // not a width: counted, nothing written
      off_l = __ldg(word_offsets + n) + r * (8 * b_l);
      const float gmn = load_scalar<T>(mn, q), gmx = load_scalar<T>(mx, q);
      const GroupParams gp = prepare_group<T>(gmn, gmx, b_l);
      store_scalar<ST>(scale, q, gp.scale);
      if (mn_out) store_scalar<ST>(mn_out, q, gmn);
      mine = lane_params<T>(gp);
    }
    // ---- runs of bundles of one width (the lanes past the end close the last run)
    int k = 0;
    while (k < kFlatGroups / kFlatBundle) {
      const int first = k * kFlatBundle;
      const int b = __shfl_sync(kFull, b_l, first);
      if (b < 0) break;
      const unsigned same = __ballot_sync(kFull, b_l == b) >> first;          // bit i: lane first + i
      const int run_lanes = same == 0xffffffffu >> first ? 32 - first : __ffs((int)~same) - 1;
      const int k1 = k + run_lanes / kFlatBundle;
      const uint32_t olo = __shfl_sync(kFull, (uint32_t)off_l, first);
      const uint32_t ohi = __shfl_sync(kFull, (uint32_t)((uint64_t)off_l >> 32), first);
      int32_t* out = packed + (int64_t)(((uint64_t)ohi << 32) | olo);
      if (k > 0) {
#pragma unroll
        for (int gi = 0; gi < kFlatBundle; ++gi)
          bufA[gi] = load_oct<T>(data + (q0 + first + gi) * kGroup + lane * kOct);
      }
#define ACTNN_CASE(B)                                                                                          \
      case B:                                                                                                  \
        pack_flat_run<T, B, MODE, CLAMP_LOW, PREFETCH>(bufA, bufB, k, k1, q0, data, mine, out, noise, key, plan, lane); \
        break;
      switch (b) {
        ACTNN_CASE(1) ACTNN_CASE(2) ACTNN_CASE(3) ACTNN_CASE(4) ACTNN_CASE(5) ACTNN_CASE(6) ACTNN_CASE(7)
        ACTNN_CASE(8)
        default:
          if (lane == 0) atomicAdd(&g_bad_width_bundles, (unsigned)(k1 - k));
          break;
      }
#undef ACTNN_CASE
      k = k1;
    }
    n0 += step_n;
    r0 += step_r;
    if (r0 >= G) { r0 -= G; ++n0; }
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
        float y = 0.f;
        if (sizeof(T) == 2 && group_reciprocal(sc, y)) {           // 16-bit statistics; warp-uniform
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = dequant_bits_recip<T>((float)code[j], sc, y, m);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = dequant_bits<T>((float)code[j], sc, m);
        }
      }
      if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ow[j] = v[j];
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) ow[k] = v[2 * k] | (v[2 * k + 1] << 16);
      }
    }
    if (gi < c.count) store_oct_streaming<T>(out + (c.q0 + gi) * kGroup + lane * kOct, o);
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

// How the flat unpack kernel deals out its tasks (32 consecutive groups each).  Block b owns tasks
// b, b + gridDim.x, b + 2 gridDim.x, ... -- a sample is 20 to 30 consecutive tasks, so every block
// meets every width in the proportion of the whole activation -- and its warps claim them one at
// a time from a counter in shared memory: a warp that met wider (slower) samples simply takes
// fewer tasks.  The last `split` tasks of a block are claimed as halves of 16 groups, which
// shortens the ragged end of the launch (an activation is only a few tasks per resident warp).
// Nothing is shared between blocks or launches.
#ifndef ACTNN_UNPACK_SPLIT
#define ACTNN_UNPACK_SPLIT 8
#endif
struct FlatClaim { int64_t task; int kb, ke; };            // bundles kb .. ke-1 of the task
struct FlatPool {
  unsigned* counters;                                      // [0] whole tasks claimed, [1] halves claimed
  unsigned whole, halves;
  bool in_halves;
  ACTNN_DEV void init(unsigned* smem2, int64_t tasks, int split_tasks) {
    counters = smem2;
    const int64_t mine = tasks > blockIdx.x ? (tasks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int64_t split = mine < split_tasks ? mine : split_tasks;
    whole = (unsigned)(mine - split);
    halves = (unsigned)(2 * split);
    in_halves = false;
    if (threadIdx.x < 2) counters[threadIdx.x] = 0u;
    __syncthreads();
  }
  ACTNN_DEV int64_t task_of(unsigned i) const { return blockIdx.x + (int64_t)i * gridDim.x; }
  ACTNN_DEV bool claim(int lane, FlatClaim& c) {
    unsigned i = 0u;
    if (!in_halves) {
      if (lane == 0) i = atomicAdd(&counters[0], 1u);
      i = __shfl_sync(kFull, i, 0);
      if (i < whole) { c.task = task_of(i); c.kb = 0; c.ke = kFlatGroups / kFlatBundle; return true; }
      in_halves = true;
    }
    if (lane == 0) i = atomicAdd(&counters[1], 1u);
    i = __shfl_sync(kFull, i, 0);
    if (i >= halves) return false;
    constexpr int kHalfBundles = kFlatGroups / kFlatBundle / 2;
    c.task = task_of(whole + (i >> 1));
    c.kb = (int)(i & 1u) * kHalfBundles;
    c.ke = c.kb + kHalfBundles;
    return true;
  }
};
// (sample, group) of group q; one 32-bit division where the activation allows it
ACTNN_DEV void split_group_index(int64_t q, int64_t G, int64_t& n, int64_t& r) {
  if (((uint64_t)q | (uint64_t)G) >> 32) { n = q / G; } else { n = (int64_t)((uint32_t)q / (uint32_t)G); }
  r = q - n * G;
}

// ---------------------------------------------------------------------------- unpack, flat tasks
// Same task shape as the flat pack: lane l owns group q0 + l of a task of 32 groups (its
// sample, width, stream position, scale and min come from coalesced loads), and eight bundles
// of four groups are decoded with the words of the next bundle already requested.  For 16-bit
// outputs at 1 or 2 bits the lane also computes the 2^B decoded values of its own group once
// per task (packed in two registers); a bundle then fetches them with two shuffles per group.
#ifndef ACTNN_UNPACK_DIRECT_FROM
#define ACTNN_UNPACK_DIRECT_FROM 6
#endif
template <typename T, int B, bool FASTDIV>
ACTNN_DEV void unpack_flat_bundle(const uint32_t (&words)[B], float sc_l, float m_l, uint32_t t01_l, uint32_t t23_l,
                                  int first, int64_t q, T* __restrict__ out, const TransposePlan& plan, int lane) {
  // from kDirect bits on every element is computed (a table of 2^B entries no longer fits a warp,
  // or costs more shuffles than the arithmetic)
  constexpr int kDirect = FASTDIV ? ACTNN_UNPACK_DIRECT_FROM : 6;
  constexpr int E = 1 << (B < kDirect ? B : 5);        // table entries per group
  constexpr int GPC = (32 / E) < kFlatBundle ? (32 / E) : kFlatBundle;   // groups served by one table
  constexpr bool PAIRS = sizeof(T) == 2 && B <= 2;
  uint32_t S[B];
#pragma unroll
  for (int k = 0; k < B; ++k) S[k] = warp_transpose32(words[k], plan);
  uint32_t entry = 0u;
#pragma unroll
  for (int gi = 0; gi < kFlatBundle; ++gi) {
    if constexpr (!PAIRS && B < kDirect) {
      if (gi % GPC == 0) {                               // (re)build the table for groups gi .. gi+GPC-1
        const int g = first + ((gi + lane / E) & (kFlatBundle - 1));
        const float sc = __shfl_sync(kFull, sc_l, g), m = __shfl_sync(kFull, m_l, g);
        entry = dequant_bits<T>((float)(lane % E), sc, m);
      }
    }
    uint32_t lo = 0u, hi = 0u;                           // this group's row
    if (gi == 0) { lo = get_bits<0 * 8 * B, (8 * B < 32 ? 8 * B : 32)>(S); if constexpr (8 * B > 32) hi = get_bits<0 * 8 * B + 32, 8 * B - 32>(S); }
    if (gi == 1) { lo = get_bits<1 * 8 * B, (8 * B < 32 ? 8 * B : 32)>(S); if constexpr (8 * B > 32) hi = get_bits<1 * 8 * B + 32, 8 * B - 32>(S); }
    if (gi == 2) { lo = get_bits<2 * 8 * B, (8 * B < 32 ? 8 * B : 32)>(S); if constexpr (8 * B > 32) hi = get_bits<2 * 8 * B + 32, 8 * B - 32>(S); }
    if (gi == 3) { lo = get_bits<3 * 8 * B, (8 * B < 32 ? 8 * B : 32)>(S); if constexpr (8 * B > 32) hi = get_bits<3 * 8 * B + 32, 8 * B - 32>(S); }
    Oct<T> o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
    if constexpr (PAIRS) {
      const uint32_t t01 = __shfl_sync(kFull, t01_l, first + gi);
      const uint32_t t23 = B == 2 ? __shfl_sync(kFull, t23_l, first + gi) : t01;
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
      if constexpr (B < kDirect) {
        const int base = (gi % GPC) * E;
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __shfl_sync(kFull, entry, base + (int)code[j]);
      } else {
        const float sc = __shfl_sync(kFull, sc_l, first + gi), m = __shfl_sync(kFull, m_l, first + gi);
        float y = 0.f;
        if (FASTDIV && group_reciprocal(sc, y)) {                 // warp-uniform: one scale per group
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = dequant_bits_recip<T>((float)code[j], sc, y, m);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = dequant_bits<T>((float)code[j], sc, m);
        }
      }
      if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ow[j] = v[j];
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) ow[k] = v[2 * k] | (v[2 * k + 1] << 16);
      }
    }
    store_oct_streaming<T>(out + (q + gi) * kGroup + lane * kOct, o);
  }
}

// A run of bundles k0 .. k1-1 of one width B (see pack_flat_run): the B words per lane of
// bundle k+1 are requested before bundle k is decoded.  `in` points at this lane's first word
// of bundle k0; a bundle is 32 * B words.
template <typename T, int B, bool FASTDIV>
ACTNN_DEV void unpack_flat_run(int k0, int k1, int64_t q0, const int32_t* __restrict__ in, float sc_l, float m_l,
                               uint32_t t01_l, uint32_t t23_l, T* __restrict__ out, const TransposePlan& plan,
                               int lane) {
  auto load = [&](uint32_t (&w)[B], const int32_t* p) {
#pragma unroll
    for (int kk = 0; kk < B; ++kk) w[kk] = (uint32_t)__ldg(p + kk * 32);
  };
  if constexpr (B <= 2 && sizeof(T) == 2) {
    // Narrow widths, 16-bit outputs: four bundles at a time are decoded as straight-line code.
    // The words of up to 8 bundles (8 * B registers) are requested up front (2 KB per warp in
    // flight instead of 256 bytes), the transposes of four bundles are issued together
    // (4 * B independent butterfly chains instead of B), and only the stores are predicated, so
    // the scheduler always has independent work.  A run that is not a multiple of four bundles
    // transposes a few zero words.
    constexpr int kHalf = kFlatGroups / kFlatBundle / 2;         // bundles decoded per pass of the loop below
    uint32_t S[kHalf][B], N2[kHalf][B];
#pragma unroll
    for (int i = 0; i < kHalf; ++i) {
#pragma unroll
      for (int kk = 0; kk < B; ++kk) {
        S[i][kk] = (k0 + i < k1) ? (uint32_t)__ldg(in + (i * B + kk) * 32) : 0u;
        N2[i][kk] = (k0 + kHalf + i < k1) ? (uint32_t)__ldg(in + ((kHalf + i) * B + kk) * 32) : 0u;
      }
    }
    // two passes over the same code (kept rolled: the straight-line body of one pass is already
    // a few thousand instructions, and the instruction cache is shared by all eight widths)
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      const int kb = k0 + half * kHalf;
      if (kb >= k1) break;
#pragma unroll
      for (int i = 0; i < kHalf; ++i) {
#pragma unroll
        for (int kk = 0; kk < B; ++kk) S[i][kk] = warp_transpose32(S[i][kk], plan);
      }
#pragma unroll
      for (int i = 0; i < kHalf; ++i) {
        const bool live = kb + i < k1;
        const int first = (kb + i < 2 * kHalf ? kb + i : 2 * kHalf - 1) * kFlatBundle;   // a lane of this warp in any case
#pragma unroll
        for (int gi = 0; gi < kFlatBundle; ++gi) {
          const uint32_t t01 = __shfl_sync(kFull, t01_l, first + gi);
          const uint32_t t23 = B == 2 ? __shfl_sync(kFull, t23_l, first + gi) : t01;
          uint32_t lo = 0u;
          if (gi == 0) lo = get_bits<0 * 8 * B, 8 * B>(S[i]);
          if (gi == 1) lo = get_bits<1 * 8 * B, 8 * B>(S[i]);
          if (gi == 2) lo = get_bits<2 * 8 * B, 8 * B>(S[i]);
          if (gi == 3) lo = get_bits<3 * 8 * B, 8 * B>(S[i]);
          Oct<T> o;
#pragma unroll
          for (int h = 0; h < 2; ++h) {                      // four elements per step
            const uint32_t y = spread_codes_to_bytes<B>((lo >> (4 * B * h)) & ((1u << (4 * B)) - 1u));
            const uint32_t sel = y * 0x22u + 0x10101010u;    // byte pair (2c, 2c+1) per element
            o.r[2 * h] = __byte_perm(t01, t23, sel);
            o.r[2 * h + 1] = __byte_perm(t01, t23, sel >> 16);
          }
          if (live) store_oct_streaming<T>(out + (q0 + (kb + i) * kFlatBundle + gi) * kGroup + lane * kOct, o);
        }
      }
#pragma unroll
      for (int i = 0; i < kHalf; ++i) {
#pragma unroll
        for (int kk = 0; kk < B; ++kk) S[i][kk] = N2[i][kk];
      }
    }
  } else {
    uint32_t wa[B], wb[B];
    load(wa, in);
    for (int k = k0; k < k1; k += 2) {
      if (k + 1 < k1) load(wb, in + 32 * B);
      unpack_flat_bundle<T, B, FASTDIV>(wa, sc_l, m_l, t01_l, t23_l, k * kFlatBundle, q0 + k * kFlatBundle, out, plan, lane);
      if (k + 1 >= k1) break;
      if (k + 2 < k1) load(wa, in + 64 * B);
      unpack_flat_bundle<T, B, FASTDIV>(wb, sc_l, m_l, t01_l, t23_l, (k + 1) * kFlatBundle, q0 + (k + 1) * kFlatBundle, out,
                               plan, lane);
      in += 64 * B;
    }
  }
}

template <typename T, typename ST>
__global__ void __launch_bounds__(kThreads, kFlatUnpackBlocks)
unpack_mixed_flat_kernel(const int32_t* __restrict__ packed, const int32_t* __restrict__ bits,
                         const int64_t* __restrict__ word_offsets, const ST* __restrict__ scale,
                         const ST* __restrict__ mn, T* __restrict__ out, int64_t Q, int64_t G) {
  const int lane = threadIdx.x & 31;
  const TransposePlan plan = make_transpose_plan(lane);
  __shared__ unsigned pool_counters[2];
  FlatPool pool;
  pool.init(pool_counters, (Q + kFlatGroups - 1) / kFlatGroups, ACTNN_UNPACK_SPLIT);

  FlatClaim claim;
  while (pool.claim(lane, claim)) {
    const int64_t q0 = claim.task * kFlatGroups;
    const int64_t q = q0 + lane;
    int b_l = -1;                                             // past the end of the activation
    int64_t off_l = 0;
    float sc_l = 1.f, m_l = 0.f;
    uint32_t t01_l = 0u, t23_l = 0u;
    if (q < Q) {
      int64_t n, r;
      split_group_index(q, G, n, r);
      b_l = __ldg(bits + n);
      if (b_l < 1 || b_l > 8) b_l = 0;                        // not a width: the pack kernel wrote nothing either
      off_l = __ldg(word_offsets + n) + r * (8 * b_l);
      sc_l = load_scalar<ST>(scale, q);
      m_l = load_scalar<ST>(mn, q);
      if constexpr (sizeof(T) == 2) {
        if (b_l == 1 || b_l == 2) {
          const uint32_t e0 = dequant_bits<T>(0.f, sc_l, m_l), e1 = dequant_bits<T>(1.f, sc_l, m_l);
          t01_l = e0 | (e1 << 16);
          if (b_l == 2) {
            const uint32_t e2 = dequant_bits<T>(2.f, sc_l, m_l), e3 = dequant_bits<T>(3.f, sc_l, m_l);
            t23_l = e2 | (e3 << 16);
          }
        }
      }
    }
    int k = claim.kb;
    while (k < claim.ke) {
      const int first = k * kFlatBundle;
      const int b = __shfl_sync(kFull, b_l, first);
      if (b < 0) break;
      const unsigned same = __ballot_sync(kFull, b_l == b) >> first;          // bit i: lane first + i
      const int run_lanes = same == 0xffffffffu >> first ? 32 - first : __ffs((int)~same) - 1;
      const int k1 = min(k + run_lanes / kFlatBundle, claim.ke);
      const uint32_t olo = __shfl_sync(kFull, (uint32_t)off_l, first);
      const uint32_t ohi = __shfl_sync(kFull, (uint32_t)((uint64_t)off_l >> 32), first);
      const int32_t* in = packed + (int64_t)(((uint64_t)ohi << 32) | olo) + lane;
#define ACTNN_CASE(B) \
      case B: unpack_flat_run<T, B, sizeof(ST) == 2>(k, k1, q0, in, sc_l, m_l, t01_l, t23_l, out, plan, lane); break;
      switch (b) {
        ACTNN_CASE(1) ACTNN_CASE(2) ACTNN_CASE(3) ACTNN_CASE(4) ACTNN_CASE(5) ACTNN_CASE(6) ACTNN_CASE(7)
        ACTNN_CASE(8)
        default: break;
      }
#undef ACTNN_CASE
      k = k1;
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

template <typename T, typename ST, int MODE, bool CLAMP_LOW>
void launch_pack_flat(const void* data, const void* mn, const void* mx, const int32_t* bits,
                      const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out, int64_t N,
                      int64_t G, const void* noise, const NoiseKey& key, cudaStream_t stream) {
  auto kernel = pack_mixed_flat_kernel<T, ST, MODE, CLAMP_LOW>;
  const int64_t tasks = (N * G + kFlatGroups - 1) / kFlatGroups;
  kernel<<<persistent_grid(kernel, kThreads, tasks), kThreads, 0, stream>>>(
      (const T*)data, (const T*)mn, (const T*)mx, bits, word_offsets, packed, (ST*)scale, (ST*)mn_out, N * G, G,
      (const T*)noise, key);
}

template <typename T, typename ST>
int launch_pack(const void* data, const void* mn, const void* mx, const int32_t* bits,
                const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out, int64_t N,
                int64_t G, int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                bool min_is_exact, cudaStream_t stream) {
  constexpr int GPB = PackShape<T>::GPB;
  const int64_t tasks = N * ((G + GPB - 1) / GPB);
  const NoiseKey key = make_noise_key(seed, offset);
  if (G % kFlatBundle == 0 && G >= kFlatGroups) {
#define ACTNN_FLAT(MODE)                                                                                     \
    if (min_is_exact)                                                                                        \
      launch_pack_flat<T, ST, MODE, false>(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G, noise, \
                                           key, stream);                                                     \
    else                                                                                                     \
      launch_pack_flat<T, ST, MODE, true>(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G, noise, \
                                          key, stream);
    if (!stochastic) { ACTNN_FLAT(kNoiseNone) }
    else if (noise) { ACTNN_FLAT(kNoiseTensor) }
    else { ACTNN_FLAT(kNoisePhilox) }
#undef ACTNN_FLAT
    return check_launch();
  }
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
  if (G % kFlatBundle == 0 && G >= kFlatGroups) {
    auto kernel = unpack_mixed_flat_kernel<T, ST>;
    const int64_t flat_tasks = (N * G + kFlatGroups - 1) / kFlatGroups;
    // sized by half tasks: a small activation spreads over twice the warps (see FlatPool)
    kernel<<<persistent_grid(kernel, kThreads, 2 * flat_tasks), kThreads, 0, stream>>>(
        packed, bits, word_offsets, (const ST*)scale, (const ST*)mn, (T*)out, N * G, G);
    return check_launch();
  }
  const int64_t tasks = N * ((G + kBundle - 1) / kBundle);
  unpack_mixed_kernel<T, ST><<<persistent_grid(unpack_mixed_kernel<T, ST>, kThreads, tasks), kThreads, 0, stream>>>(
      packed, bits, word_offsets, (const ST*)scale, (const ST*)mn, (T*)out, N, G);
  return check_launch();
}

int check_common(int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype) {
  if (N < 0 || G < 0) return ACTNN_ERR_SHAPE;
  if (group_size != kGroup && !generic_group_ok(group_size)) return ACTNN_ERR_SHAPE;
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

namespace actnn {
// `min_is_exact`: every `mn[q]` is the true minimum of its group (then the rounding itself maps
// the smallest values to code 0 and the lower clamp is dropped).
int pack_mixed_impl(const void* data, const void* mn, const void* mx, const int32_t* bits,
                    const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out, int64_t N, int64_t G,
                    int64_t group_size, int dtype, int stat_dtype, int stochastic, const void* noise, uint64_t seed,
                    uint64_t offset, bool min_is_exact, cudaStream_t s) {
  if (int st = check_common(N, G, group_size, dtype, stat_dtype)) return st;
  if (N == 0 || G == 0) return ACTNN_OK;
  if (!data || !mn || !mx || !bits || !word_offsets || !packed || !scale) return ACTNN_ERR_NULL;
  if (group_size != kGroup)
    return pack_mixed_generic(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G, group_size, dtype,
                              stat_dtype, stochastic, noise, seed, offset, s);
  const size_t al = dtype == ACTNN_F32 ? 32 : 16;
  if (!aligned(data, al) || (noise && !aligned(noise, al)) || !aligned(packed, 4)) return ACTNN_ERR_ALIGN;
  switch (dtype) {
    case ACTNN_F16:
      return launch_pack<__half, __half>(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G,
                                         stochastic, noise, seed, offset, min_is_exact, s);
    case ACTNN_BF16:
      return launch_pack<__nv_bfloat16, __nv_bfloat16>(data, mn, mx, bits, word_offsets, packed, scale, mn_out,
                                                       N, G, stochastic, noise, seed, offset, min_is_exact, s);
    default:
      if (stat_dtype == ACTNN_BF16)
        return launch_pack<float, __nv_bfloat16>(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G,
                                                 stochastic, noise, seed, offset, min_is_exact, s);
      return launch_pack<float, float>(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G,
                                       stochastic, noise, seed, offset, min_is_exact, s);
  }
}
}  // namespace actnn

extern "C" int actnn_pack_mixed(const void* data, const void* mn, const void* mx, const int32_t* bits,
                                const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out,
                                int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype,
                                int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                                actnn_stream_t stream) {
  return pack_mixed_impl(data, mn, mx, bits, word_offsets, packed, scale, mn_out, N, G, group_size, dtype,
                         stat_dtype, stochastic, noise, seed, offset, false, (cudaStream_t)stream);
}

extern "C" int actnn_bad_width_bundles(uint32_t* count) {
  if (!count) return ACTNN_ERR_NULL;
  return cudaMemcpyFromSymbol(count, g_bad_width_bundles, sizeof(unsigned)) == cudaSuccess ? ACTNN_OK
                                                                                           : ACTNN_ERR_LAUNCH;
}

extern "C" int actnn_unpack_mixed(const int32_t* packed, const int32_t* bits, const int64_t* word_offsets,
                                  const void* scale, const void* mn, void* out, int64_t N, int64_t G,
                                  int64_t group_size, int dtype, int stat_dtype, actnn_stream_t stream) {
  if (int st = check_common(N, G, group_size, dtype, stat_dtype)) return st;
  if (N == 0 || G == 0) return ACTNN_OK;
  if (!packed || !bits || !word_offsets || !scale || !mn || !out) return ACTNN_ERR_NULL;
  cudaStream_t s = (cudaStream_t)stream;
  if (group_size != kGroup)
    return unpack_mixed_generic(packed, bits, word_offsets, scale, mn, out, N, G, group_size, dtype, stat_dtype, s);
  if (!aligned(out, dtype == ACTNN_F32 ? 32 : 16) || !aligned(packed, 4)) return ACTNN_ERR_ALIGN;
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
