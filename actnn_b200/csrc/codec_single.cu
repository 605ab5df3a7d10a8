// Single-precision (uniform bit width) stream: int8 bytes packed ACROSS the batch axis.
//
// Layout (reference: quantization_cuda_kernel.cu:236-257): byte (no*G + g)*256 + d holds
// the codes of samples no*wpt + ni (wpt = 8 / bits, ni = 0..wpt-1) for position d of group
// g, sample ni at bit offset ni*bits.
//
// A warp owns (sample block no, two neighbouring groups).  Lane t owns positions
// 8t..8t+7 of each group, loads one 16/32-byte octet per (sample, group), and ORs the
// wpt samples' codes into eight bytes that it stores with one 8-byte store (256 B per
// warp, contiguous).  The fused variant gets each group's min / max from two
// redux.sync.f32 instructions on the same registers, so the activation is read once.
#include "quant_math.cuh"

namespace actnn {
namespace {

constexpr int kThreads = 256;
constexpr int kPair = 2;              // groups per warp task

template <typename T, typename ST, int BITS, bool FUSED>
__global__ void __launch_bounds__(kThreads)
pack_single_kernel(const T* __restrict__ data, const T* __restrict__ mn, const T* __restrict__ mx,
                   int8_t* __restrict__ packed, ST* __restrict__ scale, ST* __restrict__ mn_out,
                   ST* __restrict__ mx_out, int64_t N, int64_t G, const T* __restrict__ noise,
                   int stochastic, NoiseKey key, int64_t total_bytes) {
  constexpr int WPT = 8 / BITS;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t gpairs = (G + kPair - 1) / kPair;
  const int64_t nblocks = (N + WPT - 1) / WPT;
  const int64_t total = nblocks * gpairs;
  NoiseGen<T> gen(key, lane);
  if (warp == 0 && lane == 0) packed[total_bytes - 1] = 0;     // the reference's spare byte

  for (int64_t task = warp; task < total; task += nwarps) {
    const int64_t no = task / gpairs;
    const int64_t g0 = (task - no * gpairs) * kPair;
    const int cnt = (int)min((int64_t)kPair, G - g0);
    uint32_t acc[kPair][4];
#pragma unroll
    for (int gi = 0; gi < kPair; ++gi)
#pragma unroll
      for (int m = 0; m < 4; ++m) acc[gi][m] = 0u;

#pragma unroll
    for (int ni = 0; ni < WPT; ni += 2) {
      // two samples x two groups in flight
      Oct<T> x[2][kPair];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int64_t n = no * WPT + ni + s;
#pragma unroll
        for (int gi = 0; gi < kPair; ++gi)
          x[s][gi] = (s < WPT && n < N && gi < cnt)
                         ? load_oct<T>(data + (n * G + g0 + gi) * kGroup + lane * kOct) : zero_oct<T>();
      }
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (ni + s >= WPT) continue;
        const int64_t n = no * WPT + ni + s;
        if (n >= N) continue;                                   // warp-uniform
        const int64_t q0 = n * G + g0;
        // group statistics: lanes 0..1 own one group each
        float gmn = 0.f, gmx = 0.f;
        if constexpr (FUSED) {
          float a[kPair], b[kPair];
#pragma unroll
          for (int gi = 0; gi < kPair; ++gi) {
            float lo, hi;
            oct_minmax<T>(x[s][gi], lo, hi);
            a[gi] = warp_min(lo);
            b[gi] = warp_max(hi);
          }
          gmn = lane == 0 ? a[0] : a[1];
          gmx = lane == 0 ? b[0] : b[1];
        } else if (lane < cnt) {
          gmn = load_scalar<T>(mn, q0 + lane);
          gmx = load_scalar<T>(mx, q0 + lane);
        }
        GroupParams mine = {0.f, 0.f};
        if (lane < cnt) {
          mine = prepare_group<T>(gmn, gmx, BITS);
          store_scalar<ST>(scale, q0 + lane, mine.scale);
          if (mn_out) store_scalar<ST>(mn_out, q0 + lane, gmn);
          if (FUSED && mx_out) store_scalar<ST>(mx_out, q0 + lane, gmx);
        }
#pragma unroll
        for (int gi = 0; gi < kPair; ++gi) {
          GroupParams p;
          p.mn1 = __shfl_sync(kFull, mine.mn1, gi);
          p.scale = __shfl_sync(kFull, mine.scale, gi);
          if (gi < cnt) {
            Oct<T> nz;
            if (!stochastic) nz = zero_oct<T>();
            else if (noise) nz = load_oct<T>(noise + (q0 + gi) * kGroup + lane * kOct);
            else nz = gen.get((uint64_t)(q0 + gi));
            uint32_t cp[4];
            quantize_oct<T>(x[s][gi], nz, p, BITS, cp);
#pragma unroll
            for (int m = 0; m < 4; ++m) acc[gi][m] |= cp[m] << ((ni + s) * BITS);
          }
        }
      }
    }
    // acc[gi][m] holds byte 2m in its low half and byte 2m+1 in its high half
#pragma unroll
    for (int gi = 0; gi < kPair; ++gi) {
      if (gi < cnt) {
        uint2 w;
        w.x = __byte_perm(acc[gi][0], acc[gi][1], 0x6420);
        w.y = __byte_perm(acc[gi][2], acc[gi][3], 0x6420);
        *reinterpret_cast<uint2*>(packed + ((no * G + g0 + gi) * kGroup + lane * kOct)) = w;
      }
    }
  }
}

template <typename T, typename ST, int BITS>
__global__ void __launch_bounds__(kThreads)
unpack_single_kernel(const int8_t* __restrict__ packed, const ST* __restrict__ scale,
                     const ST* __restrict__ mn, T* __restrict__ out, int64_t N, int64_t G) {
  constexpr int WPT = 8 / BITS;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t nblocks = (N + WPT - 1) / WPT;
  const int64_t total = nblocks * G;

  for (int64_t task = warp; task < total; task += nwarps) {
    const int64_t no = task / G;
    const int64_t g = task - no * G;
    const uint2 w = __ldg(reinterpret_cast<const uint2*>(packed + ((no * G + g) * kGroup + lane * kOct)));
    // lane ni (< wpt) fetches the statistics of sample no*wpt + ni
    const int64_t my_n = no * WPT + (lane < WPT ? lane : 0);
    float my_scale = 1.f, my_mn = 0.f;
    if (lane < WPT && my_n < N) {
      my_scale = load_scalar<ST>(scale, my_n * G + g);
      my_mn = load_scalar<ST>(mn, my_n * G + g);
    }
#pragma unroll
    for (int ni = 0; ni < WPT; ++ni) {
      const int64_t n = no * WPT + ni;
      const float sc = __shfl_sync(kFull, my_scale, ni);
      const float m = __shfl_sync(kFull, my_mn, ni);
      uint32_t v[8];
      if constexpr (BITS <= 4) {
        const uint32_t entry = dequant_bits<T>((float)lane, sc, m);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t byte = ((j < 4 ? w.x : w.y) >> (8 * (j & 3))) & 0xffu;
          v[j] = __shfl_sync(kFull, entry, (int)((byte >> (ni * BITS)) & ((1u << BITS) - 1u)));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t byte = ((j < 4 ? w.x : w.y) >> (8 * (j & 3))) & 0xffu;
          v[j] = dequant_bits<T>((float)byte, sc, m);
        }
      }
      if (n < N) {
        Oct<T> o;
        if constexpr (sizeof(T) == 4) {
#pragma unroll
          for (int j = 0; j < 8; ++j) reinterpret_cast<uint32_t*>(&o)[j] = v[j];
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) reinterpret_cast<uint32_t*>(&o)[k] = v[2 * k] | (v[2 * k + 1] << 16);
        }
        store_oct<T>(out + (n * G + g) * kGroup + lane * kOct, o);
      }
    }
  }
}

int grid_for(int64_t warp_tasks) {
  const int64_t blocks = (warp_tasks + (kThreads / 32) - 1) / (kThreads / 32);
  const int64_t cap = (int64_t)device_info().sm_count * 8;
  return (int)max((int64_t)1, min(blocks, cap));
}

int64_t single_total_bytes(int bits, int64_t N, int64_t G) {
  const int wpt = 8 / bits;
  const int64_t n_round = (N + wpt - 1) / wpt * wpt;
  return (int64_t)bits * n_round * G * kGroup / 8 + 1;
}

template <typename T, typename ST, bool FUSED>
int launch_pack(int bits, const void* data, const void* mn, const void* mx, int8_t* packed, void* scale,
                void* mn_out, void* mx_out, int64_t N, int64_t G, int stochastic, const void* noise,
                uint64_t seed, uint64_t offset, cudaStream_t s) {
  const int wpt = 8 / bits;
  const int64_t tasks = ((N + wpt - 1) / wpt) * ((G + kPair - 1) / kPair);
  const int grid = grid_for(tasks);
  const NoiseKey key = make_noise_key(seed, offset);
  const int64_t tb = single_total_bytes(bits, N, G);
#define ACTNN_LAUNCH(BITS)                                                                        \
  pack_single_kernel<T, ST, BITS, FUSED><<<grid, kThreads, 0, s>>>(                               \
      (const T*)data, (const T*)mn, (const T*)mx, packed, (ST*)scale, (ST*)mn_out, (ST*)mx_out, N, G, \
      (const T*)noise, stochastic, key, tb)
  switch (bits) {
    case 1: ACTNN_LAUNCH(1); break;
    case 2: ACTNN_LAUNCH(2); break;
    case 4: ACTNN_LAUNCH(4); break;
    default: ACTNN_LAUNCH(8); break;
  }
#undef ACTNN_LAUNCH
  return check_launch();
}

template <typename T, typename ST>
int launch_unpack(int bits, const int8_t* packed, const void* scale, const void* mn, void* out, int64_t N,
                  int64_t G, cudaStream_t s) {
  const int wpt = 8 / bits;
  const int grid = grid_for(((N + wpt - 1) / wpt) * G);
#define ACTNN_LAUNCH(BITS)                                                                        \
  unpack_single_kernel<T, ST, BITS><<<grid, kThreads, 0, s>>>(packed, (const ST*)scale, (const ST*)mn, \
                                                              (T*)out, N, G)
  switch (bits) {
    case 1: ACTNN_LAUNCH(1); break;
    case 2: ACTNN_LAUNCH(2); break;
    case 4: ACTNN_LAUNCH(4); break;
    default: ACTNN_LAUNCH(8); break;
  }
#undef ACTNN_LAUNCH
  return check_launch();
}

int check_common(int bits, int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype) {
  if (!(bits == 1 || bits == 2 || bits == 4 || bits == 8)) return ACTNN_ERR_BITS;
  if (N < 0 || G < 0 || group_size != kGroup) return ACTNN_ERR_SHAPE;
  if (dtype < ACTNN_F32 || dtype > ACTNN_BF16) return ACTNN_ERR_DTYPE;
  if (!(stat_dtype == dtype || (dtype == ACTNN_F32 && stat_dtype == ACTNN_BF16))) return ACTNN_ERR_DTYPE;
  if (N > (int64_t)1 << 40 || G > (int64_t)1 << 40 || (G && N > ((int64_t)1 << 52) / G)) return ACTNN_ERR_SHAPE;
  return ACTNN_OK;
}

template <bool FUSED>
int pack_entry(const void* data, const void* mn, const void* mx, int bits, int8_t* packed, void* scale,
               void* mn_out, void* mx_out, int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype,
               int stochastic, const void* noise, uint64_t seed, uint64_t offset, actnn_stream_t stream) {
  if (int st = check_common(bits, N, G, group_size, dtype, stat_dtype)) return st;
  if (!packed) return ACTNN_ERR_NULL;
  cudaStream_t s = (cudaStream_t)stream;
  if (N == 0 || G == 0) {     // only the spare byte exists
    return cudaMemsetAsync(packed, 0, 1, s) == cudaSuccess ? ACTNN_OK : ACTNN_ERR_LAUNCH;
  }
  if (!data || !scale || (!FUSED && (!mn || !mx)) || (FUSED && !mn_out)) return ACTNN_ERR_NULL;
  const size_t al = dtype == ACTNN_F32 ? 32 : 16;
  if (!aligned(data, al) || (noise && !aligned(noise, al)) || !aligned(packed, 8)) return ACTNN_ERR_ALIGN;
  switch (dtype) {
    case ACTNN_F16:
      return launch_pack<__half, __half, FUSED>(bits, data, mn, mx, packed, scale, mn_out, mx_out, N, G,
                                                stochastic, noise, seed, offset, s);
    case ACTNN_BF16:
      return launch_pack<__nv_bfloat16, __nv_bfloat16, FUSED>(bits, data, mn, mx, packed, scale, mn_out, mx_out,
                                                              N, G, stochastic, noise, seed, offset, s);
    default:
      if (stat_dtype == ACTNN_BF16)
        return launch_pack<float, __nv_bfloat16, FUSED>(bits, data, mn, mx, packed, scale, mn_out, mx_out, N, G,
                                                        stochastic, noise, seed, offset, s);
      return launch_pack<float, float, FUSED>(bits, data, mn, mx, packed, scale, mn_out, mx_out, N, G,
                                              stochastic, noise, seed, offset, s);
  }
}

}  // namespace
}  // namespace actnn

using namespace actnn;

extern "C" int actnn_pack_single(const void* data, const void* mn, const void* mx, int bits, int8_t* packed,
                                 void* scale, void* mn_out, int64_t N, int64_t G, int64_t group_size, int dtype,
                                 int stat_dtype, int stochastic, const void* noise, uint64_t seed,
                                 uint64_t offset, actnn_stream_t stream) {
  return pack_entry<false>(data, mn, mx, bits, packed, scale, mn_out, nullptr, N, G, group_size, dtype,
                           stat_dtype, stochastic, noise, seed, offset, stream);
}

extern "C" int actnn_compress_single(const void* data, int bits, int8_t* packed, void* scale, void* mn_out,
                                     void* mx_out, int64_t N, int64_t G, int64_t group_size, int dtype,
                                     int stat_dtype, int stochastic, const void* noise, uint64_t seed,
                                     uint64_t offset, actnn_stream_t stream) {
  return pack_entry<true>(data, nullptr, nullptr, bits, packed, scale, mn_out, mx_out, N, G, group_size, dtype,
                          stat_dtype, stochastic, noise, seed, offset, stream);
}

extern "C" int actnn_unpack_single(const int8_t* packed, int bits, const void* scale, const void* mn, void* out,
                                   int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype,
                                   actnn_stream_t stream) {
  if (int st = check_common(bits, N, G, group_size, dtype, stat_dtype)) return st;
  if (N == 0 || G == 0) return ACTNN_OK;
  if (!packed || !scale || !mn || !out) return ACTNN_ERR_NULL;
  if (!aligned(out, dtype == ACTNN_F32 ? 32 : 16) || !aligned(packed, 8)) return ACTNN_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case ACTNN_F16: return launch_unpack<__half, __half>(bits, packed, scale, mn, out, N, G, s);
    case ACTNN_BF16: return launch_unpack<__nv_bfloat16, __nv_bfloat16>(bits, packed, scale, mn, out, N, G, s);
    default:
      if (stat_dtype == ACTNN_BF16) return launch_unpack<float, __nv_bfloat16>(bits, packed, scale, mn, out, N, G, s);
      return launch_unpack<float, float>(bits, packed, scale, mn, out, N, G, s);
  }
}
