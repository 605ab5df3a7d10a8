// Pack / unpack for group sizes other than 256 (any multiple of 32; the reference accepts
// them, quantization_cuda_kernel.cu:94,186, and exposes `group_size` in its configuration).
//
// Correctness first: one warp per group, scalar arithmetic, codes staged in shared memory.
// The arithmetic is the same contract as the 256-element kernels (quant_math.cuh), evaluated
// per element in float32 with a rounding to the activation dtype after every operation; the
// layouts are the reference's index formulas taken literally:
//   mixed  (quantization_cuda_kernel.cu:51-79):  group (n, g) starts at word
//          (P_n * G + b_n * g) * gs / 32 (P_n = bits of the samples before n); with
//          W = gs * b_n / 32, bit i of element d goes to word (d*b + i) % W, bit (d*b + i) / W;
//   single (quantization_cuda_kernel.cu:236-257): byte (no*G + g) * gs + d holds the codes of
//          samples no*wpt + ni at bit ni * bits.
// The rounding noise of element e of the flattened [N, G, gs] activation is the one the
// 256-element kernels (and actnn_noise_fill) give to flat element e.
#include "quant_math.cuh"

namespace actnn {
namespace {

constexpr int kThreads = 128;                       // four warps, one group each
constexpr int kMaxGroup = 8192;                     // elements per group the staging buffers allow

// Noise of flat element e (see the stream definition in common.cuh).
template <typename T> ACTNN_DEV float noise_scalar(const NoiseKey& key, uint64_t e) {
  constexpr int GPC = NoiseShape<T>::GPC;
  const uint64_t q = e >> 8;
  const int d = (int)(e & 255u), t = d >> 3, j = d & 7;
  const NoiseWords w = expand_call(noise_call(key, (q / GPC) * 32ull + (uint64_t)t));
  const Oct<T> o = noise_oct<T>(w, (int)(q % GPC));
  if constexpr (sizeof(T) == 4) {
    return o.f[j];
  } else {
    const uint32_t bits = (o.r[j >> 1] >> (16 * (j & 1))) & 0xffffu;
    if constexpr (DType<T>::id == ACTNN_F16) return __half2float(__ushort_as_half((unsigned short)bits));
    else return __uint_as_float(bits << 16);
  }
}

// code = int(rint(min(relu((x - mn') * scale + noise), B))), every step rounded to T.
template <typename T> ACTNN_DEV uint32_t quantize_scalar(float x, const GroupParams& p, float noise, int bits) {
  const float B = (float)((1 << bits) - 1);
  float t = round_to<T>(__fmul_rn(round_to<T>(__fsub_rn(x, p.mn1)), p.scale));
  t = round_to<T>(__fadd_rn(t, noise));
  t = (t == t) ? fminf(fmaxf(t, 0.f), B) : B;        // NaN -> B, as the fast kernels do
  return (uint32_t)__float2int_rn(t);
}

struct NoiseArgs {
  const void* tensor;                                // injected noise (same layout as the data) or NULL
  int stochastic;
  NoiseKey key;
};
template <typename T> ACTNN_DEV float noise_of(const NoiseArgs& a, int64_t e) {
  if (!a.stochastic) return 0.f;
  if (a.tensor) return load_scalar<T>((const T*)a.tensor, e);
  return noise_scalar<T>(a.key, (uint64_t)e);
}

// ---------------------------------------------------------------------------- mixed
template <typename T, typename ST>
__global__ void __launch_bounds__(kThreads)
pack_mixed_generic_kernel(const T* __restrict__ data, const T* __restrict__ mn, const T* __restrict__ mx,
                          const int32_t* __restrict__ bits, const int64_t* __restrict__ word_offsets,
                          int32_t* __restrict__ packed, ST* __restrict__ scale, ST* __restrict__ mn_out, int64_t N,
                          int64_t G, int gs, NoiseArgs nz) {
  extern __shared__ unsigned char codes_all[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  unsigned char* codes = codes_all + (size_t)wib * gs;
  const int64_t groups = N * G;
  for (int64_t q = (int64_t)blockIdx.x * (kThreads / 32) + wib; q < groups; q += (int64_t)gridDim.x * (kThreads / 32)) {
    const int64_t n = q / G, g = q - n * G;
    const int b = __ldg(bits + n);
    if (b < 1 || b > 8) continue;                    // not a width: nothing is written (warp-uniform)
    const float gmn = load_scalar<T>(mn, q), gmx = load_scalar<T>(mx, q);
    const GroupParams gp = prepare_group<T>(gmn, gmx, b);
    if (lane == 0) {
      store_scalar<ST>(scale, q, gp.scale);
      if (mn_out) store_scalar<ST>(mn_out, q, gmn);
    }
    for (int d = lane; d < gs; d += 32) {
      const int64_t e = q * gs + d;
      codes[d] = (unsigned char)quantize_scalar<T>(load_scalar<T>(data, e), gp, noise_of<T>(nz, e), b);
    }
    __syncwarp();
    const int W = gs * b / 32;
    int32_t* out = packed + __ldg(word_offsets + n) + g * W;
    for (int w = lane; w < W; w += 32) {
      uint32_t word = 0u;
      for (int p = 0; p < 32; ++p) {
        const int idx = p * W + w, d = idx / b, i = idx - d * b;
        word |= ((uint32_t)(codes[d] >> i) & 1u) << p;
      }
      out[w] = (int32_t)word;
    }
    __syncwarp();
  }
}

template <typename T, typename ST>
__global__ void __launch_bounds__(kThreads)
unpack_mixed_generic_kernel(const int32_t* __restrict__ packed, const int32_t* __restrict__ bits,
                            const int64_t* __restrict__ word_offsets, const ST* __restrict__ scale,
                            const ST* __restrict__ mn, T* __restrict__ out, int64_t N, int64_t G, int gs) {
  extern __shared__ unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  uint32_t* words = reinterpret_cast<uint32_t*>(smem_raw) + (size_t)wib * (gs / 4);      // W <= gs * 8 / 32
  const int64_t groups = N * G;
  for (int64_t q = (int64_t)blockIdx.x * (kThreads / 32) + wib; q < groups; q += (int64_t)gridDim.x * (kThreads / 32)) {
    const int64_t n = q / G, g = q - n * G;
    const int b = __ldg(bits + n);
    if (b < 1 || b > 8) continue;
    const int W = gs * b / 32;
    const int32_t* in = packed + __ldg(word_offsets + n) + g * W;
    for (int w = lane; w < W; w += 32) words[w] = (uint32_t)__ldg(in + w);
    __syncwarp();
    const float sc = load_scalar<ST>(scale, q), m = load_scalar<ST>(mn, q);
    for (int d = lane; d < gs; d += 32) {
      uint32_t code = 0u;
      for (int i = 0; i < b; ++i) {
        const int idx = d * b + i, w = idx % W, p = idx / W;
        code |= ((words[w] >> p) & 1u) << i;
      }
      const uint32_t v = dequant_bits<T>((float)code, sc, m);
      if constexpr (sizeof(T) == 4) out[q * gs + d] = __uint_as_float(v);
      else reinterpret_cast<unsigned short*>(out)[q * gs + d] = (unsigned short)v;
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------- single
// One warp per (sample block, group).  FUSED: the min / max come from the data itself.
template <typename T, typename ST, bool FUSED>
__global__ void __launch_bounds__(kThreads)
pack_single_generic_kernel(const T* __restrict__ data, const T* __restrict__ mn, const T* __restrict__ mx,
                           int8_t* __restrict__ packed, ST* __restrict__ scale, ST* __restrict__ mn_out,
                           ST* __restrict__ mx_out, int64_t N, int64_t G, int gs, int bits, int64_t total_bytes,
                           NoiseArgs nz) {
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int wpt = 8 / bits;
  const int64_t nblocks = (N + wpt - 1) / wpt, tasks = nblocks * G;
  if (blockIdx.x == 0 && threadIdx.x == 0) packed[total_bytes - 1] = 0;       // the reference's spare byte
  for (int64_t task = (int64_t)blockIdx.x * (kThreads / 32) + wib; task < tasks;
       task += (int64_t)gridDim.x * (kThreads / 32)) {
    const int64_t no = task / G, g = task - no * G;
    GroupParams gp[8];
    for (int ni = 0; ni < wpt; ++ni) {
      const int64_t n = no * wpt + ni;
      gp[ni].mn1 = 0.f; gp[ni].scale = 0.f;
      if (n >= N) continue;
      const int64_t q = n * G + g;
      float lo, hi;
      if (FUSED) {
        lo = INFINITY; hi = -INFINITY;
        for (int d = lane; d < gs; d += 32) {
          const float v = load_scalar<T>(data, q * gs + d);
          lo = fminf(lo, v); hi = fmaxf(hi, v);
        }
        lo = warp_min(lo); hi = warp_max(hi);
      } else {
        lo = load_scalar<T>(mn, q); hi = load_scalar<T>(mx, q);
      }
      gp[ni] = prepare_group<T>(lo, hi, bits);
      if (lane == 0) {
        store_scalar<ST>(scale, q, gp[ni].scale);
        if (mn_out) store_scalar<ST>(mn_out, q, lo);
        if (FUSED && mx_out) store_scalar<ST>(mx_out, q, hi);
      }
    }
    for (int d = lane; d < gs; d += 32) {
      uint32_t byte = 0u;
      for (int ni = 0; ni < wpt; ++ni) {
        const int64_t n = no * wpt + ni;
        if (n >= N) continue;
        const int64_t e = (n * G + g) * gs + d;
        byte |= quantize_scalar<T>(load_scalar<T>(data, e), gp[ni], noise_of<T>(nz, e), bits) << (ni * bits);
      }
      packed[(no * G + g) * gs + d] = (int8_t)byte;
    }
  }
}

template <typename T, typename ST>
__global__ void __launch_bounds__(kThreads)
unpack_single_generic_kernel(const int8_t* __restrict__ packed, const ST* __restrict__ scale,
                             const ST* __restrict__ mn, T* __restrict__ out, int64_t N, int64_t G, int gs, int bits) {
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int wpt = 8 / bits;
  const int64_t nblocks = (N + wpt - 1) / wpt, tasks = nblocks * G;
  for (int64_t task = (int64_t)blockIdx.x * (kThreads / 32) + wib; task < tasks;
       task += (int64_t)gridDim.x * (kThreads / 32)) {
    const int64_t no = task / G, g = task - no * G;
    for (int ni = 0; ni < wpt; ++ni) {
      const int64_t n = no * wpt + ni;
      if (n >= N) continue;
      const int64_t q = n * G + g;
      const float sc = load_scalar<ST>(scale, q), m = load_scalar<ST>(mn, q);
      for (int d = lane; d < gs; d += 32) {
        const uint32_t byte = (uint32_t)(unsigned char)__ldg(packed + (no * G + g) * gs + d);
        const uint32_t code = (byte >> (ni * bits)) & ((1u << bits) - 1u);
        const uint32_t v = dequant_bits<T>((float)code, sc, m);
        if constexpr (sizeof(T) == 4) out[q * gs + d] = __uint_as_float(v);
        else reinterpret_cast<unsigned short*>(out)[q * gs + d] = (unsigned short)v;
      }
    }
  }
}

int grid_for(int64_t warp_tasks) {
  const int64_t blocks = (warp_tasks + kThreads / 32 - 1) / (kThreads / 32);
  return (int)max((int64_t)1, min(blocks, (int64_t)device_info().sm_count * 16));
}

}  // namespace

// Dispatch over (dtype, stat dtype): F(T, ST) is a statement.
#define ACTNN_GENERIC_TYPES(dtype, stat_dtype, F)                       \
  switch (dtype) {                                                      \
    case ACTNN_F16: { F(__half, __half) } break;                        \
    case ACTNN_BF16: { F(__nv_bfloat16, __nv_bfloat16) } break;         \
    default:                                                            \
      if (stat_dtype == ACTNN_BF16) { F(float, __nv_bfloat16) }         \
      else { F(float, float) }                                          \
  }

bool generic_group_ok(int64_t gs) { return gs > 0 && gs % 32 == 0 && gs <= kMaxGroup; }

int pack_mixed_generic(const void* data, const void* mn, const void* mx, const int32_t* bits,
                       const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out, int64_t N, int64_t G,
                       int64_t gs, int dtype, int stat_dtype, int stochastic, const void* noise, uint64_t seed,
                       uint64_t offset, cudaStream_t s) {
  const NoiseArgs nz{noise, stochastic, make_noise_key(seed, offset)};
  const int smem = (kThreads / 32) * (int)gs;
#define F(T, ST)                                                                                              \
  pack_mixed_generic_kernel<T, ST><<<grid_for(N * G), kThreads, smem, s>>>(                                   \
      (const T*)data, (const T*)mn, (const T*)mx, bits, word_offsets, packed, (ST*)scale, (ST*)mn_out, N, G, (int)gs, nz);
  ACTNN_GENERIC_TYPES(dtype, stat_dtype, F)
#undef F
  return check_launch();
}

int unpack_mixed_generic(const int32_t* packed, const int32_t* bits, const int64_t* word_offsets, const void* scale,
                         const void* mn, void* out, int64_t N, int64_t G, int64_t gs, int dtype, int stat_dtype,
                         cudaStream_t s) {
  const int smem = (kThreads / 32) * (int)gs;                    // gs / 4 words per warp
#define F(T, ST)                                                                                              \
  unpack_mixed_generic_kernel<T, ST><<<grid_for(N * G), kThreads, smem, s>>>(                                 \
      packed, bits, word_offsets, (const ST*)scale, (const ST*)mn, (T*)out, N, G, (int)gs);
  ACTNN_GENERIC_TYPES(dtype, stat_dtype, F)
#undef F
  return check_launch();
}

int pack_single_generic(bool fused, const void* data, const void* mn, const void* mx, int bits, int8_t* packed,
                        void* scale, void* mn_out, void* mx_out, int64_t N, int64_t G, int64_t gs, int dtype,
                        int stat_dtype, int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                        cudaStream_t s) {
  const NoiseArgs nz{noise, stochastic, make_noise_key(seed, offset)};
  const int wpt = 8 / bits;
  const int64_t n_round = (N + wpt - 1) / wpt * wpt;
  const int64_t total_bytes = (int64_t)bits * n_round * G * gs / 8 + 1;
  const int64_t tasks = (n_round / wpt) * G;
#define F(T, ST)                                                                                              \
  if (fused)                                                                                                  \
    pack_single_generic_kernel<T, ST, true><<<grid_for(tasks), kThreads, 0, s>>>(                             \
        (const T*)data, (const T*)mn, (const T*)mx, packed, (ST*)scale, (ST*)mn_out, (ST*)mx_out, N, G, (int)gs, \
        bits, total_bytes, nz);                                                                               \
  else                                                                                                        \
    pack_single_generic_kernel<T, ST, false><<<grid_for(tasks), kThreads, 0, s>>>(                            \
        (const T*)data, (const T*)mn, (const T*)mx, packed, (ST*)scale, (ST*)mn_out, (ST*)mx_out, N, G, (int)gs, \
        bits, total_bytes, nz);
  ACTNN_GENERIC_TYPES(dtype, stat_dtype, F)
#undef F
  return check_launch();
}

int unpack_single_generic(const int8_t* packed, int bits, const void* scale, const void* mn, void* out, int64_t N,
                          int64_t G, int64_t gs, int dtype, int stat_dtype, cudaStream_t s) {
  const int wpt = 8 / bits;
  const int64_t tasks = ((N + wpt - 1) / wpt) * G;
#define F(T, ST)                                                                                              \
  unpack_single_generic_kernel<T, ST><<<grid_for(tasks), kThreads, 0, s>>>(                                   \
      packed, (const ST*)scale, (const ST*)mn, (T*)out, N, G, (int)gs, bits);
  ACTNN_GENERIC_TYPES(dtype, stat_dtype, F)
#undef F
  return check_launch();
}

}  // namespace actnn
