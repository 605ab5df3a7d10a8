// ReLU and dropout that keep one bit per element for the backward pass.
//
// Mask layout: bit (e % 8) of byte (e / 8), i.e. the natural little-endian bit order,
// padded with zero bits to whole int32 words.  (The reference keeps its own order private
// to its two kernels, quantization_cuda_kernel.cu:437 / :480, so the order is free.)
//
// A warp handles 1024 consecutive elements per step as four rows of 256: lane t loads the
// octet 8t..8t+7 of every row (four independent 16/32-byte loads), forms one keep-byte per
// row, and four shuffles regroup the 128 keep-bytes so that lane w holds mask word w of
// the block: one coalesced 128-byte mask store per 1024 elements.
#include "quant_math.cuh"

namespace actnn {
namespace {

constexpr int kThreads = 256;
constexpr int kRows = 4;
constexpr int kBlockElems = kRows * kGroup;       // 1024 elements per warp step

// keep-bits of an octet (bit j = element j is > 0)
template <typename T> ACTNN_DEV uint32_t positive_bits(const Oct<T>& o);
template <> ACTNN_DEV uint32_t positive_bits<float>(const Oct<float>& o) {
  uint32_t b = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) b |= (o.f[j] > 0.f ? 1u : 0u) << j;
  return b;
}
template <> ACTNN_DEV uint32_t positive_bits<__half>(const Oct<__half>& o) {
  const __half2 z = __float2half2_rn(0.f);
  uint32_t b = 0;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const uint32_t g = __hgt2_mask(*reinterpret_cast<const __half2*>(&o.r[m]), z) & 0x00010001u;
    b |= ((g | (g >> 15)) & 3u) << (2 * m);
  }
  return b;
}
template <> ACTNN_DEV uint32_t positive_bits<__nv_bfloat16>(const Oct<__nv_bfloat16>& o) {
  const __nv_bfloat162 z = __float2bfloat162_rn(0.f);
  uint32_t b = 0;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const uint32_t g = __hgt2_mask(*reinterpret_cast<const __nv_bfloat162*>(&o.r[m]), z) & 0x00010001u;
    b |= ((g | (g >> 15)) & 3u) << (2 * m);
  }
  return b;
}

// zero the elements whose keep-bit is clear
template <typename T> ACTNN_DEV Oct<T> select_kept(const Oct<T>& o, uint32_t keep) {
  Oct<T> r;
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int j = 0; j < 8; ++j) r.f[j] = (keep >> j) & 1u ? o.f[j] : 0.f;
  } else {
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const uint32_t k = keep >> (2 * m);
      const uint32_t msk = ((k & 1u) * 0x0000ffffu) | (((k >> 1) & 1u) * 0xffff0000u);
      r.r[m] = o.r[m] & msk;
    }
  }
  return r;
}

// multiply an octet by a float factor, rounding once to T
template <typename T> ACTNN_DEV Oct<T> scale_oct(const Oct<T>& o, float f) {
  Oct<T> r;
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int j = 0; j < 8; ++j) r.f[j] = __fmul_rn(o.f[j], f);
  } else {
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      float lo, hi;
      if constexpr (DType<T>::id == ACTNN_F16) {
        const __half2 h = *reinterpret_cast<const __half2*>(&o.r[m]);
        const __half2 q = __floats2half2_rn(__fmul_rn(__low2float(h), f), __fmul_rn(__high2float(h), f));
        r.r[m] = *reinterpret_cast<const uint32_t*>(&q);
      } else {
        lo = __uint_as_float(o.r[m] << 16);
        hi = __uint_as_float(o.r[m] & 0xffff0000u);
        const __nv_bfloat162 q = __floats2bfloat162_rn(__fmul_rn(lo, f), __fmul_rn(hi, f));
        r.r[m] = *reinterpret_cast<const uint32_t*>(&q);
      }
    }
  }
  return r;
}

// scalar tail helpers (at most 7 elements of the whole tensor go through these)
template <typename T> ACTNN_DEV Oct<T> load_partial(const T* p, int valid) {
  Oct<T> o = zero_oct<T>();
  T* e = reinterpret_cast<T*>(&o);
  for (int j = 0; j < valid; ++j) e[j] = p[j];
  return o;
}
template <typename T> ACTNN_DEV void store_partial(T* p, const Oct<T>& o, int valid) {
  const T* e = reinterpret_cast<const T*>(&o);
  for (int j = 0; j < valid; ++j) p[j] = e[j];
}

// lane t holds keep-bytes b0..b3 (row i in byte i) -> lane w gets mask word w of the block
ACTNN_DEV uint32_t bytes_to_words(uint32_t mine, int lane) {
  const int i = lane >> 3, src = (lane & 7) * 4;
  const uint32_t v0 = __shfl_sync(kFull, mine, src + 0), v1 = __shfl_sync(kFull, mine, src + 1);
  const uint32_t v2 = __shfl_sync(kFull, mine, src + 2), v3 = __shfl_sync(kFull, mine, src + 3);
  const uint32_t sel = (uint32_t)i | ((uint32_t)(4 + i) << 4);
  return __byte_perm(__byte_perm(v0, v1, sel), __byte_perm(v2, v3, sel), 0x5410);
}
// inverse: lane w holds mask word w -> lane t gets keep-bytes b0..b3 of its four octets
ACTNN_DEV uint32_t words_to_bytes(uint32_t word, int lane) {
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    const uint32_t v = __shfl_sync(kFull, word, 8 * i + (lane >> 2));
    out |= ((v >> (8 * (lane & 3))) & 0xffu) << (8 * i);
  }
  return out;
}

enum class Op { kReluFwd, kMaskBwd, kDropoutFwd };

// One kernel body for the three element-wise passes.
//   kReluFwd:    y = x > 0 ? x : 0,           mask <- (x > 0)
//   kDropoutFwd: y = keep ? x * inv : 0,      mask <- keep = (u > p)
//   kMaskBwd:    grad_in = mask ? grad_out * inv : 0      (inv = 1 for ReLU)
// One block of 1024 elements of a warp.  FULL: the block lies wholly inside the tensor, so
// there is no per-row edge handling and the four loads (and stores) sit in one basic block.
template <typename T, Op OP, bool FULL>
ACTNN_DEV void mask_block(const T* __restrict__ in, T* __restrict__ out, int32_t* __restrict__ mask,
                          int64_t numel, int64_t mask_words, int64_t blk, int lane, float inv, float p,
                          const float* __restrict__ u, const NoiseKey& key, T* __restrict__ group_mn = nullptr,
                          T* __restrict__ group_mx = nullptr) {
  const int64_t e0 = blk * kBlockElems + lane * kOct;
  Oct<T> x[kRows];
  int valid[kRows];
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    const int64_t e = e0 + (int64_t)i * kGroup;
    if constexpr (FULL) {
      valid[i] = kOct;
      x[i] = load_oct<T>(in + e);
    } else {
      valid[i] = (int)max((int64_t)0, min((int64_t)kOct, numel - e));
      if (valid[i] == kOct) x[i] = load_oct<T>(in + e);
      else if (valid[i] > 0) x[i] = load_partial<T>(in + e, valid[i]);
      else x[i] = zero_oct<T>();
    }
  }
  uint32_t keep = 0;                                 // byte i = keep-bits of row i
  if constexpr (OP == Op::kMaskBwd) {
    const int64_t w = blk * (kBlockElems / 32) + lane;
    keep = words_to_bytes((FULL || w < mask_words) ? (uint32_t)__ldg(mask + w) : 0u, lane);
  } else if constexpr (OP == Op::kReluFwd) {
#pragma unroll
    for (int i = 0; i < kRows; ++i) keep |= positive_bits<T>(x[i]) << (8 * i);
  } else {
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      const int64_t oct = (e0 + (int64_t)i * kGroup) >> 3;
      uint32_t kb = 0;
      if (u) {
#pragma unroll
        for (int j = 0; j < 8; ++j) kb |= (j < valid[i] && __ldg(u + oct * 8 + j) > p ? 1u : 0u) << j;
      } else {
        const Philox4 r = noise_call(key, (uint64_t)oct);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t k = (r.v[j >> 1] >> (16 * (j & 1))) & 0xffffu;
          kb |= ((float)(k + 1u) * (1.0f / 65536.0f) > p ? 1u : 0u) << j;
        }
      }
      keep |= kb << (8 * i);
    }
  }
  float my_mn = 0.f, my_mx = 0.f;                     // lane i: extrema of output row i (ReLU with group_mn only)
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    if (!FULL && valid[i] == 0) continue;
    Oct<T> y = select_kept<T>(x[i], (keep >> (8 * i)) & 0xffu);
    if constexpr (OP != Op::kReluFwd) { if (inv != 1.f) y = scale_oct<T>(y, inv); }
    const int64_t e = e0 + (int64_t)i * kGroup;
    if (FULL || valid[i] == kOct) store_oct<T>(out + e, y);
    else store_partial<T>(out + e, y, valid[i]);
    if constexpr (OP == Op::kReluFwd) {
      // the caller asked for the min / max of every 256 outputs (numel % 256 == 0, so a row is whole
      // or absent for the entire warp): the same reduction as the minimax kernel, on y
      if (group_mn) {
        float lo, hi;
        oct_minmax<T>(y, lo, hi);
        lo = warp_min(lo);
        hi = warp_max(hi);
        if (lane == i) { my_mn = lo; my_mx = hi; }
      }
    }
  }
  if constexpr (OP == Op::kReluFwd) {
    if (group_mn && lane < kRows) {
      const int64_t g = blk * kRows + lane;
      if (g * kGroup < numel) {
        store_scalar<T>(group_mn, g, my_mn);
        store_scalar<T>(group_mx, g, my_mx);
      }
    }
  }
  if constexpr (OP != Op::kMaskBwd) {
    // bits past numel are already zero: rows / elements beyond the end contribute 0
    uint32_t clipped = keep;
    if constexpr (!FULL) {
      clipped = 0;
#pragma unroll
      for (int i = 0; i < kRows; ++i)
        clipped |= (((keep >> (8 * i)) & 0xffu) & ((1u << valid[i]) - 1u)) << (8 * i);
    }
    const uint32_t word = bytes_to_words(clipped, lane);
    const int64_t w = blk * (kBlockElems / 32) + lane;
    if (FULL || w < mask_words) mask[w] = (int32_t)word;
  }
}

template <typename T, Op OP>
__global__ void __launch_bounds__(kThreads)
mask_kernel(const T* __restrict__ in, T* __restrict__ out, int32_t* __restrict__ mask, int64_t numel,
            float inv, float p, const float* __restrict__ u, const NoiseKey key, T* __restrict__ group_mn,
            T* __restrict__ group_mx) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t blocks = (numel + kBlockElems - 1) / kBlockElems;
  const int64_t whole = numel / kBlockElems;            // blocks that lie wholly inside the tensor
  const int64_t mask_words = (numel + 31) / 32;
  for (int64_t blk = warp; blk < blocks; blk += nwarps) {
    if (blk < whole) mask_block<T, OP, true>(in, out, mask, numel, mask_words, blk, lane, inv, p, u, key, group_mn, group_mx);
    else mask_block<T, OP, false>(in, out, mask, numel, mask_words, blk, lane, inv, p, u, key, group_mn, group_mx);
  }
}

__global__ void dropout_uniform_kernel(float* __restrict__ u, int64_t numel, const NoiseKey key) {
  const int64_t oct = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (oct * 8 >= numel) return;
  const Philox4 r = noise_call(key, (uint64_t)oct);
  for (int j = 0; j < 8 && oct * 8 + j < numel; ++j) {
    const uint32_t k = (r.v[j >> 1] >> (16 * (j & 1))) & 0xffffu;
    u[oct * 8 + j] = (float)(k + 1u) * (1.0f / 65536.0f);
  }
}

template <Op OP>
int launch(const void* in, void* out, int32_t* mask, int64_t numel, float inv, float p, const float* u,
           uint64_t seed, uint64_t offset, int dtype, actnn_stream_t stream, void* group_mn = nullptr,
           void* group_mx = nullptr) {
  if (numel < 0) return ACTNN_ERR_SHAPE;
  if (numel == 0) return ACTNN_OK;
  if (!in || !out || !mask) return ACTNN_ERR_NULL;
  const size_t al = dtype == ACTNN_F32 ? 32 : 16;
  if (!aligned(in, al) || !aligned(out, al) || !aligned(mask, 4)) return ACTNN_ERR_ALIGN;
  const int64_t blocks = (numel + kBlockElems - 1) / kBlockElems;
  const int grid = (int)max((int64_t)1, min((blocks + 7) / 8, (int64_t)device_info().sm_count * 8));
  cudaStream_t s = (cudaStream_t)stream;
  const NoiseKey key = make_noise_key(seed, offset);
  switch (dtype) {
    case ACTNN_F32:
      mask_kernel<float, OP><<<grid, kThreads, 0, s>>>((const float*)in, (float*)out, mask, numel, inv, p, u, key,
                                                       (float*)group_mn, (float*)group_mx);
      break;
    case ACTNN_F16:
      mask_kernel<__half, OP><<<grid, kThreads, 0, s>>>((const __half*)in, (__half*)out, mask, numel, inv, p, u, key,
                                                        (__half*)group_mn, (__half*)group_mx);
      break;
    case ACTNN_BF16:
      mask_kernel<__nv_bfloat16, OP><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, mask,
                                                               numel, inv, p, u, key, (__nv_bfloat16*)group_mn,
                                                               (__nv_bfloat16*)group_mx);
      break;
    default: return ACTNN_ERR_DTYPE;
  }
  return check_launch();
}

}  // namespace
}  // namespace actnn

using namespace actnn;

extern "C" int actnn_relu_forward(const void* x, void* y, int32_t* mask, int64_t numel, int dtype,
                                  actnn_stream_t stream) {
  return launch<Op::kReluFwd>(x, y, mask, numel, 1.f, 0.f, nullptr, 0, 0, dtype, stream);
}

extern "C" int actnn_relu_forward_minimax(const void* x, void* y, int32_t* mask, void* mn, void* mx, int64_t numel,
                                          int dtype, actnn_stream_t stream) {
  if (numel < 0 || numel % kGroup != 0) return ACTNN_ERR_SHAPE;
  if (numel > 0 && (!mn || !mx)) return ACTNN_ERR_NULL;
  return launch<Op::kReluFwd>(x, y, mask, numel, 1.f, 0.f, nullptr, 0, 0, dtype, stream, mn, mx);
}

extern "C" int actnn_relu_backward(const void* grad_out, const int32_t* mask, void* grad_in, int64_t numel,
                                   int dtype, actnn_stream_t stream) {
  return launch<Op::kMaskBwd>(grad_out, grad_in, const_cast<int32_t*>(mask), numel, 1.f, 0.f, nullptr, 0, 0,
                              dtype, stream);
}

extern "C" int actnn_dropout_forward(const void* x, void* y, int32_t* mask, int64_t numel, float p, int dtype,
                                     const float* u, uint64_t seed, uint64_t offset, actnn_stream_t stream) {
  if (!(p >= 0.f && p < 1.f)) return ACTNN_ERR_ARG;
  const float inv = (float)(1.0 / (1.0 - (double)p));
  return launch<Op::kDropoutFwd>(x, y, mask, numel, inv, p, u, seed, offset, dtype, stream);
}

extern "C" int actnn_dropout_backward(const void* grad_out, const int32_t* mask, void* grad_in, int64_t numel,
                                      float p, int dtype, actnn_stream_t stream) {
  if (!(p >= 0.f && p < 1.f)) return ACTNN_ERR_ARG;
  const float inv = (float)(1.0 / (1.0 - (double)p));
  return launch<Op::kMaskBwd>(grad_out, grad_in, const_cast<int32_t*>(mask), numel, inv, p, nullptr, 0, 0, dtype,
                              stream);
}

extern "C" int actnn_dropout_uniform_fill(float* u, int64_t numel, uint64_t seed, uint64_t offset,
                                          actnn_stream_t stream) {
  if (numel < 0) return ACTNN_ERR_SHAPE;
  if (numel == 0) return ACTNN_OK;
  if (!u) return ACTNN_ERR_NULL;
  const int64_t octs = (numel + 7) / 8;
  dropout_uniform_kernel<<<(unsigned)((octs + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      u, numel, make_noise_key(seed, offset));
  return check_launch();
}
