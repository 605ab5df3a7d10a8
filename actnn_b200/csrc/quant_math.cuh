// Quantize / dequantize arithmetic of the activation codec, per element type.
//
// The contract is the reference's "simulate" branch (actnn/actnn/ops.py:23-41, 56-57):
//     B      = 2^bits - 1
//     mn'    = mn - 1e-6          mx' = mx + 1e-6
//     scale  = B / (mx' - mn')
//     t      = (x - mn') * scale + noise
//     code   = int(round_half_even(min(relu(t), B)))
//     x_hat  = code / scale + mn                      (unshifted minimum)
// where PyTorch rounds every intermediate to the tensor dtype.  For float16 / bfloat16 a
// correctly rounded native operation equals "compute in float32, round to the type"
// (float32 carries more than 2p+2 bits), so the 16-bit paths run packed half2 / bfloat162
// instructions with explicit round-to-nearest forms that the compiler may not contract
// into fused multiply-adds.  Rounding to an integer is done by adding a power of two whose
// unit in the last place is 1 (1024 in float16, 1.5 * 2^23 in float32): the hardware's
// round-to-nearest-even then IS round_half_even and the code appears in the low mantissa
// bits without a float->int conversion.
#pragma once

#include "common.cuh"

namespace actnn {

// ------------------------------------------------------------------ scalar <-> type
template <typename T> ACTNN_DEV float round_to(float x);
template <> ACTNN_DEV float round_to<float>(float x) { return x; }
template <> ACTNN_DEV float round_to<__half>(float x) { return __half2float(__float2half_rn(x)); }
template <> ACTNN_DEV float round_to<__nv_bfloat16>(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

template <typename T> ACTNN_DEV float load_scalar(const T* p, int64_t i);
template <> ACTNN_DEV float load_scalar<float>(const float* p, int64_t i) { return __ldg(p + i); }
template <> ACTNN_DEV float load_scalar<__half>(const __half* p, int64_t i) {
  return __half2float(__ldg(p + i));
}
template <> ACTNN_DEV float load_scalar<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  return __bfloat162float(__ldg(p + i));
}
template <typename T> ACTNN_DEV void store_scalar(T* p, int64_t i, float v);
template <> ACTNN_DEV void store_scalar<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> ACTNN_DEV void store_scalar<__half>(__half* p, int64_t i, float v) {
  p[i] = __float2half_rn(v);
}
template <> ACTNN_DEV void store_scalar<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) {
  p[i] = __float2bfloat16_rn(v);
}

// Raw bits of a T-valued float (exact conversion), low 16 bits for the 16-bit types.
template <typename T> ACTNN_DEV uint32_t bits_of(float v);
template <> ACTNN_DEV uint32_t bits_of<float>(float v) { return __float_as_uint(v); }
template <> ACTNN_DEV uint32_t bits_of<__half>(float v) {
  return (uint32_t)__half_as_ushort(__float2half_rn(v));
}
template <> ACTNN_DEV uint32_t bits_of<__nv_bfloat16>(float v) { return __float_as_uint(v) >> 16; }

// ------------------------------------------------------------------ group parameters
struct GroupParams {
  float mn1;     // shifted minimum, a value of T
  float scale;   // a value of T
};

template <typename T> ACTNN_DEV GroupParams prepare_group(float mn, float mx, int bits) {
  const float B = round_to<T>((float)((1 << bits) - 1));
  GroupParams p;
  p.mn1 = round_to<T>(__fsub_rn(mn, 1e-6f));
  const float mx1 = round_to<T>(__fadd_rn(mx, 1e-6f));
  const float range = round_to<T>(__fsub_rn(mx1, p.mn1));
  p.scale = round_to<T>(__fdiv_rn(B, range));
  return p;
}

// One lane prepares a group and ships (mn', scale) to the others: a single 32-bit shuffle
// for 16-bit types (both values packed), two for float32.  QP<T> is the form the quantizer
// consumes (values already duplicated into both halves for the packed types).
template <typename T> struct QP { float mn1, scale; };
template <> struct QP<__half> { __half2 mn2, sc2; };
template <> struct QP<__nv_bfloat16> { __nv_bfloat162 mn2, sc2; };

struct ParamWords { uint32_t w0, w1; };
template <typename T> ACTNN_DEV ParamWords pack_params(const GroupParams& p) {
  ParamWords w;
  if constexpr (sizeof(T) == 4) {
    w.w0 = __float_as_uint(p.mn1);
    w.w1 = __float_as_uint(p.scale);
  } else {
    w.w0 = bits_of<T>(p.mn1) | (bits_of<T>(p.scale) << 16);
    w.w1 = 0u;
  }
  return w;
}
template <typename T> ACTNN_DEV QP<T> fetch_params(const ParamWords& mine, int src_lane) {
  QP<T> q;
  if constexpr (sizeof(T) == 4) {
    q.mn1 = __uint_as_float(__shfl_sync(kFull, mine.w0, src_lane));
    q.scale = __uint_as_float(__shfl_sync(kFull, mine.w1, src_lane));
  } else {
    const uint32_t u = __shfl_sync(kFull, mine.w0, src_lane);
    const uint32_t a = __byte_perm(u, u, 0x1010), b = __byte_perm(u, u, 0x3232);
    q.mn2 = *reinterpret_cast<const decltype(q.mn2)*>(&a);
    q.sc2 = *reinterpret_cast<const decltype(q.sc2)*>(&b);
  }
  return q;
}

// ------------------------------------------------------------------ octet min / max
template <typename T> ACTNN_DEV void oct_minmax(const Oct<T>& o, float& mn, float& mx);
template <> ACTNN_DEV void oct_minmax<float>(const Oct<float>& o, float& mn, float& mx) {
  mn = fminf(fminf(fminf(o.f[0], o.f[1]), fminf(o.f[2], o.f[3])),
             fminf(fminf(o.f[4], o.f[5]), fminf(o.f[6], o.f[7])));
  mx = fmaxf(fmaxf(fmaxf(o.f[0], o.f[1]), fmaxf(o.f[2], o.f[3])),
             fmaxf(fmaxf(o.f[4], o.f[5]), fmaxf(o.f[6], o.f[7])));
}
template <> ACTNN_DEV void oct_minmax<__half>(const Oct<__half>& o, float& mn, float& mx) {
  const __half2* h = reinterpret_cast<const __half2*>(o.r);
  const __half2 lo = __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]));
  const __half2 hi = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
  mn = fminf(__low2float(lo), __high2float(lo));
  mx = fmaxf(__low2float(hi), __high2float(hi));
}
template <> ACTNN_DEV void oct_minmax<__nv_bfloat16>(const Oct<__nv_bfloat16>& o, float& mn, float& mx) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(o.r);
  const __nv_bfloat162 lo = __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]));
  const __nv_bfloat162 hi = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
  mn = fminf(__low2float(lo), __high2float(lo));
  mx = fmaxf(__low2float(hi), __high2float(hi));
}

// ------------------------------------------------------------------ noise octets
// Philox fields -> eight noise values in the register format of Oct<T>.
//   16-bit types: `w0`, `w1` hold the eight bytes k0..k7 of this group's half of a call.
//   float32:      `v` holds the four words of the group's call (eight 16-bit fields).
// Both 16-bit formats count linearly through their subnormals and first normal binade: the
// bit pattern v < 2^11 (float16) or v < 2^8 (bfloat16) IS the value v * 2^-24 resp.
// v * 2^-133.  A random field masked in place is therefore already a number proportional to
// it, and one exact fused multiply-add turns it into the centred noise: one logic
// instruction and one HFMA2 per two elements.
ACTNN_DEV Oct<__half> noise_from_bytes_f16(uint32_t w0, uint32_t w1) {
  // bits (2k + 1) = (2k + 1) * 2^-24; times 2^15, minus 0.5 = (2k + 1 - 256) / 512.
  // Elements 0, 1 take k from bits 1..8 and 17..24 of the word, elements 2, 3 from the same
  // bits of the word rotated right by 8; every bit of the word is used exactly once.
  const uint32_t s_bits = 0x78007800u, c_bits = 0xB800B800u;                     // 2^15, -0.5
  const __half2 s = *reinterpret_cast<const __half2*>(&s_bits);
  const __half2 c = *reinterpret_cast<const __half2*>(&c_bits);
  Oct<__half> o;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const uint32_t w = (m < 2) ? w0 : w1;
    const uint32_t r = (m & 1) ? __funnelshift_r(w, w, 8) : w;
    const uint32_t bits = (r & 0x01FE01FEu) | 0x00010001u;
    const __half2 h = __hfma2(*reinterpret_cast<const __half2*>(&bits), s, c);
    o.r[m] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return o;
}
ACTNN_DEV float noise_float(uint32_t k, float step, float bias) {
  // float bits 0x4B000000 + (2k + 1) = 2^23 + 2k + 1; one exact fused multiply-add
  return __fmaf_rn(__uint_as_float(0x4B000000u + 2u * k + 1u), step, bias);
}
ACTNN_DEV Oct<__nv_bfloat16> noise_from_bytes_bf16(uint32_t w0, uint32_t w1) {
  // bits k = k * 2^-133; times 2^125, minus 255/512 = (2k + 1 - 256) / 512.
  // Elements 0, 1 take bytes 0 and 2 of the word, elements 2, 3 bytes 1 and 3.
  const uint32_t s_bits = 0x7E007E00u, c_bits = 0xBEFFBEFFu;                     // 2^125, -255/512
  const __nv_bfloat162 s = *reinterpret_cast<const __nv_bfloat162*>(&s_bits);
  const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&c_bits);
  Oct<__nv_bfloat16> o;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const uint32_t w = (m < 2) ? w0 : w1;
    const uint32_t bits = (m & 1) ? __byte_perm(w, 0u, 0x4341) : (w & 0x00FF00FFu);
    const __nv_bfloat162 h = __hfma2(*reinterpret_cast<const __nv_bfloat162*>(&bits), s, c);
    o.r[m] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return o;
}
ACTNN_DEV Oct<float> noise_from_fields_f32(const Philox4& v) {
  Oct<float> o;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t k = (v.v[j >> 1] >> (16 * (j & 1))) & 0xffffu;
    // (2^23 + 2k + 1) / 2^17 - 64.5 = (2k + 1 - 65536) / 131072
    o.f[j] = noise_float(k, 1.0f / 131072.0f, -64.5f);
  }
  return o;
}

// One Philox call yields four words; four more are derived as v[i] + M * v[i+1] (mod 2^32,
// M odd: one integer multiply-add each).  Any two of the eight words are jointly uniform:
// (x, y) -> (x, x + M*y) and (x, y, z) -> (x + M*y, y + M*z) are onto with uniform fibres,
// hence any two noise fields are independent and uniform and second-order statistics of the
// rounding noise equal those of independent noise at half the generator cost.  A call thus
// serves one lane for four neighbouring groups (16-bit activations, one byte per element) or
// two groups (float32, 16 bits per element).
struct NoiseWords { uint32_t e[8]; };
constexpr uint32_t kNoiseMul = 0x9E3779B1u;
ACTNN_DEV NoiseWords expand_call(const Philox4& p) {
  NoiseWords w;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    w.e[i] = p.v[i];
    w.e[4 + i] = p.v[(i + 1) & 3] * kNoiseMul + p.v[i];
  }
  return w;
}
template <typename T> struct NoiseShape { static constexpr int GPC = sizeof(T) == 2 ? 4 : 2; };   // groups per call

template <typename T> ACTNN_DEV Oct<T> noise_oct(const NoiseWords& w, int slot);
template <> ACTNN_DEV Oct<float> noise_oct<float>(const NoiseWords& w, int slot) {
  Philox4 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) v.v[i] = slot ? w.e[4 + i] : w.e[i];
  return noise_from_fields_f32(v);
}
ACTNN_DEV void pick_pair(const NoiseWords& w, int slot, uint32_t& a, uint32_t& b) {
  a = slot == 0 ? w.e[0] : slot == 1 ? w.e[2] : slot == 2 ? w.e[4] : w.e[6];
  b = slot == 0 ? w.e[1] : slot == 1 ? w.e[3] : slot == 2 ? w.e[5] : w.e[7];
}
template <> ACTNN_DEV Oct<__half> noise_oct<__half>(const NoiseWords& w, int slot) {
  uint32_t a, b;
  pick_pair(w, slot, a, b);
  return noise_from_bytes_f16(a, b);
}
template <> ACTNN_DEV Oct<__nv_bfloat16> noise_oct<__nv_bfloat16>(const NoiseWords& w, int slot) {
  uint32_t a, b;
  pick_pair(w, slot, a, b);
  return noise_from_bytes_bf16(a, b);
}

// Noise for flat group q, this lane; keeps the last call (general path, any alignment).
template <typename T> struct NoiseGen {
  static constexpr int GPC = NoiseShape<T>::GPC;
  const NoiseKey key;                  // by value: the fields stay kernel-parameter (constant bank) reads
  uint64_t cached;
  NoiseWords w;
  int lane;
  ACTNN_DEV NoiseGen(const NoiseKey& k, int lane_) : key(k), cached(~0ull), lane(lane_) {}
  ACTNN_DEV Oct<T> get(uint64_t q) {
    const uint64_t call = q / GPC;
    if (call != cached) {
      w = expand_call(noise_call(key, call * 32ull + (uint64_t)lane));
      cached = call;
    }
    return noise_oct<T>(w, (int)(q % GPC));
  }
};

// The GPC octets of the aligned block of groups starting at q (q % GPC == 0), one call.
template <typename T>
ACTNN_DEV void noise_block(const NoiseKey& key, uint64_t q, int lane, Oct<T> (&out)[NoiseShape<T>::GPC]) {
  const NoiseWords w = expand_call(noise_call(key, (q / NoiseShape<T>::GPC) * 32ull + (uint64_t)lane));
#pragma unroll
  for (int h = 0; h < NoiseShape<T>::GPC; ++h) out[h] = noise_oct<T>(w, h);
}

// ------------------------------------------------------------------ quantize one octet
// The result stays in "magic" form: the registers still carry the exponent bits of the
// rounding constant, code in the low mantissa bits.
//   float16:                    4 registers, two elements each: halves = 0x6600 + code
//   bfloat16, up to 6 bits:     4 registers, two elements each: halves = 0x4340 + code
//   float32 / bfloat16, 7-8 b.: 8 registers, one element each:  0x4B400000 + code
// Because those high bits are the same for every element, shifted sums of magic registers
// equal shifted sums of the codes plus a compile-time constant (mod 2^32): rows and bytes
// are assembled with integer multiply-adds and one constant, without masking each code.
template <typename T> struct Magic { uint32_t v[8]; };
template <> struct Magic<__half> { uint32_t v[4]; };
template <typename T> struct MagicInfo { static constexpr uint32_t bias = 0x4B400000u; static constexpr bool paired = false; };
template <> struct MagicInfo<__half> { static constexpr uint32_t bias = 0x66006600u; static constexpr bool paired = true; };
// The form actually produced for a given width.
template <typename T, int B> struct MagicFmt {
  static constexpr bool paired = false;
  static constexpr uint32_t bias = 0x4B400000u;
  static constexpr uint32_t code_mask = 0x1ffu;
};
template <int B> struct MagicFmt<__half, B> {
  static constexpr bool paired = true;
  static constexpr uint32_t bias = 0x66006600u;
  static constexpr uint32_t code_mask = 0x01ff01ffu;
};
template <int B> struct MagicFmt<__nv_bfloat16, B> {
  // 192 + t lies in [128, 256) for t in [-0.5, 63.5], where bfloat16 has spacing 1: the packed
  // add rounds to the nearest integer, ties to even, exactly like rint; 7 and 8 bits need float32
  static constexpr bool paired = B <= 6;
  static constexpr uint32_t bias = paired ? 0x43404340u : 0x4B400000u;
  static constexpr uint32_t code_mask = paired ? 0x003f003fu : 0x1ffu;
};

// CLAMP_LOW = false may be used when min really is the group minimum: then
// (x - mn') * scale + noise >= -0.5 always and the round-to-even of the magic add maps it
// to code 0 on its own.
template <typename T, bool CLAMP_LOW, int BITS>
ACTNN_DEV Magic<T> quantize_oct(const Oct<T>& x, const Oct<T>& nz, const QP<T>& p) {
  Magic<T> m;
  if constexpr (sizeof(T) == 4) {
    constexpr float B = (float)((1 << BITS) - 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = __fmul_rn(__fsub_rn(x.f[j], p.mn1), p.scale);
      t = __fadd_rn(t, nz.f[j]);
      if (CLAMP_LOW) t = fmaxf(t, 0.f);
      t = fminf(t, B);                                      // NaN -> B
      m.v[j] = __float_as_uint(__fadd_rn(t, 12582912.f));
    }
  } else if constexpr (DType<T>::id == ACTNN_F16) {
    // (2^BITS - 1) and 1536 as half2 bit patterns; 1536 = 0x6600: every t in [-0.5, 255.5]
    // lands in [1024, 2048), where the spacing is 1
    constexpr uint32_t kB[9] = {0, 0x3C003C00u, 0x42004200u, 0x47004700u, 0x4B804B80u, 0x4FC04FC0u,
                                0x53E053E0u, 0x57F057F0u, 0x5BF85BF8u};
    const uint32_t b_bits = kB[BITS], magic_bits = 0x66006600u, zero_bits = 0u;
    const __half2 B2 = *reinterpret_cast<const __half2*>(&b_bits);
    const __half2 magic2 = *reinterpret_cast<const __half2*>(&magic_bits);
    const __half2 zero2 = *reinterpret_cast<const __half2*>(&zero_bits);
    const __half2* xv = reinterpret_cast<const __half2*>(x.r);
    const __half2* nv = reinterpret_cast<const __half2*>(nz.r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      __half2 t = __hmul2_rn(__hsub2_rn(xv[k], p.mn2), p.sc2);
      t = __hadd2_rn(t, nv[k]);
      if (CLAMP_LOW) t = __hmax2(t, zero2);
      t = __hmin2(t, B2);                                   // NaN -> B
      t = __hadd2_rn(t, magic2);
      m.v[k] = *reinterpret_cast<const uint32_t*>(&t);
    }
  } else {
    // bfloat16 patterns of 2^BITS - 1
    constexpr uint32_t kB[9] = {0, 0x3F803F80u, 0x40404040u, 0x40E040E0u, 0x41704170u, 0x41F841F8u,
                                0x427C427Cu, 0x42FE42FEu, 0x437F437Fu};
    const uint32_t b_bits = kB[BITS], zero_bits = 0u, magic_bits = 0x43404340u;   // 192
    const __nv_bfloat162 B2 = *reinterpret_cast<const __nv_bfloat162*>(&b_bits);
    const __nv_bfloat162 zero2 = *reinterpret_cast<const __nv_bfloat162*>(&zero_bits);
    const __nv_bfloat162 magic2 = *reinterpret_cast<const __nv_bfloat162*>(&magic_bits);
    const __nv_bfloat162* xv = reinterpret_cast<const __nv_bfloat162*>(x.r);
    const __nv_bfloat162* nv = reinterpret_cast<const __nv_bfloat162*>(nz.r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      __nv_bfloat162 t = __hmul2_rn(__hsub2_rn(xv[k], p.mn2), p.sc2);
      t = __hadd2_rn(t, nv[k]);
      if (CLAMP_LOW) t = __hmax2(t, zero2);
      t = __hmin2(t, B2);                                   // NaN -> B
      if constexpr (MagicFmt<T, BITS>::paired) {
        t = __hadd2_rn(t, magic2);
        m.v[k] = *reinterpret_cast<const uint32_t*>(&t);
      } else {
        const uint32_t u = *reinterpret_cast<const uint32_t*>(&t);
        // bfloat16 -> float32 is a shift; 8 mantissa bits cannot hold 255 plus a round bit, so
        // the integer rounding runs in float32 (1.5 * 2^23 also absorbs t in [-0.5, 0))
        m.v[2 * k] = __float_as_uint(__fadd_rn(__uint_as_float(u << 16), 12582912.f));
        m.v[2 * k + 1] = __float_as_uint(__fadd_rn(__uint_as_float(u & 0xffff0000u), 12582912.f));
      }
    }
  }
  return m;
}

// ------------------------------------------------------------------ dequantize
// x_hat for an integer code, as the bit pattern of T (low 16 bits for 16-bit types).
template <typename T> ACTNN_DEV uint32_t dequant_bits(float code, float scale, float mn) {
  const float q = round_to<T>(__fdiv_rn(code, scale));
  return bits_of<T>(round_to<T>(__fadd_rn(q, mn)));
}

// The same for many codes of one group whose scale is a 16-bit value (float16 / bfloat16
// statistics): the reciprocal is taken once per group and every element pays three fused
// operations instead of an IEEE division,
//     y = RN(1 / s),  q0 = RN(c y),  r = c - s q0 (exact in one FMA),  q = RN(q0 + r y),
// which is the exactly rounded quotient RN(c / s) (Markstein's correction step).  Checked on the
// CPU for every code 1..255 against every finite positive float16 scale and every bfloat16 scale
// in [2^-60, 2^60]: no difference from the IEEE division.  `group_reciprocal` says whether a scale
// is inside that range (anything else -- zero, infinity, NaN, negative, huge -- keeps the division).
ACTNN_DEV bool group_reciprocal(float scale, float& y) {
  y = __frcp_rn(scale);
  return scale >= 8.673617379884035e-19f && scale <= 1.152921504606847e18f;   // [2^-60, 2^60]
}
template <typename T> ACTNN_DEV uint32_t dequant_bits_recip(float code, float scale, float y, float mn) {
  const float q0 = __fmul_rn(code, y);
  const float r = __fmaf_rn(-scale, q0, code);
  const float q = round_to<T>(__fmaf_rn(r, y, q0));
  return bits_of<T>(round_to<T>(__fadd_rn(q, mn)));
}

// ------------------------------------------------------------------ bit strings
// A lane's slice of the packed stream is a little-endian bit string held in S[0..].
template <int OFF, int NB> ACTNN_DEV void put_bits(uint32_t* S, uint32_t v) {
  constexpr int w = OFF / 32, s = OFF % 32;
  S[w] |= v << s;
  if constexpr (s + NB > 32) S[w + 1] |= v >> (32 - s);
}
template <int OFF, int NB> ACTNN_DEV uint32_t get_bits(const uint32_t* S) {
  constexpr int w = OFF / 32, s = OFF % 32;
  uint32_t v = S[w] >> s;
  if constexpr (s + NB > 32) v |= S[w + 1] << (32 - s);
  if constexpr (NB >= 32) return v;
  else return v & ((1u << NB) - 1u);
}

// sum over k of (c << (step * k)) mod 2^32, evaluated at compile time
constexpr uint32_t shifted_sum(uint32_t c, int step, int count) {
  uint32_t acc = 0;
  for (int k = 0; k < count; ++k) acc += (step * k < 32) ? (c << (step * k)) : 0u;
  return acc;
}

// The lane's row for one octet: eight B-bit codes laid end to end, code j at bit B*j.
// lo = bits 0..31, hi = bits 32..63 (only B > 4 reaches hi).
template <typename T, int B> ACTNN_DEV void row_from_magic(const Magic<T>& m, uint32_t& lo, uint32_t& hi) {
  hi = 0u;
  if constexpr (MagicFmt<T, B>::paired) {
    constexpr uint32_t bias = MagicFmt<T, B>::bias;
    if constexpr (B <= 2) {
      // even elements accumulate in the low half, odd ones in the high half
      uint32_t acc = m.v[0] + (m.v[1] << (2 * B)) + (m.v[2] << (4 * B)) + (m.v[3] << (6 * B));
      acc -= shifted_sum(bias, 2 * B, 4);
      lo = (acc | (acc >> (16 - B))) & ((1u << (8 * B)) - 1u);
    } else if constexpr (B <= 4) {
      uint32_t a = m.v[0] + (m.v[1] << (2 * B)) - shifted_sum(bias, 2 * B, 2);
      uint32_t b = m.v[2] + (m.v[3] << (2 * B)) - shifted_sum(bias, 2 * B, 2);
      a = (a | (a >> (16 - B))) & ((1u << (4 * B)) - 1u);
      b = (b | (b >> (16 - B))) & ((1u << (4 * B)) - 1u);
      lo = a | (b << (4 * B));
    } else {
      uint32_t S[2] = {0u, 0u};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t c = m.v[k] & MagicFmt<T, B>::code_mask;
        const uint32_t pr = (c | (c >> (16 - B))) & ((1u << (2 * B)) - 1u);
        if (k == 0) put_bits<0 * B, 2 * B>(S, pr);
        if (k == 1) put_bits<2 * B, 2 * B>(S, pr);
        if (k == 2) put_bits<4 * B, 2 * B>(S, pr);
        if (k == 3) put_bits<6 * B, 2 * B>(S, pr);
      }
      lo = S[0]; hi = S[1];
    }
  } else {
    constexpr uint32_t bias = MagicFmt<T, B>::bias;
    if constexpr (B <= 4) {
      uint32_t acc = m.v[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) acc += m.v[j] << (B * j);
      lo = acc - shifted_sum(bias, B, 8);
    } else if constexpr (B == 8) {
      lo = (m.v[0] + (m.v[1] << 8) + (m.v[2] << 16) + (m.v[3] << 24)) - shifted_sum(bias, 8, 4);
      hi = (m.v[4] + (m.v[5] << 8) + (m.v[6] << 16) + (m.v[7] << 24)) - shifted_sum(bias, 8, 4);
    } else {
      uint32_t S[2] = {0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t c = m.v[j] & 0x1ffu;
        if (j == 0) put_bits<0 * B, B>(S, c);
        if (j == 1) put_bits<1 * B, B>(S, c);
        if (j == 2) put_bits<2 * B, B>(S, c);
        if (j == 3) put_bits<3 * B, B>(S, c);
        if (j == 4) put_bits<4 * B, B>(S, c);
        if (j == 5) put_bits<5 * B, B>(S, c);
        if (j == 6) put_bits<6 * B, B>(S, c);
        if (j == 7) put_bits<7 * B, B>(S, c);
      }
      lo = S[0]; hi = S[1];
    }
  }
}

// Place a row (8B bits) at bit offset OFF of the bundle string S.
template <int B, int OFF> ACTNN_DEV void put_row(uint32_t* S, uint32_t lo, uint32_t hi) {
  if constexpr (8 * B <= 32) {
    put_bits<OFF, 8 * B>(S, lo);
  } else {
    put_bits<OFF, 32>(S, lo);
    put_bits<OFF + 32, 8 * B - 32>(S, hi);
  }
}

// The eight B-bit codes stored at bit offset OFF.
template <int B, int OFF> ACTNN_DEV void get_codes(const uint32_t* S, uint32_t code[8]) {
  code[0] = get_bits<OFF + 0 * B, B>(S); code[1] = get_bits<OFF + 1 * B, B>(S);
  code[2] = get_bits<OFF + 2 * B, B>(S); code[3] = get_bits<OFF + 3 * B, B>(S);
  code[4] = get_bits<OFF + 4 * B, B>(S); code[5] = get_bits<OFF + 5 * B, B>(S);
  code[6] = get_bits<OFF + 6 * B, B>(S); code[7] = get_bits<OFF + 7 * B, B>(S);
}

}  // namespace actnn
