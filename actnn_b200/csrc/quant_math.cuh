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
ACTNN_DEV Oct<__half> noise_from_bytes_f16(uint32_t w0, uint32_t w1) {
  // half bits 0x6001 | (k << 1) = 512 + k + 0.5; times 2^-8, minus 2.5 = (2k + 1 - 256) / 512
  const __half2 s = __halves2half2(__ushort_as_half(0x1C00), __ushort_as_half(0x1C00));   // 2^-8
  const __half2 c = __halves2half2(__ushort_as_half(0xC100), __ushort_as_half(0xC100));   // -2.5
  Oct<__half> o;
  const uint32_t sp[4] = {__byte_perm(w0, 0u, 0x4140), __byte_perm(w0, 0u, 0x4342),
                          __byte_perm(w1, 0u, 0x4140), __byte_perm(w1, 0u, 0x4342)};
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const uint32_t bits = sp[m] * 2u + 0x60016001u;
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
  Oct<__nv_bfloat16> o;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const uint32_t w = (m < 2) ? w0 : w1;
    const uint32_t ka = (w >> (16 * (m & 1))) & 0xffu, kb = (w >> (16 * (m & 1) + 8)) & 0xffu;
    // (2^23 + 2k + 1) / 512 - 16384.5 = (2k + 1 - 256) / 512
    const __nv_bfloat162 h = __floats2bfloat162_rn(noise_float(ka, 1.0f / 512.0f, -16384.5f),
                                                   noise_float(kb, 1.0f / 512.0f, -16384.5f));
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

// Noise for flat group q, this lane.  Keeps the last Philox call so that the two groups of
// a pair (16-bit types) cost one call.
template <typename T> struct NoiseGen {
  NoiseKey key;
  uint64_t cached;
  Philox4 ph;
  int lane;
  ACTNN_DEV NoiseGen(const NoiseKey& k, int lane_) : key(k), cached(~0ull), lane(lane_) {}
  ACTNN_DEV Oct<T> get(uint64_t q);
};
template <> ACTNN_DEV Oct<float> NoiseGen<float>::get(uint64_t q) {
  return noise_from_fields_f32(noise_call(key, q * 32ull + (uint64_t)lane));
}
template <> ACTNN_DEV Oct<__half> NoiseGen<__half>::get(uint64_t q) {
  const uint64_t pair = q >> 1;
  if (pair != cached) { ph = noise_call(key, pair * 32ull + (uint64_t)lane); cached = pair; }
  return (q & 1) ? noise_from_bytes_f16(ph.v[2], ph.v[3]) : noise_from_bytes_f16(ph.v[0], ph.v[1]);
}
template <> ACTNN_DEV Oct<__nv_bfloat16> NoiseGen<__nv_bfloat16>::get(uint64_t q) {
  const uint64_t pair = q >> 1;
  if (pair != cached) { ph = noise_call(key, pair * 32ull + (uint64_t)lane); cached = pair; }
  return (q & 1) ? noise_from_bytes_bf16(ph.v[2], ph.v[3]) : noise_from_bytes_bf16(ph.v[0], ph.v[1]);
}

// ------------------------------------------------------------------ quantize one octet
// Result: four registers, each holding two codes in the low bits of its 16-bit halves
// (element 2m in the low half, 2m+1 in the high half).
template <typename T>
ACTNN_DEV void quantize_oct(const Oct<T>& x, const Oct<T>& nz, const GroupParams& p, int bits,
                            uint32_t cp[4]);

template <>
ACTNN_DEV void quantize_oct<float>(const Oct<float>& x, const Oct<float>& nz, const GroupParams& p,
                                   int bits, uint32_t cp[4]) {
  const float B = (float)((1 << bits) - 1);
  uint32_t c[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float t = __fmul_rn(__fsub_rn(x.f[j], p.mn1), p.scale);
    t = __fadd_rn(t, nz.f[j]);
    t = fminf(fmaxf(t, 0.f), B);                            // NaN -> 0
    c[j] = __float_as_uint(__fadd_rn(t, 12582912.f)) & 0x1ffu;
  }
#pragma unroll
  for (int m = 0; m < 4; ++m) cp[m] = c[2 * m] | (c[2 * m + 1] << 16);
}

template <>
ACTNN_DEV void quantize_oct<__half>(const Oct<__half>& x, const Oct<__half>& nz, const GroupParams& p,
                                    int bits, uint32_t cp[4]) {
  const __half2 mn2 = __float2half2_rn(p.mn1), sc2 = __float2half2_rn(p.scale);
  const __half2 B2 = __float2half2_rn((float)((1 << bits) - 1));
  const __half2 zero2 = __float2half2_rn(0.f), magic2 = __float2half2_rn(1024.f);
  const __half2* xv = reinterpret_cast<const __half2*>(x.r);
  const __half2* nv = reinterpret_cast<const __half2*>(nz.r);
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    __half2 t = __hmul2_rn(__hsub2_rn(xv[m], mn2), sc2);
    t = __hadd2_rn(t, nv[m]);
    t = __hmin2(__hmax2(t, zero2), B2);                     // NaN -> 0
    t = __hadd2_rn(t, magic2);
    cp[m] = *reinterpret_cast<const uint32_t*>(&t) & 0x03ff03ffu;
  }
}

template <>
ACTNN_DEV void quantize_oct<__nv_bfloat16>(const Oct<__nv_bfloat16>& x, const Oct<__nv_bfloat16>& nz,
                                           const GroupParams& p, int bits, uint32_t cp[4]) {
  const __nv_bfloat162 mn2 = __float2bfloat162_rn(p.mn1), sc2 = __float2bfloat162_rn(p.scale);
  const __nv_bfloat162 B2 = __float2bfloat162_rn((float)((1 << bits) - 1));
  const __nv_bfloat162 zero2 = __float2bfloat162_rn(0.f);
  const __nv_bfloat162* xv = reinterpret_cast<const __nv_bfloat162*>(x.r);
  const __nv_bfloat162* nv = reinterpret_cast<const __nv_bfloat162*>(nz.r);
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    __nv_bfloat162 t = __hmul2_rn(__hsub2_rn(xv[m], mn2), sc2);
    t = __hadd2_rn(t, nv[m]);
    t = __hmin2(__hmax2(t, zero2), B2);                     // NaN -> 0
    const uint32_t u = *reinterpret_cast<const uint32_t*>(&t);
    // bfloat16 -> float32 is a shift; 8 mantissa bits cannot hold 255 + a round bit, so the
    // integer rounding runs in float32
    const uint32_t lo = __float_as_uint(__fadd_rn(__uint_as_float(u << 16), 12582912.f)) & 0x1ffu;
    const uint32_t hi = __float_as_uint(__fadd_rn(__uint_as_float(u & 0xffff0000u), 12582912.f)) & 0x1ffu;
    cp[m] = lo | (hi << 16);
  }
}

// ------------------------------------------------------------------ dequantize
// x_hat for an integer code, as the bit pattern of T (low 16 bits for 16-bit types).
template <typename T> ACTNN_DEV uint32_t dequant_bits(float code, float scale, float mn) {
  const float q = round_to<T>(__fdiv_rn(code, scale));
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
  return v & ((1u << NB) - 1u);
}

// Append the eight B-bit codes of one octet at bit offset OFF: code j at OFF + j*B.
template <int B, int OFF> ACTNN_DEV void put_codes(uint32_t* S, const uint32_t cp[4]) {
  const uint32_t p0 = (cp[0] | (cp[0] >> (16 - B))) & ((1u << (2 * B)) - 1u);
  const uint32_t p1 = (cp[1] | (cp[1] >> (16 - B))) & ((1u << (2 * B)) - 1u);
  const uint32_t p2 = (cp[2] | (cp[2] >> (16 - B))) & ((1u << (2 * B)) - 1u);
  const uint32_t p3 = (cp[3] | (cp[3] >> (16 - B))) & ((1u << (2 * B)) - 1u);
  put_bits<OFF + 0 * B, 2 * B>(S, p0);
  put_bits<OFF + 2 * B, 2 * B>(S, p1);
  put_bits<OFF + 4 * B, 2 * B>(S, p2);
  put_bits<OFF + 6 * B, 2 * B>(S, p3);
}

// The eight B-bit codes stored at bit offset OFF.
template <int B, int OFF> ACTNN_DEV void get_codes(const uint32_t* S, uint32_t code[8]) {
  code[0] = get_bits<OFF + 0 * B, B>(S); code[1] = get_bits<OFF + 1 * B, B>(S);
  code[2] = get_bits<OFF + 2 * B, B>(S); code[3] = get_bits<OFF + 3 * B, B>(S);
  code[4] = get_bits<OFF + 4 * B, B>(S); code[5] = get_bits<OFF + 5 * B, B>(S);
  code[6] = get_bits<OFF + 6 * B, B>(S); code[7] = get_bits<OFF + 7 * B, B>(S);
}

}  // namespace actnn
