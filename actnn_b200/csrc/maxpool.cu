// 2-D max pooling (NCHW) that keeps only the window-local arg-max, one int8 per output.
//
// Forward scans each window row-major and takes a strictly larger value, so the first
// maximum wins, and stores kh*KW + kw (reference: quantization_cuda_kernel.cu:644-668;
// window taps here honour dilation, which the reference's loops leave out).
// Backward is a gather: every input position visits the few windows that contain it and
// adds the gradients of those that selected it, in float32 and in a fixed order.  That
// removes the reference's zero-fill and its atomicAdd scatter
// (quantization_cuda_kernel.cu:712-733) and makes the result deterministic.
#include <type_traits>

#include "quant_math.cuh"

namespace actnn {
namespace {

struct PoolGeom {
  int H, W, Ho, Wo, KH, KW, SH, SW, PH, PW, DH, DW;
};

// n / d for n < 2^31 with one multiply-high: the backward row kernel splits a flat segment index
// into (plane, row, segment) with two of these instead of two 32-bit divisions.
struct PoolDiv { uint32_t m, s; };
PoolDiv make_pool_div(uint32_t d) {
  PoolDiv f{0, 0};
  if (d <= 1) return f;
  uint32_t s = 0;
  while (((uint64_t)1 << s) < d) ++s;
  f.m = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << s) - d)) / d + 1);
  f.s = s;
  return f;
}
ACTNN_DEV uint32_t pool_div(uint32_t n, const PoolDiv& f) { return (__umulhi(n, f.m) + n) >> f.s; }

// Blocks are persistent: x covers a plane's positions (at most a few blocks), y strides over
// the planes, and the whole grid is about 16 blocks per SM, so that the cost of launching
// blocks does not dominate planes of a few thousand positions.
dim3 plane_grid(int elems_per_plane, int64_t planes) {
  const int bx = max(1, min(8, (elems_per_plane + 255) / 256));
  const int64_t by = max((int64_t)1, min(planes, (int64_t)device_info().sm_count * 16 / bx));
  return dim3((unsigned)bx, (unsigned)by);
}

template <typename T>
__global__ void __launch_bounds__(256)
max_pool_forward_kernel(const T* __restrict__ x, T* __restrict__ y, int8_t* __restrict__ idx, int planes,
                        PoolGeom g) {
  // blockIdx.y strides over the (n, c) planes; 32-bit index arithmetic inside a plane
  const int plane_elems = g.H * g.W, out_elems = g.Ho * g.Wo;
  for (int nc = blockIdx.y; nc < planes; nc += gridDim.y) {
    const T* plane = x + (int64_t)nc * plane_elems;
    T* y_p = y + (int64_t)nc * out_elems;
    int8_t* idx_p = idx + (int64_t)nc * out_elems;
    for (int o = blockIdx.x * blockDim.x + threadIdx.x; o < out_elems; o += gridDim.x * blockDim.x) {
      const int ho = o / g.Wo, wo = o - ho * g.Wo;
      const int hb = ho * g.SH - g.PH, wb = wo * g.SW - g.PW;
      float best = -INFINITY;
      int arg = 0;
      for (int kh = 0; kh < g.KH; ++kh) {
        const int h = hb + kh * g.DH;
        if (h < 0 || h >= g.H) continue;
        for (int kw = 0; kw < g.KW; ++kw) {
          const int w = wb + kw * g.DW;
          if (w < 0 || w >= g.W) continue;
          const float v = load_scalar<T>(plane, h * g.W + w);
          if (v > best) { best = v; arg = kh * g.KW + kw; }
        }
      }
      store_scalar<T>(y_p, o, best);
      idx_p[o] = (int8_t)arg;
    }
  }
}

// Forward for K x K windows with K known at compile time and unit dilation: the K*K taps
// are loaded unconditionally (coordinates clamped into the plane, validity kept aside) so
// that all loads of a window are in flight together; the scan order and the strict
// comparison are those of the general kernel.
template <typename T, int K>
__global__ void __launch_bounds__(256)
max_pool_forward_fixed_kernel(const T* __restrict__ x, T* __restrict__ y, int8_t* __restrict__ idx, int planes,
                              PoolGeom g) {
  const int plane_elems = g.H * g.W, out_elems = g.Ho * g.Wo;
  for (int nc = blockIdx.y; nc < planes; nc += gridDim.y) {
    const T* plane = x + (int64_t)nc * plane_elems;
    T* y_p = y + (int64_t)nc * out_elems;
    int8_t* idx_p = idx + (int64_t)nc * out_elems;
    for (int o = blockIdx.x * blockDim.x + threadIdx.x; o < out_elems; o += gridDim.x * blockDim.x) {
      const int ho = o / g.Wo, wo = o - ho * g.Wo;
      const int hb = ho * g.SH - g.PH, wb = wo * g.SW - g.PW;
      float v[K * K];
      bool ok[K * K];
#pragma unroll
      for (int kh = 0; kh < K; ++kh) {
        const int h = hb + kh;
        const bool hok = h >= 0 && h < g.H;
        const int hc = min(max(h, 0), g.H - 1);
#pragma unroll
        for (int kw = 0; kw < K; ++kw) {
          const int w = wb + kw;
          ok[kh * K + kw] = hok && w >= 0 && w < g.W;
          v[kh * K + kw] = load_scalar<T>(plane, hc * g.W + min(max(w, 0), g.W - 1));
        }
      }
      float best = -INFINITY;
      int arg = 0;
#pragma unroll
      for (int t = 0; t < K * K; ++t)
        if (ok[t] && v[t] > best) { best = v[t]; arg = t; }
      store_scalar<T>(y_p, o, best);
      idx_p[o] = (int8_t)arg;
    }
  }
}

template <typename T> ACTNN_DEV void oct_values(const Oct<T>& o, float (&f)[8]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = o.f[j];
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if constexpr (std::is_same<T, __half>::value) {
        f[2 * k] = __half2float(__ushort_as_half((unsigned short)(o.r[k] & 0xffffu)));
        f[2 * k + 1] = __half2float(__ushort_as_half((unsigned short)(o.r[k] >> 16)));
      } else {
        f[2 * k] = __uint_as_float(o.r[k] << 16);
        f[2 * k + 1] = __uint_as_float(o.r[k] & 0xffff0000u);
      }
    }
  }
}

// Forward by output-row segments: K x K windows (K = 2 or 3), column stride 2, unit dilation,
// column padding P = 0 or 1, rows of W % 8 == 0 elements in a vector-aligned tensor (the pooling
// layers of the ResNets, VGGs and DenseNets).  A thread owns eight consecutive outputs of one
// output row.  Their windows cover the 16 input columns 2 wo0 .. 2 wo0 + 15 plus at most one
// column on either side, so a window row costs two vector loads and at most two scalar ones
// instead of 8 K scalar loads.  A tap outside the plane counts as -inf: with the strict
// comparison and the -inf start that is the same as skipping it.  Scan order, comparison and
// codes are those of the general kernel.
template <typename T, int K, int P>
__global__ void __launch_bounds__(256)
max_pool_forward_row_kernel(const T* __restrict__ x, T* __restrict__ y, int8_t* __restrict__ idx,
                            uint32_t total_segments, int segs_per_row, PoolGeom g, int vector_store) {
  const int out_elems = g.Ho * g.Wo, plane_elems = g.H * g.W;
  for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < total_segments; t += gridDim.x * blockDim.x) {
    const uint32_t row = t / (uint32_t)segs_per_row;
    const int seg = (int)(t - row * (uint32_t)segs_per_row);
    const uint32_t nc = row / (uint32_t)g.Ho;
    const int ho = (int)(row - nc * (uint32_t)g.Ho);
    const int wo0 = seg * 8, c0 = 2 * wo0;
    const T* plane = x + (int64_t)nc * plane_elems;
    const int hb = ho * g.SH - g.PH;
    float best[8];
    int arg[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { best[i] = -INFINITY; arg[i] = 0; }
    // the loads of all K window rows are issued before the first comparison (rows outside the
    // plane read a clamped row and are masked afterwards), so K times as many bytes are in flight
    Oct<T> lo8[K], hi8[K];
    float left[K], right[K];
    const bool whole = c0 + 16 <= g.W;
#pragma unroll
    for (int kh = 0; kh < K; ++kh) {
      const int h = min(max(hb + kh, 0), g.H - 1);
      const T* r = plane + h * g.W;
      if (whole) {
        lo8[kh] = load_oct<T>(r + c0);
        hi8[kh] = load_oct<T>(r + c0 + 8);
      }
      left[kh] = (P == 1 && c0 >= 1) ? load_scalar<T>(r, c0 - 1) : -INFINITY;
      right[kh] = (K - P == 3 && c0 + 16 < g.W) ? load_scalar<T>(r, c0 + 16) : -INFINITY;
    }
#pragma unroll
    for (int kh = 0; kh < K; ++kh) {
      const int h = hb + kh;
      if (h < 0 || h >= g.H) continue;
      float v[18];                                               // v[j]: column c0 - 1 + j
      if (whole) {
        float f[8];
        oct_values<T>(lo8[kh], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[1 + j] = f[j];
        oct_values<T>(hi8[kh], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[9 + j] = f[j];
      } else {                                                   // the last segment of a row that is not a multiple of 16
        const T* r = plane + h * g.W;
#pragma unroll
        for (int j = 0; j < 16; ++j) v[1 + j] = c0 + j < g.W ? load_scalar<T>(r, c0 + j) : -INFINITY;
      }
      v[0] = left[kh];
      v[17] = right[kh];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int kw = 0; kw < K; ++kw) {
          const float val = v[2 * i - P + kw + 1];
          if (val > best[i]) { best[i] = val; arg[i] = kh * K + kw; }
        }
      }
    }
    const int64_t o = (int64_t)nc * out_elems + ho * g.Wo + wo0;
    if (vector_store) {                                          // Wo % 8 == 0, aligned outputs
      Oct<T> out;
      if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out.f[i] = best[i];
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          out.r[k] = bits_of<T>(best[2 * k]) | (bits_of<T>(best[2 * k + 1]) << 16);   // values of T: exact
        }
      }
      store_oct<T>(y + o, out);
      uint2 codes;
      codes.x = (uint32_t)arg[0] | ((uint32_t)arg[1] << 8) | ((uint32_t)arg[2] << 16) | ((uint32_t)arg[3] << 24);
      codes.y = (uint32_t)arg[4] | ((uint32_t)arg[5] << 8) | ((uint32_t)arg[6] << 16) | ((uint32_t)arg[7] << 24);
      *reinterpret_cast<uint2*>(idx + o) = codes;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (wo0 + i < g.Wo) {
          store_scalar<T>(y, o + i, best[i]);
          idx[o + i] = (int8_t)arg[i];
        }
      }
    }
  }
}

template <typename T>
int launch_forward(const void* x, void* y, int8_t* idx, int64_t planes, const PoolGeom& g, cudaStream_t s) {
  const int out_elems = g.Ho * g.Wo;
  const bool unit = g.DH == 1 && g.DW == 1 && g.KH == g.KW;
  const int segs = (g.Wo + 7) / 8;
  const int64_t total_segments = planes * g.Ho * segs;
  if (unit && (g.KH == 2 || g.KH == 3) && g.SW == 2 && g.PW <= 1 && g.W % 8 == 0 && aligned(x, sizeof(T) * 8) &&
      total_segments < ((int64_t)1 << 31)) {
    const int vec = g.Wo % 8 == 0 && aligned(y, sizeof(T) * 8) && aligned(idx, 8);
    const int64_t blocks = (total_segments + 255) / 256;
    const int rgrid = (int)max((int64_t)1, min(blocks, (int64_t)device_info().sm_count * 16));
#define ACTNN_ROW(K, P)                                                                                       \
    max_pool_forward_row_kernel<T, K, P><<<rgrid, 256, 0, s>>>((const T*)x, (T*)y, idx, (uint32_t)total_segments, \
                                                               segs, g, vec)
    if (g.KH == 3 && g.PW == 1) ACTNN_ROW(3, 1);
    else if (g.KH == 3) ACTNN_ROW(3, 0);
    else if (g.PW == 1) ACTNN_ROW(2, 1);
    else ACTNN_ROW(2, 0);
#undef ACTNN_ROW
    return check_launch();
  }
  dim3 grid = plane_grid(out_elems, planes);
  if (unit && g.KH == 3)
    max_pool_forward_fixed_kernel<T, 3><<<grid, 256, 0, s>>>((const T*)x, (T*)y, idx, (int)planes, g);
  else if (unit && g.KH == 2)
    max_pool_forward_fixed_kernel<T, 2><<<grid, 256, 0, s>>>((const T*)x, (T*)y, idx, (int)planes, g);
  else
    max_pool_forward_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (T*)y, idx, (int)planes, g);
  return check_launch();
}

// Backward.  One block row per (n, c) plane (blockIdx.y strides over planes), threads over
// the plane's positions, all index arithmetic in 32 bits.  STRIDE / UNIT_DILATION are
// compile-time for the common geometries (stride 1 or 2, dilation 1) so that the divisions
// become shifts; STRIDE == 0 is the general case.  Only the output rows / columns whose
// window can contain the position are visited:
//   ho in [ceil((h + PH - (KH-1)*DH) / SH), floor((h + PH) / SH)].
template <typename T, int STRIDE, bool UNIT_DILATION>
__global__ void __launch_bounds__(256)
max_pool_backward_kernel(const T* __restrict__ gy, const int8_t* __restrict__ idx, T* __restrict__ gx,
                         int planes, PoolGeom g) {
  const int SH = STRIDE ? STRIDE : g.SH, SW = STRIDE ? STRIDE : g.SW;
  const int DH = UNIT_DILATION ? 1 : g.DH, DW = UNIT_DILATION ? 1 : g.DW;
  const int plane_elems = g.H * g.W, out_elems = g.Ho * g.Wo;
  const int reach_h = (g.KH - 1) * DH, reach_w = (g.KW - 1) * DW;
  for (int nc = blockIdx.y; nc < planes; nc += gridDim.y) {
    const T* gy_p = gy + (int64_t)nc * out_elems;
    const int8_t* idx_p = idx + (int64_t)nc * out_elems;
    T* gx_p = gx + (int64_t)nc * plane_elems;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < plane_elems; e += gridDim.x * blockDim.x) {
      const int h = e / g.W, w = e - h * g.W;
      const int ah = h + g.PH, aw = w + g.PW;                    // >= 0
      const int ho_hi = min(g.Ho - 1, ah / SH), wo_hi = min(g.Wo - 1, aw / SW);
      const int ho_lo = ah > reach_h ? (ah - reach_h + SH - 1) / SH : 0;
      const int wo_lo = aw > reach_w ? (aw - reach_w + SW - 1) / SW : 0;
      float acc = 0.f;
      for (int ho = ho_lo; ho <= ho_hi; ++ho) {
        const int dh = ah - ho * SH;                              // = kh * DH if this row has a tap on h
        const int kh = UNIT_DILATION ? dh : dh / DH;
        if (!UNIT_DILATION && kh * DH != dh) continue;
        for (int wo = wo_lo; wo <= wo_hi; ++wo) {
          const int dw = aw - wo * SW;
          const int kw = UNIT_DILATION ? dw : dw / DW;
          if (!UNIT_DILATION && kw * DW != dw) continue;
          const int o = ho * g.Wo + wo;
          if (idx_p[o] == (int8_t)(kh * g.KW + kw)) acc += load_scalar<T>(gy_p, o);
        }
      }
      store_scalar<T>(gx_p, e, acc);
    }
  }
}

// Backward by row segments (unit dilation, at most two window rows over an input row, at most
// NWIN window columns over eight neighbouring positions: every pooling layer of the usual
// networks).  A thread owns eight consecutive positions of one input row.  It loads the
// arg-max code and the gradient of all 2 x NWIN candidate windows unconditionally (clamped
// coordinates, validity aside), so that the loads are in flight together, decodes each code
// into (kh, kw) with two 16-entry nibble tables, and adds the gradient to the position the
// window selected if that lies in its segment.  Index arithmetic is paid once per eight
// outputs, the store is one 16-byte vector when the row allows it, and every position
// receives its terms in the general kernel's order (window rows, then columns, ascending).
// FIXED_SW / FIXED_KW / FIXED_D0 > -100: the column stride, the window width and the offset
// `wo_lo * SW - PW - w0` of the first candidate column against the segment are compile-time
// (they do not depend on the segment when 8 % SW == 0); a window then reaches only FIXED_KW
// known positions of the segment instead of being compared against all eight.
template <typename T, int NWIN, int FIXED_SW = 0, int FIXED_KW = 0, int FIXED_D0 = -100>
__global__ void __launch_bounds__(256)
max_pool_backward_row_kernel(const T* __restrict__ gy, const int8_t* __restrict__ idx, T* __restrict__ gx,
                             uint32_t total_segments, int segs_per_row, PoolGeom g, uint64_t kh_of, uint64_t kw_of,
                             int vector_store) {
  const int out_elems = g.Ho * g.Wo, plane_elems = g.H * g.W;
  const int reach_h = g.KH - 1, reach_w = g.KW - 1;
  for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < total_segments; t += gridDim.x * blockDim.x) {
    const uint32_t row = t / (uint32_t)segs_per_row;
    const int seg = (int)(t - row * (uint32_t)segs_per_row);
    const uint32_t nc = row / (uint32_t)g.H;
    const int h = (int)(row - nc * (uint32_t)g.H);
    const int w0 = seg * 8;
    const int last = min(w0 + 7, g.W - 1);
    const T* gy_p = gy + (int64_t)nc * out_elems;
    const int8_t* idx_p = idx + (int64_t)nc * out_elems;
    const int ah = h + g.PH, aw0 = w0 + g.PW;
    const int ho_hi = min(g.Ho - 1, ah / g.SH);
    const int ho_lo = ah > reach_h ? (ah - reach_h + g.SH - 1) / g.SH : 0;
    const int wo_hi = min(g.Wo - 1, (last + g.PW) / g.SW);
    const int wo_lo = aw0 > reach_w ? (aw0 - reach_w + g.SW - 1) / g.SW : 0;
    int code[2][NWIN];
    float grad[2][NWIN];
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int hoc = min(ho_lo + a, g.Ho - 1);
#pragma unroll
      for (int b = 0; b < NWIN; ++b) {
        const int o = hoc * g.Wo + min(wo_lo + b, g.Wo - 1);
        code[a][b] = idx_p[o];
        grad[a][b] = load_scalar<T>(gy_p, o);
      }
    }
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int ho = ho_lo + a;
      const int kh_need = ah - ho * g.SH;                        // the tap row this input row is in that window row
#pragma unroll
      for (int b = 0; b < NWIN; ++b) {
        const int wo = wo_lo + b;
        const int c = code[a][b] & 15;
        const int kh = (int)((kh_of >> (4 * c)) & 15), kw = (int)((kw_of >> (4 * c)) & 15);
        const bool live = ho <= ho_hi && wo <= wo_hi && kh == kh_need;
        if constexpr (FIXED_D0 > -100) {
#pragma unroll
          for (int t = 0; t < FIXED_KW; ++t) {
            constexpr int kFirst = FIXED_D0;
            const int j = kFirst + FIXED_SW * b + t;             // compile-time after unrolling
            if (j >= 0 && j < 8) acc[j] += (live && kw == t) ? grad[a][b] : 0.f;
          }
        } else {
          const int target = live ? wo * g.SW - g.PW + kw - w0 : -1;   // position inside the segment
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += target == j ? grad[a][b] : 0.f;
        }
      }
    }
    T* out = gx + (int64_t)nc * plane_elems + h * g.W + w0;
    if (vector_store) {                                        // W % 8 == 0 and a 16-byte aligned tensor
      if constexpr (sizeof(T) == 2) {
        uint4 v;
        uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          T lo, hi;
          store_scalar<T>(&lo, 0, acc[2 * k]);
          store_scalar<T>(&hi, 0, acc[2 * k + 1]);
          pv[k] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&lo)) |
                  ((uint32_t)(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
        }
        *reinterpret_cast<uint4*>(out) = v;
      } else {
        *reinterpret_cast<float4*>(out) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (w0 + j < g.W) store_scalar<T>(out, j, acc[j]);
    }
  }
}

// Backward by row segments for the geometries of the forward row kernel (K x K windows with
// K = 2 or 3, stride 2, unit dilation, column padding P = 0 or 1, W % 8 == 0).  A thread owns
// eight consecutive positions w0 .. w0 + 7 of one input row.  At most two window rows contain
// the row, and the window columns that reach the segment are w0 / 2 + BLO .. w0 / 2 + BHI with
// BLO = -1 for (K, P) = (3, 0), else 0, and BHI = 4 for P = 1, else 3: the four columns
// w0 / 2 .. w0 / 2 + 3 come with one vector load of the codes and one of the gradients, the
// fifth with a scalar load.  Window column b reaches the positions 2 b - P .. 2 b - P + K - 1 of
// the segment, known at compile time.  Every position receives its terms in the general
// kernel's order (window rows, then columns, ascending).
template <typename T, int K, int P>
__global__ void __launch_bounds__(256)
max_pool_backward_s2_kernel(const T* __restrict__ gy, const int8_t* __restrict__ idx, T* __restrict__ gx,
                            uint32_t total_segments, int segs_per_row, PoolGeom g, int vector_load, PoolDiv by_segs,
                            PoolDiv by_rows) {
  constexpr int BLO = (K == 3 && P == 0) ? -1 : 0, BHI = P == 1 ? 4 : 3, NB = BHI - BLO + 1;
  const int out_elems = g.Ho * g.Wo, plane_elems = g.H * g.W;
  for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < total_segments; t += gridDim.x * blockDim.x) {
    const uint32_t row = pool_div(t, by_segs);
    const int seg = (int)(t - row * (uint32_t)segs_per_row);
    const uint32_t nc = pool_div(row, by_rows);
    const int h = (int)(row - nc * (uint32_t)g.H);
    const int w0 = seg * 8, b0 = seg * 4;
    const T* gy_p = gy + (int64_t)nc * out_elems;
    const int8_t* idx_p = idx + (int64_t)nc * out_elems;
    const int ah = h + g.PH;
    const int ho_hi = min(g.Ho - 1, ah / 2);
    const int ho_lo = ah > K - 1 ? (ah - (K - 1) + 1) / 2 : 0;
    int code[2][NB];
    float grad[2][NB];
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int base = min(ho_lo + a, g.Ho - 1) * g.Wo;
      if (vector_load && b0 + 4 <= g.Wo) {
        const uint32_t c4 = __ldg(reinterpret_cast<const uint32_t*>(idx_p + base + b0));
        float f[4];
        if constexpr (sizeof(T) == 4) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(gy_p + base + b0));
          f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
        } else {
          const uint2 v = __ldg(reinterpret_cast<const uint2*>(gy_p + base + b0));
          const uint32_t r[2] = {v.x, v.y};
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            if constexpr (std::is_same<T, __half>::value) {
              f[2 * k] = __half2float(__ushort_as_half((unsigned short)(r[k] & 0xffffu)));
              f[2 * k + 1] = __half2float(__ushort_as_half((unsigned short)(r[k] >> 16)));
            } else {
              f[2 * k] = __uint_as_float(r[k] << 16);
              f[2 * k + 1] = __uint_as_float(r[k] & 0xffff0000u);
            }
          }
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          code[a][b - BLO] = (int)((c4 >> (8 * b)) & 0xffu);
          grad[a][b - BLO] = f[b];
        }
      } else {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int o = base + min(b0 + b, g.Wo - 1);
          code[a][b - BLO] = idx_p[o];
          grad[a][b - BLO] = load_scalar<T>(gy_p, o);
        }
      }
      if constexpr (BLO < 0) {
        const int o = base + max(b0 - 1, 0);
        code[a][0] = idx_p[o];
        grad[a][0] = load_scalar<T>(gy_p, o);
      }
      if constexpr (BHI > 3) {
        const int o = base + min(b0 + 4, g.Wo - 1);
        code[a][NB - 1] = idx_p[o];
        grad[a][NB - 1] = load_scalar<T>(gy_p, o);
      }
    }
    // Position j (column w0 + j) is tap (j + P) % 2 of window column (j + P) / 2 and, for K = 3 and
    // an even j + P, also tap 2 of the column before: one or two candidates per window row, each
    // a comparison of the stored code with the code that would name this position.
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int ho = ho_lo + a;
      const int first_code = ho <= ho_hi ? (ah - ho * 2) * K : -64;   // code of tap column 0 in this input row
      if (b0 + BLO < 0 || b0 + BHI >= g.Wo) {                      // first / last segments of a row only
#pragma unroll
        for (int bi = 0; bi < NB; ++bi) {
          const int wo = b0 + bi + BLO;
          if (wo < 0 || wo >= g.Wo) code[a][bi] = -1;              // a clamped load, not a window
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int q = j + P, b_hi = q >> 1, kw_hi = q & 1;         // compile-time after unrolling
        if (K == 3 && kw_hi == 0 && b_hi - 1 >= BLO) {
          if (code[a][b_hi - 1 - BLO] == first_code + 2) acc[j] += grad[a][b_hi - 1 - BLO];
        }
        if (b_hi <= BHI) {
          if (code[a][b_hi - BLO] == first_code + kw_hi) acc[j] += grad[a][b_hi - BLO];
        }
      }
    }
    Oct<T> out;
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int j = 0; j < 8; ++j) out.f[j] = acc[j];
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        out.r[k] = bits_of<T>(round_to<T>(acc[2 * k])) | (bits_of<T>(round_to<T>(acc[2 * k + 1])) << 16);
      }
    }
    store_oct<T>(gx + (int64_t)nc * plane_elems + h * g.W + w0, out);
  }
}

template <typename T>
int launch_backward(const void* gy, const int8_t* idx, void* gx, int64_t planes, const PoolGeom& g, cudaStream_t s) {
  const int plane_elems = g.H * g.W;
  const bool unit = g.DH == 1 && g.DW == 1;
  const int p = (int)planes;
  // window columns that can touch eight neighbouring positions: positions aw0 .. aw0 + 7 see
  // columns ceil((aw0 - (KW-1)) / SW) .. floor((aw0 + 7) / SW), at most (7 + KW-1) / SW + 1 of them
  const int nwin = (7 + g.KW - 1) / g.SW + 1;
  const int segs = (g.W + 7) / 8;
  const int64_t total_segments = planes * g.H * segs;
  if (unit && g.KH == g.KW && (g.KH == 2 || g.KH == 3) && g.SH == 2 && g.SW == 2 && g.PW <= 1 && g.W % 8 == 0 &&
      aligned(gx, sizeof(T) * 8) && total_segments < ((int64_t)1 << 31)) {
    const int vec = g.Wo % 4 == 0 && aligned(gy, sizeof(T) * 4) && aligned(idx, 4);
    const int64_t blocks = (total_segments + 255) / 256;
    const int grid = (int)max((int64_t)1, min(blocks, (int64_t)device_info().sm_count * 16));
#define ACTNN_S2(K, P)                                                                                      \
    max_pool_backward_s2_kernel<T, K, P><<<grid, 256, 0, s>>>((const T*)gy, idx, (T*)gx, (uint32_t)total_segments, \
                                                              segs, g, vec, make_pool_div((uint32_t)segs),         \
                                                              make_pool_div((uint32_t)g.H))
    if (g.KH == 3 && g.PW == 1) ACTNN_S2(3, 1);
    else if (g.KH == 3) ACTNN_S2(3, 0);
    else if (g.PW == 1) ACTNN_S2(2, 1);
    else ACTNN_S2(2, 0);
#undef ACTNN_S2
    return check_launch();
  }
  if (unit && (g.KH + g.SH - 1) / g.SH <= 2 && nwin <= 10 && total_segments < ((int64_t)1 << 31)) {
    uint64_t kh_of = 0, kw_of = 0;                               // code -> (kh, kw), one nibble each
    for (int c = 0; c < g.KH * g.KW; ++c) {
      kh_of |= (uint64_t)(c / g.KW) << (4 * c);
      kw_of |= (uint64_t)(c % g.KW) << (4 * c);
    }
    const int vec = g.W % 8 == 0 && aligned(gx, 16);
    const int64_t blocks = (total_segments + 255) / 256;
    const int grid = (int)max((int64_t)1, min(blocks, (int64_t)device_info().sm_count * 16));
    if (g.KW == 3 && g.SW == 2 && g.PW == 1)                     // the stem pooling of the ResNets: offset -1 always
      max_pool_backward_row_kernel<T, 5, 2, 3, -1><<<grid, 256, 0, s>>>((const T*)gy, idx, (T*)gx,
                                                                        (uint32_t)total_segments, segs, g, kh_of,
                                                                        kw_of, vec);
    else if (nwin <= 6)
      max_pool_backward_row_kernel<T, 6><<<grid, 256, 0, s>>>((const T*)gy, idx, (T*)gx, (uint32_t)total_segments,
                                                              segs, g, kh_of, kw_of, vec);
    else
      max_pool_backward_row_kernel<T, 10><<<grid, 256, 0, s>>>((const T*)gy, idx, (T*)gx, (uint32_t)total_segments,
                                                               segs, g, kh_of, kw_of, vec);
    return check_launch();
  }
  dim3 grid = plane_grid(plane_elems, planes);
  if (unit && g.SH == 2 && g.SW == 2)
    max_pool_backward_kernel<T, 2, true><<<grid, 256, 0, s>>>((const T*)gy, idx, (T*)gx, p, g);
  else if (unit && g.SH == 1 && g.SW == 1)
    max_pool_backward_kernel<T, 1, true><<<grid, 256, 0, s>>>((const T*)gy, idx, (T*)gx, p, g);
  else if (unit)
    max_pool_backward_kernel<T, 0, true><<<grid, 256, 0, s>>>((const T*)gy, idx, (T*)gx, p, g);
  else
    max_pool_backward_kernel<T, 0, false><<<grid, 256, 0, s>>>((const T*)gy, idx, (T*)gx, p, g);
  return check_launch();
}

int check_geom(int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int SH, int SW, int PH, int PW, int DH,
               int DW, PoolGeom* g) {
  if (N < 0 || C < 0 || H <= 0 || W <= 0 || H > (1 << 30) || W > (1 << 30)) return ACTNN_ERR_SHAPE;
  if (KH <= 0 || KW <= 0 || SH <= 0 || SW <= 0 || PH < 0 || PW < 0 || DH <= 0 || DW <= 0) return ACTNN_ERR_ARG;
  if (KH * KW >= 16) return ACTNN_ERR_ARG;                      // quantization.cc:162
  const int64_t Ho = (H + 2 * PH - (int64_t)DH * (KH - 1) - 1) / SH + 1;
  const int64_t Wo = (W + 2 * PW - (int64_t)DW * (KW - 1) - 1) / SW + 1;
  if (Ho <= 0 || Wo <= 0) return ACTNN_ERR_SHAPE;
  *g = PoolGeom{(int)H, (int)W, (int)Ho, (int)Wo, KH, KW, SH, SW, PH, PW, DH, DW};
  return ACTNN_OK;
}

}  // namespace
}  // namespace actnn

using namespace actnn;

extern "C" int actnn_max_pool2d_forward(const void* x, void* y, int8_t* idx, int64_t N, int64_t C, int64_t H,
                                        int64_t W, int KH, int KW, int SH, int SW, int PH, int PW, int DH, int DW,
                                        int dtype, actnn_stream_t stream) {
  PoolGeom g;
  if (int st = check_geom(N, C, H, W, KH, KW, SH, SW, PH, PW, DH, DW, &g)) return st;
  const int64_t total = N * C * g.Ho * g.Wo;
  if (total == 0) return ACTNN_OK;
  if (!x || !y || !idx) return ACTNN_ERR_NULL;
  if (N * C > 0x7fffffff || H * W > 0x7fffffff) return ACTNN_ERR_SHAPE;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case ACTNN_F32: return launch_forward<float>(x, y, idx, N * C, g, s);
    case ACTNN_F16: return launch_forward<__half>(x, y, idx, N * C, g, s);
    case ACTNN_BF16: return launch_forward<__nv_bfloat16>(x, y, idx, N * C, g, s);
    default: return ACTNN_ERR_DTYPE;
  }
}

extern "C" int actnn_max_pool2d_backward(const void* grad_out, const int8_t* idx, void* grad_in, int64_t N,
                                         int64_t C, int64_t H, int64_t W, int KH, int KW, int SH, int SW, int PH,
                                         int PW, int DH, int DW, int dtype, actnn_stream_t stream) {
  PoolGeom g;
  if (int st = check_geom(N, C, H, W, KH, KW, SH, SW, PH, PW, DH, DW, &g)) return st;
  const int64_t total = N * C * H * W;
  const int64_t planes = N * C;
  if (total == 0) return ACTNN_OK;
  if (!grad_out || !idx || !grad_in) return ACTNN_ERR_NULL;
  if (planes > 0x7fffffff || H * W > 0x7fffffff) return ACTNN_ERR_SHAPE;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case ACTNN_F32: return launch_backward<float>(grad_out, idx, grad_in, planes, g, s);
    case ACTNN_F16: return launch_backward<__half>(grad_out, idx, grad_in, planes, g, s);
    case ACTNN_BF16: return launch_backward<__nv_bfloat16>(grad_out, idx, grad_in, planes, g, s);
    default: return ACTNN_ERR_DTYPE;
  }
}
