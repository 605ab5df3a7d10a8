// 2-D max pooling (NCHW) that keeps only the window-local arg-max, one int8 per output.
//
// Forward scans each window row-major and takes a strictly larger value, so the first
// maximum wins, and stores kh*KW + kw (reference: quantization_cuda_kernel.cu:644-668;
// window taps here honour dilation, which the reference's loops leave out).
// Backward is a gather: every input position visits the few windows that contain it and
// adds the gradients of those that selected it, in float32 and in a fixed order.  That
// removes the reference's zero-fill and its atomicAdd scatter
// (quantization_cuda_kernel.cu:712-733) and makes the result deterministic.
#include "quant_math.cuh"

namespace actnn {
namespace {

struct PoolGeom {
  int H, W, Ho, Wo, KH, KW, SH, SW, PH, PW, DH, DW;
};

template <typename T>
__global__ void __launch_bounds__(256)
max_pool_forward_kernel(const T* __restrict__ x, T* __restrict__ y, int8_t* __restrict__ idx, int64_t total,
                        PoolGeom g) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t id = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; id < total; id += stride) {
    const int wo = (int)(id % g.Wo);
    const int64_t t = id / g.Wo;
    const int ho = (int)(t % g.Ho);
    const int64_t nc = t / g.Ho;
    const T* plane = x + nc * ((int64_t)g.H * g.W);
    const int hb = ho * g.SH - g.PH, wb = wo * g.SW - g.PW;
    float best = -INFINITY;
    int arg = 0;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int h = hb + kh * g.DH;
      if (h < 0 || h >= g.H) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int w = wb + kw * g.DW;
        if (w < 0 || w >= g.W) continue;
        const float v = load_scalar<T>(plane, (int64_t)h * g.W + w);
        if (v > best) { best = v; arg = kh * g.KW + kw; }
      }
    }
    store_scalar<T>(y, id, best);
    idx[id] = (int8_t)arg;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
max_pool_backward_kernel(const T* __restrict__ gy, const int8_t* __restrict__ idx, T* __restrict__ gx,
                         int64_t total, PoolGeom g) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t id = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; id < total; id += stride) {
    const int w = (int)(id % g.W);
    const int64_t t = id / g.W;
    const int h = (int)(t % g.H);
    const int64_t nc = t / g.H;
    const int64_t obase = nc * ((int64_t)g.Ho * g.Wo);
    float acc = 0.f;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int hh = h + g.PH - kh * g.DH;
      if (hh < 0 || hh % g.SH != 0) continue;
      const int ho = hh / g.SH;
      if (ho >= g.Ho) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int ww = w + g.PW - kw * g.DW;
        if (ww < 0 || ww % g.SW != 0) continue;
        const int wo = ww / g.SW;
        if (wo >= g.Wo) continue;
        const int64_t o = obase + (int64_t)ho * g.Wo + wo;
        if (idx[o] == (int8_t)(kh * g.KW + kw)) acc += load_scalar<T>(gy, o);
      }
    }
    store_scalar<T>(gx, id, acc);
  }
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

int grid_for(int64_t total) {
  return (int)max((int64_t)1, min((total + 255) / 256, (int64_t)device_info().sm_count * 16));
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
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case ACTNN_F32:
      max_pool_forward_kernel<float><<<grid_for(total), 256, 0, s>>>((const float*)x, (float*)y, idx, total, g);
      break;
    case ACTNN_F16:
      max_pool_forward_kernel<__half><<<grid_for(total), 256, 0, s>>>((const __half*)x, (__half*)y, idx, total, g);
      break;
    case ACTNN_BF16:
      max_pool_forward_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>((const __nv_bfloat16*)x,
                                                                            (__nv_bfloat16*)y, idx, total, g);
      break;
    default: return ACTNN_ERR_DTYPE;
  }
  return check_launch();
}

extern "C" int actnn_max_pool2d_backward(const void* grad_out, const int8_t* idx, void* grad_in, int64_t N,
                                         int64_t C, int64_t H, int64_t W, int KH, int KW, int SH, int SW, int PH,
                                         int PW, int DH, int DW, int dtype, actnn_stream_t stream) {
  PoolGeom g;
  if (int st = check_geom(N, C, H, W, KH, KW, SH, SW, PH, PW, DH, DW, &g)) return st;
  const int64_t total = N * C * H * W;
  if (total == 0) return ACTNN_OK;
  if (!grad_out || !idx || !grad_in) return ACTNN_ERR_NULL;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case ACTNN_F32:
      max_pool_backward_kernel<float><<<grid_for(total), 256, 0, s>>>((const float*)grad_out, idx, (float*)grad_in,
                                                                      total, g);
      break;
    case ACTNN_F16:
      max_pool_backward_kernel<__half><<<grid_for(total), 256, 0, s>>>((const __half*)grad_out, idx,
                                                                       (__half*)grad_in, total, g);
      break;
    case ACTNN_BF16:
      max_pool_backward_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(
          (const __nv_bfloat16*)grad_out, idx, (__nv_bfloat16*)grad_in, total, g);
      break;
    default: return ACTNN_ERR_DTYPE;
  }
  return check_launch();
}
