// Shared device helpers for the actnn_b200 kernels (sm_100a only).
//
// Everything on this path is a streaming codec bound by HBM bandwidth, so the helpers are
// about moving bytes well: 128/256-bit global loads and stores, one-instruction warp
// min/max (redux.sync.f32, new with sm_100a), a 32x32 bit-matrix transpose across the
// lanes of a warp (the packed layouts are "lane ballots", see quant_math.cuh), and a
// counter-based Philox generator that lives entirely in registers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/actnn_b200.h"

#define ACTNN_HD __host__ __device__ __forceinline__
#define ACTNN_DEV __device__ __forceinline__

namespace actnn {

constexpr int kGroup = 256;          // elements per quantization group on the fast paths
constexpr int kOct = 8;              // consecutive elements one lane owns inside a group
constexpr unsigned kFull = 0xffffffffu;

// ------------------------------------------------------------------ dtype plumbing
template <typename T> struct DType;
template <> struct DType<float> { static constexpr int id = ACTNN_F32; };
template <> struct DType<__half> { static constexpr int id = ACTNN_F16; };
template <> struct DType<__nv_bfloat16> { static constexpr int id = ACTNN_BF16; };

static inline int dtype_size(int dtype) { return dtype == ACTNN_F32 ? 4 : 2; }

// Eight consecutive elements of T, as they sit in registers after one vector load.
template <typename T> struct Oct { uint32_t r[4]; };          // 16-bit types: 4 x (lo, hi)
template <> struct Oct<float> { float f[8]; };

#ifdef __CUDACC__
// ------------------------------------------------------------------ vector memory ops
// Streaming loads bypass L1 allocation: every byte of the activation is touched once.
template <typename T> ACTNN_DEV Oct<T> load_oct(const T* p) {
  Oct<T> o;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(o.r[0]), "=r"(o.r[1]), "=r"(o.r[2]), "=r"(o.r[3]) : "l"(p));
  return o;
}
template <> ACTNN_DEV Oct<float> load_oct<float>(const float* p) {
  Oct<float> o;     // one 256-bit load (sm_100): 32 lanes x 32 B = 1 KiB contiguous per warp
  asm volatile("ld.global.nc.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(o.f[0]), "=f"(o.f[1]), "=f"(o.f[2]), "=f"(o.f[3]),
                 "=f"(o.f[4]), "=f"(o.f[5]), "=f"(o.f[6]), "=f"(o.f[7]) : "l"(p));
  return o;
}
template <typename T> ACTNN_DEV void store_oct(T* p, const Oct<T>& o) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};"
               :: "l"(p), "r"(o.r[0]), "r"(o.r[1]), "r"(o.r[2]), "r"(o.r[3]) : "memory");
}
template <> ACTNN_DEV void store_oct<float>(float* p, const Oct<float>& o) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               :: "l"(p), "f"(o.f[0]), "f"(o.f[1]), "f"(o.f[2]), "f"(o.f[3]),
                  "f"(o.f[4]), "f"(o.f[5]), "f"(o.f[6]), "f"(o.f[7]) : "memory");
}
// Streaming ("evict first") stores for the decoders: a decoded activation is several times the
// size of what was read to produce it and nothing in the kernel reads it back, so its lines
// should not push the packed input out of the L2.  Measured on a B200, decoding 205 MB:
// 54.8 -> 47.0 microseconds.
template <typename T> ACTNN_DEV void store_oct_streaming(T* p, const Oct<T>& o) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
               :: "l"(p), "r"(o.r[0]), "r"(o.r[1]), "r"(o.r[2]), "r"(o.r[3]) : "memory");
}
template <> ACTNN_DEV void store_oct_streaming<float>(float* p, const Oct<float>& o) {
  asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               :: "l"(p), "f"(o.f[0]), "f"(o.f[1]), "f"(o.f[2]), "f"(o.f[3]),
                  "f"(o.f[4]), "f"(o.f[5]), "f"(o.f[6]), "f"(o.f[7]) : "memory");
}
template <typename T> ACTNN_DEV Oct<T> zero_oct() {
  Oct<T> o;
  for (int i = 0; i < 4; ++i) o.r[i] = 0u;
  return o;
}
template <> ACTNN_DEV Oct<float> zero_oct<float>() {
  Oct<float> o;
  for (int i = 0; i < 8; ++i) o.f[i] = 0.f;
  return o;
}

// ------------------------------------------------------------------ bulk copies into shared memory
// A warp stages its next inputs with the bulk-copy engine (cp.async.bulk, completion counted
// in bytes on an mbarrier) so that no register waits on DRAM.  Addresses are 32-bit shared
// window addresses; source, destination and size must be multiples of 16 bytes.
ACTNN_DEV uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
ACTNN_DEV void mbar_init(uint32_t bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(arrivals) : "memory");
}
ACTNN_DEV void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async;" ::: "memory");
}
ACTNN_DEV void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
ACTNN_DEV void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// One attempt may sleep in hardware for up to about kBulkWaitHintNs before it reports failure.
constexpr uint32_t kBulkWaitHintNs = 20000u;
ACTNN_DEV bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity), "r"(kBulkWaitHintNs) : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity, at most kBulkWaitTries attempts (each attempt
// itself sleeps in hardware for a bounded time).  false = gave up.
constexpr uint32_t kBulkWaitTries = 1u << 16;
ACTNN_DEV bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kBulkWaitTries; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
template <typename T> ACTNN_DEV Oct<T> lds_oct(uint32_t addr) {
  Oct<T> o;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(o.r[0]), "=r"(o.r[1]), "=r"(o.r[2]), "=r"(o.r[3]) : "r"(addr));
  return o;
}
template <> ACTNN_DEV Oct<float> lds_oct<float>(uint32_t addr) {
  Oct<float> o;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(o.f[0]), "=f"(o.f[1]), "=f"(o.f[2]), "=f"(o.f[3]) : "r"(addr));
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(o.f[4]), "=f"(o.f[5]), "=f"(o.f[6]), "=f"(o.f[7]) : "r"(addr + 16u));
  return o;
}

// ------------------------------------------------------------------ warp reductions
ACTNN_DEV float warp_min(float v) {
  float r;
  asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
ACTNN_DEV float warp_max(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

// ------------------------------------------------------------------ 32x32 bit transpose
// Lane r holds row r of a 32x32 bit matrix (bit c = column c).  Afterwards lane r holds
// column r of the original (bit c = original lane c, bit r).  Five butterfly stages; per
// stage one shuffle, one funnel shift (a rotate) and one LOP3 bit-select.
// The stages that exchange half-words and bytes are one byte-permute each.
struct TransposePlan {
  uint32_t sel16, sel8;   // byte selectors of the stages s = 16 and s = 8
  uint32_t keep[3];       // bits this lane keeps at stage s = 4, 2, 1
  uint32_t rot[3];        // left-rotate applied to the partner's word
};
ACTNN_DEV TransposePlan make_transpose_plan(int lane) {
  TransposePlan p;
  p.sel16 = (lane & 16) ? 0x3276u : 0x5410u;
  p.sel8 = (lane & 8) ? 0x3715u : 0x6240u;
  const uint32_t m[3] = {0x0f0f0f0fu, 0x33333333u, 0x55555555u};
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const int s = 4 >> k;
    const bool low = (lane & s) == 0;
    p.keep[k] = low ? m[k] : ~m[k];
    p.rot[k] = low ? s : 32 - s;
  }
  return p;
}
ACTNN_DEV uint32_t warp_transpose32(uint32_t x, const TransposePlan& p) {
  x = __byte_perm(x, __shfl_xor_sync(kFull, x, 16), p.sel16);
  x = __byte_perm(x, __shfl_xor_sync(kFull, x, 8), p.sel8);
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const uint32_t y = __shfl_xor_sync(kFull, x, 4 >> k);
    const uint32_t ry = __funnelshift_l(y, y, p.rot[k]);
    x = (x & p.keep[k]) | (ry & ~p.keep[k]);
  }
  return x;
}
#endif  // __CUDACC__

// ------------------------------------------------------------------ Philox4x32-10
// Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3" (SC'11).
// The ten round keys depend only on the seed, so the host expands them once and passes
// them as kernel parameters: in the kernel they are constant-bank operands of the XORs
// and the key schedule costs no instructions.
struct Philox4 { uint32_t v[4]; };
struct NoiseKey {
  uint32_t k0[10], k1[10];   // round keys
  uint32_t o0, o1;           // the 64-bit offset, upper half of the counter
};

static inline NoiseKey make_noise_key(uint64_t seed, uint64_t offset) {
  NoiseKey k;
  uint32_t a = (uint32_t)seed, b = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    k.k0[r] = a; k.k1[r] = b;
    a += 0x9E3779B9u; b += 0xBB67AE85u;
  }
  k.o0 = (uint32_t)offset; k.o1 = (uint32_t)(offset >> 32);
  return k;
}

#ifdef __CUDACC__
ACTNN_DEV Philox4 noise_call(const NoiseKey& key, uint64_t c) {
  uint32_t c0 = (uint32_t)c, c1 = (uint32_t)(c >> 32), c2 = key.o0, c3 = key.o1;
#ifndef ACTNN_PHILOX_ROUNDS
#define ACTNN_PHILOX_ROUNDS 10
#endif
#pragma unroll
  for (int r = 0; r < ACTNN_PHILOX_ROUNDS; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    c0 = (uint32_t)(p1 >> 32) ^ c1 ^ key.k0[r];
    c1 = (uint32_t)p1;
    c2 = (uint32_t)(p0 >> 32) ^ c3 ^ key.k1[r];
    c3 = (uint32_t)p0;
  }
  Philox4 o;
  o.v[0] = c0; o.v[1] = c1; o.v[2] = c2; o.v[3] = c3;
  return o;
}
#endif

// Rounding-noise stream, indexed by position in the padded [N, G, 256] activation:
// flat group q, position d in the group, lane t = d / 8, j = d % 8.
//   counter = (lo32(c), hi32(c), lo32(offset), hi32(offset)), key = (lo32(seed), hi32(seed));
//   the call's four output words v[0..3] are extended to eight, e[i] = v[i] and
//   e[4 + i] = v[i] + 0x9E3779B1 * v[(i + 1) % 4] mod 2^32 (see quant_math.cuh for why that
//   is sound);
//   16-bit activations: c = (q / 4) * 32 + t; word w = e[2h + j / 4], h = q % 4, p = j % 4;
//     float16:  k = bits 1..8 (p even) or 17..24 (p odd) of w rotated right by 8 * (p / 2);
//     bfloat16: k = byte 2 * (p % 2) + p / 2 of w;
//     noise = (2k + 1 - 256) / 512.
//   float32 activations: c = (q / 2) * 32 + t; 16-bit field j of the words e[4h .. 4h + 3],
//     h = q % 2, is k; noise = (2k + 1 - 65536) / 131072.
// Both are odd multiples of the step, symmetric about zero, strictly inside (-0.5, 0.5)
// and exactly representable in the activation dtype.  The resolution follows the dtype:
// (x - min) * scale carries at most 11 (float16) or 8 (bfloat16) significant bits.

// ------------------------------------------------------------------ host-side launch helpers
struct DeviceInfo { int sm_count; };
const DeviceInfo& device_info();                   // api.cu (per current device, cached)
int check_launch();                                // api.cu: cudaPeekAtLastError -> status
unsigned* bulk_wait_counter();                     // api.cu: device counter of bulk-copy waits that gave up

// codec_mixed.cu: actnn_pack_mixed with one more promise from the caller, `min_is_exact`
// (every mn[q] is the true minimum of its group, as after actnn_minimax).
int pack_mixed_impl(const void* data, const void* mn, const void* mx, const int32_t* bits,
                    const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out, int64_t N, int64_t G,
                    int64_t group_size, int dtype, int stat_dtype, int stochastic, const void* noise, uint64_t seed,
                    uint64_t offset, bool min_is_exact, cudaStream_t stream);

// stats.cu: actnn_minimax with two extras for the one-call compress: rows walked from the
// last to the first (`reverse`), and a word zeroed by the kernel (`clear_word`, the ticket of
// the next kernel).
int minimax_impl(const void* data, void* mn, void* mx, int64_t rows, int64_t cols, int dtype, int reverse,
                 unsigned* clear_word, cudaStream_t stream);
// stats.cu: sensitivities (actnn_range_sqr) and the greedy allocation (actnn_calc_precision, unit
// weights, with word offsets) of one layer in one launch; `ticket` must be zero when it starts
// and is zero again when it ends.
bool range_greedy_supported(int64_t N, int initial_bits);
int range_greedy_impl(const void* mn, const void* mx, int64_t N, int64_t G, int stat_dtype, float range_factor,
                      float coeff, const float* grad_scale, float* C, unsigned* ticket, int initial_bits,
                      double target, int32_t* b_out, int64_t* word_offsets, int64_t group_size, cudaStream_t stream);

// codec_generic.cu: the codec for group sizes other than 256 (multiples of 32), one warp per group.
bool generic_group_ok(int64_t group_size);
int pack_mixed_generic(const void* data, const void* mn, const void* mx, const int32_t* bits,
                       const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out, int64_t N, int64_t G,
                       int64_t gs, int dtype, int stat_dtype, int stochastic, const void* noise, uint64_t seed,
                       uint64_t offset, cudaStream_t s);
int unpack_mixed_generic(const int32_t* packed, const int32_t* bits, const int64_t* word_offsets, const void* scale,
                         const void* mn, void* out, int64_t N, int64_t G, int64_t gs, int dtype, int stat_dtype,
                         cudaStream_t s);
int pack_single_generic(bool fused, const void* data, const void* mn, const void* mx, int bits, int8_t* packed,
                        void* scale, void* mn_out, void* mx_out, int64_t N, int64_t G, int64_t gs, int dtype,
                        int stat_dtype, int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                        cudaStream_t s);
int unpack_single_generic(const int8_t* packed, int bits, const void* scale, const void* mn, void* out, int64_t N,
                          int64_t G, int64_t gs, int dtype, int stat_dtype, cudaStream_t s);

static inline bool aligned(const void* p, size_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

#ifdef __CUDACC__
// Grid for a persistent warp-task kernel: as many blocks as can be resident at once
// (SMs x blocks per SM), so that there is a single wave and no under-filled tail, but no
// more than the tasks need.  The occupancy query is cached per kernel and device.
// `dynamic_smem` > 0 also raises the kernel's dynamic shared memory limit to that size.
int cached_blocks_per_sm(const void* kernel, int threads, int dynamic_smem);   // api.cu

template <typename Kernel>
int persistent_grid(Kernel kernel, int threads, int64_t warp_tasks, int dynamic_smem = 0) {
  const int per_sm = cached_blocks_per_sm((const void*)kernel, threads, dynamic_smem);
  const int64_t resident = (int64_t)device_info().sm_count * per_sm;
  const int64_t needed = (warp_tasks + threads / 32 - 1) / (threads / 32);
  const int64_t grid = needed < resident ? needed : resident;
  return (int)(grid < 1 ? 1 : grid);
}
#endif

}  // namespace actnn
