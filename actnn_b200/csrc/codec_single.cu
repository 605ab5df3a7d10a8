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
#include <cstdlib>

#include "quant_math.cuh"

namespace actnn {
namespace {

constexpr int kThreads = 256;

// Byte accumulators for one group: sample ni's magic registers are added in shifted left
// by ni*BITS.  The exponent bits of the rounding constant add up to a compile-time
// constant that is subtracted up front, so no per-code masking is needed.
template <typename T, int BITS> struct ByteAcc {
  static constexpr int WPT = 8 / BITS;
  using Fmt = MagicFmt<T, BITS>;
  static constexpr int R = Fmt::paired ? 4 : 8;
  uint32_t a[R];
  ACTNN_DEV ByteAcc() {
#pragma unroll
    for (int i = 0; i < R; ++i) a[i] = 0u - shifted_sum(Fmt::bias, BITS, WPT);
  }
  template <int NI> ACTNN_DEV void add(const Magic<T>& m) {
#pragma unroll
    for (int i = 0; i < R; ++i) a[i] += m.v[i] << (NI * BITS);
  }
  template <int NI> ACTNN_DEV void add_missing() {       // a sample past the end: code 0 everywhere
#pragma unroll
    for (int i = 0; i < R; ++i) a[i] += Fmt::bias << (NI * BITS);
  }
  ACTNN_DEV uint2 bytes() const {
    uint2 w;
    if constexpr (Fmt::paired) {                         // a[k] = byte 2k | byte 2k+1 << 16
      w.x = __byte_perm(a[0], a[1], 0x6420);
      w.y = __byte_perm(a[2], a[3], 0x6420);
    } else {                                             // a[j] = byte j
      w.x = a[0] + (a[1] << 8) + (a[2] << 16) + (a[3] << 24);
      w.y = a[4] + (a[5] << 8) + (a[6] << 16) + (a[7] << 24);
    }
    return w;
  }
};

// Walks (sample block, group pair) tasks without 64-bit divisions.
struct PairWalker {
  int64_t no, blocks;
  int r, per, step_n, step_r;
  ACTNN_DEV PairWalker(int64_t warp, int64_t nwarps, int64_t blocks_, int64_t per_) : blocks(blocks_) {
    per = (int)per_;
    no = warp / per;
    r = (int)(warp - no * per);
    step_n = (int)(nwarps / per);
    step_r = (int)(nwarps - (int64_t)step_n * per);
  }
  ACTNN_DEV bool valid() const { return no < blocks; }
  ACTNN_DEV void next() {
    no += step_n;
    r += step_r;
    if (r >= per) { r -= per; ++no; }
  }
};

// Shape of one warp task.  A task covers GP neighbouring groups of one block of wpt
// samples and is worked off in ROUNDS rounds of SS samples; a round holds OCTS = SS * GP
// octets per lane in registers.  All their group statistics are prepared together: lane o
// (< OCTS) owns octet o = s * GP + gi, does the one division, and ships the result.
template <typename T, int BITS> struct TaskShape {
  static constexpr int WPT = 8 / BITS;
  static constexpr int OCTS = sizeof(T) == 2 ? 8 : 4;
  // at least one Philox call's worth of neighbouring groups (4 for 16-bit types, 2 for float32)
  static constexpr int SS = WPT < 2 ? 1 : 2;
  static constexpr int GP = OCTS / SS;
  static constexpr int ROUNDS = WPT / SS;
};

// STAGED (whole tasks only): a round's OCTS octets per lane are SS contiguous runs of GP
// groups in global memory.  Lane 0 asks the bulk-copy engine for the NEXT round's runs
// while the warp works on the current one, into the warp's own two-stage ring in shared
// memory, and every lane then reads its 16 / 32 bytes per octet from there; completion is
// counted in bytes on one mbarrier per stage.  No register waits on DRAM, so the integer
// pipe stays fed.
constexpr int kStages = 2;
// PHILOX (whole tasks, direct loads): the noise is known at compile time to come from the
// generator, so the body of a round has no branch on `stochastic` / `noise` and the compiler
// can interleave the generator's dependent chain with the arithmetic of neighbouring octets.
template <typename T, typename ST, int BITS, bool FUSED, bool FULL, bool STAGED, bool PHILOX = false>
__global__ void __launch_bounds__(kThreads, (MagicInfo<T>::paired && !PHILOX) ? 3 : 2)
pack_single_kernel(const T* __restrict__ data, const T* __restrict__ mn, const T* __restrict__ mx,
                   int8_t* __restrict__ packed, ST* __restrict__ scale, ST* __restrict__ mn_out,
                   ST* __restrict__ mx_out, int64_t N, int64_t G, const T* __restrict__ noise,
                   int stochastic, const NoiseKey key, int64_t total_bytes, unsigned* __restrict__ gave_up) {
  using Sh = TaskShape<T, BITS>;
  constexpr int WPT = Sh::WPT, OCTS = Sh::OCTS, SS = Sh::SS, GP = Sh::GP, ROUNDS = Sh::ROUNDS;
  static_assert(GP % NoiseShape<T>::GPC == 0, "a task covers whole Philox calls");
  static_assert(!STAGED || FULL, "staging copies whole tasks");
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t gblocks = (G + GP - 1) / GP;
  const int64_t nblocks = (N + WPT - 1) / WPT;
  NoiseGen<T> gen(key, lane);
  if (warp == 0 && lane == 0) packed[total_bytes - 1] = 0;     // the reference's spare byte
  // the octet this lane prepares statistics for
  const int my_s = lane / GP, my_gi = lane % GP;

  // ---- staging ring of this warp
  extern __shared__ __align__(128) unsigned char staging[];
  constexpr uint32_t kRoundBytes = OCTS * kGroup * sizeof(T);
  constexpr uint32_t kRunBytes = GP * kGroup * sizeof(T);
  uint32_t ring = 0, bars = 0, round_no = 0;
  PairWalker ahead(warp, nwarps, nblocks, gblocks);
  int ahead_rd = 0;
  auto request = [&](uint32_t stage) {                         // lane 0: the round `ahead` points at
    const int64_t a_n0 = ahead.no * WPT + ahead_rd * SS, a_g0 = (int64_t)ahead.r * GP;
    const uint32_t bar = bars + 8u * stage, dst = ring + stage * kRoundBytes;
    mbar_expect_tx(bar, kRoundBytes);
#pragma unroll
    for (int s = 0; s < SS; ++s) bulk_load(dst + s * kRunBytes, data + ((a_n0 + s) * G + a_g0) * kGroup, kRunBytes, bar);
  };
  auto advance = [&]() {
    if (++ahead_rd == ROUNDS) { ahead_rd = 0; ahead.next(); }
  };
  if constexpr (STAGED) {
    const uint32_t wib = threadIdx.x >> 5;
    ring = smem_addr(staging) + wib * kStages * kRoundBytes;
    bars = smem_addr(staging) + (kThreads / 32) * kStages * kRoundBytes + wib * kStages * 8u;
    if (lane == 0) {
#pragma unroll
      for (int st = 0; st < kStages; ++st) mbar_init(bars + 8u * st, 1u);
      mbar_init_fence();
    }
    __syncwarp();
    if (ahead.valid()) {
      if (lane == 0) request(0u);
      advance();
    }
  }

  for (PairWalker walk(warp, nwarps, nblocks, gblocks); walk.valid(); walk.next()) {
    const int64_t no = walk.no;
    const int64_t g0 = (int64_t)walk.r * GP;
    const int cnt = FULL ? GP : (int)min((int64_t)GP, G - g0);
    ByteAcc<T, BITS> acc[GP];

#pragma unroll
    for (int rd = 0; rd < ROUNDS; ++rd) {
      const int64_t n0 = no * WPT + rd * SS;
      Oct<T> x[STAGED ? 1 : OCTS] = {};                 // staged rounds are read from shared memory where used
      uint32_t stage_base = 0;
      auto octet = [&](int o) -> Oct<T> {
        if constexpr (STAGED) return lds_oct<T>(stage_base + (uint32_t)(o * kGroup * sizeof(T)));
        else return x[o];
      };
      if constexpr (STAGED) {
        const uint32_t stage = round_no & 1u, parity = (round_no >> 1) & 1u;
        __syncwarp();                                   // every lane has read the other stage
        if (ahead.valid()) {
          if (lane == 0) request(stage ^ 1u);
          advance();
        }
        if (!__all_sync(kFull, mbar_wait(bars + 8u * stage, parity))) {
          mbar_wait(bars + 8u * stage, parity);         // one more bounded wait for the copy in flight
          if (lane == 0) atomicAdd(gave_up, 1u);
          return;
        }
        stage_base = ring + stage * kRoundBytes + (uint32_t)(lane * kOct * sizeof(T));
        ++round_no;
      } else {
#pragma unroll
        for (int o = 0; o < OCTS; ++o) {
          const int s = o / GP, gi = o % GP;
          const bool ok = FULL || (n0 + s < N && gi < cnt);
          x[o] = ok ? load_oct<T>(data + ((n0 + s) * G + g0 + gi) * kGroup + lane * kOct) : zero_oct<T>();
        }
      }
      // ---- statistics of the OCTS groups, one per lane
      float gmn = 0.f, gmx = 0.f;
      const bool mine_ok = lane < OCTS && (FULL || (n0 + my_s < N && my_gi < cnt));
      const int64_t my_q = (n0 + my_s) * G + g0 + my_gi;
      if constexpr (FUSED) {
#pragma unroll
        for (int o = 0; o < OCTS; ++o) {
          float lo, hi;
          oct_minmax<T>(octet(o), lo, hi);
          lo = warp_min(lo);
          hi = warp_max(hi);
          if (lane == o) { gmn = lo; gmx = hi; }
        }
      } else if (mine_ok) {
        gmn = load_scalar<T>(mn, my_q);
        gmx = load_scalar<T>(mx, my_q);
      }
      ParamWords mine = {0u, 0u};
      if (mine_ok) {
        const GroupParams gp = prepare_group<T>(gmn, gmx, BITS);
        store_scalar<ST>(scale, my_q, gp.scale);
        if (mn_out) store_scalar<ST>(mn_out, my_q, gmn);
        if (FUSED && mx_out) store_scalar<ST>(mx_out, my_q, gmx);
        mine = pack_params<T>(gp);
      }
      // ---- quantize and merge into the byte accumulators
      Oct<T> nzb[NoiseShape<T>::GPC];                   // one call's worth of noise octets
#pragma unroll
      for (int o = 0; o < OCTS; ++o) {
        const int s = o / GP, gi = o % GP;
        const QP<T> qp = fetch_params<T>(mine, o);
        const bool ok = FULL || (n0 + s < N && gi < cnt);
        Oct<T> nz;
        const int64_t q = (n0 + s) * G + g0 + gi;
        if constexpr (PHILOX) {
          static_assert(!PHILOX || FULL, "the generator-only variant covers whole tasks");
          if (gi % NoiseShape<T>::GPC == 0) noise_block<T>(gen.key, (uint64_t)q, lane, nzb);
          nz = nzb[gi % NoiseShape<T>::GPC];
        } else if (!stochastic || !ok) nz = zero_oct<T>();
        else if (noise) nz = load_oct<T>(noise + q * kGroup + lane * kOct);
        else if (!FULL) nz = gen.get((uint64_t)q);
        else {                                          // FULL: q - gi is a multiple of the groups per call
          if (gi % NoiseShape<T>::GPC == 0) noise_block<T>(gen.key, (uint64_t)q, lane, nzb);
          nz = nzb[gi % NoiseShape<T>::GPC];
        }
        // with the true minimum in hand the low clamp is implied by the rounding
        const Magic<T> m = quantize_oct<T, !FUSED, BITS>(octet(o), nz, qp);
#define ACTNN_ADD(K)                                                               \
        if constexpr (K < WPT) {                                                   \
          if (rd * SS + s == K) {                                                  \
            if (ok) acc[gi].template add<K>(m);                                    \
            else acc[gi].template add_missing<K>();                                \
          }                                                                        \
        }
        ACTNN_ADD(0) ACTNN_ADD(1) ACTNN_ADD(2) ACTNN_ADD(3) ACTNN_ADD(4) ACTNN_ADD(5) ACTNN_ADD(6) ACTNN_ADD(7)
#undef ACTNN_ADD
      }
    }
#pragma unroll
    for (int gi = 0; gi < GP; ++gi) {
      if (FULL || gi < cnt)
        *reinterpret_cast<uint2*>(packed + ((no * G + g0 + gi) * kGroup + lane * kOct)) = acc[gi].bytes();
    }
  }
}

// Unpack: a warp owns (sample block, group).  Lane t reads its eight bytes once; the table
// of all wpt samples x 2^BITS codes is computed by the first wpt * 2^BITS lanes together
// (one IEEE division per lane), and for 16-bit outputs with BITS <= 2 a byte-permute
// selects two decoded elements per instruction.
template <typename T, typename ST, int BITS>
__global__ void __launch_bounds__(kThreads, 4)
unpack_single_kernel(const int8_t* __restrict__ packed, const ST* __restrict__ scale,
                     const ST* __restrict__ mn, T* __restrict__ out, int64_t N, int64_t G) {
  constexpr int WPT = 8 / BITS;
  constexpr int E = 1 << BITS;
  constexpr bool TABLE = BITS <= 4;                        // BITS == 8: divide per element
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t nblocks = (N + WPT - 1) / WPT;

  // The packed stream is an eighth of the output or less, so a task's loads are small; to
  // keep enough bytes in flight each warp issues the loads of DEPTH tasks before it decodes
  // the first of them.
  constexpr int DEPTH = 2;
  const int my_s = TABLE ? lane / E : lane;                // lane l serves sample no*wpt + my_s
  PairWalker walk(warp, nwarps, nblocks, G);
  while (walk.valid()) {
    int64_t t_no[DEPTH], t_g[DEPTH];
    uint2 t_w[DEPTH];
    float t_sc[DEPTH], t_m[DEPTH];
    bool t_ok[DEPTH];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      t_ok[d] = walk.valid();
      t_no[d] = walk.no;
      t_g[d] = walk.r;
      t_w[d] = make_uint2(0u, 0u);
      t_sc[d] = 1.f;
      t_m[d] = 0.f;
      if (t_ok[d]) {
        t_w[d] = __ldg(reinterpret_cast<const uint2*>(packed + ((t_no[d] * G + t_g[d]) * kGroup + lane * kOct)));
        const int64_t my_n = t_no[d] * WPT + my_s;
        if (my_s < WPT && my_n < N) {
          t_sc[d] = load_scalar<ST>(scale, my_n * G + t_g[d]);
          t_m[d] = load_scalar<ST>(mn, my_n * G + t_g[d]);
        }
        walk.next();
      }
    }
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      if (!t_ok[d]) break;                                 // warp-uniform
      const int64_t no = t_no[d], g = t_g[d];
      const uint2 w = t_w[d];
      const float sc = t_sc[d], m = t_m[d];
      uint32_t entry = 0u, pairs = 0u;
      if constexpr (TABLE) {
        entry = dequant_bits<T>((float)(lane % E), sc, m);
        if constexpr (sizeof(T) == 2 && BITS <= 2) pairs = entry | (__shfl_down_sync(kFull, entry, 1) << 16);
      }
#pragma unroll
      for (int ni = 0; ni < WPT; ++ni) {
        const int64_t n = no * WPT + ni;
        Oct<T> o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
        if constexpr (sizeof(T) == 2 && BITS <= 2) {
          const uint32_t t01 = __shfl_sync(kFull, pairs, ni * E);
          const uint32_t t23 = BITS == 2 ? __shfl_sync(kFull, pairs, ni * E + 2) : t01;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t y = ((h ? w.y : w.x) >> (ni * BITS)) & (0x01010101u * (uint32_t)(E - 1));
            const uint32_t sel = y * 0x22u + 0x10101010u;
            ow[2 * h] = __byte_perm(t01, t23, sel);
            ow[2 * h + 1] = __byte_perm(t01, t23, sel >> 16);
          }
        } else {
          uint32_t v[8];
          const float sc_n = TABLE ? 0.f : __shfl_sync(kFull, sc, ni), m_n = TABLE ? 0.f : __shfl_sync(kFull, m, ni);
          float y_n = 0.f;                                       // 16-bit statistics: one reciprocal per group
          const bool recip = !TABLE && sizeof(ST) == 2 && group_reciprocal(sc_n, y_n);   // warp-uniform
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t code = ((((j < 4) ? w.x : w.y) >> (8 * (j & 3))) >> (ni * BITS)) & (uint32_t)(E - 1);
            if constexpr (TABLE) v[j] = __shfl_sync(kFull, entry, ni * E + (int)code);
            else v[j] = recip ? dequant_bits_recip<T>((float)code, sc_n, y_n, m_n) : dequant_bits<T>((float)code, sc_n, m_n);
          }
          if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int j = 0; j < 8; ++j) ow[j] = v[j];
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) ow[k] = v[2 * k] | (v[2 * k + 1] << 16);
          }
        }
        if (n < N) store_oct_streaming<T>(out + (n * G + g) * kGroup + lane * kOct, o);
      }
    }
  }
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
  const NoiseKey key = make_noise_key(seed, offset);
  const int64_t tb = single_total_bytes(bits, N, G);
  unsigned* gave_up = bulk_wait_counter();
  // The staged variant is opt-in (environment ACTNN_STAGED_PACK=1): measured on a B200 it
  // removes the waits on DRAM but not the kernel's real limit, instruction issue, and its
  // start-up (every warp waits for its first round) costs more than that gains on tensors
  // of ~100 MB.  Bulk copies want 16-byte aligned runs and whole tasks.
  static const bool staged_wanted = [] {
    const char* v = getenv("ACTNN_STAGED_PACK");
    return v && v[0] == '1';
  }();
  const bool can_stage = staged_wanted && gave_up != nullptr && aligned(data, 16);
#define ACTNN_LAUNCH(BITS)                                                                          \
  {                                                                                                 \
    using Sh = TaskShape<T, BITS>;                                                                  \
    constexpr int smem = (kThreads / 32) * (kStages * Sh::OCTS * kGroup * (int)sizeof(T) + kStages * 8); \
    const int64_t tasks = ((N + Sh::WPT - 1) / Sh::WPT) * ((G + Sh::GP - 1) / Sh::GP);              \
    const bool full = N % Sh::WPT == 0 && G % Sh::GP == 0;                                          \
    if (full && can_stage && stochastic && !noise) {                                                \
      auto kernel = pack_single_kernel<T, ST, BITS, FUSED, true, true, true>;                       \
      const int grid = persistent_grid(kernel, kThreads, tasks, smem);                              \
      kernel<<<grid, kThreads, smem, s>>>((const T*)data, (const T*)mn, (const T*)mx, packed, (ST*)scale, \
                                          (ST*)mn_out, (ST*)mx_out, N, G, (const T*)noise, stochastic, key, tb, \
                                          gave_up);                                                 \
    } else if (full && can_stage) {                                                                 \
      auto kernel = pack_single_kernel<T, ST, BITS, FUSED, true, true>;                             \
      const int grid = persistent_grid(kernel, kThreads, tasks, smem);                              \
      kernel<<<grid, kThreads, smem, s>>>((const T*)data, (const T*)mn, (const T*)mx, packed, (ST*)scale, \
                                          (ST*)mn_out, (ST*)mx_out, N, G, (const T*)noise, stochastic, key, tb, \
                                          gave_up);                                                 \
    } else if (full && stochastic && !noise) {                                                      \
      auto kernel = pack_single_kernel<T, ST, BITS, FUSED, true, false, true>;                      \
      kernel<<<persistent_grid(kernel, kThreads, tasks), kThreads, 0, s>>>(                         \
          (const T*)data, (const T*)mn, (const T*)mx, packed, (ST*)scale, (ST*)mn_out, (ST*)mx_out, N, G, \
          (const T*)noise, stochastic, key, tb, gave_up);                                           \
    } else if (full) {                                                                              \
      auto kernel = pack_single_kernel<T, ST, BITS, FUSED, true, false>;                            \
      kernel<<<persistent_grid(kernel, kThreads, tasks), kThreads, 0, s>>>(                         \
          (const T*)data, (const T*)mn, (const T*)mx, packed, (ST*)scale, (ST*)mn_out, (ST*)mx_out, N, G, \
          (const T*)noise, stochastic, key, tb, gave_up);                                           \
    } else {                                                                                        \
      auto kernel = pack_single_kernel<T, ST, BITS, FUSED, false, false>;                           \
      kernel<<<persistent_grid(kernel, kThreads, tasks), kThreads, 0, s>>>(                         \
          (const T*)data, (const T*)mn, (const T*)mx, packed, (ST*)scale, (ST*)mn_out, (ST*)mx_out, N, G, \
          (const T*)noise, stochastic, key, tb, gave_up);                                           \
    }                                                                                               \
  }
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
  const int64_t tasks = ((N + wpt - 1) / wpt) * G;
#define ACTNN_LAUNCH(BITS)                                                                        \
  unpack_single_kernel<T, ST, BITS><<<persistent_grid(unpack_single_kernel<T, ST, BITS>, kThreads, tasks), \
                                      kThreads, 0, s>>>(packed, (const ST*)scale, (const ST*)mn, (T*)out, N, G)
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
  if (N < 0 || G < 0 || (group_size != kGroup && !generic_group_ok(group_size))) return ACTNN_ERR_SHAPE;
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
  if (group_size != kGroup)
    return pack_single_generic(FUSED, data, mn, mx, bits, packed, scale, mn_out, mx_out, N, G, group_size, dtype,
                               stat_dtype, stochastic, noise, seed, offset, s);
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
  cudaStream_t s = (cudaStream_t)stream;
  if (group_size != kGroup)
    return unpack_single_generic(packed, bits, scale, mn, out, N, G, group_size, dtype, stat_dtype, s);
  if (!aligned(out, dtype == ACTNN_F32 ? 32 : 16) || !aligned(packed, 8)) return ACTNN_ERR_ALIGN;
  switch (dtype) {
    case ACTNN_F16: return launch_unpack<__half, __half>(bits, packed, scale, mn, out, N, G, s);
    case ACTNN_BF16: return launch_unpack<__nv_bfloat16, __nv_bfloat16>(bits, packed, scale, mn, out, N, G, s);
    default:
      if (stat_dtype == ACTNN_BF16) return launch_unpack<float, __nv_bfloat16>(bits, packed, scale, mn, out, N, G, s);
      return launch_unpack<float, float>(bits, packed, scale, mn, out, N, G, s);
  }
}
