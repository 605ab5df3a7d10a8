// The whole adaptive (per-sample bit width) compress of one activation behind one call:
// per-group min/max -> per-sample sensitivity -> greedy bit allocation -> scale, stochastic
// rounding and mixed-precision pack.  Three kernel launches on the caller's stream, no host
// synchronisation, no allocation: the per-group min / max that only live between the first
// and the last kernel go to a workspace the caller provides.
#include <atomic>

#include "quant_math.cuh"

using namespace actnn;

extern "C" int64_t actnn_compress_mixed_workspace(int64_t N, int64_t G, int dtype) {
  if (N < 0 || G < 0 || dtype < ACTNN_F32 || dtype > ACTNN_BF16) return -1;
  if (G && N > ((int64_t)1 << 52) / G) return -1;
  // min and max of every group in the activation dtype, each rounded up to 256 bytes, and 256
  // bytes for the ticket of the sensitivity / allocation kernel
  const int64_t one = (N * G * dtype_size(dtype) + 255) / 256 * 256;
  return 2 * one + 256;
}

extern "C" int actnn_compress_mixed(const void* data, int32_t* packed, void* scale, void* mn_out,
                                    int32_t* bits_out, int64_t* word_offsets_out, float* C_out, void* workspace,
                                    int64_t workspace_bytes, int64_t N, int64_t G, int64_t group_size, int dtype,
                                    int stat_dtype, float range_factor, float coeff, const float* grad_scale,
                                    int initial_bits, double target, int stochastic, const void* noise,
                                    uint64_t seed, uint64_t offset, actnn_stream_t stream) {
  if (N < 0 || G < 0 || (group_size != kGroup && !generic_group_ok(group_size))) return ACTNN_ERR_SHAPE;
  if (dtype < ACTNN_F32 || dtype > ACTNN_BF16) return ACTNN_ERR_DTYPE;
  if (initial_bits < 1 || initial_bits > 8) return ACTNN_ERR_BITS;
  if (N == 0 || G == 0) return ACTNN_OK;
  if (!data || !packed || !scale || !mn_out || !bits_out || !word_offsets_out || !C_out || !workspace)
    return ACTNN_ERR_NULL;
  const int64_t need = actnn_compress_mixed_workspace(N, G, dtype);
  if (workspace_bytes < need) return ACTNN_ERR_CAPACITY;
  if (!aligned(workspace, 256)) return ACTNN_ERR_ALIGN;
  const int64_t one = (need - 256) / 2;
  void* mn = workspace;
  void* mx = (char*)workspace + one;
  unsigned* ticket = (unsigned*)((char*)workspace + 2 * one);
  cudaStream_t s = (cudaStream_t)stream;
  const bool fused_alloc = range_greedy_supported(N, initial_bits);
  // pass 1 walks the activation from its end to its start, pass 2 (the pack) from the start:
  // what the first pass read last is what the second finds in the L2
  int st = minimax_impl(data, mn, mx, N * G, group_size, dtype, 1, fused_alloc ? ticket : nullptr, s);
  if (st) return st;
  if (fused_alloc) {
    st = range_greedy_impl(mn, mx, N, G, dtype, range_factor, coeff, grad_scale, C_out, ticket, initial_bits, target,
                           bits_out, word_offsets_out, group_size, s);
    if (st) return st;
  } else {
    st = actnn_range_sqr(mn, mx, N, G, dtype, range_factor, coeff, grad_scale, C_out, stream);
    if (st) return st;
    st = actnn_calc_precision(C_out, nullptr, N, initial_bits, target, bits_out, word_offsets_out, G, group_size,
                              nullptr, 0, stream);
    if (st) return st;
  }
  return pack_mixed_impl(data, mn, mx, bits_out, word_offsets_out, packed, scale, mn_out, N, G, group_size, dtype,
                         stat_dtype, stochastic, noise, seed, offset, true, (cudaStream_t)stream);
}

// The same compress when the per-group min / max already exist (actnn_batch_norm_stats_minimax
// produces them in the pass that computes the batch-norm statistics): sensitivities + greedy
// allocation, then the pack.  `ticket_workspace`: 256 bytes, 256-byte aligned.
static int compress_prestat(const void* data, const void* mn, const void* mx, int32_t* packed, void* scale,
                            void* mn_out, int32_t* bits_out, int64_t* word_offsets_out, float* C_out,
                            void* ticket_workspace, int64_t N, int64_t G, int64_t group_size, int dtype,
                            int stat_dtype, float range_factor, float coeff, const float* grad_scale,
                            int initial_bits, double target, int stochastic, const void* noise, uint64_t seed,
                            uint64_t offset, actnn_stream_t stream, bool clear_ticket) {
  if (N < 0 || G < 0 || (group_size != kGroup && !generic_group_ok(group_size))) return ACTNN_ERR_SHAPE;
  if (dtype < ACTNN_F32 || dtype > ACTNN_BF16) return ACTNN_ERR_DTYPE;
  if (initial_bits < 1 || initial_bits > 8) return ACTNN_ERR_BITS;
  if (N == 0 || G == 0) return ACTNN_OK;
  if (!data || !mn || !mx || !packed || !scale || !mn_out || !bits_out || !word_offsets_out || !C_out ||
      !ticket_workspace)
    return ACTNN_ERR_NULL;
  if (!aligned(ticket_workspace, 256)) return ACTNN_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  int st;
  if (range_greedy_supported(N, initial_bits)) {
    if (clear_ticket && cudaMemsetAsync(ticket_workspace, 0, sizeof(unsigned), s) != cudaSuccess)
      return ACTNN_ERR_LAUNCH;
    st = range_greedy_impl(mn, mx, N, G, dtype, range_factor, coeff, grad_scale, C_out, (unsigned*)ticket_workspace,
                           initial_bits, target, bits_out, word_offsets_out, group_size, s);
    if (st) return st;
  } else {
    st = actnn_range_sqr(mn, mx, N, G, dtype, range_factor, coeff, grad_scale, C_out, stream);
    if (st) return st;
    st = actnn_calc_precision(C_out, nullptr, N, initial_bits, target, bits_out, word_offsets_out, G, group_size,
                              nullptr, 0, stream);
    if (st) return st;
  }
  return pack_mixed_impl(data, mn, mx, bits_out, word_offsets_out, packed, scale, mn_out, N, G, group_size, dtype,
                         stat_dtype, stochastic, noise, seed, offset, true, s);
}

extern "C" int actnn_compress_mixed_prestat(const void* data, const void* mn, const void* mx, int32_t* packed,
                                            void* scale, void* mn_out, int32_t* bits_out, int64_t* word_offsets_out,
                                            float* C_out, void* ticket_workspace, int64_t N, int64_t G,
                                            int64_t group_size, int dtype, int stat_dtype, float range_factor,
                                            float coeff, const float* grad_scale, int initial_bits, double target,
                                            int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                                            actnn_stream_t stream) {
  return compress_prestat(data, mn, mx, packed, scale, mn_out, bits_out, word_offsets_out, C_out, ticket_workspace, N,
                          G, group_size, dtype, stat_dtype, range_factor, coeff, grad_scale, initial_bits, target,
                          stochastic, noise, seed, offset, stream, true);
}

// The same with a ticket word the caller keeps for this purpose only: zero before the first call
// (one cudaMemset when it is allocated), left at zero by every call (the block that takes the last
// ticket resets it), never touched by anything else, used by one stream at a time.  Saves the
// per-call clear: one memory operation less in the stream of every layer.
extern "C" int actnn_compress_mixed_prestat_kept(const void* data, const void* mn, const void* mx, int32_t* packed,
                                                 void* scale, void* mn_out, int32_t* bits_out,
                                                 int64_t* word_offsets_out, float* C_out, void* ticket_workspace,
                                                 int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype,
                                                 float range_factor, float coeff, const float* grad_scale,
                                                 int initial_bits, double target, int stochastic, const void* noise,
                                                 uint64_t seed, uint64_t offset, actnn_stream_t stream) {
  return compress_prestat(data, mn, mx, packed, scale, mn_out, bits_out, word_offsets_out, C_out, ticket_workspace, N,
                          G, group_size, dtype, stat_dtype, range_factor, coeff, grad_scale, initial_bits, target,
                          stochastic, noise, seed, offset, stream, false);
}

// ------------------------------------------------------------------------------------------
// The same compress for callers that have no way to provide scratch memory.
//
// Some users of this library only ever hold pointers that somebody else handed to them: a
// plug-in inside a host framework that owns every byte of device memory and exposes no
// allocator to it, or a job whose device memory was carved up in advance by a memory plan
// so that any further cudaMalloc may fail or disturb the plan.  For them the per-group
// min / max that live between the four kernels go to a fixed array inside the library
// instead of a caller workspace.  The price: the array (kStaticScratchBytes) is resident on
// every GPU that loads the library until the process exits, and the problem size is capped.
namespace {

// 4 MiB of min / max (N * G <= 1 Mi groups of 16-bit data) and the 256-byte ticket block
constexpr int64_t kStaticScratchBytes = (4 << 20) + 256;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device, looked up once per device.  In
// host code the array's name is only a handle, not an address a kernel could use.
int static_scratch_address(void** out) {
  // one slot per device; the address is published with release / acquire so that a thread
  // that sees it set also sees a complete value (the look-up itself is idempotent)
  static std::atomic<void*> addr[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return ACTNN_ERR_ARG;
  void* p = addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return ACTNN_ERR_LAUNCH;
    addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return ACTNN_OK;
}

}  // namespace

extern "C" int64_t actnn_compress_mixed_static_capacity(void) { return kStaticScratchBytes; }

extern "C" int actnn_compress_mixed_static(const void* data, int32_t* packed, void* scale, void* mn_out,
                                           int32_t* bits_out, int64_t* word_offsets_out, float* C_out, int64_t N,
                                           int64_t G, int64_t group_size, int dtype, int stat_dtype,
                                           float range_factor, float coeff, const float* grad_scale,
                                           int initial_bits, double target, int stochastic, const void* noise,
                                           uint64_t seed, uint64_t offset, actnn_stream_t stream) {
  const int64_t need = actnn_compress_mixed_workspace(N, G, dtype);
  if (need < 0) return (N < 0 || G < 0) ? ACTNN_ERR_SHAPE : ACTNN_ERR_DTYPE;
  if (need > kStaticScratchBytes) return ACTNN_ERR_CAPACITY;
  void* scratch = nullptr;
  if (int st = static_scratch_address(&scratch)) return st;
  return actnn_compress_mixed(data, packed, scale, mn_out, bits_out, word_offsets_out, C_out, scratch,
                              kStaticScratchBytes, N, G, group_size, dtype, stat_dtype, range_factor, coeff,
                              grad_scale, initial_bits, target, stochastic, noise, seed, offset, stream);
}
