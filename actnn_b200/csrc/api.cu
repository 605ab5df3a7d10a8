// Status strings, cached device properties, launch checking and the noise export.
#include <atomic>
#include <mutex>

#include "quant_math.cuh"

namespace actnn {

const DeviceInfo& device_info() {
  // Immutable per-device facts, filled on first use.  Racing first calls write the same
  // values; the flag is published with release / acquire so that a reader that sees it set
  // also sees the value.
  static DeviceInfo info[64];
  static std::atomic<bool> ready[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!ready[dev].load(std::memory_order_acquire)) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    DeviceInfo fresh;
    fresh.sm_count = sms;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    if (!ready[dev].load(std::memory_order_relaxed)) {
      info[dev] = fresh;
      ready[dev].store(true, std::memory_order_release);
    }
  }
  return info[dev];
}

// Kernels that stage inputs with bulk copies bound every wait on an mbarrier; a wait that
// runs out adds one here and the warp stops.  Zero in every healthy run.
__device__ unsigned g_bulk_wait_gave_up;

unsigned* bulk_wait_counter() {
  static std::atomic<unsigned*> addr[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  unsigned* p = addr[dev].load(std::memory_order_acquire);
  if (!p) {
    void* q = nullptr;
    if (cudaGetSymbolAddress(&q, g_bulk_wait_gave_up) == cudaSuccess) {
      p = (unsigned*)q;
      addr[dev].store(p, std::memory_order_release);
    }
  }
  return p;
}

// cudaGetLastError also clears a launch error, so one refused launch does not fail every later call.
int check_launch() { return cudaGetLastError() == cudaSuccess ? ACTNN_OK : ACTNN_ERR_LAUNCH; }

// Resident blocks per SM of a kernel (by entry address) on the current device, asked of the
// occupancy calculator once and kept.  A first use with dynamic shared memory also raises
// the kernel's limit to that size.
int cached_blocks_per_sm(const void* kernel, int threads, int dynamic_smem) {
  struct Entry { const void* fn; int dev; int n; };
  static Entry table[512];
  static int used = 0;
  static std::mutex lock;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> guard(lock);
  for (int i = 0; i < used; ++i)
    if (table[i].fn == kernel && table[i].dev == dev) return table[i].n;
  int n = 0;
  if (dynamic_smem > 0) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic_smem);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, dynamic_smem) != cudaSuccess || n <= 0) n = 1;
  if (used < 512) table[used++] = Entry{kernel, dev, n};
  return n;
}

namespace {

// One thread per octet of the padded [N, G, 256] activation.
template <typename T>
__global__ void noise_fill_kernel(T* __restrict__ out, int64_t numel, const NoiseKey key) {
  const int64_t oct = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (oct * kOct >= numel) return;
  const uint64_t q = (uint64_t)(oct >> 5);        // 32 octets per 256-element group
  NoiseGen<T> gen(key, (int)(oct & 31));
  const Oct<T> nz = gen.get(q);
  const T* e = reinterpret_cast<const T*>(&nz);
  for (int j = 0; j < kOct && oct * kOct + j < numel; ++j) out[oct * kOct + j] = e[j];
}

}  // namespace
}  // namespace actnn

using namespace actnn;

extern "C" const char* actnn_status_string(int status) {
  switch (status) {
    case ACTNN_OK: return "ok";
    case ACTNN_ERR_NULL: return "a required pointer is NULL";
    case ACTNN_ERR_DTYPE: return "unsupported dtype (float32, float16 and bfloat16 are accepted; statistics must "
                                 "match the data dtype, or be bfloat16 for float32 data)";
    case ACTNN_ERR_SHAPE: return "invalid shape (negative size, overflow, or a group size other than 256; minimax "
                                 "needs cols % 32 == 0 and cols > 32)";
    case ACTNN_ERR_BITS: return "unsupported bit width (single precision: 1, 2, 4, 8; mixed precision: 1..8)";
    case ACTNN_ERR_ALIGN: return "pointer not aligned for vector access (16 bytes; 32 for float32 data)";
    case ACTNN_ERR_ARG: return "invalid argument";
    case ACTNN_ERR_LAUNCH: return "CUDA launch failed";
    case ACTNN_ERR_CAPACITY: return "problem exceeds a fixed internal capacity";
    default: return "unknown status";
  }
}

extern "C" int actnn_abi_version(void) { return 3; }

extern "C" int actnn_bulk_wait_failures(uint32_t* count) {
  if (!count) return ACTNN_ERR_NULL;
  unsigned* p = bulk_wait_counter();
  if (!p) return ACTNN_ERR_LAUNCH;
  return cudaMemcpy(count, p, sizeof(unsigned), cudaMemcpyDeviceToHost) == cudaSuccess ? ACTNN_OK : ACTNN_ERR_LAUNCH;
}

extern "C" int actnn_noise_fill(void* noise, int64_t numel, int dtype, uint64_t seed, uint64_t offset,
                                actnn_stream_t stream) {
  if (numel < 0) return ACTNN_ERR_SHAPE;
  if (numel == 0) return ACTNN_OK;
  if (!noise) return ACTNN_ERR_NULL;
  const int64_t octs = (numel + kOct - 1) / kOct;
  const unsigned grid = (unsigned)((octs + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  const NoiseKey key = make_noise_key(seed, offset);
  switch (dtype) {
    case ACTNN_F32: noise_fill_kernel<float><<<grid, 256, 0, s>>>((float*)noise, numel, key); break;
    case ACTNN_F16: noise_fill_kernel<__half><<<grid, 256, 0, s>>>((__half*)noise, numel, key); break;
    case ACTNN_BF16: noise_fill_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)noise, numel, key); break;
    default: return ACTNN_ERR_DTYPE;
  }
  return check_launch();
}
