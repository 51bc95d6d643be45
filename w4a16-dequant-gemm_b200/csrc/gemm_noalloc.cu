// w4b_gemm_w4_noalloc: the stream GEMM for callers that must not allocate.
//
// Who needs it: code that runs where cudaMalloc / cudaFree are off limits - a
// process whose memory pool has claimed the whole device (an allocation would
// simply fail), or a serving loop that forbids allocations and the implicit
// device synchronisation of cudaFree once warm-up is over. The regular entry
// (w4b_gemm_w4) grows library scratch with cudaMalloc on demand; this one keeps
// the stream kernel's scratch (the FP32 fragments of panels split between CTAs,
// their arrival counters, the arranged activations and a status word) in a fixed array that is part of the
// library image. Every device that loads the library holds those kNoAllocBytes
// until the process exits.
//
// Limits: only shapes the stream kernel serves (K % 512 == 0, N >= 64, group
// size 32 / 64 / 128, 16-byte aligned q / scales / x), and only sizes whose
// scratch fits the array. With passes = ceil(M / 16) and mt = 2 when a pass holds
// more than 8 rows, else 1:  passes * ceil(N / 64) * 4 counters <= 65,536;
// passes * min(units, SMs) * mt * 4096 bytes of fragments <= 3 MiB; and, unless
// the activation rows stay resident in shared memory (one or two rows of a few thousand activations),
// passes * (K / 512) * (8704 * mt + 256) bytes of arranged activations <= 1 MiB
// (e.g. M <= 16, K <= 28,672, N <= 1,000,000 fits). Anything else is rejected
// with W4B_INVALID and a message; nothing falls back to an allocating path.
//
// The first call on a device resolves the array's device address and clears the
// counters with a memset on the caller's stream; make that call before any
// stream capture. All calls share the one array, which keeps what the last call
// left in it: the kernel re-zeroes the counters it used, and calls whose kernels
// overlap on the GPU race on the array, exactly like concurrent calls of the
// regular entry race on the library scratch. A bounded wait that gave up inside
// this entry's kernel shows in w4b_device_status() like any other.
#include "../../include/w4b_abi.h"

#include <atomic>
#include <mutex>

#include "w4b_kernels.h"

namespace {

constexpr size_t kStatusBytes = 256;
constexpr size_t kCounterBytes = 256 * 1024;        // 65,536 per-tile arrival counters
constexpr size_t kFragmentBytes = 3 * 1024 * 1024;  // parked FP32 fragments
constexpr size_t kBlockBytes = 1024 * 1024;         // arranged activations (M > 1 or long K)
constexpr size_t kNoAllocBytes = kStatusBytes + kCounterBytes + kFragmentBytes + kBlockBytes;

// Host code sees only a stand-in for this symbol: its device address is taken
// with cudaGetSymbolAddress below, never with the & operator.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
std::atomic<unsigned char*> g_base[kMaxDevices];
std::mutex g_mu;

int fail(int code, const char* msg) {
  w4b::set_last_error(msg);  // read back through w4b_last_error()
  return code;
}

}  // namespace

extern "C" int w4b_gemm_w4_noalloc(const w4b_packed_w4* p, const void* x, void* c, int M, void* stream) {
  using namespace w4b;
  if (!p) return fail(W4B_INVALID, "gemm noalloc: null descriptor");
  if (p->N < 1 || p->K < 1) return fail(W4B_INVALID, "gemm noalloc: bad dims");
  if (p->gs < 8 || p->gs % 8 != 0) return fail(W4B_INVALID, "gemm noalloc: gs must be a multiple of 8");
  if (p->G != (p->K + p->gs - 1) / p->gs) return fail(W4B_INVALID, "gemm noalloc: G inconsistent with K, gs");
  if (!p->q || !p->scales || !x || !c) return fail(W4B_INVALID, "gemm noalloc: null pointer");
  if (!p->symmetric && !p->zeros) return fail(W4B_INVALID, "gemm noalloc: asymmetric without zeros");
  if (p->symmetric && p->zeros) return fail(W4B_INVALID, "gemm noalloc: symmetric carries no zeros");
  if (M < 1) return fail(W4B_INVALID, "gemm noalloc: bad M");
  if (!stream_gemm_supported(p->N, p->K, p->gs, p->q, p->scales, x))
    return fail(W4B_INVALID,
                "gemm noalloc: shape not served by the stream kernel (needs K % 512 == 0, N >= 64, "
                "gs in {32, 64, 128}, 16-byte aligned q / scales / x); use w4b_gemm_w4");

  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(W4B_CUDA, "gemm noalloc: cudaGetDevice failed");
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return fail(W4B_CUDA, "gemm noalloc: device attribute query failed");
  StreamPlan plan;
  stream_gemm_plan(p->N, p->K, M, p->gs, sms, &plan);
  if (plan.ws_bytes > kFragmentBytes)
    return fail(W4B_INVALID, "gemm noalloc: M too large for the fixed scratch (fragments exceed 3 MiB)");
  if (plan.xa_bytes > kBlockBytes)
    return fail(W4B_INVALID, "gemm noalloc: M * K too large for the fixed scratch (activation blocks exceed 1 MiB)");
  if (plan.counter_ints * sizeof(int) > kCounterBytes)
    return fail(W4B_INVALID, "gemm noalloc: N * passes too large for the fixed scratch (more than 65,536 tile counters)");

  int launches = 0;
  unsigned char* base = g_base[dev].load(std::memory_order_acquire);
  if (!base) {  // once per device, with that device current
    std::lock_guard<std::mutex> lk(g_mu);
    base = g_base[dev].load(std::memory_order_acquire);
    if (!base) {
      unsigned char* ptr = nullptr;
      const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
      if (e != cudaSuccess || !ptr) return fail(W4B_CUDA, "gemm noalloc: cudaGetSymbolAddress failed");
      // the counters (and the status word) must start at zero; the kernel re-zeroes what it uses. The clear is
      // ordered before the first kernel because it goes to the same stream.
      if (cudaMemsetAsync(ptr, 0, kStatusBytes + kCounterBytes, (cudaStream_t)stream) != cudaSuccess)
        return fail(W4B_CUDA, "gemm noalloc: clearing the counters failed");
      g_base[dev].store(ptr, std::memory_order_release);
      base = ptr;
    }
  }
  const cudaError_t e = stream_gemm_launch(
      p->symmetric ? 0 : 1, p->gs, p->q, p->scales, p->zeros, p->N, p->K, p->G, (const __half*)x, (__half*)c, M,
      nullptr, plan, (float*)(base + kStatusBytes + kCounterBytes), (int*)(base + kStatusBytes),
      base + kStatusBytes + kCounterBytes + kFragmentBytes, (int*)base, launch_overlap(), (cudaStream_t)stream, &launches);
  if (e != cudaSuccess) return fail(W4B_CUDA, cudaGetErrorString(e));
  count_launches(launches);
  return W4B_OK;
}

namespace w4b {
// For w4b_device_status(): the fixed array's status word and counter region on `dev`, once the entry has been
// used there (null before).
void noalloc_regions(int dev, int** status, void** counters, size_t* counter_bytes) {
  unsigned char* base = dev >= 0 && dev < kMaxDevices ? g_base[dev].load(std::memory_order_acquire) : nullptr;
  *status = (int*)base;
  *counters = base ? base + kStatusBytes : nullptr;
  *counter_bytes = kCounterBytes;
}
}  // namespace w4b
