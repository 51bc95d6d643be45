// w4b_gemm_w4_noalloc: the stream GEMM for callers that must not allocate.
//
// Who needs it: code that runs where cudaMalloc / cudaFree are off limits -
// inside a region being captured into a CUDA graph, inside a framework whose
// memory pool owns the whole device, or in a serving loop with a hard "no
// allocation, no implicit device synchronisation after warm-up" rule. The
// regular entry (w4b_gemm_w4) grows library scratch with cudaMalloc on demand;
// this one keeps the stream kernel's scratch (the FP32 fragments of panels split
// between CTAs, their arrival counters and the status word) in a fixed array
// that is part of the library image. Every device that loads the library holds
// those kNoAllocBytes until the process exits.
//
// Limits: only shapes the stream kernel serves (K % 256 == 0, N >= 64, group
// size 32 / 64 / 128, 16-byte aligned q / scales / x), and only sizes whose
// scratch fits the array (see the two checks below; e.g. M <= 16 with
// N <= 1,000,000 always fits on a 148-SM part). Anything else is rejected with
// W4B_INVALID and a message; nothing falls back to an allocating path.
//
// The first call on a device resolves the array's device address (and clears
// the counters once); make that call before any stream capture. All calls share
// the one array: calls whose kernels overlap on the GPU race on it, exactly like
// concurrent calls of the regular entry race on the library scratch.
#include "../../include/w4b_abi.h"

#include <mutex>

#include "w4b_kernels.h"

namespace {

constexpr size_t kStatusBytes = 256;
constexpr size_t kCounterBytes = 256 * 1024;        // 65,536 per-tile arrival counters
constexpr size_t kFragmentBytes = 3 * 1024 * 1024;  // parked FP32 fragments
constexpr size_t kNoAllocBytes = kStatusBytes + kCounterBytes + kFragmentBytes;

// Host code sees only a stand-in for this symbol: its device address is taken
// with cudaGetSymbolAddress below, never with the & operator.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_base[kMaxDevices];
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
                "gemm noalloc: shape not served by the stream kernel (needs K % 256 == 0, N >= 64, "
                "gs in {32, 64, 128}, 16-byte aligned q / scales / x); use w4b_gemm_w4");

  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(W4B_CUDA, "gemm noalloc: cudaGetDevice failed");
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return fail(W4B_CUDA, "gemm noalloc: device attribute query failed");
  StreamPlan plan;
  stream_gemm_plan(p->N, p->K, M, sms, &plan);
  if (plan.ws_bytes > kFragmentBytes)
    return fail(W4B_INVALID, "gemm noalloc: M too large for the fixed scratch (fragments exceed 3 MiB)");
  if (plan.counter_ints * sizeof(int) > kCounterBytes)
    return fail(W4B_INVALID, "gemm noalloc: N * passes too large for the fixed scratch (more than 65,536 tile counters)");

  if (!g_base[dev]) {  // once per device, with that device current
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_base[dev]) {
      unsigned char* ptr = nullptr;
      const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
      if (e != cudaSuccess || !ptr) return fail(W4B_CUDA, "gemm noalloc: cudaGetSymbolAddress failed");
      // the counters (and the status word) must start at zero; the kernel re-zeroes what it uses
      if (cudaMemset(ptr, 0, kStatusBytes + kCounterBytes) != cudaSuccess)
        return fail(W4B_CUDA, "gemm noalloc: clearing the counters failed");
      g_base[dev] = ptr;
    }
  }
  unsigned char* base = g_base[dev];
  const cudaError_t e = stream_gemm_launch(
      p->symmetric ? 0 : 1, p->gs, p->q, p->scales, p->zeros, p->N, p->K, p->G, (const __half*)x, (__half*)c, M,
      nullptr, plan, (float*)(base + kStatusBytes + kCounterBytes), (int*)(base + kStatusBytes), (int*)base,
      launch_overlap(), (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(W4B_CUDA, cudaGetErrorString(e));
  return W4B_OK;
}
