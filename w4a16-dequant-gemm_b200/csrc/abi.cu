// The C ABI of libw4b200 (include/w4b_abi.h): argument validation with the
// reference's reject-before-touching contract, per-device scratch, routing
// between the kernels, and error reporting. No kernel lives in this file.
#include "../../include/w4b_abi.h"

#include <limits.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "w4b_kernels.h"

namespace {

using namespace w4b;

thread_local char g_err[512] = "";
std::atomic<unsigned long long> g_launches{0};
std::atomic<int> g_overlap{0};  // w4b_set_launch_overlap

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(W4B_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define INVALID(...) return fail(W4B_INVALID, __VA_ARGS__)
#define CUDA_TRY(expr, what)                         \
  do {                                               \
    const cudaError_t e_ = (expr);                   \
    if (e_ != cudaSuccess) return cuda_fail(e_, what); \
  } while (0)

// The crossover between the stream kernel and the tensor kernel under
// W4B_PATH_AUTO (the reference's DISPATCH_MMA_MIN_M, include/w4/dispatch.cuh:25).
constexpr int kMmaMinM = 17;

// Grow-only device buffer. Like the reference's function-static scratch
// (include/w4/fused.cuh:55-66) it is shared by all calls on a device.
struct Scratch {
  void* ptr = nullptr;
  size_t cap = 0;
  // Grows to at least `bytes`; `zero` clears a newly allocated buffer.
  cudaError_t reserve(size_t bytes, bool zero) {
    if (bytes <= cap) return cudaSuccess;
    void* nb = nullptr;
    size_t want = bytes < 4096 ? 4096 : bytes;
    cudaError_t e = cudaMalloc(&nb, want);
    if (e != cudaSuccess) return e;
    if (zero) {
      e = cudaMemset(nb, 0, want);
      if (e != cudaSuccess) {
        cudaFree(nb);
        return e;
      }
    }
    if (ptr) cudaFree(ptr);  // implicit device synchronisation: no kernel still uses it
    ptr = nb;
    cap = want;
    return cudaSuccess;
  }
};

struct DeviceCtx {
  bool ready = false;
  int sm_count = 0;
  int* status = nullptr;  // device status word written by bounded waits
  Scratch gemm_ws;        // FP32 partial fragments of split panels
  Scratch gemm_counters;  // arrival counters, zero between launches
  Scratch gemm_xa;        // arranged activations of the stream GEMM's streamed form
  Scratch tensor_counters;  // per-tile arrival counters of the tensor GEMM's split-K form, zero between launches
  Scratch attn_ws;        // (m, l, acc[D]) partials of split sequences
  Scratch io_x, io_c;     // device staging of the host-buffer entry
  Scratch gemm_xpad;      // zero-padded activation rows of the padded-K entries
};

constexpr int kMaxDevices = 64;
DeviceCtx g_ctx[kMaxDevices];
std::mutex g_mu;

int get_ctx(DeviceCtx** out) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return fail(W4B_CUDA, "device index %d out of range", dev);
  DeviceCtx& c = g_ctx[dev];
  if (!c.ready) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!c.ready) {
      CUDA_TRY(cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev), "device attribute");
      int major = 0;
      CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev), "device attribute");
      if (major != 10)
        return fail(W4B_CUDA, "libw4b200 is built for sm_100a only; device %d has compute capability %d.x", dev,
                    major);
      CUDA_TRY(cudaMalloc((void**)&c.status, sizeof(int)), "status word");
      CUDA_TRY(cudaMemset(c.status, 0, sizeof(int)), "status word");
      c.ready = true;
    }
  }
  *out = &c;
  return W4B_OK;
}

// ---- validation, in the reference's order (fused.cuh:175-193, mma.cuh:237-254) ----

int check_w4(const w4b_packed_w4* p, const char* who) {
  if (!p) INVALID("%s: null descriptor", who);
  if (p->N < 1 || p->K < 1) INVALID("%s: bad dims", who);
  if (p->gs < 8 || p->gs % 8 != 0) INVALID("%s: gs must be a multiple of 8", who);
  if (p->G != (p->K + p->gs - 1) / p->gs) INVALID("%s: G inconsistent with K, gs", who);
  if (!p->q || !p->scales) INVALID("%s: null pointer", who);
  if (!p->symmetric && !p->zeros) INVALID("%s: asymmetric without zeros", who);
  if (p->symmetric && p->zeros) INVALID("%s: symmetric carries no zeros", who);
  return W4B_OK;
}

int check_mx(const w4b_packed_mx* p, const char* who) {  // mxfused.cuh:32-37
  if (!p) INVALID("%s: null descriptor", who);
  if (p->N < 1 || p->K < 1) INVALID("%s: bad dims", who);
  if (p->B != (p->K + 31) / 32) INVALID("%s: B inconsistent with K", who);
  if (!p->q || !p->scales) INVALID("%s: null pointer", who);
  return W4B_OK;
}

// Which reference entry's launch bounds apply to a call (fused vs mma) and
// which kernel serves it.
int resolve_path(int path, int M) {
  if (path == W4B_PATH_AUTO) return M < kMmaMinM ? W4B_PATH_STREAM : W4B_PATH_TENSOR;
  return path;
}

int check_gemm_bounds(int N, int M, int entry, const char* who) {
  if (M < 1) INVALID("%s: bad M", who);
  if (entry == W4B_PATH_TENSOR) {  // mma.cuh:252-254
    if (M > 65535 * 64 || N > INT_MAX - 64) INVALID("%s: launch grid out of range", who);
  } else {  // fused.cuh:187-194
    const int mtile = M <= 1 ? 1 : (M <= 2 ? 2 : 4);
    const int rpw = M <= 4 ? 1 : 4;
    if (M > 65535 * mtile || N > INT_MAX - 8 * rpw) INVALID("%s: launch grid out of range", who);
  }
  return W4B_OK;
}

// Chooses the kernel: the requested one when the shape fits it, else the other fast
// kernel, else generic. `w_out` matters because the tensor kernel's hook stores 16 bytes.
int route_kernel(int entry, int N, int K, int gs_or_0, const void* q, const void* scales, const void* x,
                 const void* w_out = nullptr) {
  if (entry == W4B_PATH_GENERIC) return W4B_PATH_GENERIC;
  const bool tensor_ok = tensor_gemm_supported(N, K, q, x) && (((uintptr_t)w_out & 15u) == 0);
  const bool stream_ok = stream_gemm_supported(N, K, gs_or_0, q, scales, x);
  if (entry == W4B_PATH_TENSOR) return tensor_ok ? W4B_PATH_TENSOR : (stream_ok ? W4B_PATH_STREAM : W4B_PATH_GENERIC);
  return stream_ok ? W4B_PATH_STREAM : W4B_PATH_GENERIC;
}

int run_gemm(int fmt, int gs, const uint32_t* q, const void* scales, const uint32_t* zeros, int N, int K, int G,
             const void* x, void* c, int M, int entry, cudaStream_t stream, void* w_out, const char* who,
             const StreamPeers* peers = nullptr) {
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  const int kernel = route_kernel(entry, N, K, fmt == 2 ? 0 : gs, q, scales, x, w_out);
  if (peers && kernel != W4B_PATH_STREAM)
    return fail(W4B_INVALID, "%s: the exchange form needs a shape of the stream kernel (K %% 512 == 0, N >= 64, gs 32/64/128, "
                "16-byte aligned q / scales / x)", who);
  if (kernel == W4B_PATH_TENSOR) {
    TensorPlan tplan;
    tensor_gemm_plan(N, K, M, ctx->sm_count, &tplan);
    CUDA_TRY(ctx->gemm_ws.reserve(tplan.ws_bytes, false), "gemm workspace");
    CUDA_TRY(ctx->tensor_counters.reserve(tplan.counter_ints * sizeof(int), true), "gemm counters");
    CUDA_TRY(tensor_gemm_launch(fmt, gs, q, scales, zeros, N, K, G, (const __half*)x, (__half*)c, M, (__half*)w_out,
                                tplan, (float*)ctx->gemm_ws.ptr, (int*)ctx->tensor_counters.ptr, ctx->status, stream),
             who);
    g_launches += 1;
    return W4B_OK;
  }
  if (kernel == W4B_PATH_STREAM) {
    StreamPlan plan;
    stream_gemm_plan(N, K, M, fmt == 2 ? 0 : gs, ctx->sm_count, &plan);
    CUDA_TRY(ctx->gemm_ws.reserve(plan.ws_bytes, false), "gemm workspace");
    CUDA_TRY(ctx->gemm_counters.reserve(plan.counter_ints * sizeof(int), true), "gemm counters");
    CUDA_TRY(ctx->gemm_xa.reserve(plan.xa_bytes, false), "gemm activation blocks");
    int launches = 0;
    CUDA_TRY(stream_gemm_launch(fmt, gs, q, scales, zeros, N, K, G, (const __half*)x, (__half*)c, M,
                                (__half*)w_out, plan, (float*)ctx->gemm_ws.ptr, (int*)ctx->gemm_counters.ptr,
                                ctx->gemm_xa.ptr, ctx->status, g_overlap.load() != 0, stream, &launches, peers),
             who);
    g_launches += (unsigned long long)launches;
    return W4B_OK;
  }
  CUDA_TRY(generic_gemm_launch(fmt, gs, q, scales, zeros, N, K, G, (const __half*)x, (__half*)c, M,
                               (__half*)w_out, stream),
           who);
  g_launches += 1;
  return W4B_OK;
}

}  // namespace

namespace w4b {
void set_last_error(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }
bool launch_overlap() { return g_overlap.load() != 0; }
void count_launches(int n) { g_launches += (unsigned long long)n; }
}  // namespace w4b

extern "C" {

const char* w4b_last_error(void) { return g_err; }

int w4b_dispatch_mma_min_m(void) { return kMmaMinM; }

unsigned long long w4b_launch_count(void) { return g_launches.load(); }

int w4b_set_launch_overlap(int on) { return g_overlap.exchange(on ? 1 : 0); }

int w4b_launch_overlap(void) { return g_overlap.load(); }

int w4b_device_status(void) {
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return -rc;
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cuda_fail(cudaGetLastError(), "cudaDeviceSynchronize");
    return -W4B_CUDA;
  }
  int st = 0;
  if (cudaMemcpy(&st, ctx->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -W4B_CUDA;
  // the no-allocation entry keeps its own status word (and counters) in its fixed array
  int dev = 0, st2 = 0;
  int* na_status = nullptr;
  void* na_counters = nullptr;
  size_t na_bytes = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) noalloc_regions(dev, &na_status, &na_counters, &na_bytes);
  if (na_status && cudaMemcpy(&st2, na_status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -W4B_CUDA;
  if (st != 0 || st2 != 0) {
    // A kernel that gave up may have left arrival counters behind: clear them, or every later launch that
    // shares a panel between CTAs would take stale fragments for fresh ones.
    cudaMemset(ctx->status, 0, sizeof(int));
    if (ctx->gemm_counters.ptr) cudaMemset(ctx->gemm_counters.ptr, 0, ctx->gemm_counters.cap);
    if (ctx->tensor_counters.ptr) cudaMemset(ctx->tensor_counters.ptr, 0, ctx->tensor_counters.cap);
    if (na_status) {
      cudaMemset(na_status, 0, sizeof(int));
      cudaMemset(na_counters, 0, na_bytes);
    }
  }
  return st != 0 ? st : st2;
}

int w4b_gemm_w4_route(const w4b_packed_w4* p, int M, int path, const void* x) {
  if (check_w4(p, "route") || M < 1) return -1;
  return route_kernel(resolve_path(path, M), p->N, p->K, p->gs, p->q, p->scales, x);
}

int w4b_gemm_mx_route(const w4b_packed_mx* p, int M, int path, const void* x) {
  if (check_mx(p, "route") || M < 1) return -1;
  return route_kernel(resolve_path(path, M), p->N, p->K, 0, p->q, p->scales, x);
}

int w4b_gemm_w4(const w4b_packed_w4* p, const void* x, void* c, int M, int path, void* stream, void* w_out) {
  if (path < W4B_PATH_AUTO || path > W4B_PATH_GENERIC) INVALID("gemm: unknown path %d", path);
  if (int rc = check_w4(p, "gemm")) return rc;
  if (!x || !c) INVALID("gemm: null pointer");
  if (M < 1) INVALID("gemm: bad M");
  const int entry = resolve_path(path, M);
  if (int rc = check_gemm_bounds(p->N, M, entry, "gemm")) return rc;
  return run_gemm(p->symmetric ? 0 : 1, p->gs, p->q, p->scales, p->zeros, p->N, p->K, p->G, x, c, M, entry,
                  (cudaStream_t)stream, w_out, "gemm kernel");
}

int w4b_gemm_mx(const w4b_packed_mx* p, const void* x, void* c, int M, int path, void* stream, void* w_out) {
  if (path < W4B_PATH_AUTO || path > W4B_PATH_GENERIC) INVALID("gemm_mx: unknown path %d", path);
  if (int rc = check_mx(p, "gemm_mx")) return rc;
  if (!x || !c) INVALID("gemm_mx: null pointer");
  if (M < 1) INVALID("gemm_mx: bad M");
  const int entry = resolve_path(path, M);
  if (int rc = check_gemm_bounds(p->N, M, entry, "gemm_mx")) return rc;
  return run_gemm(2, 32, p->q, p->scales, nullptr, p->N, p->K, p->B, x, c, M, entry, (cudaStream_t)stream, w_out,
                  "gemm_mx kernel");
}

int w4b_gemm_w4_hostio(const w4b_packed_w4* p, const void* x_host, void* c_host, int M, int path, void* stream) {
  if (path < W4B_PATH_AUTO || path > W4B_PATH_GENERIC) INVALID("gemm hostio: unknown path %d", path);
  if (int rc = check_w4(p, "gemm hostio")) return rc;
  if (!x_host || !c_host) INVALID("gemm hostio: null pointer");
  if (M < 1) INVALID("gemm hostio: bad M");
  const int entry = resolve_path(path, M);
  if (int rc = check_gemm_bounds(p->N, M, entry, "gemm hostio")) return rc;
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  const size_t xb = (size_t)M * p->K * sizeof(__half), cb = (size_t)M * p->N * sizeof(__half);
  CUDA_TRY(ctx->io_x.reserve(xb, false), "hostio x staging");
  // A page-locked output buffer is written by the kernel itself (every CTA stores its slice of c
  // straight over PCIe); pageable memory goes through a device staging buffer and a copy.
  void* c_dev = nullptr;
  {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, c_host) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer)
      c_dev = at.devicePointer;
    else
      (void)cudaGetLastError();
  }
  const bool direct = c_dev != nullptr;
  if (!direct) {
    CUDA_TRY(ctx->io_c.reserve(cb, false), "hostio c staging");
    c_dev = ctx->io_c.ptr;
  }
  cudaStream_t st = (cudaStream_t)stream;
  CUDA_TRY(cudaMemcpyAsync(ctx->io_x.ptr, x_host, xb, cudaMemcpyHostToDevice, st), "hostio h2d");
  if (int rc = run_gemm(p->symmetric ? 0 : 1, p->gs, p->q, p->scales, p->zeros, p->N, p->K, p->G, ctx->io_x.ptr, c_dev,
                        M, entry, st, nullptr, "gemm kernel"))
    return rc;
  if (!direct) CUDA_TRY(cudaMemcpyAsync(c_host, c_dev, cb, cudaMemcpyDeviceToHost, st), "hostio d2h");
  CUDA_TRY(cudaStreamSynchronize(st), "hostio sync");
  return W4B_OK;
}

int w4b_dequant_w4(const w4b_packed_w4* p, void* w, void* stream) {
  // dequant.cuh:62-82 (null check precedes the mode checks there)
  if (!p) INVALID("dequant: null descriptor");
  if (p->N < 1 || p->K < 1) INVALID("dequant: bad dims");
  if (p->gs < 8 || p->gs % 8 != 0) INVALID("dequant: gs must be a multiple of 8");
  if (p->G != (p->K + p->gs - 1) / p->gs) INVALID("dequant: G inconsistent with K, gs");
  if (!p->q || !p->scales || !w) INVALID("dequant: null pointer");
  if (!p->symmetric && !p->zeros) INVALID("dequant: asymmetric without zeros");
  if (p->symmetric && p->zeros) INVALID("dequant: symmetric carries no zeros");
  if ((long long)p->N * words(p->K) >= (1LL << 31)) INVALID("dequant: N*words(K) exceeds 2^31");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  CUDA_TRY(dequant_w4_launch(p->q, (const __half*)p->scales, p->zeros, p->N, p->K, p->gs, p->G, p->symmetric,
                             (__half*)w, (cudaStream_t)stream),
           "dequant kernel");
  g_launches += 1;
  return W4B_OK;
}

int w4b_dequant_mx(const w4b_packed_mx* p, void* w, void* stream) {
  if (int rc = check_mx(p, "mx dequant")) return rc;  // mxfused.cuh:57-69
  if (!w) INVALID("mx dequant: null output");
  if ((long long)p->N * words(p->K) >= (1LL << 31)) INVALID("mx dequant: N*words(K) exceeds 2^31");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  CUDA_TRY(dequant_mx_launch(p->q, p->scales, p->N, p->K, p->B, (__half*)w, (cudaStream_t)stream),
           "mx dequant kernel");
  g_launches += 1;
  return W4B_OK;
}

int w4b_dequant_f8(const uint8_t* q, const uint16_t* s, void* w, int S, int D, int gs, void* stream) {
  // kvflash.cuh:435-457
  if (S < 1 || D < 1) INVALID("f8 dequant: bad dims");
  if (gs < 8 || gs % 8 != 0) INVALID("f8 dequant: gs must be a multiple of 8");
  if (!q || !s || !w) INVALID("f8 dequant: null pointer");
  if ((long long)S * ((D + 3) / 4) >= (1LL << 31)) INVALID("f8 dequant: S*words4(D) exceeds 2^31");
  if (D % 4 != 0) INVALID("f8 dequant: D must be a multiple of 4");
  if ((uintptr_t)q % 4 != 0) INVALID("f8 dequant: q must be 4-byte aligned");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  CUDA_TRY(dequant_f8_launch(q, (const __half*)s, (__half*)w, S, D, gs, (cudaStream_t)stream), "f8 dequant kernel");
  g_launches += 1;
  return W4B_OK;
}

// ---- device-side quantizers and KV append (no device counterpart in the reference) ------------

int w4b_quantize_w4(const void* w, int w_is_f16, int N, int K, int gs, int symmetric, uint32_t* q, uint16_t* scales,
                    uint32_t* zeros, void* stream) {
  // the host quantizer's shape contract (pack.hpp:66-75)
  if (N < 1 || K < 1) INVALID("quantize: bad dims");
  if (gs < 8 || gs % 8 != 0) INVALID("quantize: gs must be a multiple of 8");
  if (!w || !q || !scales) INVALID("quantize: null pointer");
  if (!symmetric && !zeros) INVALID("quantize: asymmetric without zeros");
  if (symmetric && zeros) INVALID("quantize: symmetric carries no zeros");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  CUDA_TRY(quantize_w4_launch(w, w_is_f16, N, K, gs, symmetric ? 1 : 0, 1, 0, q, (__half*)scales, zeros, ctx->status,
                              (cudaStream_t)stream),
           "quantize kernel");
  g_launches += 1;
  return W4B_OK;
}

int w4b_quantize_mx(const void* w, int w_is_f16, int N, int K, uint32_t* q, uint8_t* scales, void* stream) {
  if (N < 1 || K < 1) INVALID("quantize_mx: bad dims");  // mx.hpp:73-77
  if (!w || !q || !scales) INVALID("quantize_mx: null pointer");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  CUDA_TRY(quantize_mx_launch(w, w_is_f16, N, K, q, scales, ctx->status, (cudaStream_t)stream), "quantize_mx kernel");
  g_launches += 1;
  return W4B_OK;
}

int w4b_quantize_f8(const void* x, int x_is_f16, int rows, int D, int gs, uint8_t* q, uint16_t* scales, void* stream) {
  if (rows < 1 || D < 1) INVALID("quantize_f8: bad dims");  // kvfp8.hpp:72-80
  if (gs < 8 || gs % 8 != 0) INVALID("quantize_f8: gs must be a multiple of 8");
  if (!x || !q || !scales) INVALID("quantize_f8: null pointer");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  CUDA_TRY(quantize_f8_launch(x, x_is_f16, rows, D, gs, 1, 0, q, (__half*)scales, ctx->status, (cudaStream_t)stream),
           "quantize_f8 kernel");
  g_launches += 1;
  return W4B_OK;
}

int w4b_kv_append_w4(const w4b_kv_w4* p, long long row, long long slab_rows, const void* k_new, const void* v_new,
                     int new_is_f16, void* stream) {
  if (!p) INVALID("kv append: null descriptor");
  if (p->H < 1 || p->D < 1) INVALID("kv append: bad dims");
  if (p->gs < 8 || p->gs % 8 != 0) INVALID("kv append: gs must be a multiple of 8");
  if (p->G != (p->D + p->gs - 1) / p->gs) INVALID("kv append: G inconsistent with D, gs");
  if (!p->q_k || !p->s_k || !p->q_v || !p->s_v || !k_new || !v_new) INVALID("kv append: null pointer");
  if (!p->symmetric && (!p->z_k || !p->z_v)) INVALID("kv append: asymmetric without zeros");
  if (p->symmetric && (p->z_k || p->z_v)) INVALID("kv append: symmetric carries zeros");
  if (slab_rows < 1 || row < 0 || row >= slab_rows) INVALID("kv append: row outside the head slab");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  const int sym = p->symmetric ? 1 : 0;
  CUDA_TRY(quantize_w4_launch(k_new, new_is_f16, p->H, p->D, p->gs, sym, slab_rows, row, (uint32_t*)p->q_k, (__half*)p->s_k,
                              (uint32_t*)p->z_k, ctx->status, (cudaStream_t)stream),
           "kv append kernel");
  CUDA_TRY(quantize_w4_launch(v_new, new_is_f16, p->H, p->D, p->gs, sym, slab_rows, row, (uint32_t*)p->q_v, (__half*)p->s_v,
                              (uint32_t*)p->z_v, ctx->status, (cudaStream_t)stream),
           "kv append kernel");
  g_launches += 2;
  return W4B_OK;
}

int w4b_kv_append_f8(const w4b_kv_f8* p, long long row, const void* k_new, const void* v_new, int new_is_f16,
                     void* stream) {
  if (!p) INVALID("kv f8 append: null descriptor");
  if (p->H < 1 || p->S < 1 || p->D < 1) INVALID("kv f8 append: bad dims");
  if (p->gs < 8 || p->gs % 8 != 0) INVALID("kv f8 append: gs must be a multiple of 8");
  if (p->G != (p->D + p->gs - 1) / p->gs) INVALID("kv f8 append: G inconsistent with D, gs");
  if (!p->q_k || !p->s_k || !p->q_v || !p->s_v || !k_new || !v_new) INVALID("kv f8 append: null pointer");
  if (row < 0 || row >= p->S) INVALID("kv f8 append: row outside the head slab");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  CUDA_TRY(quantize_f8_launch(k_new, new_is_f16, p->H, p->D, p->gs, p->S, row, (uint8_t*)p->q_k, (__half*)p->s_k, ctx->status,
                              (cudaStream_t)stream),
           "kv f8 append kernel");
  CUDA_TRY(quantize_f8_launch(v_new, new_is_f16, p->H, p->D, p->gs, p->S, row, (uint8_t*)p->q_v, (__half*)p->s_v, ctx->status,
                              (cudaStream_t)stream),
           "kv f8 append kernel");
  g_launches += 2;
  return W4B_OK;
}

// ---- offline re-layout: the matrix zero-extended along K (no counterpart in the reference) ----

int w4b_relayout_k(int K) {
  if (K < 1 || K > INT_MAX - 511) return -1;
  return (K + 511) / 512 * 512;
}

int w4b_relayout_w4(const w4b_packed_w4* src, const w4b_packed_w4* dst, void* stream) {
  if (int rc = check_w4(src, "relayout source")) return rc;
  if (int rc = check_w4(dst, "relayout destination")) return rc;
  if (dst->N != src->N || dst->gs != src->gs || (dst->symmetric != 0) != (src->symmetric != 0))
    INVALID("relayout: the destination must keep N, gs and the mode of the source");
  if (dst->K < src->K) INVALID("relayout: destination K %d below the source's %d", dst->K, src->K);
  if (dst->q == src->q || dst->scales == src->scales || (dst->zeros && dst->zeros == src->zeros))
    INVALID("relayout: in place is not supported");
  int launches = 0;
  CUDA_TRY(relayout_launch(src->symmetric ? 0 : 1, src->gs, src->q, src->scales, src->zeros, src->N, src->K, src->G,
                           (uint32_t*)dst->q, (void*)dst->scales, (uint32_t*)dst->zeros, dst->K, dst->G,
                           (cudaStream_t)stream, &launches),
           "relayout kernel");
  g_launches += (unsigned long long)launches;
  return W4B_OK;
}

int w4b_relayout_mx(const w4b_packed_mx* src, const w4b_packed_mx* dst, void* stream) {
  if (int rc = check_mx(src, "relayout_mx source")) return rc;
  if (int rc = check_mx(dst, "relayout_mx destination")) return rc;
  if (dst->N != src->N) INVALID("relayout_mx: the destination must keep N");
  if (dst->K < src->K) INVALID("relayout_mx: destination K %d below the source's %d", dst->K, src->K);
  if (dst->q == src->q || dst->scales == src->scales) INVALID("relayout_mx: in place is not supported");
  int launches = 0;
  CUDA_TRY(relayout_launch(2, 32, src->q, src->scales, nullptr, src->N, src->K, src->B, (uint32_t*)dst->q,
                           (void*)dst->scales, nullptr, dst->K, dst->B, (cudaStream_t)stream, &launches),
           "relayout_mx kernel");
  g_launches += (unsigned long long)launches;
  return W4B_OK;
}

namespace {
// Pads x (M rows of K_x halves) to the descriptor's K in library scratch; *xp is x itself when nothing is to pad.
int pad_activations(const void* x, int K_x, int K, int M, cudaStream_t st, const void** xp, const char* who) {
  if (K_x < 1 || K_x > K) INVALID("%s: K_x must be in 1..K of the descriptor", who);
  if (K_x == K) {
    *xp = x;
    return W4B_OK;
  }
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  CUDA_TRY(ctx->gemm_xpad.reserve((size_t)M * K * sizeof(__half), false), "padded activations");
  CUDA_TRY(pad_rows_launch((const __half*)x, (__half*)ctx->gemm_xpad.ptr, M, K_x, K, st), "pad kernel");
  g_launches += 1;
  *xp = ctx->gemm_xpad.ptr;
  return W4B_OK;
}
}  // namespace

int w4b_gemm_w4_padded(const w4b_packed_w4* p, const void* x, int K_x, void* c, int M, int path, void* stream) {
  if (path < W4B_PATH_AUTO || path > W4B_PATH_GENERIC) INVALID("gemm padded: unknown path %d", path);
  if (int rc = check_w4(p, "gemm padded")) return rc;
  if (!x || !c) INVALID("gemm padded: null pointer");
  if (M < 1) INVALID("gemm padded: bad M");
  const int entry = resolve_path(path, M);
  if (int rc = check_gemm_bounds(p->N, M, entry, "gemm padded")) return rc;
  const void* xp = nullptr;
  if (int rc = pad_activations(x, K_x, p->K, M, (cudaStream_t)stream, &xp, "gemm padded")) return rc;
  return run_gemm(p->symmetric ? 0 : 1, p->gs, p->q, p->scales, p->zeros, p->N, p->K, p->G, xp, c, M, entry,
                  (cudaStream_t)stream, nullptr, "gemm kernel");
}

int w4b_gemm_mx_padded(const w4b_packed_mx* p, const void* x, int K_x, void* c, int M, int path, void* stream) {
  if (path < W4B_PATH_AUTO || path > W4B_PATH_GENERIC) INVALID("gemm_mx padded: unknown path %d", path);
  if (int rc = check_mx(p, "gemm_mx padded")) return rc;
  if (!x || !c) INVALID("gemm_mx padded: null pointer");
  if (M < 1) INVALID("gemm_mx padded: bad M");
  const int entry = resolve_path(path, M);
  if (int rc = check_gemm_bounds(p->N, M, entry, "gemm_mx padded")) return rc;
  const void* xp = nullptr;
  if (int rc = pad_activations(x, K_x, p->K, M, (cudaStream_t)stream, &xp, "gemm_mx padded")) return rc;
  return run_gemm(2, 32, p->q, p->scales, nullptr, p->N, p->K, p->B, xp, c, M, entry, (cudaStream_t)stream, nullptr,
                  "gemm_mx kernel");
}

// ---- decode attention ------------------------------------------------------

namespace {

constexpr int kKvMaxS = 4096;      // kvattention.cuh:36 (single-block entries only)
constexpr int kKvMaxD = 512;       // kvattention.cuh:37
constexpr int kFlashTile = 256;    // kvflash.cuh:35: bounds S through the reference's grid.y

int check_kv_w4(const w4b_kv_w4* p, bool single, const char* who) {  // kvattention.cuh:50-67, kvflash.cuh:37-54
  if (!p) INVALID("%s: null descriptor", who);
  if (p->H < 1 || p->S < 1 || p->D < 1) INVALID("%s: bad dims", who);
  if (single && p->S > kKvMaxS) INVALID("%s: S exceeds the shared-memory bound", who);
  if (p->D > kKvMaxD) INVALID("%s: D exceeds the shared-memory bound", who);
  if (p->gs < 8 || p->gs % 8 != 0) INVALID("%s: gs must be a multiple of 8", who);
  if (p->G != (p->D + p->gs - 1) / p->gs) INVALID("%s: G inconsistent with D, gs", who);
  if (!p->q_k || !p->s_k || !p->q_v || !p->s_v) INVALID("%s: null pointer", who);
  if (!p->symmetric && (!p->z_k || !p->z_v)) INVALID("%s: asymmetric without zeros", who);
  if (p->symmetric && (p->z_k || p->z_v)) INVALID("%s: symmetric carries no zeros", who);
  if (!single && p->S > 65535 * kFlashTile) INVALID("%s: S exceeds the tile-grid bound", who);
  return W4B_OK;
}

int run_attn(const AttnSource& src, const void* q, void* out, int H, int S, int D, cudaStream_t stream,
             void* k_out, void* v_out, const char* who) {
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  const int splits = attn_flash_splits(H, S, ctx->sm_count);
  CUDA_TRY(ctx->attn_ws.reserve(attn_flash_ws_bytes(H, D, splits), false), "attention workspace");
  int launches = 0;
  CUDA_TRY(attn_flash_launch(src, (const __half*)q, (__half*)out, H, S, D, splits, (float*)ctx->attn_ws.ptr,
                             (__half*)k_out, (__half*)v_out, stream, &launches),
           who);
  g_launches += (unsigned long long)launches;
  return W4B_OK;
}

AttnSource w4_source(const w4b_kv_w4* p) {
  AttnSource s;
  memset(&s, 0, sizeof(s));
  s.fmt = p->symmetric ? ATTN_W4_SYM : ATTN_W4_ASYM;
  s.k = p->q_k;
  s.v = p->q_v;
  s.s_k = (const __half*)p->s_k;
  s.s_v = (const __half*)p->s_v;
  s.z_k = p->z_k;
  s.z_v = p->z_v;
  s.gs = p->gs;
  s.G = p->G;
  s.slab_rows = p->S;
  return s;
}

int fp16_attn(const void* q, const void* k16, const void* v16, void* out, int H, int S, int D, void* stream,
              bool single, const char* who) {
  if (H < 1 || S < 1 || D < 1) INVALID("%s: bad dims", who);  // kvflash.cuh:368-377, kvattention.cuh:229-236
  if (single && S > kKvMaxS) INVALID("%s: S exceeds the shared-memory bound", who);
  if (D > kKvMaxD) INVALID("%s: D exceeds the shared-memory bound", who);
  if (!single && S > 65535 * kFlashTile) INVALID("%s: S exceeds the tile-grid bound", who);
  if (!q || !k16 || !v16 || !out) INVALID("%s: null pointer", who);
  AttnSource s;
  memset(&s, 0, sizeof(s));
  s.fmt = ATTN_FP16;
  s.k = k16;
  s.v = v16;
  s.slab_rows = S;
  return run_attn(s, q, out, H, S, D, (cudaStream_t)stream, nullptr, nullptr, who);
}

}  // namespace

int w4b_attn_flash_fp16(const void* q, const void* k16, const void* v16, void* out, int H, int S, int D,
                        void* stream) {
  return fp16_attn(q, k16, v16, out, H, S, D, stream, false, "kv flash fp16");
}

int w4b_attn_single_fp16(const void* q, const void* k16, const void* v16, void* out, int H, int S, int D,
                         void* stream) {
  return fp16_attn(q, k16, v16, out, H, S, D, stream, true, "kv fp16");
}

int w4b_attn_flash_w4(const w4b_kv_w4* p, const void* q, void* out, void* stream, void* k_out, void* v_out) {
  if (int rc = check_kv_w4(p, false, "kv flash")) return rc;
  if (!q || !out) INVALID("kv flash w4: null pointer");
  return run_attn(w4_source(p), q, out, p->H, p->S, p->D, (cudaStream_t)stream, k_out, v_out, "kv flash w4");
}

int w4b_attn_single_w4(const w4b_kv_w4* p, const void* q, void* out, void* stream, void* k_out, void* v_out) {
  if (int rc = check_kv_w4(p, true, "kv")) return rc;
  if (!q || !out) INVALID("kv w4: null pointer");
  return run_attn(w4_source(p), q, out, p->H, p->S, p->D, (cudaStream_t)stream, k_out, v_out, "kv w4");
}

int w4b_attn_flash_f8(const w4b_kv_f8* p, const void* q, void* out, void* stream, void* k_out, void* v_out) {
  // kvflash.cuh:398-411,572-582
  if (!p) INVALID("kv f8 flash: null descriptor");
  if (p->H < 1 || p->S < 1 || p->D < 1) INVALID("kv f8 flash: bad dims");
  if (p->D > kKvMaxD) INVALID("kv f8 flash: D exceeds the shared bound");
  if (p->gs < 8 || p->gs % 8 != 0) INVALID("kv f8 flash: gs must be a multiple of 8");
  if (p->G != (p->D + p->gs - 1) / p->gs) INVALID("kv f8 flash: G inconsistent with D, gs");
  if (!p->q_k || !p->s_k || !p->q_v || !p->s_v) INVALID("kv f8 flash: null pointer");
  if (p->S > 65535 * kFlashTile) INVALID("kv f8 flash: S exceeds the tile-grid bound");
  if (!q || !out) INVALID("kv f8 flash: null io pointer");
  if (p->D % 4 != 0) INVALID("kv f8 flash: D must be a multiple of 4");
  if ((uintptr_t)p->q_k % 4 != 0 || (uintptr_t)p->q_v % 4 != 0) INVALID("kv f8 flash: cache bases 4-byte aligned");
  if ((long long)p->S * ((p->D + 3) / 4) >= (1LL << 31)) INVALID("kv f8 flash: S*words4(D) exceeds 2^31");
  AttnSource s;
  memset(&s, 0, sizeof(s));
  s.fmt = ATTN_F8;
  s.k = p->q_k;
  s.v = p->q_v;
  s.s_k = (const __half*)p->s_k;
  s.s_v = (const __half*)p->s_v;
  s.gs = p->gs;
  s.G = p->G;
  s.slab_rows = p->S;
  return run_attn(s, q, out, p->H, p->S, p->D, (cudaStream_t)stream, k_out, v_out, "kv f8 flash");
}

int w4b_attn_flash_w4_paged(const w4b_kv_w4* p, const int* bt, int page, int npages, const void* q, void* out,
                            void* stream, void* k_out, void* v_out) {
  // kvflash.cuh:733-754
  if (!p) INVALID("kv paged flash: null descriptor");
  if (p->H < 1 || p->S < 1 || p->D < 1) INVALID("kv paged flash: bad dims");
  if (p->D > kKvMaxD) INVALID("kv paged flash: D exceeds the shared bound");
  if (p->gs < 8 || p->gs % 8 != 0) INVALID("kv paged flash: gs must be a multiple of 8");
  if (p->G != (p->D + p->gs - 1) / p->gs) INVALID("kv paged flash: G inconsistent with D, gs");
  if (!p->q_k || !p->s_k || !p->q_v || !p->s_v || !bt) INVALID("kv paged flash: null pointer");
  if (!p->symmetric && (!p->z_k || !p->z_v)) INVALID("kv paged flash: asymmetric without zeros");
  if (p->symmetric && (p->z_k || p->z_v)) INVALID("kv paged flash: symmetric carries zeros");
  if (page < 1 || npages < 1 || (unsigned long long)npages * (unsigned long long)page < (unsigned long long)p->S)
    INVALID("kv paged flash: bad page geometry");
  if ((long long)npages * page >= (1LL << 31)) INVALID("kv paged flash: pool rows exceed 2^31");
  if (p->S > 65535 * kFlashTile) INVALID("kv paged flash: S exceeds tile-grid bound");
  if (!q || !out) INVALID("kv paged flash: null io");
  AttnSource s = w4_source(p);
  s.bt = bt;
  s.page = page;
  s.slab_rows = (long long)npages * page;
  return run_attn(s, q, out, p->H, p->S, p->D, (cudaStream_t)stream, k_out, v_out, "kv paged flash");
}

int w4b_attn_flash_w4_paged_batched(const w4b_kv_w4* p, const int* bt, int bt_stride, const int* seq_lens, int nseq,
                                    int max_seq_len, int page, int npages, const void* q, void* out, void* stream) {
  // the per-sequence contract of w4b_attn_flash_w4_paged (kvflash.cuh:733-754) with p->S ignored
  if (!p) INVALID("kv paged batched: null descriptor");
  if (p->H < 1 || p->D < 1) INVALID("kv paged batched: bad dims");
  if (nseq < 1 || max_seq_len < 1) INVALID("kv paged batched: bad sequence count or length");
  if (p->D > kKvMaxD) INVALID("kv paged batched: D exceeds the shared bound");
  if (p->gs < 8 || p->gs % 8 != 0) INVALID("kv paged batched: gs must be a multiple of 8");
  if (p->G != (p->D + p->gs - 1) / p->gs) INVALID("kv paged batched: G inconsistent with D, gs");
  if (!p->q_k || !p->s_k || !p->q_v || !p->s_v || !bt || !seq_lens) INVALID("kv paged batched: null pointer");
  if (!p->symmetric && (!p->z_k || !p->z_v)) INVALID("kv paged batched: asymmetric without zeros");
  if (p->symmetric && (p->z_k || p->z_v)) INVALID("kv paged batched: symmetric carries zeros");
  if (page < 1 || npages < 1 || (unsigned long long)npages * (unsigned long long)page < (unsigned long long)max_seq_len)
    INVALID("kv paged batched: bad page geometry");
  if ((long long)npages * page >= (1LL << 31)) INVALID("kv paged batched: pool rows exceed 2^31");
  if (max_seq_len > 65535 * kFlashTile) INVALID("kv paged batched: sequence exceeds tile-grid bound");
  if (bt_stride < (max_seq_len + page - 1) / page) INVALID("kv paged batched: block-table rows shorter than the longest sequence");
  if ((long long)nseq * p->H > INT_MAX) INVALID("kv paged batched: too many (sequence, head) rows");
  if (!q || !out) INVALID("kv paged batched: null io");
  AttnSource s = w4_source(p);
  s.bt = bt;
  s.page = page;
  s.slab_rows = (long long)npages * page;
  if (!attn_mma_supported(s, p->D, q, nullptr, nullptr))
    INVALID("kv paged batched: served for D = 64 / 128, gs = 32 / 64 / 128 and 16-byte aligned caches and q; "
            "call w4b_attn_flash_w4_paged per sequence otherwise");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  const int max_splits = attn_flash_splits(attn_batched_rows(nseq, p->H), max_seq_len, ctx->sm_count);
  CUDA_TRY(ctx->attn_ws.reserve(attn_flash_ws_bytes(nseq * p->H, p->D, max_splits), false), "attention workspace");
  int launches = 0;
  CUDA_TRY(attn_flash_batched_launch(s, (const __half*)q, (__half*)out, p->H, p->D, nseq, seq_lens, bt_stride, max_splits,
                                     ctx->sm_count, (float*)ctx->attn_ws.ptr, (cudaStream_t)stream, &launches),
           "kv paged batched");
  g_launches += (unsigned long long)launches;
  return W4B_OK;
}

// ---- all-gather over peer memory (no reference counterpart) --------------------------------

int w4b_peer_alloc(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes == 0) INVALID("peer alloc: null pointer or empty size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  void* p = nullptr;
  CUDA_TRY(cudaMalloc(&p, bytes), "peer alloc");
  CUDA_TRY(cudaMemset(p, 0, bytes), "peer alloc clear");
  CUDA_TRY(cudaDeviceSynchronize(), "peer alloc clear");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "peer alloc: cudaIpcGetMemHandle");
  }
  memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return W4B_OK;
}

int w4b_peer_open(const void* handle64, void** ptr) {
  if (!ptr || !handle64) INVALID("peer open: null pointer");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "peer open: cudaIpcOpenMemHandle");
  return W4B_OK;
}

int w4b_peer_close(void* ptr) {
  if (!ptr) INVALID("peer close: null pointer");
  CUDA_TRY(cudaIpcCloseMemHandle(ptr), "peer close");
  return W4B_OK;
}

int w4b_peer_free(void* ptr) {
  if (!ptr) INVALID("peer free: null pointer");
  CUDA_TRY(cudaFree(ptr), "peer free");
  return W4B_OK;
}

int w4b_allgather_push(const void* src, size_t bytes, void* const* dst, void* const* flag_dst, const void* flags_local,
                       void* counters, int rank, int world, int wait_now, void* stream) {
  if (world < 2 || world > kMaxPeers) INVALID("allgather push: world must be 2..%d", kMaxPeers);
  if (rank < 0 || rank >= world) INVALID("allgather push: rank out of range");
  if (!src || !dst || !flag_dst || !flags_local || !counters) INVALID("allgather push: null pointer");
  if (bytes == 0 || bytes % 16 != 0 || ((uintptr_t)src & 15u)) INVALID("allgather push: slice must be 16-byte sized and aligned");
  if (((uintptr_t)flags_local | (uintptr_t)counters) & 7u) INVALID("allgather push: flags must be 8-byte aligned");
  PeerPush pp;
  memset(&pp, 0, sizeof(pp));
  for (int p = 0; p < world; ++p) {
    if (p == rank) continue;
    if (!dst[p] || !flag_dst[p] || ((uintptr_t)dst[p] & 15u) || ((uintptr_t)flag_dst[p] & 7u))
      INVALID("allgather push: bad destination for peer %d", p);
    pp.dst[p] = dst[p];
    pp.flag_dst[p] = flag_dst[p];
  }
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  pp.src = src;
  pp.n16 = bytes / 16;
  pp.flags_local = flags_local;
  pp.counters = (unsigned long long*)counters;
  pp.rank = rank;
  pp.world = world;
  pp.wait_now = wait_now ? 1 : 0;
  pp.status = ctx->status;
  CUDA_TRY(peer_push_launch(pp, (cudaStream_t)stream), "allgather push kernel");
  g_launches += 1;
  return W4B_OK;
}

int w4b_gemm_w4_push(const w4b_packed_w4* p, const void* x, void* c, int M, void* const* c_peer, void* const* flag_dst,
                     const void* flags_local, void* counters, void* done, int rank, int world, void* stream) {
  if (int rc = check_w4(p, "gemm push")) return rc;
  if (!x || !c) INVALID("gemm push: null pointer");
  if ((uintptr_t)c & 15u) INVALID("gemm push: the slice buffer must be 16-byte aligned");
  if (M < 1 || M > 16) INVALID("gemm push: M must be 1..16 (the stream kernel's single pass)");
  if (int rc = check_gemm_bounds(p->N, M, W4B_PATH_STREAM, "gemm push")) return rc;
  if (world < 2 || world > kMaxPeers) INVALID("gemm push: world must be 2..%d", kMaxPeers);
  if (rank < 0 || rank >= world) INVALID("gemm push: rank out of range");
  if (!c_peer || !flag_dst || !flags_local || !counters || !done) INVALID("gemm push: null pointer");
  if ((((uintptr_t)flags_local | (uintptr_t)counters) & 7u) || ((uintptr_t)done & 3u))
    INVALID("gemm push: flags must be 8-byte aligned, the completion counter 4-byte aligned");
  StreamPeers sp;
  memset(&sp, 0, sizeof(sp));
  for (int r = 0; r < world; ++r) {
    if (r == rank) continue;
    if (!c_peer[r] || !flag_dst[r] || ((uintptr_t)c_peer[r] & 15u) || ((uintptr_t)flag_dst[r] & 7u))
      INVALID("gemm push: bad destination for peer %d", r);
    sp.c_peer[r] = (__half*)c_peer[r];
    sp.flag_dst[r] = (unsigned long long*)flag_dst[r];
  }
  sp.world = world;
  sp.rank = rank;
  sp.flags_local = flags_local;
  sp.counters = (unsigned long long*)counters;
  sp.done = (int*)done;
  return run_gemm(p->symmetric ? 0 : 1, p->gs, p->q, p->scales, p->zeros, p->N, p->K, p->G, x, c, M, W4B_PATH_STREAM,
                  (cudaStream_t)stream, nullptr, "gemm push", &sp);
}

int w4b_gemm_w4_carry(const w4b_packed_w4* p, const void* x, void* c, int M, const void* prev, size_t prev_bytes,
                      void* const* prev_peer, void* const* flag_dst, const void* flags_local, void* counters, void* done,
                      int rank, int world, void* stream) {
  if (int rc = check_w4(p, "gemm carry")) return rc;
  if (!x || !c) INVALID("gemm carry: null pointer");
  if (M < 1 || M > 16) INVALID("gemm carry: M must be 1..16 (the stream kernel's single pass)");
  if (int rc = check_gemm_bounds(p->N, M, W4B_PATH_STREAM, "gemm carry")) return rc;
  if (world < 2 || world > kMaxPeers) INVALID("gemm carry: world must be 2..%d", kMaxPeers);
  if (rank < 0 || rank >= world) INVALID("gemm carry: rank out of range");
  if (!flags_local || !counters || !done) INVALID("gemm carry: null pointer");
  if ((((uintptr_t)flags_local | (uintptr_t)counters) & 7u) || ((uintptr_t)done & 3u))
    INVALID("gemm carry: flags must be 8-byte aligned, the completion counter 4-byte aligned");
  if (prev_bytes && (!prev || !prev_peer || !flag_dst)) INVALID("gemm carry: a slice to carry needs its source and destinations");
  if (prev_bytes % 2 != 0 || ((uintptr_t)prev & 15u)) INVALID("gemm carry: the carried slice must be 16-byte aligned FP16 data");
  StreamPeers sp;
  memset(&sp, 0, sizeof(sp));
  for (int r = 0; r < world && prev_bytes; ++r) {
    if (r == rank) continue;
    if (!prev_peer[r] || !flag_dst[r] || ((uintptr_t)prev_peer[r] & 15u) || ((uintptr_t)flag_dst[r] & 7u))
      INVALID("gemm carry: bad destination for peer %d", r);
    sp.c_peer[r] = (__half*)prev_peer[r];
    sp.flag_dst[r] = (unsigned long long*)flag_dst[r];
  }
  sp.world = world;
  sp.rank = rank;
  sp.flags_local = flags_local;
  sp.counters = (unsigned long long*)counters;
  sp.done = (int*)done;
  sp.carry = 1;
  sp.prev_src = (const __half*)prev;
  sp.prev_bytes = prev_bytes;
  return run_gemm(p->symmetric ? 0 : 1, p->gs, p->q, p->scales, p->zeros, p->N, p->K, p->G, x, c, M, W4B_PATH_STREAM,
                  (cudaStream_t)stream, nullptr, "gemm carry", &sp);
}

int w4b_allgather_wait(const void* flags_local, const void* counters, int rank, int world, void* stream) {
  if (world < 2 || world > kMaxPeers) INVALID("allgather wait: world must be 2..%d", kMaxPeers);
  if (rank < 0 || rank >= world) INVALID("allgather wait: rank out of range");
  if (!flags_local || !counters || (((uintptr_t)flags_local | (uintptr_t)counters) & 7u))
    INVALID("allgather wait: flags must be non-null and 8-byte aligned");
  DeviceCtx* ctx = nullptr;
  if (int rc = get_ctx(&ctx)) return rc;
  CUDA_TRY(peer_wait_launch(flags_local, (const unsigned long long*)counters, rank, world, ctx->status,
                            (cudaStream_t)stream),
           "allgather wait kernel");
  g_launches += 1;
  return W4B_OK;
}

}  // extern "C"
