// extern "C" shim over the REFERENCE project's own host headers.
//
// Test infrastructure only. Compiled (by oracle/Makefile, target `ref`) against
// the reference tree where it lies — nothing of the reference is copied into
// this repository — into oracle/_ref/libw4ref.so. It exists to (1) pin the
// plain-C restatement in w4_oracle.c bit-for-bit against the reference,
// (2) produce the committed golden vectors, and (3) time the reference's CPU
// path (quantize / dequant_all / gemm_oracle, attention_reference) on all host
// cores by handing disjoint row or head slices to the reference's unmodified,
// single-threaded functions from several threads.
//
// Signatures mirror the orc_* functions of w4_oracle.c one to one.
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <thread>
#include <vector>

#include "w4/kvcache.hpp"
#include "w4/kvfp8.hpp"
#include "w4/kvpaged.hpp"
#include "w4/mx.hpp"
#include "w4/pack.hpp"

namespace {

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::invalid_argument&) {
    return 1;
  } catch (...) {
    return 2;
  }
}

std::vector<__half> halves(const uint16_t* p, size_t n) {
  std::vector<__half> v(n);
  std::memcpy(v.data(), p, n * 2);
  return v;
}

w4::PackedW make_packed(int N, int K, int gs, int G, int symmetric, const uint32_t* q,
                        const uint16_t* scales, const uint32_t* zeros) {
  w4::PackedW p;
  p.N = N;
  p.K = K;
  p.gs = gs;
  p.G = G;
  p.symmetric = symmetric != 0;
  if (N > 0 && K > 0 && G > 0) {
    p.q.assign(q, q + (size_t)N * w4::words(K));
    p.scales = halves(scales, (size_t)N * G);
    if (zeros) p.zeros.assign(zeros, zeros + (size_t)N * w4::words(G));
  }
  return p;
}

}  // namespace

extern "C" {

uint16_t ref_f32_to_f16(float f) {
  const __half h = __float2half_rn(f);
  uint16_t u;
  std::memcpy(&u, &h, 2);
  return u;
}

float ref_f16_to_f32(uint16_t u) {
  __half h;
  std::memcpy(&h, &u, 2);
  return __half2float(h);
}

void ref_normal_f64(double* out, size_t count, uint64_t seed) {
  const auto v = w4::normal_weights((int)count, seed);
  std::memcpy(out, v.data(), count * sizeof(double));
}

void ref_normal_f16(uint16_t* out, size_t count, uint64_t seed) {
  const auto v = w4::normal_activations((int)count, seed);
  std::memcpy(out, v.data(), count * 2);
}

uint16_t ref_dequant_one(uint16_t s, int q, int z) {
  __half h;
  std::memcpy(&h, &s, 2);
  const __half r = w4::dequant_one(h, q, z);
  uint16_t u;
  std::memcpy(&u, &r, 2);
  return u;
}

uint16_t ref_dequant_one_mx(uint8_t se, int q) {
  const __half r = w4::mx::dequant_one_mx(se, q);
  uint16_t u;
  std::memcpy(&u, &r, 2);
  return u;
}

uint16_t ref_dequant_one_f8(uint16_t s, uint8_t b) {
  __half h;
  std::memcpy(&h, &s, 2);
  const __half r = w4::kv8::dequant_one_f8(h, b);
  uint16_t u;
  std::memcpy(&u, &r, 2);
  return u;
}

uint8_t ref_encode_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

int ref_quantize_w4(const double* w, int N, int K, int gs, int symmetric, uint32_t* q,
                    uint16_t* scales, uint32_t* zeros) {
  return guarded([&] {
    const size_t n = (N > 0 && K > 0) ? (size_t)N * K : 0;
    const auto p = w4::quantize(std::vector<double>(w, w + n), N, K, gs, symmetric != 0);
    std::memcpy(q, p.q.data(), p.q.size() * 4);
    std::memcpy(scales, p.scales.data(), p.scales.size() * 2);
    if (!p.symmetric) std::memcpy(zeros, p.zeros.data(), p.zeros.size() * 4);
  });
}

int ref_dequant_all_w4(int N, int K, int gs, int G, int symmetric, const uint32_t* q,
                       const uint16_t* scales, const uint32_t* zeros, uint16_t* w) {
  return guarded([&] {
    const auto p = make_packed(N, K, gs, G, symmetric, q, scales, zeros);
    const auto d = w4::dequant_all(p);
    std::memcpy(w, d.data(), d.size() * 2);
  });
}

int ref_gemm_oracle(const uint16_t* x, int M, int K, const uint16_t* w, int N, double* c) {
  return guarded([&] {
    const auto r = w4::gemm_oracle(halves(x, (size_t)M * K), M, K, halves(w, (size_t)N * K), N);
    std::memcpy(c, r.data(), r.size() * sizeof(double));
  });
}

// Row-sliced threads over the reference's serial gemm_oracle; c is M x N row-major.
int ref_gemm_oracle_mt(const uint16_t* x, int M, int K, const uint16_t* w, int N, double* c,
                       int threads) {
  if (threads < 1) threads = 1;
  if (threads > N) threads = N;
  const auto xv = halves(x, (size_t)M * K);
  std::vector<int> rc((size_t)threads, 0);
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&, t] {
      rc[t] = guarded([&] {
        const int n0 = (int)((int64_t)N * t / threads), n1 = (int)((int64_t)N * (t + 1) / threads);
        if (n1 <= n0) return;
        const auto r = w4::gemm_oracle(xv, M, K, halves(w + (size_t)n0 * K, (size_t)(n1 - n0) * K), n1 - n0);
        for (int m = 0; m < M; ++m)
          std::memcpy(c + (size_t)m * N + n0, r.data() + (size_t)m * (n1 - n0), (size_t)(n1 - n0) * 8);
      });
    });
  for (auto& th : pool) th.join();
  for (int v : rc)
    if (v) return v;
  return 0;
}

int ref_quantize_mx(const double* w, int N, int K, uint32_t* q, uint8_t* scales) {
  return guarded([&] {
    const size_t n = (N > 0 && K > 0) ? (size_t)N * K : 0;
    const auto p = w4::mx::quantize_mx(std::vector<double>(w, w + n), N, K);
    std::memcpy(q, p.q.data(), p.q.size() * 4);
    std::memcpy(scales, p.scales.data(), p.scales.size());
  });
}

int ref_dequant_all_mx(int N, int K, int B, const uint32_t* q, const uint8_t* scales, uint16_t* w) {
  return guarded([&] {
    w4::mx::PackedWm p;
    p.N = N;
    p.K = K;
    p.B = B;
    if (N > 0 && K > 0 && B > 0) {
      p.q.assign(q, q + (size_t)N * w4::words(K));
      p.scales.assign(scales, scales + (size_t)N * B);
    }
    const auto d = w4::mx::dequant_all_mx(p);
    std::memcpy(w, d.data(), d.size() * 2);
  });
}

int ref_quantize_cache_w4(const double* k, const double* v, int H, int S, int D, int gs,
                          int symmetric, uint32_t* q_k, uint16_t* s_k, uint32_t* z_k,
                          uint32_t* q_v, uint16_t* s_v, uint32_t* z_v) {
  return guarded([&] {
    const size_t n = (H > 0 && S > 0 && D > 0) ? (size_t)H * S * D : 0;
    const auto c = w4::kv::quantize_cache(std::vector<double>(k, k + n), std::vector<double>(v, v + n),
                                          H, S, D, gs, symmetric != 0);
    std::memcpy(q_k, c.q_k.data(), c.q_k.size() * 4);
    std::memcpy(q_v, c.q_v.data(), c.q_v.size() * 4);
    std::memcpy(s_k, c.s_k.data(), c.s_k.size() * 2);
    std::memcpy(s_v, c.s_v.data(), c.s_v.size() * 2);
    if (!c.symmetric) {
      std::memcpy(z_k, c.z_k.data(), c.z_k.size() * 4);
      std::memcpy(z_v, c.z_v.data(), c.z_v.size() * 4);
    }
  });
}

static w4::kv::KVCacheW4 make_cache(int H, int S, int D, int gs, int G, int symmetric,
                                    const uint32_t* q_k, const uint16_t* s_k, const uint32_t* z_k,
                                    const uint32_t* q_v, const uint16_t* s_v, const uint32_t* z_v) {
  w4::kv::KVCacheW4 c;
  c.H = H;
  c.S = S;
  c.D = D;
  c.gs = gs;
  c.G = G;
  c.symmetric = symmetric != 0;
  const size_t nq = (size_t)H * S * w4::words(D), ns = (size_t)H * S * G,
               nz = (size_t)H * S * w4::words(G);
  c.q_k.assign(q_k, q_k + nq);
  c.q_v.assign(q_v, q_v + nq);
  c.s_k = halves(s_k, ns);
  c.s_v = halves(s_v, ns);
  if (!c.symmetric) {
    c.z_k.assign(z_k, z_k + nz);
    c.z_v.assign(z_v, z_v + nz);
  }
  return c;
}

// attention_reference over a W4 cache; also returns the dequantised heads when
// kd / vd are non-null (dequant_head per head, H*S*D FP16 each).
int ref_attention_w4(const uint16_t* q, int H, int S, int D, int gs, int G, int symmetric,
                     const uint32_t* q_k, const uint16_t* s_k, const uint32_t* z_k,
                     const uint32_t* q_v, const uint16_t* s_v, const uint32_t* z_v, double* out,
                     uint16_t* kd, uint16_t* vd) {
  return guarded([&] {
    const auto c = make_cache(H, S, D, gs, G, symmetric, q_k, s_k, z_k, q_v, s_v, z_v);
    const auto r = w4::kv::attention_reference(halves(q, (size_t)H * D), c);
    std::memcpy(out, r.data(), r.size() * 8);
    for (int h = 0; h < H && (kd || vd); ++h) {
      if (kd) {
        const auto d = w4::kv::dequant_head(c, h, false);
        std::memcpy(kd + (size_t)h * S * D, d.data(), d.size() * 2);
      }
      if (vd) {
        const auto d = w4::kv::dequant_head(c, h, true);
        std::memcpy(vd + (size_t)h * S * D, d.data(), d.size() * 2);
      }
    }
  });
}

int ref_quantize_cache_f8(const double* k, const double* v, int H, int S, int D, int gs,
                          uint8_t* q_k, uint16_t* s_k, uint8_t* q_v, uint16_t* s_v) {
  return guarded([&] {
    const size_t n = (H > 0 && S > 0 && D > 0) ? (size_t)H * S * D : 0;
    const auto c = w4::kv8::quantize_cache_f8(std::vector<double>(k, k + n),
                                              std::vector<double>(v, v + n), H, S, D, gs);
    std::memcpy(q_k, c.q_k.data(), c.q_k.size());
    std::memcpy(q_v, c.q_v.data(), c.q_v.size());
    std::memcpy(s_k, c.s_k.data(), c.s_k.size() * 2);
    std::memcpy(s_v, c.s_v.data(), c.s_v.size() * 2);
  });
}

int ref_attention_f8(const uint16_t* q, int H, int S, int D, int gs, int G, const uint8_t* q_k,
                     const uint16_t* s_k, const uint8_t* q_v, const uint16_t* s_v, double* out,
                     uint16_t* kd, uint16_t* vd) {
  return guarded([&] {
    w4::kv8::KVCacheF8 c;
    c.H = H;
    c.S = S;
    c.D = D;
    c.gs = gs;
    c.G = G;
    const size_t nq = (size_t)H * S * D, ns = (size_t)H * S * G;
    c.q_k.assign(q_k, q_k + nq);
    c.q_v.assign(q_v, q_v + nq);
    c.s_k = halves(s_k, ns);
    c.s_v = halves(s_v, ns);
    const auto r = w4::kv8::attention_reference_f8(halves(q, (size_t)H * D), c);
    std::memcpy(out, r.data(), r.size() * 8);
    for (int h = 0; h < H && (kd || vd); ++h) {
      if (kd) {
        const auto d = w4::kv8::dequant_head_f8(c, h, false);
        std::memcpy(kd + (size_t)h * S * D, d.data(), d.size() * 2);
      }
      if (vd) {
        const auto d = w4::kv8::dequant_head_f8(c, h, true);
        std::memcpy(vd + (size_t)h * S * D, d.data(), d.size() * 2);
      }
    }
  });
}

// paged_from_contiguous on a W4 cache; pool outputs sized H*lpages*page rows.
int ref_paged_from_contiguous(int H, int S, int D, int gs, int G, int symmetric,
                              const uint32_t* q_k, const uint16_t* s_k, const uint32_t* z_k,
                              const uint32_t* q_v, const uint16_t* s_v, const uint32_t* z_v,
                              int page, const int* bt, int nbt, uint32_t* pq_k, uint16_t* ps_k,
                              uint32_t* pz_k, uint32_t* pq_v, uint16_t* ps_v, uint32_t* pz_v) {
  return guarded([&] {
    const auto c = make_cache(H, S, D, gs, G, symmetric, q_k, s_k, z_k, q_v, s_v, z_v);
    const auto p = w4::kv::paged_from_contiguous(c, page, std::vector<int>(bt, bt + nbt));
    w4::kv::validate_paged(p);
    std::memcpy(pq_k, p.q_k.data(), p.q_k.size() * 4);
    std::memcpy(pq_v, p.q_v.data(), p.q_v.size() * 4);
    std::memcpy(ps_k, p.s_k.data(), p.s_k.size() * 2);
    std::memcpy(ps_v, p.s_v.data(), p.s_v.size() * 2);
    if (!p.symmetric) {
      std::memcpy(pz_k, p.z_k.data(), p.z_k.size() * 4);
      std::memcpy(pz_v, p.z_v.data(), p.z_v.size() * 4);
    }
  });
}

// The reference's CPU path for one W4 GEMM, row-sliced over `threads`:
// quantize -> dequant_all -> gemm_oracle, each phase timed (seconds, wall).
// wd (N*K FP16) and c (M*N FP64) receive the results.
int ref_cpu_path_w4(const double* w, const uint16_t* x, int M, int N, int K, int gs, int symmetric,
                    int threads, int do_quantize, const uint32_t* q_in, const uint16_t* s_in,
                    const uint32_t* z_in, uint16_t* wd, double* c, double* seconds /*[3]*/);

}  // extern "C"

#include <chrono>

namespace {
double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

extern "C" int ref_cpu_path_w4(const double* w, const uint16_t* x, int M, int N, int K, int gs,
                               int symmetric, int threads, int do_quantize, const uint32_t* q_in,
                               const uint16_t* s_in, const uint32_t* z_in, uint16_t* wd, double* c,
                               double* seconds) {
  if (threads < 1) threads = 1;
  if (threads > N) threads = N;
  const int G = (K + gs - 1) / gs;
  std::vector<w4::PackedW> parts((size_t)threads);
  std::vector<int> rc((size_t)threads, 0);
  auto span = [&](int t, int& n0, int& n1) {
    n0 = (int)((int64_t)N * t / threads);
    n1 = (int)((int64_t)N * (t + 1) / threads);
  };
  auto run = [&](auto&& body) {
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) pool.emplace_back([&, t] { rc[t] = guarded([&] { body(t); }); });
    for (auto& th : pool) th.join();
    for (int v : rc)
      if (v) return v;
    return 0;
  };
  double t0 = now_s();
  int r = run([&](int t) {
    int n0, n1;
    span(t, n0, n1);
    if (do_quantize) {
      parts[t] = w4::quantize(std::vector<double>(w + (size_t)n0 * K, w + (size_t)n1 * K), n1 - n0, K,
                              gs, symmetric != 0);
    } else {
      parts[t] = make_packed(n1 - n0, K, gs, G, symmetric, q_in + (size_t)n0 * w4::words(K),
                             s_in + (size_t)n0 * G,
                             symmetric ? nullptr : z_in + (size_t)n0 * w4::words(G));
    }
  });
  if (r) return r;
  double t1 = now_s();
  seconds[0] = do_quantize ? t1 - t0 : 0.0;
  r = run([&](int t) {
    int n0, n1;
    span(t, n0, n1);
    const auto d = w4::dequant_all(parts[t]);
    std::memcpy(wd + (size_t)n0 * K, d.data(), d.size() * 2);
  });
  if (r) return r;
  double t2 = now_s();
  seconds[1] = t2 - t1;
  r = ref_gemm_oracle_mt(x, M, K, wd, N, c, threads);
  seconds[2] = now_s() - t2;
  return r;
}
