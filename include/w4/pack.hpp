#pragma once
// Drop-in host header: the packed W4A16 weight format, its host quantizer, the
// reference dequantisation and the FP64 GEMM oracle, with the names, signatures
// and throw contracts of the reference's include/w4/pack.hpp (format :3-14,
// words :33, PackedW :35-41, accessors :43-53, dequant_one :58-60, quantize
// :64-130, validate_packed :134-148, dequant_all :150-161, gemm_oracle :166-184,
// seeded generators :186-200). Written from the format's definition; it shares
// no code with the GPU kernels, which are checked against it.
//
//   q       8 codes per uint32, word w of row n holds k = 8w .. 8w+7, low nibble first
//   scales  FP16, one per (row, group); group g covers k in [g*gs, min((g+1)*gs, K))
//   zeros   asymmetric only: one code per (row, group), packed like q along the groups
//   value   w = scale * (q - z),  z = 8 in symmetric mode
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <random>
#include <stdexcept>
#include <vector>

#if defined(__CUDACC__)
#define W4_HD __host__ __device__
#else
#define W4_HD
#endif

namespace w4 {

W4_HD inline int words(int n) { return (n + 7) / 8; }

struct PackedW {
  int N = 0, K = 0, gs = 0, G = 0;
  bool symmetric = true;
  std::vector<uint32_t> q;
  std::vector<__half> scales;
  std::vector<uint32_t> zeros;
};

namespace detail {
inline int code_at(const std::vector<uint32_t>& packed, size_t row_words, int n, int i) {
  return (int)((packed[(size_t)n * row_words + (size_t)(i >> 3)] >> ((i & 7) * 4)) & 0xFu);
}
inline void put_code(std::vector<uint32_t>& packed, size_t row_words, int n, int i, int code) {
  packed[(size_t)n * row_words + (size_t)(i >> 3)] |= (uint32_t)code << ((i & 7) * 4);
}
inline int clamp_code(long v) { return (int)std::max(0L, std::min(15L, v)); }
inline void require(bool ok, const char* what) {
  if (!ok) throw std::invalid_argument(what);
}
}  // namespace detail

inline int get_q(const PackedW& p, int n, int k) { return detail::code_at(p.q, (size_t)words(p.K), n, k); }
inline int get_z(const PackedW& p, int n, int g) { return detail::code_at(p.zeros, (size_t)words(p.G), n, g); }
inline int zero_point(const PackedW& p, int n, int g) { return p.symmetric ? 8 : get_z(p, n, g); }

// The one dequantisation step: exact float product, one rounding to FP16.
W4_HD inline __half dequant_one(__half s, int q, int z) {
  return __float2half_rn(__half2float(s) * (float)(q - z));
}

inline PackedW quantize(const std::vector<double>& w, int N, int K, int gs, bool symmetric) {
  using detail::require;
  require(N >= 1 && K >= 1, "quantize: bad dims");
  require(gs >= 8 && gs % 8 == 0, "quantize: gs must be a multiple of 8");
  require(w.size() == (size_t)N * (size_t)K, "quantize: size");
  require(std::all_of(w.begin(), w.end(), [](double v) { return std::isfinite(v); }), "quantize: non-finite input");

  PackedW p;
  p.N = N;
  p.K = K;
  p.gs = gs;
  p.G = (K + gs - 1) / gs;
  p.symmetric = symmetric;
  p.q.assign((size_t)N * words(K), 0u);
  p.scales.assign((size_t)N * p.G, __float2half_rn(0.0f));
  if (!symmetric) p.zeros.assign((size_t)N * words(p.G), 0u);

  for (int n = 0; n < N; ++n) {
    const double* row = w.data() + (size_t)n * K;
    for (int g = 0; g < p.G; ++g) {
      const int k0 = g * gs, k1 = std::min(K, k0 + gs);
      const auto mm = std::minmax_element(row + k0, row + k1);
      double lo = *mm.first, hi = *mm.second;
      if (!symmetric) {  // the range must bracket zero so that the zero point is a code
        lo = std::min(lo, 0.0);
        hi = std::max(hi, 0.0);
      }
      const double span = symmetric ? std::max(std::fabs(lo), std::fabs(hi)) / 7.0 : (hi - lo) / 15.0;
      const bool flat = symmetric ? (lo == 0.0 && hi == 0.0) : !(hi > lo);
      const __half stored = __float2half_rn((float)(flat ? 1.0 : span));
      const float sf = __half2float(stored);  // codes are rounded against the scale actually stored
      require(std::isfinite(sf) && !(sf == 0.0f && !flat), "quantize: group scale outside FP16 range");
      const int z = symmetric ? 8 : detail::clamp_code(std::lround(-lo / (double)sf));
      p.scales[(size_t)n * p.G + g] = stored;
      for (int k = k0; k < k1; ++k)
        detail::put_code(p.q, (size_t)words(K), n, k, detail::clamp_code(std::lround(row[k] / (double)sf) + z));
      if (!symmetric) detail::put_code(p.zeros, (size_t)words(p.G), n, g, z);
    }
  }
  return p;
}

inline void validate_packed(const PackedW& p) {
  using detail::require;
  require(p.N >= 1 && p.K >= 1, "packed: bad dims");
  require(p.gs >= 8 && p.gs % 8 == 0, "packed: gs must be a multiple of 8");
  require(p.G == (p.K + p.gs - 1) / p.gs, "packed: G inconsistent with K, gs");
  require(p.q.size() == (size_t)p.N * (size_t)words(p.K), "packed: q size");
  require(p.scales.size() == (size_t)p.N * (size_t)p.G, "packed: scales size");
  require(p.symmetric || p.zeros.size() == (size_t)p.N * (size_t)words(p.G), "packed: zeros size");
  require(!p.symmetric || p.zeros.empty(), "packed: symmetric carries no zeros");
}

inline std::vector<__half> dequant_all(const PackedW& p) {
  validate_packed(p);
  std::vector<__half> out((size_t)p.N * p.K);
  for (int n = 0; n < p.N; ++n)
    for (int g = 0; g < p.G; ++g) {
      const __half s = p.scales[(size_t)n * p.G + g];
      const int z = zero_point(p, n, g);
      for (int k = g * p.gs, k1 = std::min(p.K, k + p.gs); k < k1; ++k)
        out[(size_t)n * p.K + k] = dequant_one(s, get_q(p, n, k), z);
    }
  return out;
}

// C[m,n] = sum_k x[m,k] * w[n,k], accumulated in FP64 in ascending k.
inline std::vector<double> gemm_oracle(const std::vector<__half>& x, int M, int K, const std::vector<__half>& w,
                                       int N) {
  using detail::require;
  require(M >= 1 && N >= 1 && K >= 1, "gemm_oracle: bad dims");
  require(x.size() == (size_t)M * (size_t)K && w.size() == (size_t)N * (size_t)K, "gemm_oracle: size");
  std::vector<double> c((size_t)M * N);
  for (int m = 0; m < M; ++m) {
    const __half* xr = x.data() + (size_t)m * K;
    for (int n = 0; n < N; ++n) {
      const __half* wr = w.data() + (size_t)n * K;
      double acc = 0.0;
      for (int k = 0; k < K; ++k) acc += (double)__half2float(xr[k]) * (double)__half2float(wr[k]);
      c[(size_t)m * N + n] = acc;
    }
  }
  return c;
}

inline std::vector<double> normal_weights(int count, uint64_t seed) {
  std::mt19937_64 rng(seed);
  std::normal_distribution<double> dist(0.0, 1.0);
  std::vector<double> v((size_t)count);
  std::generate(v.begin(), v.end(), [&] { return dist(rng); });
  return v;
}

inline std::vector<__half> normal_activations(int count, uint64_t seed) {
  std::mt19937_64 rng(seed);
  std::normal_distribution<double> dist(0.0, 1.0);
  std::vector<__half> v((size_t)count);
  std::generate(v.begin(), v.end(), [&] { return __float2half_rn((float)dist(rng)); });
  return v;
}

}  // namespace w4
