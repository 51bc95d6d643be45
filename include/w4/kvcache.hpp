#pragma once
// Drop-in host header: the W4 KV cache (H head slabs of the packed W4 format, rows
// are positions, the packed axis is the head dimension), its quantizer and the
// FP64 decode-attention reference, with the names and contracts of the reference's
// include/w4/kvcache.hpp (KVCacheW4 :28-34, validate_cache :36-55, quantize_cache
// :60-108, dequant_head :111-135, attention_reference :141-175).
#include <cuda_fp16.h>

#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <vector>

#include "pack.hpp"

namespace w4::kv {

struct KVCacheW4 {
  int H = 0, S = 0, D = 0, gs = 0, G = 0;
  bool symmetric = true;
  std::vector<uint32_t> q_k, q_v;  // H slabs of S * words(D)
  std::vector<__half> s_k, s_v;    // H slabs of S * G
  std::vector<uint32_t> z_k, z_v;  // H slabs of S * words(G), asymmetric only
};

inline void validate_cache(const KVCacheW4& c) {
  using w4::detail::require;
  require(c.H >= 1 && c.S >= 1 && c.D >= 1, "cache: bad dims");
  require(c.gs >= 8 && c.gs % 8 == 0, "cache: gs must be a multiple of 8");
  require(c.G == (c.D + c.gs - 1) / c.gs, "cache: G inconsistent with D, gs");
  const size_t rows = (size_t)c.H * c.S;
  require(c.q_k.size() == rows * words(c.D) && c.q_v.size() == rows * words(c.D), "cache: q size");
  require(c.s_k.size() == rows * c.G && c.s_v.size() == rows * c.G, "cache: scales size");
  if (c.symmetric)
    require(c.z_k.empty() && c.z_v.empty(), "cache: symmetric carries no zeros");
  else
    require(c.z_k.size() == rows * words(c.G) && c.z_v.size() == rows * words(c.G), "cache: zeros size");
}

namespace detail {
// One head of one side as a stand-alone PackedW (positions are its rows).
inline PackedW head_view(const KVCacheW4& c, int h, bool vside) {
  PackedW p;
  p.N = c.S;
  p.K = c.D;
  p.gs = c.gs;
  p.G = c.G;
  p.symmetric = c.symmetric;
  const auto cut = [&](const auto& src, size_t per_row) {
    using V = std::decay_t<decltype(src)>;
    const size_t n = (size_t)c.S * per_row;
    return V(src.begin() + (size_t)h * n, src.begin() + (size_t)(h + 1) * n);
  };
  p.q = cut(vside ? c.q_v : c.q_k, (size_t)words(c.D));
  p.scales = cut(vside ? c.s_v : c.s_k, (size_t)c.G);
  if (!c.symmetric) p.zeros = cut(vside ? c.z_v : c.z_k, (size_t)words(c.G));
  return p;
}

// softmax(q.k / sqrt(D)) . v for one head over FP16-exact K / V rows, all in FP64
inline void attend(const __half* q, const std::vector<__half>& k, const std::vector<__half>& v, int S, int D,
                   double* out) {
  const double inv = 1.0 / std::sqrt((double)D);
  std::vector<double> p((size_t)S);
  double top = -INFINITY;
  for (int t = 0; t < S; ++t) {
    double acc = 0.0;
    for (int d = 0; d < D; ++d) acc += (double)__half2float(q[d]) * (double)__half2float(k[(size_t)t * D + d]);
    p[t] = acc * inv;
    top = std::max(top, p[t]);
  }
  double denom = 0.0;
  for (int t = 0; t < S; ++t) denom += (p[t] = std::exp(p[t] - top));
  for (int t = 0; t < S; ++t) p[t] /= denom;
  for (int d = 0; d < D; ++d) {
    double acc = 0.0;
    for (int t = 0; t < S; ++t) acc += p[t] * (double)__half2float(v[(size_t)t * D + d]);
    out[d] = acc;
  }
}
}  // namespace detail

// k and v are H*S*D doubles, head-major then position-major; each head is quantised
// by w4::quantize, which carries the NaN / scale-range / dims contracts.
inline KVCacheW4 quantize_cache(const std::vector<double>& k, const std::vector<double>& v, int H, int S, int D,
                                int gs, bool symmetric) {
  using w4::detail::require;
  require(H >= 1 && S >= 1 && D >= 1, "quantize_cache: bad dims");
  require(gs >= 8 && gs % 8 == 0, "quantize_cache: gs must be a multiple of 8");
  const size_t per_head = (size_t)S * D;
  require(k.size() == (size_t)H * per_head && v.size() == (size_t)H * per_head, "quantize_cache: size");
  KVCacheW4 c;
  c.H = H;
  c.S = S;
  c.D = D;
  c.gs = gs;
  c.G = (D + gs - 1) / gs;
  c.symmetric = symmetric;
  for (int side = 0; side < 2; ++side) {
    const std::vector<double>& src = side ? v : k;
    auto& qs = side ? c.q_v : c.q_k;
    auto& ss = side ? c.s_v : c.s_k;
    auto& zs = side ? c.z_v : c.z_k;
    for (int h = 0; h < H; ++h) {
      const PackedW p = quantize(std::vector<double>(src.begin() + (size_t)h * per_head,
                                                     src.begin() + (size_t)(h + 1) * per_head),
                                 S, D, gs, symmetric);
      qs.insert(qs.end(), p.q.begin(), p.q.end());
      ss.insert(ss.end(), p.scales.begin(), p.scales.end());
      zs.insert(zs.end(), p.zeros.begin(), p.zeros.end());
    }
  }
  return c;
}

inline std::vector<__half> dequant_head(const KVCacheW4& c, int h, bool vside) {
  validate_cache(c);
  w4::detail::require(h >= 0 && h < c.H, "dequant_head: h");
  return dequant_all(detail::head_view(c, h, vside));
}

// q is H*D FP16; the result is H*D doubles.
inline std::vector<double> attention_reference(const std::vector<__half>& q, const KVCacheW4& c) {
  validate_cache(c);
  w4::detail::require(q.size() == (size_t)c.H * c.D, "attention_reference: q size");
  std::vector<double> out((size_t)c.H * c.D, 0.0);
  for (int h = 0; h < c.H; ++h)
    detail::attend(q.data() + (size_t)h * c.D, dequant_head(c, h, false), dequant_head(c, h, true), c.S, c.D,
                   out.data() + (size_t)h * c.D);
  return out;
}

}  // namespace w4::kv
