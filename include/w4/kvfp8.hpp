#pragma once
// Drop-in host header: the FP8 (E4M3) KV cache - one byte per element, one FP16
// scale per (position, group) - with the names and contracts of the reference's
// include/w4/kvfp8.hpp (KVCacheF8 :36-40, decode_f8_e4m3 :42-47, dequant_one_f8
// :51-53, validate_cache_f8 :55-68, quantize_cache_f8 :70-128, dequant_head_f8
// :131-146, attention_reference_f8 :150-184).
//
// Decode is exact in float: exponent field 0 -> m * 2^-9, otherwise (8 + m) * 2^(e-10).
// The quantizer scales a group by amax / 448 (nothing saturates) and rounds elements
// with the toolkit's round-to-nearest-even, saturate-to-finite conversion.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <vector>

#include "kvcache.hpp"
#include "pack.hpp"

namespace w4::kv8 {

struct KVCacheF8 {
  int H = 0, S = 0, D = 0, gs = 0, G = 0;
  std::vector<uint8_t> q_k, q_v;  // H slabs of S * D bytes
  std::vector<__half> s_k, s_v;   // H slabs of S * G
};

W4_HD inline float decode_f8_e4m3(uint8_t b) {
  const int e = (b >> 3) & 0xF, m = b & 7;
  const float mag = e == 0 ? ldexpf((float)m, -9) : ldexpf((float)(8 + m), e - 10);
  return (b & 0x80) ? -mag : mag;
}

W4_HD inline __half dequant_one_f8(__half s, uint8_t b) {
  return __float2half_rn(__half2float(s) * decode_f8_e4m3(b));
}

inline void validate_cache_f8(const KVCacheF8& c) {
  using w4::detail::require;
  require(c.H >= 1 && c.S >= 1 && c.D >= 1, "cache f8: bad dims");
  require(c.gs >= 8 && c.gs % 8 == 0, "cache f8: gs must be a multiple of 8");
  require(c.G == (c.D + c.gs - 1) / c.gs, "cache f8: G inconsistent with D, gs");
  const size_t rows = (size_t)c.H * c.S;
  require(c.q_k.size() == rows * c.D && c.q_v.size() == rows * c.D, "cache f8: q size");
  require(c.s_k.size() == rows * c.G && c.s_v.size() == rows * c.G, "cache f8: scales size");
}

inline KVCacheF8 quantize_cache_f8(const std::vector<double>& k, const std::vector<double>& v, int H, int S, int D,
                                   int gs) {
  using w4::detail::require;
  require(H >= 1 && S >= 1 && D >= 1, "quantize_cache_f8: bad dims");
  require(gs >= 8 && gs % 8 == 0, "quantize_cache_f8: gs must be a multiple of 8");
  const size_t total = (size_t)H * S * D;
  require(k.size() == total && v.size() == total, "quantize_cache_f8: size");
  for (const auto* src : {&k, &v})
    for (const double x : *src) require(std::isfinite(x), "quantize_cache_f8: non-finite input");
  KVCacheF8 c;
  c.H = H;
  c.S = S;
  c.D = D;
  c.gs = gs;
  c.G = (D + gs - 1) / gs;
  const size_t rows = (size_t)H * S;
  for (int side = 0; side < 2; ++side) {
    const std::vector<double>& src = side ? v : k;
    auto& codes = side ? c.q_v : c.q_k;
    auto& scales = side ? c.s_v : c.s_k;
    codes.assign(total, 0);
    scales.assign(rows * c.G, __float2half_rn(0.0f));
    for (size_t row = 0; row < rows; ++row) {
      const double* x = src.data() + row * D;
      for (int g = 0; g < c.G; ++g) {
        const int d0 = g * gs, d1 = std::min(D, d0 + gs);
        double amax = 0.0;
        for (int d = d0; d < d1; ++d) amax = std::max(amax, std::fabs(x[d]));
        const __half stored = __float2half_rn((float)(amax > 0.0 ? amax / 448.0 : 1.0));
        const float sf = __half2float(stored);
        require(std::isfinite(sf) && !(sf == 0.0f && amax > 0.0), "quantize_cache_f8: group scale outside FP16 range");
        scales[row * c.G + g] = stored;
        for (int d = d0; d < d1; ++d)
          codes[row * D + d] =
              (uint8_t)__nv_cvt_float_to_fp8((float)(x[d] / (double)sf), __NV_SATFINITE, __NV_E4M3);
      }
    }
  }
  return c;
}

inline std::vector<__half> dequant_head_f8(const KVCacheF8& c, int h, bool vside) {
  validate_cache_f8(c);
  w4::detail::require(h >= 0 && h < c.H, "dequant_head_f8: h");
  const auto& codes = vside ? c.q_v : c.q_k;
  const auto& scales = vside ? c.s_v : c.s_k;
  std::vector<__half> out((size_t)c.S * c.D);
  for (int t = 0; t < c.S; ++t) {
    const size_t row = (size_t)h * c.S + t;
    for (int d = 0; d < c.D; ++d)
      out[(size_t)t * c.D + d] = dequant_one_f8(scales[row * c.G + d / c.gs], codes[row * c.D + d]);
  }
  return out;
}

inline std::vector<double> attention_reference_f8(const std::vector<__half>& q, const KVCacheF8& c) {
  validate_cache_f8(c);
  w4::detail::require(q.size() == (size_t)c.H * c.D, "attention_reference_f8: q size");
  std::vector<double> out((size_t)c.H * c.D, 0.0);
  for (int h = 0; h < c.H; ++h)
    w4::kv::detail::attend(q.data() + (size_t)h * c.D, dequant_head_f8(c, h, false), dequant_head_f8(c, h, true),
                           c.S, c.D, out.data() + (size_t)h * c.D);
  return out;
}

}  // namespace w4::kv8
