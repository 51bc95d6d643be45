#pragma once
// Drop-in host header: the MXFP4 packed format (E2M1 elements, one E8M0 scale per
// 32-element block), its host quantizer and reference dequantisation, with the
// names and contracts of the reference's include/w4/mx.hpp (MX_BLOCK :36, kE2M1
// :39, PackedWm :41-45, dequant_one_mx :56-63, blocks :65, quantize_mx :71-119,
// validate_packed_mx :121-129, dequant_all_mx :131-140).
//
//   q       codes packed like the W4 format; code = sign << 3 | magnitude index
//   scales  one byte per (row, block): value 2^(byte - 127); 255 is never produced
//   value   w = 2^(byte-127) * {0, .5, 1, 1.5, 2, 3, 4, 6}[code & 7], negated when code & 8
#include <cuda_fp16.h>

#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <vector>

#include "pack.hpp"

namespace w4::mx {

constexpr int MX_BLOCK = 32;
constexpr float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

struct PackedWm {
  int N = 0, K = 0, B = 0;
  std::vector<uint32_t> q;
  std::vector<uint8_t> scales;
};

// Branch-free decode (no table indexed at run time): exponent field ee = idx >> 1,
// mantissa m = idx & 1; ee == 0 is the subnormal m/2, otherwise (2 + m) * 2^(ee-2).
// The sign goes onto the magnitude, so code 8 is minus zero. One rounding to FP16.
W4_HD inline __half dequant_one_mx(uint8_t se, int q) {
  const int idx = q & 7, ee = idx >> 1, m = idx & 1;
  const float mag = ee == 0 ? ldexpf((float)m, -1) : ldexpf((float)(2 + m), ee - 2);
  const float scale = ldexpf(1.0f, (int)se - 127);
  return __float2half_rn(scale * ((q & 8) ? -mag : mag));
}

W4_HD inline int blocks(int K) { return (K + MX_BLOCK - 1) / MX_BLOCK; }

inline int get_q(const PackedWm& p, int n, int k) { return w4::detail::code_at(p.q, (size_t)words(p.K), n, k); }

inline PackedWm quantize_mx(const std::vector<double>& w, int N, int K) {
  using w4::detail::require;
  require(N >= 1 && K >= 1, "quantize_mx: bad dims");
  require(w.size() == (size_t)N * (size_t)K, "quantize_mx: size");
  for (const double v : w) require(std::isfinite(v), "quantize_mx: non-finite input");
  PackedWm p;
  p.N = N;
  p.K = K;
  p.B = blocks(K);
  p.q.assign((size_t)N * words(K), 0u);
  p.scales.assign((size_t)N * p.B, 0);
  for (int n = 0; n < N; ++n) {
    const double* row = w.data() + (size_t)n * K;
    for (int b = 0; b < p.B; ++b) {
      const int k0 = b * MX_BLOCK, k1 = std::min(K, k0 + MX_BLOCK);
      double amax = 0.0;
      for (int k = k0; k < k1; ++k) amax = std::max(amax, std::fabs(row[k]));
      // smallest power of two with amax / 2^e <= 6: no element saturates
      int e = 0;
      if (amax > 0.0) {
        e = (int)std::ceil(std::log2(amax / 6.0));
        while (amax > 6.0 * std::ldexp(1.0, e)) ++e;  // log2 may land one low at exact powers of two
        require(e <= 127, "quantize_mx: block scale outside E8M0 range");
        e = std::max(e, -127);
      }
      p.scales[(size_t)n * p.B + b] = (uint8_t)(e + 127);
      const double s = std::ldexp(1.0, e);
      for (int k = k0; k < k1; ++k) {
        const double v = row[k] / s, av = std::fabs(v);
        int best = 0;  // nearest magnitude; a tie keeps the lower index
        for (int i = 1; i < 8; ++i)
          if (std::fabs((double)kE2M1[i] - av) < std::fabs((double)kE2M1[best] - av)) best = i;
        w4::detail::put_code(p.q, (size_t)words(K), n, k, (std::signbit(v) ? 8 : 0) | best);
      }
    }
  }
  return p;
}

inline void validate_packed_mx(const PackedWm& p) {
  using w4::detail::require;
  require(p.N >= 1 && p.K >= 1, "packed mx: bad dims");
  require(p.B == blocks(p.K), "packed mx: B inconsistent with K");
  require(p.q.size() == (size_t)p.N * (size_t)words(p.K), "packed mx: q size");
  require(p.scales.size() == (size_t)p.N * (size_t)p.B, "packed mx: scales size");
}

inline std::vector<__half> dequant_all_mx(const PackedWm& p) {
  validate_packed_mx(p);
  std::vector<__half> out((size_t)p.N * p.K);
  for (int n = 0; n < p.N; ++n)
    for (int k = 0; k < p.K; ++k)
      out[(size_t)n * p.K + k] = dequant_one_mx(p.scales[(size_t)n * p.B + k / MX_BLOCK], get_q(p, n, k));
  return out;
}

}  // namespace w4::mx
