/*
 * CPU oracle for the fused-dequant hot path: packed W4 / MXFP4 weight formats,
 * W4 / FP8-E4M3 / paged-W4 KV caches, reference dequantisation and the FP64
 * GEMM / decode-attention references.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is a plain-C restatement of the
 * reference project's host-side algorithms, used only as the checker in the
 * test-suite, in the smoke check and as the timed CPU baseline of the
 * benchmark. Nothing in the shipped GPU path links, loads or calls it.
 *
 * Parity is pinned: the restatement is compared bit-for-bit against the
 * reference's own headers compiled into a shared object (oracle/ref_shim.cpp,
 * built where the reference tree is present) and against committed golden
 * vectors produced by that shared object (tests/golden).
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the reference project's root). All functions return 0 on success and
 * ORC_INVALID (1) where the reference throws std::invalid_argument.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_OK 0
#define ORC_INVALID 1

/* ------------------------------------------------------------------------ */
/* IEEE binary16 <-> binary32, round-to-nearest-even.                        */
/* Stand-ins for the toolkit's host __float2half_rn / __half2float, which    */
/* the reference calls at include/w4/pack.hpp:59,106-107.                    */
/* ------------------------------------------------------------------------ */

uint16_t orc_f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t absx = x & 0x7FFFFFFFu;
  if (absx > 0x7F800000u) return (uint16_t)(sign | 0x7FFFu); /* NaN (toolkit's canonical) */
  if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* >= 65520 rounds to inf */
  if (absx < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25 rounds to zero */
  const int e = (int)(absx >> 23) - 127;                      /* unbiased exponent */
  uint32_t mant = (absx & 0x7FFFFFu) | 0x800000u;             /* 24-bit significand */
  int shift;                                                  /* bits dropped */
  uint32_t base;
  if (e >= -14) { /* normal half */
    shift = 13;
    base = (uint32_t)(e + 15) << 10;
    mant &= 0x7FFFFFu; /* implicit bit goes into the exponent field */
  } else {        /* subnormal half: value = mant * 2^(e-23), unit 2^-24 */
    shift = 13 + (-14 - e);
    base = 0;
  }
  uint32_t q = mant >> shift;
  const uint32_t rem = mant & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q += 1; /* carries ripple into the exponent */
  return (uint16_t)(sign | (base + q));
}

float orc_f16_to_f32(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 0x1Fu;
  const uint32_t m = h & 0x3FFu;
  uint32_t x;
  if (e == 0) {
    if (m == 0) {
      x = sign;
    } else { /* subnormal: renormalise */
      int k = 0;
      uint32_t mm = m;
      while (!(mm & 0x400u)) {
        mm <<= 1;
        ++k;
      }
      x = sign | ((uint32_t)(127 - 15 + 1 - k) << 23) | ((mm & 0x3FFu) << 13);
    }
  } else if (e == 31) {
    x = sign | 0x7F800000u | (m << 13);
  } else {
    x = sign | ((e + 112u) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &x, 4);
  return f;
}

/* ------------------------------------------------------------------------ */
/* Seeded inputs: 64-bit Mersenne twister + polar-method normal deviates,    */
/* the same stream std::mt19937_64 + std::normal_distribution<double>(0,1)   */
/* produce in the reference's generators (include/w4/pack.hpp:186-200).      */
/* ------------------------------------------------------------------------ */

typedef struct {
  uint64_t mt[312];
  int idx;
  int have_saved;
  double saved;
} orc_rng;

static void rng_seed(orc_rng* r, uint64_t seed) {
  r->mt[0] = seed;
  for (int i = 1; i < 312; ++i)
    r->mt[i] = 6364136223846793005ULL * (r->mt[i - 1] ^ (r->mt[i - 1] >> 62)) + (uint64_t)i;
  r->idx = 312;
  r->have_saved = 0;
  r->saved = 0.0;
}

static uint64_t rng_u64(orc_rng* r) {
  if (r->idx >= 312) {
    for (int i = 0; i < 312; ++i) {
      const uint64_t y = (r->mt[i] & 0xFFFFFFFF80000000ULL) | (r->mt[(i + 1) % 312] & 0x7FFFFFFFULL);
      r->mt[i] = r->mt[(i + 156) % 312] ^ (y >> 1) ^ ((y & 1ULL) ? 0xB5026F5AA96619E9ULL : 0ULL);
    }
    r->idx = 0;
  }
  uint64_t y = r->mt[r->idx++];
  y ^= (y >> 29) & 0x5555555555555555ULL;
  y ^= (y << 17) & 0x71D67FFFEDA60000ULL;
  y ^= (y << 37) & 0xFFF7EEE000000000ULL;
  y ^= (y >> 43);
  return y;
}

/* One 64-bit draw mapped to [0,1): draw / 2^64 in double, clamped below 1. */
static double rng_unit(orc_rng* r) {
  double u = (double)rng_u64(r) / 18446744073709551616.0;
  if (u >= 1.0) u = nextafter(1.0, 0.0);
  return u;
}

static double rng_normal(orc_rng* r) {
  if (r->have_saved) {
    r->have_saved = 0;
    return r->saved;
  }
  double x, y, r2;
  do {
    x = 2.0 * rng_unit(r) - 1.0;
    y = 2.0 * rng_unit(r) - 1.0;
    r2 = x * x + y * y;
  } while (r2 > 1.0 || r2 == 0.0);
  const double mult = sqrt(-2.0 * log(r2) / r2);
  r->saved = x * mult;
  r->have_saved = 1;
  return y * mult;
}

/* normal_weights (pack.hpp:186-192): count N(0,1) doubles. */
void orc_normal_f64(double* out, size_t count, uint64_t seed) {
  orc_rng r;
  rng_seed(&r, seed);
  for (size_t i = 0; i < count; ++i) out[i] = rng_normal(&r);
}

/* normal_activations (pack.hpp:194-200): N(0,1) rounded through float to FP16. */
void orc_normal_f16(uint16_t* out, size_t count, uint64_t seed) {
  orc_rng r;
  rng_seed(&r, seed);
  for (size_t i = 0; i < count; ++i) out[i] = orc_f32_to_f16((float)rng_normal(&r));
}

/* ------------------------------------------------------------------------ */
/* W4 packed format (pack.hpp:33-60).                                        */
/* ------------------------------------------------------------------------ */

int orc_words(int n) { return (n + 7) / 8; } /* pack.hpp:33 */

static int nib(const uint32_t* base, size_t word0, int idx) { /* pack.hpp:43-49 */
  return (int)((base[word0 + (size_t)(idx / 8)] >> (4 * (idx % 8))) & 0xF);
}

/* dequant_one (pack.hpp:58-60): float product, one RNE rounding to FP16. */
uint16_t orc_dequant_one(uint16_t s, int q, int z) {
  return orc_f32_to_f16(orc_f16_to_f32(s) * (float)(q - z));
}

static double dmin(double a, double b) { return b < a ? b : a; } /* std::min */
static double dmax(double a, double b) { return a < b ? b : a; } /* std::max */

/* quantize (pack.hpp:64-130). q: N*words(K), scales: N*G, zeros: N*words(G)
 * (asymmetric only; may be NULL when symmetric). Outputs are fully written. */
int orc_quantize_w4(const double* w, int N, int K, int gs, int symmetric, uint32_t* q,
                    uint16_t* scales, uint32_t* zeros) {
  if (N < 1 || K < 1) return ORC_INVALID;
  if (gs < 8 || gs % 8 != 0) return ORC_INVALID;
  const size_t total = (size_t)N * (size_t)K;
  for (size_t i = 0; i < total; ++i)
    if (!isfinite(w[i])) return ORC_INVALID;
  const int G = (K + gs - 1) / gs;
  const int wk = orc_words(K), wg = orc_words(G);
  memset(q, 0, (size_t)N * wk * sizeof(uint32_t));
  for (size_t i = 0; i < (size_t)N * G; ++i) scales[i] = 0;
  if (!symmetric) memset(zeros, 0, (size_t)N * wg * sizeof(uint32_t));

  for (int n = 0; n < N; ++n) {
    const double* row = w + (size_t)n * K;
    for (int g = 0; g < G; ++g) {
      const int k0 = g * gs, k1 = (k0 + gs < K) ? k0 + gs : K;
      double lo = row[k0], hi = lo;
      for (int k = k0 + 1; k < k1; ++k) {
        lo = dmin(lo, row[k]);
        hi = dmax(hi, row[k]);
      }
      if (!symmetric) { /* bracket zero (pack.hpp:93-98) */
        lo = dmin(lo, 0.0);
        hi = dmax(hi, 0.0);
      }
      double s;
      if (symmetric) {
        const double amax = dmax(fabs(lo), fabs(hi));
        s = amax > 0.0 ? amax / 7.0 : 1.0;
      } else {
        s = hi > lo ? (hi - lo) / 15.0 : 1.0;
      }
      const uint16_t sh = orc_f32_to_f16((float)s);
      const float sf = orc_f16_to_f32(sh);
      const int nonzero = symmetric ? (lo != 0.0 || hi != 0.0) : (hi != lo);
      if (!isfinite(sf) || (sf == 0.0f && nonzero)) return ORC_INVALID; /* pack.hpp:110-112 */
      int z = 8;
      if (!symmetric) {
        z = (int)lround(-lo / (double)sf);
        z = z < 0 ? 0 : (z > 15 ? 15 : z);
      }
      scales[(size_t)n * G + g] = sh;
      for (int k = k0; k < k1; ++k) {
        int c = (int)lround(row[k] / (double)sf) + z;
        c = c < 0 ? 0 : (c > 15 ? 15 : c);
        q[(size_t)n * wk + k / 8] |= (uint32_t)c << (4 * (k % 8));
      }
      if (!symmetric) zeros[(size_t)n * wg + g / 8] |= (uint32_t)z << (4 * (g % 8));
    }
  }
  return ORC_OK;
}

/* validate_packed (pack.hpp:134-148), minus the container-size checks that
 * have no meaning for raw pointers; the pointer/mode pairing stands in for
 * "symmetric carries no zeros". */
static int w4_shape_ok(int N, int K, int gs, int G, int symmetric, const uint32_t* q,
                       const uint16_t* scales, const uint32_t* zeros) {
  if (N < 1 || K < 1) return 0;
  if (gs < 8 || gs % 8 != 0) return 0;
  if (G != (K + gs - 1) / gs) return 0;
  if (!q || !scales) return 0;
  if (!symmetric && !zeros) return 0;
  if (symmetric && zeros) return 0;
  return 1;
}

/* dequant_all (pack.hpp:150-161): w is N*K FP16, the bitwise target. */
int orc_dequant_all_w4(int N, int K, int gs, int G, int symmetric, const uint32_t* q,
                       const uint16_t* scales, const uint32_t* zeros, uint16_t* w) {
  if (!w4_shape_ok(N, K, gs, G, symmetric, q, scales, zeros) || !w) return ORC_INVALID;
  const int wk = orc_words(K), wg = orc_words(G);
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const int g = k / gs;
      const int z = symmetric ? 8 : nib(zeros, (size_t)n * wg, g);
      w[(size_t)n * K + k] = orc_dequant_one(scales[(size_t)n * G + g], nib(q, (size_t)n * wk, k), z);
    }
  return ORC_OK;
}

/* gemm_oracle (pack.hpp:166-184): C[m,n] = sum_k x[m,k]*w[n,k], FP64, k ascending. */
static void gemm_rows(const uint16_t* x, int M, int K, const uint16_t* w, int N, int n0, int n1,
                      double* c) {
  /* widen x once; the per-element products are unchanged */
  double* xd = (double*)malloc((size_t)M * K * sizeof(double));
  for (size_t i = 0; i < (size_t)M * K; ++i) xd[i] = (double)orc_f16_to_f32(x[i]);
  double* wd = (double*)malloc((size_t)K * sizeof(double));
  for (int n = n0; n < n1; ++n) {
    for (int k = 0; k < K; ++k) wd[k] = (double)orc_f16_to_f32(w[(size_t)n * K + k]);
    for (int m = 0; m < M; ++m) {
      double acc = 0.0;
      const double* xr = xd + (size_t)m * K;
      for (int k = 0; k < K; ++k) acc += xr[k] * wd[k];
      c[(size_t)m * N + n] = acc;
    }
  }
  free(wd);
  free(xd);
}

int orc_gemm_oracle(const uint16_t* x, int M, int K, const uint16_t* w, int N, double* c) {
  if (M < 1 || N < 1 || K < 1 || !x || !w || !c) return ORC_INVALID;
  gemm_rows(x, M, K, w, N, 0, N, c);
  return ORC_OK;
}

typedef struct {
  const uint16_t* x;
  const uint16_t* w;
  double* c;
  int M, K, N, n0, n1;
} gemm_job;

static void* gemm_thread(void* arg) {
  gemm_job* j = (gemm_job*)arg;
  gemm_rows(j->x, j->M, j->K, j->w, j->N, j->n0, j->n1, j->c);
  return NULL;
}

/* Row-parallel gemm_oracle: every c[m,n] is still one in-order k-sum, so the
 * result is bit-identical to the serial function for any thread count. */
int orc_gemm_oracle_mt(const uint16_t* x, int M, int K, const uint16_t* w, int N, double* c,
                       int threads) {
  if (M < 1 || N < 1 || K < 1 || !x || !w || !c) return ORC_INVALID;
  if (threads < 1) threads = 1;
  if (threads > N) threads = N;
  if (threads > 256) threads = 256;
  pthread_t tid[256];
  gemm_job job[256];
  for (int t = 0; t < threads; ++t) {
    job[t] = (gemm_job){x, w, c, M, K, N, (int)((int64_t)N * t / threads),
                        (int)((int64_t)N * (t + 1) / threads)};
    pthread_create(&tid[t], NULL, gemm_thread, &job[t]);
  }
  for (int t = 0; t < threads; ++t) pthread_join(tid[t], NULL);
  return ORC_OK;
}

/* ------------------------------------------------------------------------ */
/* MXFP4 (include/w4/mx.hpp).                                                */
/* ------------------------------------------------------------------------ */

static const double kMag[8] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0}; /* mx.hpp:39 */

int orc_blocks(int K) { return (K + 31) / 32; } /* mx.hpp:65 */

/* dequant_one_mx (mx.hpp:56-63): exact float product 2^(se-127) * e2m1, the
 * sign applied to the magnitude (code 8 is -0), one RNE rounding to FP16. */
uint16_t orc_dequant_one_mx(uint8_t se, int q) {
  const int i = q & 7;
  const float mag = (i >> 1) == 0 ? ldexpf((float)(i & 1), -1) : ldexpf((float)(2 + (i & 1)), (i >> 1) - 2);
  const float s = ldexpf(1.0f, (int)se - 127);
  const float v = (q & 8) ? -mag : mag;
  return orc_f32_to_f16(s * v);
}

/* quantize_mx (mx.hpp:71-119). q: N*words(K), scales: N*blocks(K) E8M0 bytes. */
int orc_quantize_mx(const double* w, int N, int K, uint32_t* q, uint8_t* scales) {
  if (N < 1 || K < 1) return ORC_INVALID;
  const size_t total = (size_t)N * (size_t)K;
  for (size_t i = 0; i < total; ++i)
    if (!isfinite(w[i])) return ORC_INVALID;
  const int B = orc_blocks(K), wk = orc_words(K);
  memset(q, 0, (size_t)N * wk * sizeof(uint32_t));
  memset(scales, 0, (size_t)N * B);
  for (int n = 0; n < N; ++n) {
    const double* row = w + (size_t)n * K;
    for (int b = 0; b < B; ++b) {
      const int k0 = b * 32, k1 = (k0 + 32 < K) ? k0 + 32 : K;
      double amax = 0.0;
      for (int k = k0; k < k1; ++k) amax = dmax(amax, fabs(row[k]));
      int e = 0;
      if (amax > 0.0) {
        e = (int)ceil(log2(amax / 6.0));
        while (amax > 6.0 * ldexp(1.0, e)) ++e; /* no-saturation insurance (mx.hpp:93-96) */
        if (e > 127) return ORC_INVALID;
        if (e < -127) e = -127;
      }
      const double s = ldexp(1.0, e);
      scales[(size_t)n * B + b] = (uint8_t)(e + 127);
      for (int k = k0; k < k1; ++k) {
        const double v = row[k] / s;
        const double av = fabs(v);
        int idx = 0; /* nearest magnitude, ties to the lower index (mx.hpp:108-112) */
        for (int i = 1; i < 8; ++i)
          if (fabs(kMag[i] - av) < fabs(kMag[idx] - av)) idx = i;
        const int code = (signbit(v) ? 8 : 0) | idx;
        q[(size_t)n * wk + k / 8] |= (uint32_t)code << (4 * (k % 8));
      }
    }
  }
  return ORC_OK;
}

/* dequant_all_mx (mx.hpp:131-140) with validate_packed_mx's shape rules (:121-129). */
int orc_dequant_all_mx(int N, int K, int B, const uint32_t* q, const uint8_t* scales, uint16_t* w) {
  if (N < 1 || K < 1 || B != orc_blocks(K) || !q || !scales || !w) return ORC_INVALID;
  const int wk = orc_words(K);
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k)
      w[(size_t)n * K + k] = orc_dequant_one_mx(scales[(size_t)n * B + k / 32], nib(q, (size_t)n * wk, k));
  return ORC_OK;
}

/* ------------------------------------------------------------------------ */
/* W4 KV cache (include/w4/kvcache.hpp): H slabs of the W4 format, rows are  */
/* positions, the packed axis is the head dimension.                         */
/* ------------------------------------------------------------------------ */

/* quantize_cache (kvcache.hpp:60-108): per-head quantize of both sides.
 * k, v: H*S*D doubles. Outputs per side: q H*S*words(D), s H*S*G, z H*S*words(G). */
int orc_quantize_cache_w4(const double* k, const double* v, int H, int S, int D, int gs,
                          int symmetric, uint32_t* q_k, uint16_t* s_k, uint32_t* z_k,
                          uint32_t* q_v, uint16_t* s_v, uint32_t* z_v) {
  if (H < 1 || S < 1 || D < 1) return ORC_INVALID;
  if (gs < 8 || gs % 8 != 0) return ORC_INVALID;
  const int G = (D + gs - 1) / gs;
  const size_t oq = (size_t)S * orc_words(D), os = (size_t)S * G, oz = (size_t)S * orc_words(G);
  for (int h = 0; h < H; ++h) {
    const size_t src = (size_t)h * S * D;
    int rc = orc_quantize_w4(k + src, S, D, gs, symmetric, q_k + h * oq, s_k + h * os,
                             symmetric ? NULL : z_k + h * oz);
    if (rc) return rc;
    rc = orc_quantize_w4(v + src, S, D, gs, symmetric, q_v + h * oq, s_v + h * os,
                         symmetric ? NULL : z_v + h * oz);
    if (rc) return rc;
  }
  return ORC_OK;
}

/* dequant_head (kvcache.hpp:111-135) for every head: out is H*S*D FP16. */
int orc_dequant_cache_w4(int H, int S, int D, int gs, int G, int symmetric, const uint32_t* q,
                         const uint16_t* s, const uint32_t* z, uint16_t* out) {
  if (H < 1 || S < 1 || D < 1) return ORC_INVALID;
  const size_t oq = (size_t)S * orc_words(D), os = (size_t)S * G, oz = (size_t)S * orc_words(G);
  for (int h = 0; h < H; ++h) {
    const int rc = orc_dequant_all_w4(S, D, gs, G, symmetric, q + h * oq, s + h * os,
                                      symmetric ? NULL : z + h * oz, out + (size_t)h * S * D);
    if (rc) return rc;
  }
  return ORC_OK;
}

/* attention_reference (kvcache.hpp:141-175) and attention_reference_f8
 * (kvfp8.hpp:150-184) share this body: FP64 scores / sqrt(D), max-subtracted
 * softmax, sum_t p_t v_t, over the dequantised (FP16-exact) K and V [H][S][D]. */
static void attn_heads(const uint16_t* q, const uint16_t* kd, const uint16_t* vd, int h0, int h1,
                       int S, int D, double* out) {
  const double inv_sqrt_d = 1.0 / sqrt((double)D);
  double* scores = (double*)malloc((size_t)S * sizeof(double));
  for (int h = h0; h < h1; ++h) {
    const uint16_t* kh = kd + (size_t)h * S * D;
    const uint16_t* vh = vd + (size_t)h * S * D;
    double smax = -INFINITY;
    for (int t = 0; t < S; ++t) {
      double acc = 0.0;
      for (int d = 0; d < D; ++d)
        acc += (double)orc_f16_to_f32(q[(size_t)h * D + d]) * (double)orc_f16_to_f32(kh[(size_t)t * D + d]);
      scores[t] = acc * inv_sqrt_d;
      smax = dmax(smax, scores[t]);
    }
    double denom = 0.0;
    for (int t = 0; t < S; ++t) {
      scores[t] = exp(scores[t] - smax);
      denom += scores[t];
    }
    for (int t = 0; t < S; ++t) scores[t] /= denom;
    for (int d = 0; d < D; ++d) {
      double acc = 0.0;
      for (int t = 0; t < S; ++t) acc += scores[t] * (double)orc_f16_to_f32(vh[(size_t)t * D + d]);
      out[(size_t)h * D + d] = acc;
    }
  }
  free(scores);
}

typedef struct {
  const uint16_t *q, *kd, *vd;
  double* out;
  int h0, h1, S, D;
} attn_job;

static void* attn_thread(void* arg) {
  attn_job* j = (attn_job*)arg;
  attn_heads(j->q, j->kd, j->vd, j->h0, j->h1, j->S, j->D, j->out);
  return NULL;
}

/* Heads are independent, so the head-parallel run is bit-identical to serial. */
int orc_attention_reference(const uint16_t* q, const uint16_t* kd, const uint16_t* vd, int H, int S,
                            int D, double* out, int threads) {
  if (H < 1 || S < 1 || D < 1 || !q || !kd || !vd || !out) return ORC_INVALID;
  if (threads < 1) threads = 1;
  if (threads > H) threads = H;
  if (threads > 256) threads = 256;
  pthread_t tid[256];
  attn_job job[256];
  for (int t = 0; t < threads; ++t) {
    job[t] = (attn_job){q, kd, vd, out, (int)((int64_t)H * t / threads),
                        (int)((int64_t)H * (t + 1) / threads), S, D};
    pthread_create(&tid[t], NULL, attn_thread, &job[t]);
  }
  for (int t = 0; t < threads; ++t) pthread_join(tid[t], NULL);
  return ORC_OK;
}

/* ------------------------------------------------------------------------ */
/* FP8 E4M3 KV cache (include/w4/kvfp8.hpp).                                 */
/* ------------------------------------------------------------------------ */

/* decode_f8_e4m3 (kvfp8.hpp:42-47): exact in float. */
float orc_decode_e4m3(uint8_t b) {
  const int e = (b >> 3) & 0xF, m = b & 7;
  const float mag = (e == 0) ? ldexpf((float)m, -9) : ldexpf((float)(8 + m), e - 10);
  return (b & 0x80) ? -mag : mag;
}

/* dequant_one_f8 (kvfp8.hpp:51-53). */
uint16_t orc_dequant_one_f8(uint16_t s, uint8_t b) {
  return orc_f32_to_f16(orc_f16_to_f32(s) * orc_decode_e4m3(b));
}

/* float -> E4M3, round-to-nearest-even, saturate-to-finite: the conversion the
 * quantizer takes from the toolkit at kvfp8.hpp:119-121. Magnitudes above
 * 448 + half an ulp (464) clamp to 0x7E; at or below half the smallest
 * subnormal (2^-10) they become zero; the sign bit is always carried. */
uint8_t orc_encode_e4m3(float x) {
  uint32_t xb;
  memcpy(&xb, &x, 4);
  const uint8_t sign = (uint8_t)((xb >> 31) << 7);
  if ((xb & 0x7FFFFFFFu) > 0x7F800000u) return (uint8_t)(sign | 0x7F);
  const double a = fabs((double)x);
  uint8_t code;
  if (a <= ldexp(1.0, -10)) {
    code = 0;
  } else if (a > 464.0) {
    code = 0x7E;
  } else if (a >= ldexp(1.0, -6)) {
    int ex;
    const double fr = frexp(a, &ex); /* a = fr * 2^ex, fr in [0.5, 1) */
    int e = ex - 1;                  /* a = m * 2^e,  m in [1, 2)    */
    int r = (int)nearbyint((fr * 2.0 - 1.0) * 8.0); /* ties to even under the default mode */
    if (r == 8) {
      r = 0;
      ++e;
    }
    code = (uint8_t)(((e + 7) << 3) | r);
  } else {
    code = (uint8_t)nearbyint(a * 512.0); /* units of 2^-9; 8 lands on the first normal */
  }
  return (uint8_t)(code | sign);
}

/* quantize_cache_f8 (kvfp8.hpp:70-128). k, v: H*S*D doubles; outputs per side:
 * bytes H*S*D, scales H*S*G. */
int orc_quantize_cache_f8(const double* k, const double* v, int H, int S, int D, int gs,
                          uint8_t* q_k, uint16_t* s_k, uint8_t* q_v, uint16_t* s_v) {
  if (H < 1 || S < 1 || D < 1) return ORC_INVALID;
  if (gs < 8 || gs % 8 != 0) return ORC_INVALID;
  const size_t total = (size_t)H * S * D;
  for (size_t i = 0; i < total; ++i)
    if (!isfinite(k[i])) return ORC_INVALID;
  for (size_t i = 0; i < total; ++i)
    if (!isfinite(v[i])) return ORC_INVALID;
  const int G = (D + gs - 1) / gs;
  for (int side = 0; side < 2; ++side) {
    const double* src = side ? v : k;
    uint8_t* qc = side ? q_v : q_k;
    uint16_t* sc = side ? s_v : s_k;
    for (size_t row = 0; row < (size_t)H * S; ++row) {
      const double* base = src + row * D;
      for (int g = 0; g < G; ++g) {
        const int d0 = g * gs, d1 = (d0 + gs < D) ? d0 + gs : D;
        double amax = 0.0;
        for (int d = d0; d < d1; ++d) amax = dmax(amax, fabs(base[d]));
        const double s = amax > 0.0 ? amax / 448.0 : 1.0;
        const uint16_t sh = orc_f32_to_f16((float)s);
        const float sf = orc_f16_to_f32(sh);
        if (!isfinite(sf) || (sf == 0.0f && amax > 0.0)) return ORC_INVALID;
        sc[row * G + g] = sh;
        for (int d = d0; d < d1; ++d) qc[row * D + d] = orc_encode_e4m3((float)(base[d] / (double)sf));
      }
    }
  }
  return ORC_OK;
}

/* dequant_head_f8 (kvfp8.hpp:131-146) for every head: out is H*S*D FP16. */
int orc_dequant_cache_f8(int H, int S, int D, int gs, int G, const uint8_t* q, const uint16_t* s,
                         uint16_t* out) {
  if (H < 1 || S < 1 || D < 1 || gs < 8 || gs % 8 != 0 || G != (D + gs - 1) / gs) return ORC_INVALID;
  if (!q || !s || !out) return ORC_INVALID;
  for (size_t row = 0; row < (size_t)H * S; ++row)
    for (int d = 0; d < D; ++d) out[row * D + d] = orc_dequant_one_f8(s[row * G + d / gs], q[row * D + d]);
  return ORC_OK;
}

/* ------------------------------------------------------------------------ */
/* Paged W4 KV cache (include/w4/kvpaged.hpp).                               */
/* ------------------------------------------------------------------------ */

/* paged_from_contiguous (kvpaged.hpp:72-134): logical page i of every head
 * lands at physical page bt[i]; the pool has exactly lpages = ceil(S/page)
 * pages per head and rows past S in the last page stay zero. `row_words` is
 * the number of 32-bit (or 16-bit, via `elem`) elements per position, so the
 * same routine scatters codes, scales and zeros. */
int orc_paged_scatter(const void* src, void* dst, int H, int S, int page, const int* bt,
                      int row_elems, int elem_bytes) {
  if (H < 1 || S < 1 || page < 1 || !src || !dst || !bt) return ORC_INVALID;
  const size_t lpages = ((size_t)S + (size_t)page - 1) / (size_t)page;
  char* seen = (char*)calloc(lpages, 1);
  for (size_t i = 0; i < lpages; ++i) {
    if (bt[i] < 0 || (size_t)bt[i] >= lpages || seen[bt[i]]++) {
      free(seen);
      return ORC_INVALID; /* kvpaged.hpp:81-84 */
    }
  }
  free(seen);
  const size_t rb = (size_t)row_elems * elem_bytes;
  const size_t pool_rows = lpages * (size_t)page;
  memset(dst, 0, (size_t)H * pool_rows * rb);
  for (int h = 0; h < H; ++h)
    for (size_t lp = 0; lp < lpages; ++lp)
      for (int j = 0; j < page; ++j) {
        const size_t t = lp * page + j;
        if (t >= (size_t)S) break;
        const size_t drow = (size_t)bt[lp] * page + j;
        memcpy((char*)dst + ((size_t)h * pool_rows + drow) * rb,
               (const char*)src + ((size_t)h * S + t) * rb, rb);
      }
  return ORC_OK;
}

/* validate_paged's block-table rules (kvpaged.hpp:36-67): table length is
 * ceil(S/page) by construction here; entries in [0, npages), no repeats,
 * pool at least as large as the table. */
int orc_validate_block_table(const int* bt, int S, int page, int npages) {
  if (S < 1 || page < 1 || npages < 1 || !bt) return ORC_INVALID;
  const size_t lpages = ((size_t)S + (size_t)page - 1) / (size_t)page;
  if ((size_t)npages < lpages) return ORC_INVALID;
  char* seen = (char*)calloc((size_t)npages, 1);
  int rc = ORC_OK;
  for (size_t i = 0; i < lpages; ++i)
    if (bt[i] < 0 || bt[i] >= npages || seen[bt[i]]++) {
      rc = ORC_INVALID;
      break;
    }
  free(seen);
  return rc;
}
