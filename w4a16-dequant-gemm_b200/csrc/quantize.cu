// Device-side quantizers: the reference's host quantizers (quantize, include/w4/pack.hpp:64-130; quantize_mx,
// include/w4/mx.hpp:71-119; the per-side loop of quantize_cache_f8, include/w4/kvfp8.hpp:70-128) as CUDA kernels
// that produce the same bits from the same values, plus the append of one token's K / V rows to a (paged) W4 or
// FP8 cache - what a decode loop needs between two attention calls (the reference quantises caches on the host
// only, include/w4/kvcache.hpp:60-108).
//
// The arithmetic is the host's, operation for operation, in FP64: group minimum / maximum (order-independent),
// scale = amax / 7 or (hi - lo) / 15 rounded through float to FP16, zero point and codes by lround of the FP64
// quotient against the stored scale. Inputs are FP64 (what the host quantizers take) or FP16 (what a model
// produces; converted exactly). A value the host quantizer throws on (NaN / infinity, a scale that overflows FP16
// or underflows to zero on a non-zero group, an MX exponent above 127) cannot throw here: the kernel records
// ST_QUANT_INVALID in the device status word, which w4b_device_status() returns, and the group's output is zero.
//
// One warp per (row, group). Rows are written at row * out_mul + out_add of the destination, so the same kernels
// fill a whole matrix (1, 0) and one position of every head slab of a cache (slab rows, position's row).
#include <cuda_fp8.h>

#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {
namespace {

constexpr int QZ_WARPS = 8;

template <typename T>
__device__ __forceinline__ double as_f64(T v);
template <>
__device__ __forceinline__ double as_f64<double>(double v) {
  return v;
}
template <>
__device__ __forceinline__ double as_f64<__half>(__half v) {
  return (double)__half2float(v);
}

__device__ __forceinline__ double warp_min(double v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmin(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}
__device__ __forceinline__ double warp_max(double v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}

struct QuantRows {
  int N, K, gs, G;
  long long out_mul, out_add;  // destination row of source row n: n * out_mul + out_add
  int* status;
};

// W4: q rows of words(K) words, scales rows of G halves, zeros rows of words(G) words. The groups of a row share
// zero words: each replaces its own nibble atomically, and the row's last group clears the unused nibbles behind
// it, so the destination needs no clearing beforehand.
template <typename T>
__global__ void __launch_bounds__(32 * QZ_WARPS)
    quantize_w4_kernel(const T* __restrict__ w, QuantRows a, int symmetric, uint32_t* __restrict__ q,
                       __half* __restrict__ scales, uint32_t* __restrict__ zeros) {
  const long long item = (long long)blockIdx.x * QZ_WARPS + (threadIdx.x >> 5);
  if (item >= (long long)a.N * a.G) return;  // warp-uniform
  const int lane = threadIdx.x & 31;
  const int n = (int)(item / a.G), g = (int)(item - (long long)n * a.G);
  const int k0 = g * a.gs, k1 = min(k0 + a.gs, a.K);
  const T* row = w + (size_t)n * a.K;
  const long long orow = (long long)n * a.out_mul + a.out_add;
  const int wk = words(a.K), wg = words(a.G);

  double lo = as_f64(row[k0]), hi = lo;
  bool finite = true;
  for (int k = k0 + lane; k < k1; k += 32) {
    const double v = as_f64(row[k]);
    finite = finite && isfinite(v);
    lo = fmin(lo, v);
    hi = fmax(hi, v);
  }
  lo = warp_min(lo);
  hi = warp_max(hi);
  finite = __all_sync(0xffffffffu, finite);
  if (!symmetric) {  // bracket zero
    lo = fmin(lo, 0.0);
    hi = fmax(hi, 0.0);
  }
  double s;
  if (symmetric) {
    const double amax = fmax(fabs(lo), fabs(hi));
    s = amax > 0.0 ? amax / 7.0 : 1.0;
  } else {
    s = hi > lo ? (hi - lo) / 15.0 : 1.0;
  }
  const __half sh = __float2half_rn((float)s);
  const float sf = __half2float(sh);
  const bool nonzero = symmetric ? (lo != 0.0 || hi != 0.0) : (hi != lo);
  const bool bad = !finite || !isfinite(sf) || (sf == 0.0f && nonzero);
  if (bad && lane == 0) atomicExch(a.status, ST_QUANT_INVALID);
  int z = 8;
  if (!symmetric && !bad) {
    z = (int)lround(-lo / (double)sf);
    z = z < 0 ? 0 : (z > 15 ? 15 : z);
  }
  if (lane == 0) {
    scales[orow * a.G + g] = bad ? __ushort_as_half((unsigned short)0) : sh;
    if (!symmetric) {
      uint32_t* zw = zeros + orow * wg + (g >> 3);
      const int sh = 4 * (g & 7);
      atomicAnd(zw, ~(0xFu << sh));
      if (!bad) atomicOr(zw, (uint32_t)z << sh);
      if (g == a.G - 1 && (g & 7) != 7) atomicAnd(zw, (1u << (sh + 4)) - 1u);
    }
  }
  // codes: a lane builds whole words (the group starts on a word boundary: gs % 8 == 0)
  for (int w0 = (k0 >> 3) + lane; 8 * w0 < k1; w0 += 32) {
    uint32_t word = 0;
    if (!bad) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = 8 * w0 + j;
        if (k < k1) {
          int c = (int)lround(as_f64(row[k]) / (double)sf) + z;
          c = c < 0 ? 0 : (c > 15 ? 15 : c);
          word |= (uint32_t)c << (4 * j);
        }
      }
    }
    q[orow * wk + w0] = word;
  }
}

// MXFP4: warp per (row, 32-block), lane per element.
template <typename T>
__global__ void __launch_bounds__(32 * QZ_WARPS)
    quantize_mx_kernel(const T* __restrict__ w, QuantRows a, uint32_t* __restrict__ q, uint8_t* __restrict__ scales) {
  const long long item = (long long)blockIdx.x * QZ_WARPS + (threadIdx.x >> 5);
  if (item >= (long long)a.N * a.G) return;
  const int lane = threadIdx.x & 31;
  const int n = (int)(item / a.G), b = (int)(item - (long long)n * a.G);
  const int k = 32 * b + lane;
  const bool in = k < a.K;
  const double x = in ? as_f64(w[(size_t)n * a.K + k]) : 0.0;
  const bool finite = __all_sync(0xffffffffu, isfinite(x));
  const double amax = warp_max(fabs(x));
  // e = the smallest integer with 6 * 2^e >= amax: what ceil(log2(amax / 6)) followed by the reference's
  // no-saturation loop yields; worked out here without trusting the last bit of log2
  int e = 0;
  if (amax > 0.0) {
    e = (int)ceil(log2(amax / 6.0));
    while (amax > 6.0 * ldexp(1.0, e)) ++e;
    while (amax <= 6.0 * ldexp(1.0, e - 1)) --e;
  }
  const bool bad = !finite || e > 127;
  if (bad && lane == 0) atomicExch(a.status, ST_QUANT_INVALID);
  if (e < -127) e = -127;
  const long long orow = (long long)n * a.out_mul + a.out_add;
  if (lane == 0) scales[orow * a.G + b] = bad ? 0 : (uint8_t)(e + 127);
  uint32_t code = 0;
  if (in && !bad) {
    const double v = x / ldexp(1.0, e);
    const double av = fabs(v);
    const double mag[8] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0};
    int idx = 0;  // nearest magnitude, ties to the lower index
#pragma unroll
    for (int i = 1; i < 8; ++i)
      if (fabs(mag[i] - av) < fabs(mag[idx] - av)) idx = i;
    code = (uint32_t)((signbit(v) ? 8 : 0) | idx);
  }
  uint32_t word = code << (4 * (lane & 7));
  word |= __shfl_xor_sync(0xffffffffu, word, 1);
  word |= __shfl_xor_sync(0xffffffffu, word, 2);
  word |= __shfl_xor_sync(0xffffffffu, word, 4);
  if ((lane & 7) == 0 && 8 * (4 * b + (lane >> 3)) < a.K) q[orow * words(a.K) + 4 * b + (lane >> 3)] = word;
}

// FP8 E4M3 with an FP16 scale per (row, group): scale = amax / 448, codes by the toolkit's conversion
// (round to nearest even, saturate to finite), the call the reference makes on the host.
template <typename T>
__global__ void __launch_bounds__(32 * QZ_WARPS)
    quantize_f8_kernel(const T* __restrict__ x, QuantRows a, uint8_t* __restrict__ q, __half* __restrict__ scales) {
  const long long item = (long long)blockIdx.x * QZ_WARPS + (threadIdx.x >> 5);
  if (item >= (long long)a.N * a.G) return;
  const int lane = threadIdx.x & 31;
  const int n = (int)(item / a.G), g = (int)(item - (long long)n * a.G);
  const int d0 = g * a.gs, d1 = min(d0 + a.gs, a.K);
  const T* row = x + (size_t)n * a.K;
  double amax = 0.0;
  bool finite = true;
  for (int d = d0 + lane; d < d1; d += 32) {
    const double v = as_f64(row[d]);
    finite = finite && isfinite(v);
    amax = fmax(amax, fabs(v));
  }
  amax = warp_max(amax);
  finite = __all_sync(0xffffffffu, finite);
  const double s = amax > 0.0 ? amax / 448.0 : 1.0;
  const __half sh = __float2half_rn((float)s);
  const float sf = __half2float(sh);
  const bool bad = !finite || !isfinite(sf) || (sf == 0.0f && amax > 0.0);
  if (bad && lane == 0) atomicExch(a.status, ST_QUANT_INVALID);
  const long long orow = (long long)n * a.out_mul + a.out_add;
  if (lane == 0) scales[orow * a.G + g] = bad ? __ushort_as_half((unsigned short)0) : sh;
  for (int d = d0 + lane; d < d1; d += 32)
    q[orow * a.K + d] = bad ? 0 : (uint8_t)__nv_cvt_float_to_fp8((float)(as_f64(row[d]) / (double)sf), __NV_SATFINITE, __NV_E4M3);
}

unsigned blocks_for(long long items) { return (unsigned)((items + QZ_WARPS - 1) / QZ_WARPS); }

}  // namespace

cudaError_t quantize_w4_launch(const void* w, int f16, int N, int K, int gs, int symmetric, long long out_mul,
                               long long out_add, uint32_t* q, __half* scales, uint32_t* zeros, int* status,
                               cudaStream_t stream) {
  QuantRows a{N, K, gs, (K + gs - 1) / gs, out_mul, out_add, status};
  const unsigned grid = blocks_for((long long)N * a.G);
  if (f16)
    quantize_w4_kernel<__half><<<grid, 32 * QZ_WARPS, 0, stream>>>((const __half*)w, a, symmetric, q, scales, zeros);
  else
    quantize_w4_kernel<double><<<grid, 32 * QZ_WARPS, 0, stream>>>((const double*)w, a, symmetric, q, scales, zeros);
  return cudaGetLastError();
}

cudaError_t quantize_mx_launch(const void* w, int f16, int N, int K, uint32_t* q, uint8_t* scales, int* status,
                               cudaStream_t stream) {
  QuantRows a{N, K, 32, (K + 31) / 32, 1, 0, status};
  const unsigned grid = blocks_for((long long)N * a.G);
  if (f16)
    quantize_mx_kernel<__half><<<grid, 32 * QZ_WARPS, 0, stream>>>((const __half*)w, a, q, scales);
  else
    quantize_mx_kernel<double><<<grid, 32 * QZ_WARPS, 0, stream>>>((const double*)w, a, q, scales);
  return cudaGetLastError();
}

cudaError_t quantize_f8_launch(const void* x, int f16, int rows, int D, int gs, long long out_mul, long long out_add,
                               uint8_t* q, __half* scales, int* status, cudaStream_t stream) {
  QuantRows a{rows, D, gs, (D + gs - 1) / gs, out_mul, out_add, status};
  const unsigned grid = blocks_for((long long)rows * a.G);
  if (f16)
    quantize_f8_kernel<__half><<<grid, 32 * QZ_WARPS, 0, stream>>>((const __half*)x, a, q, scales);
  else
    quantize_f8_kernel<double><<<grid, 32 * QZ_WARPS, 0, stream>>>((const double*)x, a, q, scales);
  return cudaGetLastError();
}

}  // namespace w4b
