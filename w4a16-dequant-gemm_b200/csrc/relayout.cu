// Offline re-layout of packed weights: the same matrix zero-extended along K, in the same packed format
// (include/w4/pack.hpp:3-14, include/w4/mx.hpp:10-14), so that its row pitches become multiples of 16 bytes and K
// a multiple of 512 - what the TMA-fed kernels need. A matrix whose K the fast kernels cannot address (K = 4100:
// 2052-byte rows) is converted once, and every GEMM against it runs on the stream / tensor kernel with the
// activation rows padded by zeros. The reference has no counterpart: its kernels take any K with scalar loads.
//
// The added columns dequantise to +0 exactly: inside the source's partial last group they carry the group's zero
// point (asymmetric), 8 (symmetric) or the E2M1 code of +0 (MXFP4); whole new groups get scale 0 (W4) or 2^0
// (MXFP4) with zero codes. Everything in the destination is written, so it needs no clearing beforehand.
#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {
namespace {

constexpr int RL_THREADS = 256;

__device__ __forceinline__ uint32_t nibble_of(const uint32_t* __restrict__ row, int i) {
  return (row[i >> 3] >> ((i & 7) * 4)) & 15u;
}

// fmt: 0 = W4 symmetric, 1 = W4 asymmetric, 2 = MXFP4. One thread per destination code word.
__global__ void __launch_bounds__(RL_THREADS)
    relayout_codes_kernel(int fmt, const uint32_t* __restrict__ src_q, const uint32_t* __restrict__ src_zeros,
                          uint32_t* __restrict__ dst_q, int N, int K, int gs, int G, int wk_src, int wk_dst, int wg_src) {
  const long long i = (long long)blockIdx.x * RL_THREADS + threadIdx.x;
  if (i >= (long long)N * wk_dst) return;
  const int n = (int)(i / wk_dst), w = (int)(i % wk_dst);
  const int k0 = w * 8;
  uint32_t v;
  if (k0 + 8 <= K) {
    v = src_q[(size_t)n * wk_src + w];
  } else {
    const uint32_t s = k0 < K ? src_q[(size_t)n * wk_src + w] : 0u;
    v = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int k = k0 + j;
      uint32_t code;
      if (k < K) {
        code = (s >> (4 * j)) & 15u;
      } else if (fmt == 2) {
        code = 0u;
      } else if (fmt == 0) {
        code = 8u;
      } else {
        const int g = k / gs;
        code = g < G ? nibble_of(src_zeros + (size_t)n * wg_src, g) : 0u;
      }
      v |= code << (4 * j);
    }
  }
  dst_q[i] = v;
}

// One thread per destination scale. W4: FP16 bit patterns, new groups 0. MXFP4: E8M0 bytes, new blocks 127.
__global__ void __launch_bounds__(RL_THREADS)
    relayout_scales_kernel(int mx, const void* __restrict__ src, void* __restrict__ dst, int N, int G_src, int G_dst) {
  const long long i = (long long)blockIdx.x * RL_THREADS + threadIdx.x;
  if (i >= (long long)N * G_dst) return;
  const int n = (int)(i / G_dst), g = (int)(i % G_dst);
  if (mx)
    ((uint8_t*)dst)[i] = g < G_src ? ((const uint8_t*)src)[(size_t)n * G_src + g] : (uint8_t)127;
  else
    ((uint16_t*)dst)[i] = g < G_src ? ((const uint16_t*)src)[(size_t)n * G_src + g] : (uint16_t)0;
}

// One thread per destination word of zero points (asymmetric W4).
__global__ void __launch_bounds__(RL_THREADS)
    relayout_zeros_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int N, int G_src, int wg_src,
                          int wg_dst) {
  const long long i = (long long)blockIdx.x * RL_THREADS + threadIdx.x;
  if (i >= (long long)N * wg_dst) return;
  const int n = (int)(i / wg_dst), w = (int)(i % wg_dst);
  uint32_t v = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int g = w * 8 + j;
    if (g < G_src) v |= nibble_of(src + (size_t)n * wg_src, g) << (4 * j);
  }
  dst[i] = v;
}

// Activation rows of K halves to rows of Kp halves, zeros behind column K.
__global__ void __launch_bounds__(RL_THREADS)
    pad_rows_kernel(const __half* __restrict__ x, __half* __restrict__ xp, int M, int K, int Kp) {
  const long long i = (long long)blockIdx.x * RL_THREADS + threadIdx.x;
  if (i >= (long long)M * Kp) return;
  const int m = (int)(i / Kp), k = (int)(i % Kp);
  xp[i] = k < K ? x[(size_t)m * K + k] : __ushort_as_half((unsigned short)0);
}

inline unsigned blocks_for(long long items) { return (unsigned)((items + RL_THREADS - 1) / RL_THREADS); }

}  // namespace

cudaError_t relayout_launch(int fmt, int gs, const uint32_t* src_q, const void* src_scales, const uint32_t* src_zeros,
                            int N, int K, int G, uint32_t* dst_q, void* dst_scales, uint32_t* dst_zeros, int Kp, int Gp,
                            cudaStream_t stream, int* launches) {
  const int wk_src = (K + 7) / 8, wk_dst = (Kp + 7) / 8, wg_src = (G + 7) / 8, wg_dst = (Gp + 7) / 8;
  relayout_codes_kernel<<<blocks_for((long long)N * wk_dst), RL_THREADS, 0, stream>>>(
      fmt, src_q, src_zeros, dst_q, N, K, gs, G, wk_src, wk_dst, wg_src);
  relayout_scales_kernel<<<blocks_for((long long)N * Gp), RL_THREADS, 0, stream>>>(fmt == 2 ? 1 : 0, src_scales,
                                                                                  dst_scales, N, G, Gp);
  *launches = 2;
  if (fmt == 1) {
    relayout_zeros_kernel<<<blocks_for((long long)N * wg_dst), RL_THREADS, 0, stream>>>(src_zeros, dst_zeros, N, G,
                                                                                       wg_src, wg_dst);
    *launches = 3;
  }
  return cudaGetLastError();
}

cudaError_t pad_rows_launch(const __half* x, __half* xp, int M, int K, int Kp, cudaStream_t stream) {
  pad_rows_kernel<<<blocks_for((long long)M * Kp), RL_THREADS, 0, stream>>>(x, xp, M, K, Kp);
  return cudaGetLastError();
}

}  // namespace w4b
