// Shape-agnostic fused dequant GEMM: serves every shape the packed formats
// allow (ragged K, K % 8 != 0, any group size that is a multiple of 8, N or M
// of any size, buffers with only natural alignment). It is the safety net
// behind the stream and tensor kernels, not a fast path.
//
// One warp per weight row: lanes stride the row's packed words, decode each
// word once with the scalar definition of the format and feed up to eight
// activation rows (FP32 FMA); a shuffle tree then adds the 32 lane sums in a
// fixed order, so results are reproducible bit for bit.
#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {
namespace {

constexpr int GG_WARPS = 8;
constexpr int GG_MTILE = 8;

template <int FMT>  // 0 W4 sym, 1 W4 asym, 2 MX
__global__ void __launch_bounds__(32 * GG_WARPS)
    generic_gemm_kernel(const uint32_t* __restrict__ q, const void* __restrict__ scales,
                        const uint32_t* __restrict__ zeros, int N, int K, int gs, int G,
                        const __half* __restrict__ x, __half* __restrict__ c, int M, __half* __restrict__ w_out) {
  const int lane = threadIdx.x & 31;
  const long long n = (long long)blockIdx.x * GG_WARPS + (threadIdx.x >> 5);
  if (n >= N) return;  // warp-uniform
  const int wpr = words(K);
  const int wG = words(G);
  const uint32_t* qrow = q + n * wpr;

  for (int m0 = (int)blockIdx.y * GG_MTILE; m0 < M; m0 += (int)gridDim.y * GG_MTILE) {
    float acc[GG_MTILE];
#pragma unroll
    for (int i = 0; i < GG_MTILE; ++i) acc[i] = 0.0f;
    const int mt = min(GG_MTILE, M - m0);
    for (int w = lane; w < wpr; w += 32) {
      const int k0 = 8 * w;
      const uint32_t qw = qrow[w];
      __half s = __ushort_as_half((unsigned short)0);
      int z = 8;
      uint32_t se = 0;
      if (FMT == 2) {
        se = ((const uint8_t*)scales)[n * G + (k0 >> 5)];
      } else {
        const int grp = k0 / gs;
        s = ((const __half*)scales)[n * G + grp];
        if (FMT == 1) z = (int)((zeros[n * wG + (grp >> 3)] >> (4 * (grp & 7))) & 0xFu);
      }
      const int lim = min(8, K - k0);
      for (int j = 0; j < lim; ++j) {
        const int code = (int)((qw >> (4 * j)) & 0xFu);
        const __half wj = FMT == 2 ? dq_mx_scalar(se, code) : dq_w4_scalar(s, code, z);
        if (w_out != nullptr && m0 == 0) w_out[n * K + k0 + j] = wj;
        const float wf = __half2float(wj);
#pragma unroll
        for (int i = 0; i < GG_MTILE; ++i)
          if (i < mt) acc[i] = fmaf(wf, __half2float(x[(size_t)(m0 + i) * K + k0 + j]), acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < GG_MTILE; ++i) {
      float v = acc[i];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == 0 && i < mt) c[(size_t)(m0 + i) * N + n] = __float2half_rn(v);
    }
  }
}

}  // namespace

cudaError_t generic_gemm_launch(int fmt, int gs, const uint32_t* q, const void* scales, const uint32_t* zeros,
                                int N, int K, int G, const __half* x, __half* c, int M, __half* w_out,
                                cudaStream_t stream) {
  const unsigned gx = (unsigned)(((long long)N + GG_WARPS - 1) / GG_WARPS);
  long long gy = ((long long)M + GG_MTILE - 1) / GG_MTILE;
  if (gy > 64) gy = 64;  // the kernel strides over the remaining m-tiles
  const dim3 grid(gx, (unsigned)gy);
  if (fmt == 0)
    generic_gemm_kernel<0><<<grid, 32 * GG_WARPS, 0, stream>>>(q, scales, zeros, N, K, gs, G, x, c, M, w_out);
  else if (fmt == 1)
    generic_gemm_kernel<1><<<grid, 32 * GG_WARPS, 0, stream>>>(q, scales, zeros, N, K, gs, G, x, c, M, w_out);
  else
    generic_gemm_kernel<2><<<grid, 32 * GG_WARPS, 0, stream>>>(q, scales, zeros, N, K, 32, G, x, c, M, w_out);
  return cudaGetLastError();
}

}  // namespace w4b
