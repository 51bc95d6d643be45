// Shape-agnostic fused dequant GEMMs: they serve every shape the packed formats
// allow (ragged K, K % 8 != 0, any group size that is a multiple of 8, N or M
// of any size, buffers with only natural alignment) - what the stream and tensor
// kernels, which need 16-byte row pitches for TMA, cannot take.
//
// generic_gemm_kernel: one warp per weight row, lanes stride the row's packed
// words, decode each word with the scalar definition of the format and feed up to
// eight activation rows (FP32 FMA); a shuffle tree then adds the 32 lane sums in a
// fixed order, so results are reproducible bit for bit. It serves everything,
// including the w_out hook.
//
// row_gemm_kernel: the same warp-per-row walk made fast for the common ragged case
// (power-of-two group size or MXFP4, no hook, activations that fit in shared
// memory): persistent CTAs stage the activation tile once as FP32 (zero-padded to
// whole words, so a half-used last word needs no special case), every lane keeps
// four coalesced 4-byte loads in flight, words are decoded with the register
// decoders (bit-identical to the scalar definitions) and accumulated in FP32.
#include <atomic>

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

constexpr int RG_THREADS = 512;
constexpr int RG_UNROLL = 4;
constexpr size_t RG_SMEM_MAX = 100 * 1024;  // two CTAs per SM

template <int FMT, int MT>
__global__ void __launch_bounds__(RG_THREADS, 2)
    row_gemm_kernel(const uint32_t* __restrict__ q, const void* __restrict__ scales,
                    const uint32_t* __restrict__ zeros, int N, int K, int gshift, int G,
                    const __half* __restrict__ x, __half* __restrict__ c, int M) {
  extern __shared__ __align__(16) float xs[];  // [MT][8 * words(K)]
  const int lane = threadIdx.x & 31;
  const int wpr = words(K);
  const int kpad = 8 * wpr;
  const int wG = words(G);
  const int warps_total = (int)gridDim.x * (RG_THREADS / 32);
  const int warp0 = (int)blockIdx.x * (RG_THREADS / 32) + (threadIdx.x >> 5);
  const W4Consts kc = w4_consts();

  for (int m0 = (int)blockIdx.y * MT; m0 < M; m0 += (int)gridDim.y * MT) {
    __syncthreads();  // the previous tile's readers are done
    for (int i = threadIdx.x; i < MT * kpad; i += RG_THREADS) {
      const int m = i / kpad, k = i - m * kpad;
      xs[i] = (m0 + m < M && k < K) ? __half2float(x[(size_t)(m0 + m) * K + k]) : 0.0f;
    }
    __syncthreads();
    for (long long n = warp0; n < N; n += warps_total) {
      const uint32_t* qrow = q + n * wpr;
      float acc[MT];
#pragma unroll
      for (int i = 0; i < MT; ++i) acc[i] = 0.0f;
      for (int w0 = lane; w0 < wpr; w0 += 32 * RG_UNROLL) {
        uint32_t qw[RG_UNROLL];
#pragma unroll
        for (int u = 0; u < RG_UNROLL; ++u) {
          const int w = w0 + 32 * u;
          qw[u] = w < wpr ? __ldg(qrow + w) : 0u;
        }
#pragma unroll
        for (int u = 0; u < RG_UNROLL; ++u) {
          const int w = w0 + 32 * u;
          if (w >= wpr) break;
          __half2 h[4];
          if (FMT == 2) {
            dq_mx_word(qw[u], mx_block(((const uint8_t*)scales)[n * G + (w >> 2)]), h);
          } else {
            const int grp = (8 * w) >> gshift;
            const __half s = ((const __half*)scales)[n * G + grp];
            const uint32_t z = FMT == 1 ? ((__ldg(zeros + n * wG + (grp >> 3)) >> (4 * (grp & 7))) & 0xFu) : 8u;
            dq_w4_word(qw[u], w4_group(s, z), kc, h);
          }
          // h[i] = (weight 8w + i, weight 8w + i + 4)
          float wf[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            wf[i] = f.x;
            wf[i + 4] = f.y;
          }
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const float4 xa = *reinterpret_cast<const float4*>(xs + m * kpad + 8 * w);
            const float4 xb = *reinterpret_cast<const float4*>(xs + m * kpad + 8 * w + 4);
            float a = acc[m];
            a = fmaf(wf[0], xa.x, a);
            a = fmaf(wf[1], xa.y, a);
            a = fmaf(wf[2], xa.z, a);
            a = fmaf(wf[3], xa.w, a);
            a = fmaf(wf[4], xb.x, a);
            a = fmaf(wf[5], xb.y, a);
            a = fmaf(wf[6], xb.z, a);
            a = fmaf(wf[7], xb.w, a);
            acc[m] = a;
          }
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float v = acc[m];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0 && m0 + m < M) c[(size_t)(m0 + m) * N + n] = __float2half_rn(v);
      }
    }
  }
}

template <int FMT>
cudaError_t row_gemm_launch(int dev, int mt, dim3 grid, size_t smem, const uint32_t* q, const void* scales,
                            const uint32_t* zeros, int N, int K, int gshift, int G, const __half* x, __half* c, int M,
                            cudaStream_t stream) {
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
#define W4B_ROW_CASE(MT)                                                                                          \
  case MT: {                                                                                                      \
    static std::atomic<bool> configured[64]; /* the opt-in is a per-device attribute of the function */          \
    if (!configured[dev].load(std::memory_order_acquire)) {                                                       \
      const cudaError_t e = cudaFuncSetAttribute(row_gemm_kernel<FMT, MT>,                                        \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RG_SMEM_MAX);  \
      if (e != cudaSuccess) return e;                                                                             \
      configured[dev].store(true, std::memory_order_release);                                                     \
    }                                                                                                             \
    row_gemm_kernel<FMT, MT><<<grid, RG_THREADS, smem, stream>>>(q, scales, zeros, N, K, gshift, G, x, c, M);     \
    return cudaGetLastError();                                                                                    \
  }
  switch (mt) {
    W4B_ROW_CASE(1)
    W4B_ROW_CASE(2)
    W4B_ROW_CASE(4)
    W4B_ROW_CASE(8)
  }
#undef W4B_ROW_CASE
  return cudaErrorInvalidValue;
}

}  // namespace

// The fast ragged kernel's activation tile: the largest of 8 / 4 / 2 / 1 rows (no more than M needs) that fits
// half an SM's shared memory; 0 when not even one row fits or the shape needs the slow kernel.
static int row_gemm_tile(int fmt, int gs, int K, int M, const __half* w_out) {
  if (w_out != nullptr) return 0;
  if (fmt != 2 && (gs & (gs - 1)) != 0) return 0;
  const size_t row = (size_t)8 * (size_t)((K + 7) / 8) * sizeof(float);
  int mt = 8;
  while (mt > 1 && (mt / 2 >= M || (size_t)mt * row > RG_SMEM_MAX)) mt /= 2;
  return (size_t)mt * row <= RG_SMEM_MAX ? mt : 0;
}

cudaError_t generic_gemm_launch(int fmt, int gs, const uint32_t* q, const void* scales, const uint32_t* zeros,
                                int N, int K, int G, const __half* x, __half* c, int M, __half* w_out,
                                cudaStream_t stream) {
  if (const int mt = row_gemm_tile(fmt, gs, K, M, w_out)) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    const long long tiles = ((long long)M + mt - 1) / mt;
    const long long row_blocks = ((long long)N + RG_THREADS / 32 - 1) / (RG_THREADS / 32);
    long long gx = 2LL * sms, gy = 1;
    if (gx > row_blocks) gx = row_blocks;
    while (gy < tiles && gy < 64 && gx * gy * 2 <= 2LL * sms) gy *= 2;  // few rows: spread the m-tiles instead
    const dim3 grid((unsigned)gx, (unsigned)gy);
    const size_t smem = (size_t)mt * 8 * (size_t)((K + 7) / 8) * sizeof(float);
    int gshift = 0;
    while (fmt != 2 && (1 << gshift) < gs) ++gshift;
    if (fmt == 0) return row_gemm_launch<0>(dev, mt, grid, smem, q, scales, zeros, N, K, gshift, G, x, c, M, stream);
    if (fmt == 1) return row_gemm_launch<1>(dev, mt, grid, smem, q, scales, zeros, N, K, gshift, G, x, c, M, stream);
    return row_gemm_launch<2>(dev, mt, grid, smem, q, scales, zeros, N, K, 5, G, x, c, M, stream);
  }
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
