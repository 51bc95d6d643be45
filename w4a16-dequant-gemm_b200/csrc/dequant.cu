// Stand-alone dequantisation kernels: the two-pass comparator of the reference
// (dequant_kernel, include/w4/dequant.cuh:40-60; dequant_kernel_mx,
// include/w4/mxfused.cuh:41-55; dequant_kernel_f8, include/w4/kvflash.cuh:415-433)
// and the vehicle of the bitwise gate.
//
// Two code paths per format, both bit-identical to the host reference:
//  * vector path (K % 32 == 0, group size % 32 == 0, 16-byte aligned buffers):
//    a thread reads 16 bytes of codes (32 weights), decodes them with the same
//    register decoders the GEMM kernels use, and writes four 16-byte stores;
//  * scalar path (any shape the format allows): a thread per packed word with
//    the scalar definition of the format.
#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {
namespace {

// out[i] = (w[i], w[i+4])  ->  eight consecutive halves
__device__ __forceinline__ uint4 unpair(const __half2 o[4]) {
  uint4 r;
  r.x = __byte_perm(h2_as_u32(o[0]), h2_as_u32(o[1]), 0x5410);
  r.y = __byte_perm(h2_as_u32(o[2]), h2_as_u32(o[3]), 0x5410);
  r.z = __byte_perm(h2_as_u32(o[0]), h2_as_u32(o[1]), 0x7632);
  r.w = __byte_perm(h2_as_u32(o[2]), h2_as_u32(o[3]), 0x7632);
  return r;
}

__global__ void dequant_w4_vec_kernel(const uint4* __restrict__ q, const __half* __restrict__ scales,
                                      const uint32_t* __restrict__ zeros, int K, int gs, int G, int symmetric,
                                      long long nvec, uint4* __restrict__ w) {
  const int vpr = K >> 5;  // 16-byte code vectors per row
  const int wG = words(G);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    const long long n = v / vpr;
    const int j = (int)(v - n * vpr);
    const int grp = (32 * j) / gs;
    const __half s = scales[n * G + grp];
    const uint32_t z = symmetric ? 8u : ((zeros[n * wG + (grp >> 3)] >> (4 * (grp & 7))) & 0xFu);
    const W4Group g = w4_group(s, z);
    const uint4 codes = __ldg(q + v);
    const uint32_t cw[4] = {codes.x, codes.y, codes.z, codes.w};
    uint4* dst = w + v * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 o[4];
      dq_w4_word(cw[i], g, o);
      dst[i] = unpair(o);
    }
  }
}

__global__ void dequant_w4_scalar_kernel(const uint32_t* __restrict__ q, const __half* __restrict__ scales,
                                         const uint32_t* __restrict__ zeros, int K, int gs, int G,
                                         int symmetric, long long nwords, __half* __restrict__ w) {
  const int wpr = words(K);
  const int wG = words(G);
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < nwords;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / wpr;
    const int k0 = 8 * (int)(idx - n * wpr);
    const int grp = k0 / gs;
    const __half s = scales[n * G + grp];
    const int z = symmetric ? 8 : (int)((zeros[n * wG + (grp >> 3)] >> (4 * (grp & 7))) & 0xFu);
    const uint32_t qw = q[idx];
    __half* out = w + n * K + k0;
    const int lim = min(8, K - k0);
    for (int j = 0; j < lim; ++j) out[j] = dq_w4_scalar(s, (int)((qw >> (4 * j)) & 0xFu), z);
  }
}

__global__ void dequant_mx_vec_kernel(const uint4* __restrict__ q, const uint8_t* __restrict__ scales, int K,
                                      int B, long long nvec, uint4* __restrict__ w) {
  const int vpr = K >> 5;  // one vector == one 32-element block
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    const long long n = v / vpr;
    const int j = (int)(v - n * vpr);
    const MxBlock b = mx_block(scales[n * B + j]);
    const uint4 codes = __ldg(q + v);
    const uint32_t cw[4] = {codes.x, codes.y, codes.z, codes.w};
    uint4* dst = w + v * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 o[4];
      dq_mx_word(cw[i], b, o);
      dst[i] = unpair(o);
    }
  }
}

__global__ void dequant_mx_scalar_kernel(const uint32_t* __restrict__ q, const uint8_t* __restrict__ scales,
                                         int K, int B, long long nwords, __half* __restrict__ w) {
  const int wpr = words(K);
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < nwords;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / wpr;
    const int k0 = 8 * (int)(idx - n * wpr);
    const uint32_t se = scales[n * B + (k0 >> 5)];
    const uint32_t qw = q[idx];
    __half* out = w + n * K + k0;
    const int lim = min(8, K - k0);
    for (int j = 0; j < lim; ++j) out[j] = dq_mx_scalar(se, (int)((qw >> (4 * j)) & 0xFu));
  }
}

// One head of an FP8 cache: a thread per four bytes (D % 4 == 0 by contract).
__global__ void dequant_f8_kernel(const uint32_t* __restrict__ q, const __half* __restrict__ s,
                                  __half* __restrict__ w, long long nquads, int D, int gs, int G) {
  const int qpr = D >> 2;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < nquads;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / qpr;
    const int d0 = 4 * (int)(idx - t * qpr);
    const __half sc = s[t * G + d0 / gs];
    const uint32_t qw = q[idx];
    __half* out = w + t * D + d0;
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = dq_f8_scalar(sc, (qw >> (8 * j)) & 0xFFu);
  }
}

unsigned grid_for(long long items, int block) {
  long long g = (items + block - 1) / block;
  const long long cap = 148LL * 32;  // grid-stride loops; a few waves of CTAs
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (unsigned)g;
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

}  // namespace

cudaError_t dequant_w4_launch(const uint32_t* q, const __half* scales, const uint32_t* zeros, int N, int K,
                              int gs, int G, int symmetric, __half* w, cudaStream_t stream) {
  if (K % 32 == 0 && gs % 32 == 0 && aligned16(q) && aligned16(w)) {
    const long long nvec = (long long)N * (K >> 5);
    dequant_w4_vec_kernel<<<grid_for(nvec, 256), 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(q), scales, zeros, K, gs, G, symmetric, nvec, reinterpret_cast<uint4*>(w));
  } else {
    const long long nwords = (long long)N * words(K);
    dequant_w4_scalar_kernel<<<grid_for(nwords, 256), 256, 0, stream>>>(q, scales, zeros, K, gs, G, symmetric,
                                                                       nwords, w);
  }
  return cudaGetLastError();
}

cudaError_t dequant_mx_launch(const uint32_t* q, const uint8_t* scales, int N, int K, int B, __half* w,
                              cudaStream_t stream) {
  if (K % 32 == 0 && aligned16(q) && aligned16(w)) {
    const long long nvec = (long long)N * (K >> 5);
    dequant_mx_vec_kernel<<<grid_for(nvec, 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(q), scales, K,
                                                                   B, nvec, reinterpret_cast<uint4*>(w));
  } else {
    const long long nwords = (long long)N * words(K);
    dequant_mx_scalar_kernel<<<grid_for(nwords, 256), 256, 0, stream>>>(q, scales, K, B, nwords, w);
  }
  return cudaGetLastError();
}

cudaError_t dequant_f8_launch(const uint8_t* q, const __half* s, __half* w, int S, int D, int gs,
                              cudaStream_t stream) {
  const long long nquads = (long long)S * (D >> 2);
  dequant_f8_kernel<<<grid_for(nquads, 256), 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(q), s, w, nquads,
                                                               D, gs, (D + gs - 1) / gs);
  return cudaGetLastError();
}

}  // namespace w4b
