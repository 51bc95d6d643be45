#pragma once
// Drop-in GPU header: the MXFP4 entries of the reference's include/w4/mxfused.cuh
// (DevicePackedWm :26-30, validate_mx :32-37, dequant_mx :57-69, gemm_fused_mx
// :166-198, gemm_mma_mx :291-307) over the C ABI of libw4b200.
#include "fused.cuh"
#include "mma.cuh"
#include "mx.hpp"

namespace w4::gpu {

struct DevicePackedWm {
  int N, K, B;  // B = mx::blocks(K)
  const uint32_t* q;
  const uint8_t* scales;
};
static_assert(sizeof(DevicePackedWm) == sizeof(w4b_packed_mx), "descriptor layouts must agree");

inline const w4b_packed_mx* abi(const DevicePackedWm& p) { return reinterpret_cast<const w4b_packed_mx*>(&p); }

inline void validate_mx(const DevicePackedWm& p) {
  if (p.N < 1 || p.K < 1) throw std::invalid_argument("mx: bad dims");
  if (p.B != mx::blocks(p.K)) throw std::invalid_argument("mx: B inconsistent with K");
  if (!p.q || !p.scales) throw std::invalid_argument("mx: null pointer");
}

inline void dequant_mx(const DevicePackedWm& p, __half* w, cudaStream_t stream = 0) {
  abi_check(w4b_dequant_mx(abi(p), w, stream));
}

inline void gemm_fused_mx(const DevicePackedWm& p, const __half* x, __half* c, int M, cudaStream_t stream = 0,
                          __half* w_out = nullptr) {
  abi_check(w4b_gemm_mx(abi(p), x, c, M, W4B_PATH_STREAM, stream, w_out));
}

inline void gemm_mma_mx(const DevicePackedWm& p, const __half* x, __half* c, int M, cudaStream_t stream = 0,
                        __half* w_out = nullptr) {
  abi_check(w4b_gemm_mx(abi(p), x, c, M, W4B_PATH_TENSOR, stream, w_out));
}

}  // namespace w4::gpu
