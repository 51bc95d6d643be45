#pragma once
// Drop-in GPU header: the stream / tensor dispatcher (reference
// include/w4/dispatch.cuh:25-43). The crossover is the library's, re-measured on
// B200: w4b_dispatch_mma_min_m() returns the same value as this constant.
#include "fused.cuh"
#include "mma.cuh"
#include "mxfused.cuh"

namespace w4::gpu {

// M below this goes to the stream kernel; M at or above goes to the tensor kernel.
constexpr int DISPATCH_MMA_MIN_M = 17;

inline void gemm(const DevicePackedW& p, const __half* x, __half* c, int M, cudaStream_t stream = 0,
                 __half* w_out = nullptr) {
  abi_check(w4b_gemm_w4(abi(p), x, c, M, W4B_PATH_AUTO, stream, w_out));
}

inline void gemm_mx(const DevicePackedWm& p, const __half* x, __half* c, int M, cudaStream_t stream = 0,
                    __half* w_out = nullptr) {
  abi_check(w4b_gemm_mx(abi(p), x, c, M, W4B_PATH_AUTO, stream, w_out));
}

}  // namespace w4::gpu
