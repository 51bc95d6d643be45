#pragma once
// Drop-in GPU header: gemm_fused (reference include/w4/fused.cuh:172-214) served by
// the HBM-streaming kernel of libw4b200 (generic kernel for shapes outside its family).
#include "dequant.cuh"

namespace w4::gpu {

inline void gemm_fused(const DevicePackedW& p, const __half* x, __half* c, int M, cudaStream_t stream = 0,
                       __half* w_out = nullptr) {
  abi_check(w4b_gemm_w4(abi(p), x, c, M, W4B_PATH_STREAM, stream, w_out));
}

}  // namespace w4::gpu
