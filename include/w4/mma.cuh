#pragma once
// Drop-in GPU header: gemm_mma (reference include/w4/mma.cuh:234-260) served by the
// tcgen05 / TMEM kernel of libw4b200. The tile constants keep the reference's names
// (:59-61) and describe that kernel: 128 weight rows per CTA, K chunks of 64; the
// launch bound the reference derives from its 64-row m-tile is kept by the library.
#include "dequant.cuh"

namespace w4::gpu {

constexpr int MMA_TILE_M = 64;
constexpr int MMA_TILE_N = 128;
constexpr int MMA_CHUNK_K = 64;

inline void gemm_mma(const DevicePackedW& p, const __half* x, __half* c, int M, cudaStream_t stream = 0,
                     __half* w_out = nullptr) {
  abi_check(w4b_gemm_w4(abi(p), x, c, M, W4B_PATH_TENSOR, stream, w_out));
}

}  // namespace w4::gpu
