// Host-callable launchers of the CUDA kernels (one translation unit each).
// Internal to libw4b200; the public surface is include/w4b_abi.h.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace w4b {

// 32-bit words that hold n 4-bit codes (the reference's words(), include/w4/pack.hpp:33).
__host__ __device__ __forceinline__ int words(int n) { return (n + 7) >> 3; }

// ---- abi.cu ------------------------------------------------------------------
// Sets the calling thread's message returned by w4b_last_error().
void set_last_error(const char* msg);
// The process-wide launch-overlap setting (w4b_set_launch_overlap).
bool launch_overlap();
// Adds to the count returned by w4b_launch_count().
void count_launches(int n);

// ---- gemm_noalloc.cu -----------------------------------------------------------
void noalloc_regions(int dev, int** status, void** counters, size_t* counter_bytes);

// ---- dequant.cu -----------------------------------------------------------
cudaError_t dequant_w4_launch(const uint32_t* q, const __half* scales, const uint32_t* zeros, int N, int K,
                              int gs, int G, int symmetric, __half* w, cudaStream_t stream);
cudaError_t dequant_mx_launch(const uint32_t* q, const uint8_t* scales, int N, int K, int B, __half* w,
                              cudaStream_t stream);
cudaError_t dequant_f8_launch(const uint8_t* q, const __half* s, __half* w, int S, int D, int gs,
                              cudaStream_t stream);

// ---- quantize.cu ---------------------------------------------------------------
// f16: the source holds FP16 values, else FP64. Destination row of source row n: n * out_mul + out_add.
cudaError_t quantize_w4_launch(const void* w, int f16, int N, int K, int gs, int symmetric, long long out_mul,
                               long long out_add, uint32_t* q, __half* scales, uint32_t* zeros, int* status,
                               cudaStream_t stream);
cudaError_t quantize_mx_launch(const void* w, int f16, int N, int K, uint32_t* q, uint8_t* scales, int* status,
                               cudaStream_t stream);
cudaError_t quantize_f8_launch(const void* x, int f16, int rows, int D, int gs, long long out_mul, long long out_add,
                               uint8_t* q, __half* scales, int* status, cudaStream_t stream);

// ---- relayout.cu ---------------------------------------------------------------
// The matrix zero-extended along K to Kp columns (Gp groups / blocks per row) in the same packed format.
// fmt: 0 = W4 symmetric, 1 = W4 asymmetric, 2 = MXFP4 (gs ignored).
cudaError_t relayout_launch(int fmt, int gs, const uint32_t* src_q, const void* src_scales, const uint32_t* src_zeros,
                            int N, int K, int G, uint32_t* dst_q, void* dst_scales, uint32_t* dst_zeros, int Kp, int Gp,
                            cudaStream_t stream, int* launches);
// x (M rows of K halves) to xp (M rows of Kp halves), zeros behind column K.
cudaError_t pad_rows_launch(const __half* x, __half* xp, int M, int K, int Kp, cudaStream_t stream);

// ---- gemm_generic.cu --------------------------------------------------------
// fmt: 0 = W4 symmetric, 1 = W4 asymmetric, 2 = MXFP4 (gs ignored, G = blocks per row).
cudaError_t generic_gemm_launch(int fmt, int gs, const uint32_t* q, const void* scales, const uint32_t* zeros,
                                int N, int K, int G, const __half* x, __half* c, int M, __half* w_out,
                                cudaStream_t stream);

// ---- gemm_stream.cu ---------------------------------------------------------
// Exchange form of the stream GEMM (column-parallel ranks, one process per GPU): besides c, every output element
// is stored to the same offset of each peer's copy, and the grid's last warp posts the step flags.
struct StreamPeers {
  int world, rank;                      // world == 0: no exchange
  __half* c_peer[8];                    // rank p's copy of this rank's slice (null for this rank)
  unsigned long long* flag_dst[8];      // rank p's flag word for this rank
  const void* flags_local;              // this rank's flag words, one uint64 per peer
  unsigned long long* counters;         // steps pushed to each peer so far, one uint64 per rank
  int* done;                            // grid completion counter in this rank's arena, zero between launches
  // carry form: the grid delivers the PREVIOUS step's slice (prev_src, finished by the previous grid) into c_peer
  // beside its own GEMM and posts that step; nothing is sent from the epilogue. prev_bytes == 0: nothing to carry.
  int carry;
  const __half* prev_src;
  size_t prev_bytes;
};
struct StreamPlan {
  int streamed;       // 1: activations arranged by a pre-pass and streamed with the units; 0: resident in shared memory
  int rows_per_pass;  // activation rows per pass
  int mt;             // 8-row m-tiles per pass (1 or 2)
  int passes;         // grid.y
  int stages;         // ring depth
  int P, C;           // panels of 64 rows, units of 512 k per panel
  long long U;        // work units
  int grid_x;         // persistent CTAs
  int xpitch;
  size_t smem;
  size_t xa_bytes;      // arranged activations of the streamed form (0 in the resident form)
  size_t ws_bytes;      // FP32 partial-fragment slots
  size_t counter_ints;  // per-(pass, tile) arrival counters, zero between launches
};
bool stream_gemm_supported(int N, int K, int gs_or_0_for_mx, const void* q, const void* scales,
                           const void* x);
void stream_gemm_plan(int N, int K, int M, int gs_or_0_for_mx, int sm_count, StreamPlan* plan);
cudaError_t stream_gemm_launch(int fmt, int gs, const uint32_t* q, const void* scales, const uint32_t* zeros,
                               int N, int K, int G, const __half* x, __half* c, int M, __half* w_out,
                               const StreamPlan& plan, float* ws, int* counters, void* xa, int* status,
                               bool overlap, cudaStream_t stream, int* launches, const StreamPeers* peers = nullptr);

// ---- gemm_tensor.cu ---------------------------------------------------------
struct TensorPlan {
  int splits;           // CTAs that share a tile's K range
  size_t ws_bytes;      // FP32 partial tiles (0 when splits == 1)
  size_t counter_ints;  // per-tile arrival counters, zero between launches
};
void tensor_gemm_plan(int N, int K, int M, int sm_count, TensorPlan* plan);
bool tensor_gemm_supported(int N, int K, const void* q, const void* x);
// The caller has sized ws / counters by the plan; counters are all zero between launches.
cudaError_t tensor_gemm_launch(int fmt, int gs, const uint32_t* q, const void* scales, const uint32_t* zeros, int N,
                               int K, int G, const __half* x, __half* c, int M, __half* w_out, const TensorPlan& plan,
                               float* ws, int* counters, int* status, cudaStream_t stream);

// ---- attn_flash.cu ----------------------------------------------------------
enum : int { ATTN_FP16 = 0, ATTN_W4_SYM = 1, ATTN_W4_ASYM = 2, ATTN_F8 = 3 };
// Where the K / V rows of one call live. Head h owns rows [h*slab_rows, (h+1)*slab_rows)
// of every array; logical position t is row t, or bt[t/page]*page + t%page when bt != null.
struct AttnSource {
  int fmt;
  const void* k;        // FP16: halves [rows][D]; W4: uint32 [rows][words(D)]; F8: bytes [rows][D]
  const void* v;
  const __half* s_k;    // W4 / F8: [rows][G]
  const __half* s_v;
  const uint32_t* z_k;  // W4 asymmetric: [rows][words(G)]
  const uint32_t* z_v;
  int gs, G;
  const int* bt;
  int page;
  long long slab_rows;
};
// Slices per head of the split-S pass (the same on the host and, for the batched form, on the device).
__host__ __device__ inline int attn_flash_splits(int H, int S, int sm_count, int per_sm = 14) {
  // About per_sm CTAs per SM over the whole grid (3.5 waves at four resident CTAs per SM: a CTA pays its query
  // loads, its first block's latency and its merge once, and with eight waves of short slices that was a
  // quarter of its time - B*H = 256, S = 8192: 19 slices 97.7 us, 8 slices 90.8 us), but slices as long as
  // possible - 256 positions (four steps per warp), else 128, else 64 - as long as that still gives every SM two
  // CTAs.
  long long want = ((long long)per_sm * sm_count + H - 1) / H;
  // (no slice longer than 4096 positions: with few, long CTAs the last partial wave costs more than the merges
  // saved - B*H = 512, S = 32768: 5 slices 620 us, 8 slices 596 us)
  if (want < (S + 4095) / 4096) want = (S + 4095) / 4096;
  long long cap = 1;
  for (int slice = 256; slice >= 64; slice >>= 1) {
    cap = (S + slice - 1) / slice;
    if (cap * H >= 2LL * sm_count) break;
  }
  if (want > cap) want = cap;
  if (want > 65535) want = 65535;
  if (want < 1) want = 1;
  return (int)want;
}
// The batched paged form serves eight sequences of a head per CTA, so it cuts every sequence's slices for
// ceil(nseq / 8) * H independent rows (a single sequence: H, the geometry of the single-sequence entry).
__host__ __device__ inline int attn_batched_rows(int nseq, int H) { return ((nseq + 7) / 8) * H; }
size_t attn_flash_ws_bytes(int H, int D, int splits);
cudaError_t attn_flash_launch(const AttnSource& src, const __half* q, __half* out, int H, int S, int D, int splits,
                              float* ws, __half* k_out, __half* v_out, cudaStream_t stream, int* launches);

cudaError_t attn_flash_batched_launch(const AttnSource& src, const __half* q, __half* out, int H, int D, int nseq,
                                      const int* seq_lens, int bt_stride, int max_splits, int sm_count, float* ws,
                                      cudaStream_t stream, int* launches);

// ---- attn_mma.cu ------------------------------------------------------------
// The tensor-pipe form of the flash pass for D = 64 / 128 and group sizes 32 / 64 / 128;
// same workspace layout and split combine as attn_flash.cu.
bool attn_mma_supported(const AttnSource& src, int D, const void* q, const void* k_out, const void* v_out);
cudaError_t attn_mma_launch(const AttnSource& src, const __half* q, __half* out, int H, int S, int D, int splits,
                            float* ws, __half* k_out, __half* v_out, cudaStream_t stream);

cudaError_t attn_mma_batched_launch(const AttnSource& src, const __half* q, __half* out, int H, int D, int nseq,
                                    const int* seq_lens, int bt_stride, int max_splits, int sm_count, float* ws,
                                    cudaStream_t stream);

// ---- peer_gather.cu ---------------------------------------------------------
constexpr int kMaxPeers = 8;
struct PeerPush {
  const void* src;                // this rank's slice (in its own arena)
  size_t n16;                     // its size in 16-byte units
  void* dst[kMaxPeers];           // where the slice goes in rank p's arena
  void* flag_dst[kMaxPeers];      // rank p's flag word for this rank
  const void* flags_local;        // this rank's flag words, one per peer (uint64)
  unsigned long long* counters;   // steps pushed to each peer, one uint64 per rank (start at zero)
  int rank, world;
  int wait_now;                   // also wait for the peers' slices of this step (else: of the previous one only)
  int* status;
};
cudaError_t peer_push_launch(const PeerPush& p, cudaStream_t stream);
cudaError_t peer_wait_launch(const void* flags_local, const unsigned long long* counters, int rank, int world,
                             int* status, cudaStream_t stream);

}  // namespace w4b
