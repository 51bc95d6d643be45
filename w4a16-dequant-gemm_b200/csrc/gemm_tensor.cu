// Fused dequant GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for M
// at or above the crossover: the replacement of the reference's WMMA kernels
// mma_kernel / mma_kernel_mx (include/w4/mma.cuh:63-232,
// include/w4/mxfused.cuh:203-289). Only here is the path a dense contraction.
//
// One CTA owns a tile of 128 weight rows (the UMMA M dimension, "swap-AB": the
// dequantised W tile is the A operand) by up to 256 activation rows (the UMMA N
// dimension; x is the B operand) and walks K in chunks of 64:
//
//   warp 16 (producer)  TMA: the chunk's packed codes (128 rows x 32 B) and the
//                       chunk of x (Mpad rows x 128 B, 128-byte swizzle, rows past
//                       M zero-filled) into a ring of stages;
//   warps 0-15 (decode) four groups of four warps take chunks in turn; thread t decodes row
//                       (t & 127) of its group's chunk (8 words -> 64 halves, the same
//                       register decoders as every other kernel, bit-identical to
//                       dequant_one) and stores them into the canonical K-major
//                       128-byte-swizzled FP16 operand tile; fence.proxy.async. The
//                       groups' scales / zero points are fetched one chunk ahead,
//                       outside the wait for the codes;
//   warp 17 (MMA)       one thread issues 4 x tcgen05.mma.kind::f16 (M=128, N=Mpad,
//                       K=16) per chunk, accumulating FP32 in TMEM, and
//                       tcgen05.commit's the stage back to the producer;
//   warps 0-15 (epilogue) tcgen05.ld the accumulator (lane = weight row; warps w, w + 4, ...
//                       share a lane quarter and take alternate column blocks),
//                       convert to FP16 and store c[m*N + n] (a warp writes 32
//                       consecutive n).
//
// When the tiles alone would leave most SMs idle (N of a few thousand), the K range of a tile is split between
// several CTAs (grid.z): each writes its FP32 partial tile to a workspace, bumps the tile's counter, and the CTA
// that arrives last adds the partials in split order - fixed, so the output is bit-identical from run to run -
// and stores FP16.
//
// Shapes served: K % 32 == 0 (16-byte row pitch of q and x), 16-byte aligned q / x,
// any N, any M (grid.y tiles M by 256), any group size the format allows. The K
// tail (K % 64 != 0) is zero-filled by TMA on both operands.
// Every wait is bounded; a kernel that gives up still frees its TMEM.
#include <cuda.h>

#include <atomic>

#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {
namespace {

constexpr int TK_ROWS = 128;   // weight rows per CTA = UMMA M
constexpr int TK_KC = 64;      // k per chunk = one 128-byte swizzle row of FP16
constexpr int TK_A_BYTES = TK_ROWS * 128;
constexpr int TK_Q_BYTES = TK_ROWS * (TK_KC / 2);
constexpr int TK_GROUPS = 4;                        // decode groups of four warps; group g takes chunks g, g + 4, ...
constexpr int TK_DECODERS = 4 * TK_GROUPS;
constexpr int TK_THREADS = 32 * (TK_DECODERS + 2);  // + TMA producer + MMA issuer
constexpr int TK_MAX_STAGES = 8;   // (a multiple of TK_GROUPS, see the launcher)

struct TensorParams {
  const uint32_t* q;
  const void* scales;
  const uint32_t* zeros;
  __half* c;
  __half* w_out;
  int N, K, M, gs, G;
  int gshift;  // log2(gs) when gs is a power of two >= 32, else -1
  int mpad;    // UMMA N: activation rows per CTA rounded up to 16
  int mtile;   // activation rows per CTA (<= 256)
  int stages;
  uint32_t tx_bytes;  // bytes the two TMA boxes of a chunk deliver (boxes are clipped to N and M)
  int splits;         // CTAs that share a tile's K range (grid.z)
  float* ws;          // splits > 1: partial tiles [tile][split][column][128 rows]
  int* counters;      // splits > 1: one arrival counter per tile, zero between launches
  int* status;
};

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
  // K-major, 128-byte swizzle: 8-row atoms of 1024 bytes; LBO = 1 (unused), version 1
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// (The form without the disable-output-lane vector: with that operand an instruction occupied the issuing thread
// for 185 cycles instead of 152, whatever the tile's width - measured in isolation.)
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

// A operand in tensor memory (lane = row, 32-bit column = two consecutive k), B through a shared-memory descriptor
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(db), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

// 32 columns of this thread's lane
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t v[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
      "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
      "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
      "r"(v[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t v[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// out[i] = (w[i], w[i+4]) -> eight consecutive halves
__device__ __forceinline__ uint4 unpair(const __half2 o[4]) {
  uint4 r;
  r.x = __byte_perm(h2_as_u32(o[0]), h2_as_u32(o[1]), 0x5410);
  r.y = __byte_perm(h2_as_u32(o[2]), h2_as_u32(o[3]), 0x5410);
  r.z = __byte_perm(h2_as_u32(o[0]), h2_as_u32(o[1]), 0x7632);
  r.w = __byte_perm(h2_as_u32(o[2]), h2_as_u32(o[3]), 0x7632);
  return r;
}

template <int FMT, bool HOOK>  // FMT: 0 W4 symmetric, 1 W4 asymmetric, 2 MXFP4
__global__ void __launch_bounds__(TK_THREADS, 1)
    tensor_gemm_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_x,
                       const TensorParams a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int stages = a.stages;
  const uint32_t x_bytes = (uint32_t)a.mpad * 128u;
  const uint32_t stage_bytes = x_bytes + TK_Q_BYTES;
  const uint32_t sm_base = smem_u32(smem);
  auto x_tile = [&](int s) { return sm_base + (uint32_t)s * stage_bytes; };
  auto q_tile = [&](int s) { return x_tile(s) + x_bytes; };
  const uint32_t sm_bar = sm_base + (uint32_t)stages * stage_bytes;
  auto load_full = [&](int s) { return sm_bar + 8u * (uint32_t)s; };
  auto a_ready = [&](int s) { return sm_bar + 8u * (uint32_t)(TK_MAX_STAGES + s); };
  auto stage_free = [&](int s) { return sm_bar + 8u * (uint32_t)(2 * TK_MAX_STAGES + s); };
  const uint32_t acc_ready = sm_bar + 8u * (uint32_t)(3 * TK_MAX_STAGES);
  const uint32_t tmem_slot = acc_ready + 8u;  // where tcgen05.alloc writes the TMEM base address
  const uint32_t last_slot = tmem_slot + 4u;  // split-K: whether this CTA arrived last at its tile's counter

  const int n0 = (int)blockIdx.x * TK_ROWS;
  const int m0 = (int)blockIdx.y * a.mtile;
  // this CTA's chunks: an equal share of the tile's K range
  const int all_chunks = (a.K + TK_KC - 1) / TK_KC;
  const int kc_begin = (int)((long long)all_chunks * blockIdx.z / a.splits);
  const int nchunks = (int)((long long)all_chunks * (blockIdx.z + 1) / a.splits) - kc_begin;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(load_full(s), 1);
      mbar_init(a_ready(s), 4);  // the four warps of the group that decodes the chunk
      mbar_init(stage_free(s), 1);
    }
    mbar_init(acc_ready, 1);
    mbar_init_fence();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_x);
  }
  // TMEM: the Mpad accumulator columns, then one decoded operand tile (128 rows x 64 k = 32 columns) per stage;
  // a power-of-two column count >= 32
  uint32_t ncols = 32;
  while (ncols < (uint32_t)a.mpad + 32u * (uint32_t)stages) ncols <<= 1;
  if (wid == TK_DECODERS + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem_acc;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_acc) : "r"(tmem_slot) : "memory");

  if (wid == TK_DECODERS) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int kc = 0; kc < nchunks; ++kc) {
        if (!mbar_wait(stage_free(s), ph ^ 1u, a.status, ST_TENSOR_TIMEOUT)) break;
        mbar_arrive_expect_tx(load_full(s), a.tx_bytes);
        tma_load_2d(q_tile(s), &tmap_q, (kc_begin + kc) * (TK_KC / 8), n0, load_full(s));
        tma_load_2d(x_tile(s), &tmap_x, (kc_begin + kc) * TK_KC, m0, load_full(s));
        if (++s == stages) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (wid == TK_DECODERS + 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      // instruction descriptor: D = F32, A = B = F16, both K-major, N = Mpad, M = 128
      const uint32_t idesc = (1u << 4) | ((uint32_t)(a.mpad >> 3) << 17) | ((uint32_t)(TK_ROWS >> 4) << 24);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int kc = 0; kc < nchunks && ok; ++kc) {
        if (!mbar_wait(a_ready(s), ph, a.status, ST_TENSOR_TIMEOUT)) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t db = make_smem_desc(x_tile(s));
        const uint32_t ta = tmem_acc + (uint32_t)a.mpad + 32u * (uint32_t)s;
#pragma unroll
        for (int k = 0; k < TK_KC / 16; ++k)  // 16 k = 8 columns of the operand tile, 32 bytes inside the swizzle row of x
          umma_f16_ts(tmem_acc, ta + 8u * k, db + 2u * k, idesc, kc > 0 || k > 0);
        umma_commit(stage_free(s));  // arrives when the MMAs above have read the stage
        if (++s == stages) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (ok) umma_commit(acc_ready);
    }
  } else {
    // ------------------------- decode warps 0..7 -------------------------
    // TK_GROUPS groups of four warps take chunks in turn (group = tid >> 7), so one group's waits,
    // fences and arrivals overlap the other groups' decoding. Thread t decodes row r = t & 127
    // of its group's chunks: 8 packed words -> 64 halves.
    const int r = tid & (TK_ROWS - 1);  // row of the tile == TMEM lane
    const int hf = tid >> 7;
    const int n = min(n0 + r, a.N - 1);
    const W4Consts kc4 = w4_consts();
    const int wG = words(a.G);
    // Group sizes that are powers of two >= 32 (and MXFP4's blocks) have one group per 32 k:
    // the two groups of a chunk are fetched one chunk ahead, outside the wait for the codes.
    const int gshift = FMT == 2 ? 5 : a.gshift;
    const bool pow2 = gshift >= 5;
    auto group_of = [&](int kc, int h) { return min(((kc_begin + kc) * TK_KC + 32 * h) >> gshift, a.G - 1); };
    auto fetch_w4 = [&](int grp) {
      const __half sc = ((const __half*)a.scales)[(size_t)n * a.G + grp];
      const uint32_t z = FMT == 0 ? 8u : ((a.zeros[(size_t)n * wG + (grp >> 3)] >> (4 * (grp & 7))) & 0xFu);
      return w4_group(sc, z);
    };
    W4Group gnext[2] = {w4_group(__ushort_as_half((unsigned short)0), 8u), w4_group(__ushort_as_half((unsigned short)0), 8u)};
    uint32_t enext[2] = {0, 0};
    auto prefetch = [&](int kc) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (FMT == 2)
          enext[h] = ((const uint8_t*)a.scales)[(size_t)n * a.G + group_of(kc, h)];
        else
          gnext[h] = fetch_w4(group_of(kc, h));
      }
    };
    if (pow2 && hf < nchunks) prefetch(hf);
    int s = hf % stages;
    uint32_t ph = (uint32_t)(hf / stages) & 1u;
    bool ok = true;
    for (int kc = hf; kc < nchunks; kc += TK_GROUPS) {
      const W4Group gcur[2] = {gnext[0], gnext[1]};
      const uint32_t ecur[2] = {enext[0], enext[1]};
      if (pow2 && kc + TK_GROUPS < nchunks) prefetch(kc + TK_GROUPS);
      if (!mbar_wait(load_full(s), ph, a.status, ST_TENSOR_TIMEOUT)) {
        ok = false;
        break;
      }
      const uint4 c0 = lds128(q_tile(s) + (uint32_t)r * 32u), c1 = lds128(q_tile(s) + (uint32_t)r * 32u + 16u);
      const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      uint32_t arow[32];  // this row's 64 decoded halves
      const MxBlock mcur[2] = {mx_block(ecur[0]), mx_block(ecur[1])};
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const int k0 = (kc_begin + kc) * TK_KC + 8 * w;
        __half2 o[4];
        if (FMT == 2) {
          dq_mx_word(cw[w], mcur[w >> 2], o);
        } else if (pow2) {
          dq_w4_word(cw[w], gcur[w >> 2], kc4, o);
        } else {
          dq_w4_word(cw[w], fetch_w4(min(k0 / a.gs, a.G - 1)), kc4, o);
        }
        const uint4 v = unpair(o);
        arow[4 * w] = v.x, arow[4 * w + 1] = v.y, arow[4 * w + 2] = v.z, arow[4 * w + 3] = v.w;
        if (HOOK && blockIdx.y == 0 && n0 + r < a.N && k0 < a.K)  // K % 8 == 0: whole words are in range
          *reinterpret_cast<uint4*>(a.w_out + (size_t)(n0 + r) * a.K + k0) = v;
      }
      // the row goes to lane r of the stage's operand tile in tensor memory (the warp's lane quarter)
      tmem_st32(tmem_acc + ((uint32_t)((wid & 3) * 32) << 16) + (uint32_t)a.mpad + 32u * (uint32_t)s, arow);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(a_ready(s));
      s += TK_GROUPS;
      while (s >= stages) {  // the ring is walked TK_GROUPS stages at a time
        s -= stages;
        ph ^= 1u;
      }
    }
    // ------------------------------ epilogue ------------------------------
    if (ok && mbar_wait(acc_ready, 0u, a.status, ST_TENSOR_TIMEOUT)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // warps w, w + 4, ... own the same TMEM lane quarter and take alternate 16-column blocks
      const uint32_t lane_base = (uint32_t)((wid & 3) * 32) << 16;
      for (int cb = 16 * hf; cb < a.mpad; cb += 16 * TK_GROUPS) {
        uint32_t v[16];
        tmem_ld16(tmem_acc + lane_base + (uint32_t)cb, v);
        if (a.splits > 1) {  // FP32 partial of this split: [tile][split][column][row], a warp writes 32 rows
          float* part = a.ws + ((((size_t)blockIdx.y * gridDim.x + blockIdx.x) * a.splits + blockIdx.z) * a.mpad + cb) * TK_ROWS + r;
#pragma unroll
          for (int i = 0; i < 16; ++i) __stcg(part + (size_t)i * TK_ROWS, __uint_as_float(v[i]));
        } else if (n0 + r < a.N) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = m0 + cb + i;
            if (cb + i < a.mtile && m < a.M) a.c[(size_t)m * a.N + n0 + r] = __float2half_rn(__uint_as_float(v[i]));
          }
        }
      }
    }
  }
  if (a.splits > 1) {
    // The split that arrives last at the tile's counter adds all partials in split order and stores the tile.
    __threadfence();  // this CTA's partial is visible before its arrival is counted
    __syncthreads();
    int* cnt = a.counters + (size_t)blockIdx.y * gridDim.x + blockIdx.x;
    if (tid == 0) {
      const int prev = atomicAdd(cnt, 1);
      const uint32_t last = prev == a.splits - 1 ? 1u : 0u;
      if (last) *cnt = 0;  // ready for the next launch
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(last_slot), "r"(last) : "memory");
    }
    __syncthreads();
    uint32_t is_last;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(is_last) : "r"(last_slot) : "memory");
    if (is_last && wid < TK_DECODERS) {
      __threadfence();
      const float* base = a.ws + (((size_t)blockIdx.y * gridDim.x + blockIdx.x) * a.splits) * (size_t)a.mpad * TK_ROWS;
      const int r = tid & (TK_ROWS - 1);
      // eight columns at a time, their loads in flight together (one dependent load after the other, this loop
      // cost more than the tile's MMAs); every column still adds its partials in split order
      for (int col0 = 8 * (tid >> 7); col0 < a.mtile && m0 + col0 < a.M; col0 += 8 * (TK_DECODERS / 4)) {
        float sum[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) sum[i] = 0.0f;
        for (int sp = 0; sp < a.splits; ++sp)
#pragma unroll
          for (int i = 0; i < 8; ++i) sum[i] += __ldcg(base + ((size_t)sp * a.mpad + col0 + i) * TK_ROWS + r);
        if (n0 + r < a.N) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (col0 + i < a.mtile && m0 + col0 + i < a.M) a.c[(size_t)(m0 + col0 + i) * a.N + n0 + r] = __float2half_rn(sum[i]);
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (wid == TK_DECODERS + 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(ncols) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

template <int FMT, bool HOOK>
cudaError_t launch_one(const CUtensorMap& tq, const CUtensorMap& tx, const TensorParams& tp, dim3 grid, size_t smem,
                       cudaStream_t stream) {
  auto kern = tensor_gemm_kernel<FMT, HOOK>;
  // The shared-memory opt-in is a per-device attribute of the function: set it once on every device used.
  static std::atomic<bool> configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev].load(std::memory_order_acquire)) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return e;
    configured[dev].store(true, std::memory_order_release);
  }
  kern<<<grid, TK_THREADS, smem, stream>>>(tq, tx, tp);
  return cudaGetLastError();
}

}  // namespace

// CTAs per tile along K: 1 when the tiles fill at least half the SMs, else enough to fill them, with at least
// 8 chunks (512 k) per CTA.
void tensor_gemm_plan(int N, int K, int M, int sm_count, TensorPlan* plan) {
  const int mtile = M < 256 ? M : 256, mpad = (mtile + 15) / 16 * 16;
  const long long tiles = (long long)((N + TK_ROWS - 1) / TK_ROWS) * ((M + mtile - 1) / mtile);
  const int chunks = (K + TK_KC - 1) / TK_KC;
  int splits = 1;
  if (tiles * 2 <= sm_count) {
    splits = (int)(sm_count / tiles);
    if (splits > chunks / 8) splits = chunks / 8;
    if (splits < 1) splits = 1;
  }
  plan->splits = splits;
  plan->ws_bytes = splits > 1 ? (size_t)tiles * splits * mpad * TK_ROWS * sizeof(float) : 0;
  plan->counter_ints = splits > 1 ? (size_t)tiles : 0;
}

bool tensor_gemm_supported(int N, int K, const void* q, const void* x) {
  if (N < 1 || K < 32 || K % 32 != 0) return false;
  if (((uintptr_t)q | (uintptr_t)x) & 15u) return false;
  return encode_tiled() != nullptr;
}

cudaError_t tensor_gemm_launch(int fmt, int gs, const uint32_t* q, const void* scales, const uint32_t* zeros, int N,
                               int K, int G, const __half* x, __half* c, int M, __half* w_out, const TensorPlan& plan,
                               float* ws, int* counters, int* status, cudaStream_t stream) {
  TensorParams tp;
  tp.splits = plan.splits;
  tp.ws = ws;
  tp.counters = counters;
  tp.q = q;
  tp.scales = scales;
  tp.zeros = zeros;
  tp.c = c;
  tp.w_out = w_out;
  tp.N = N;
  tp.K = K;
  tp.M = M;
  tp.gs = gs;
  tp.gshift = -1;
  for (int b = 5; b < 31; ++b)
    if (gs == (1 << b)) tp.gshift = b;
  tp.G = G;
  tp.mtile = M < 256 ? M : 256;
  tp.mpad = (tp.mtile + 15) / 16 * 16;
  const size_t stage_bytes = (size_t)tp.mpad * 128 + TK_Q_BYTES;  // (the decoded tile lives in tensor memory)
  int stages = (int)((232448 - 1024 - 8 * (3 * TK_MAX_STAGES + 2)) / stage_bytes);
  if (tp.mpad + 32 * stages > 512) stages = (512 - tp.mpad) / 32;  // tensor memory: accumulator + one operand tile per stage
  // The ring depth is a multiple of the number of decode groups, so that a stage is always decoded by the
  // same group: a group then waits for fill n of a stage only after it has consumed fill n - 1 (an mbarrier
  // phase may be awaited at most one phase ahead - with more groups than stages a group would "pass" a wait
  // for a fill that has not even started; six groups over four stages faulted that way).
  stages = stages > TK_MAX_STAGES ? TK_MAX_STAGES : stages;
  tp.stages = stages / TK_GROUPS * TK_GROUPS;
  if (tp.stages < TK_GROUPS) return cudaErrorInvalidConfiguration;  // cannot happen: a stage is at most 52 KB
  tp.status = status;
  const size_t smem = 1024 + (size_t)tp.stages * stage_bytes + 8 * (3 * TK_MAX_STAGES + 2);

  CUtensorMap tq, tx;
  {
    const cuuint64_t gdim[2] = {(cuuint64_t)(K / 8), (cuuint64_t)N};
    const cuuint64_t gstride[1] = {(cuuint64_t)(K / 8) * 4};
    const cuuint32_t box[2] = {TK_KC / 8, (cuuint32_t)(N < TK_ROWS ? N : TK_ROWS)};  // a box never exceeds the tensor
    const cuuint32_t estr[2] = {1, 1};
    tp.tx_bytes = box[1] * (TK_KC / 2);
    if (encode_tiled()(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)q, gdim, gstride, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  {
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t gstride[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {TK_KC, (cuuint32_t)(M < tp.mpad ? M : tp.mpad)};
    const cuuint32_t estr[2] = {1, 1};
    tp.tx_bytes += box[1] * 128;
    if (encode_tiled()(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)x, gdim, gstride, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  const dim3 grid((unsigned)((N + TK_ROWS - 1) / TK_ROWS), (unsigned)((M + tp.mtile - 1) / tp.mtile),
                  (unsigned)plan.splits);
  const bool hook = w_out != nullptr;
  if (fmt == 0)
    return hook ? launch_one<0, true>(tq, tx, tp, grid, smem, stream) : launch_one<0, false>(tq, tx, tp, grid, smem, stream);
  if (fmt == 1)
    return hook ? launch_one<1, true>(tq, tx, tp, grid, smem, stream) : launch_one<1, false>(tq, tx, tp, grid, smem, stream);
  return hook ? launch_one<2, true>(tq, tx, tp, grid, smem, stream) : launch_one<2, false>(tq, tx, tp, grid, smem, stream);
}

}  // namespace w4b
