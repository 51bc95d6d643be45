// HBM-streaming fused dequant GEMM for decode-sized M (the replacement of the
// reference's SIMT kernels fused_kernel / fused_kernel_mx,
// include/w4/fused.cuh:68-170 and include/w4/mxfused.cuh:74-164).
//
// The packed weights are the whole cost: every byte of q / scales / zeros is
// read from HBM exactly once, and the kernel is organised so that this stream
// never stalls.
//
//  * Work unit = 128 rows x 256 k of packed codes = one 16 KB 2-D TMA box
//    (cp.async.bulk.tensor, 128-byte swizzle, no multicast). The units of the
//    whole matrix are numbered panel-major / chunk-fastest and cut into equal
//    contiguous ranges, one per persistent CTA (one CTA per SM), so all SMs
//    finish together whatever N and K are ("stream-K").
//  * Warp 8 is the producer: per unit it issues the TMA box plus 4..16-byte
//    cp.async copies of the unit's scales / zero words into a ring of up to 12
//    stages; full/empty mbarriers hand stages over. With ~200 KB of ring per SM
//    the loads of a CTA's whole share are in flight almost from the start.
//  * Warps 0..7 are consumers; warp w owns rows 16w..16w+15 of every unit. A
//    lane decodes packed words in registers (w4b_common.cuh: no tables, no
//    local memory) straight into mma.sync m16n8k16 A fragments; the activations
//    sit in shared memory, pre-arranged once per CTA in the decoder's pairing,
//    and are the B fragments; FP32 accumulators live in registers across the
//    units of a panel. At M = 1 the budget is ~2.8 issue slots per weight at
//    full HBM rate, which rules out per-weight FP32 FMAs: the contraction has
//    to ride the tensor pipe even though the kernel is bandwidth-bound.
//  * A panel whose K range is split between CTAs is finished deterministically:
//    every contributor parks its FP32 fragment in a workspace slot and bumps
//    the tile's counter; the last arriver adds the slots in CTA order (never
//    in arrival order) and writes FP16. Outputs are therefore bit-identical
//    from run to run.
//
// Shapes served: K % 256 == 0, N >= 128, W4 group size 32 / 64 / 128 (MXFP4:
// its fixed 32-element blocks), 16-byte aligned q / scales / x. Anything else
// is routed to the generic kernel by the dispatcher.
#include <cuda.h>

#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {

namespace {

constexpr int SK_ROWS = 128;
constexpr int SK_KC = 256;
constexpr int SK_STAGE_Q = SK_ROWS * SK_KC / 2;  // 16384 bytes of codes per unit
constexpr int SK_META_SCALES = SK_ROWS * 16;     // <= 8 FP16 scales or 8 E8M0 bytes per row
constexpr int SK_META = SK_META_SCALES + SK_ROWS * 4;  // + one zero word per row
constexpr int SK_CONSUMERS = 8;
constexpr int SK_THREADS = 32 * (SK_CONSUMERS + 1);
constexpr int SK_MAX_STAGES = 12;

enum : int { F_W4_SYM = 0, F_W4_ASYM = 1, F_MX = 2 };

struct StreamParams {
  const uint32_t* q;
  const void* scales;
  const uint32_t* zeros;
  const __half* x;
  __half* c;
  __half* w_out;
  int N, K, M;
  int G;       // scales per row: groups (W4) or 32-blocks (MX)
  int C, P;    // 256-k chunks per row, 128-row panels
  long long U; // units = P * C
  int stages;
  int xrows;   // activation rows per pass (<= 8*MT); pass y covers rows y*xrows ...
  int xpitch;  // bytes between activation rows in shared memory (== 64 mod 128)
  float* ws;
  int* counters;
  int* status;
};

__device__ __forceinline__ long long unit_begin(long long U, int b, int grid) {
  return U * (long long)b / grid;
}
// The CTA whose range holds unit t (ranges are [U*b/grid, U*(b+1)/grid)).
__device__ __forceinline__ int unit_owner(long long U, long long t, int grid) {
  return (int)(((t + 1) * grid + U - 1) / U) - 1;
}

template <int FMT, int GS>
struct Groups;  // per-row decode constants of one unit: [0] for words 0-3, [1] for words 4-7

template <int GS>
struct Groups<F_W4_SYM, GS> {
  W4Group g[2];
  __device__ __forceinline__ void load(uint32_t meta_row, uint32_t /*zero_row*/, int c, int /*ch*/) {
    constexpr int NGU = SK_KC / GS;
    const int gi = GS == 128 ? (c >> 1) : (GS == 64 ? c : 2 * c);
    unsigned short s0, s1;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s0) : "r"(meta_row + 2 * gi));
    g[0] = w4_group(__ushort_as_half(s0), 8u);
    if (NGU == 8) {
      asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s1) : "r"(meta_row + 2 * gi + 2));
      g[1] = w4_group(__ushort_as_half(s1), 8u);
    } else {
      g[1] = g[0];
    }
  }
  __device__ __forceinline__ void decode(uint32_t w, int half, __half2 out[4]) const {
    dq_w4_word(w, g[half], out);
  }
};

template <int GS>
struct Groups<F_W4_ASYM, GS> {
  W4Group g[2];
  __device__ __forceinline__ void load(uint32_t meta_row, uint32_t zero_row, int c, int ch) {
    constexpr int NGU = SK_KC / GS;
    const int gi = GS == 128 ? (c >> 1) : (GS == 64 ? c : 2 * c);
    unsigned short s0, s1;
    uint32_t zw;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s0) : "r"(meta_row + 2 * gi));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zw) : "r"(zero_row));
    const int nib = (ch * NGU + gi) & 7;  // group index within its zero word
    g[0] = w4_group(__ushort_as_half(s0), (zw >> (4 * nib)) & 0xFu);
    if (NGU == 8) {
      asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s1) : "r"(meta_row + 2 * gi + 2));
      g[1] = w4_group(__ushort_as_half(s1), (zw >> (4 * nib + 4)) & 0xFu);
    } else {
      g[1] = g[0];
    }
  }
  __device__ __forceinline__ void decode(uint32_t w, int half, __half2 out[4]) const {
    dq_w4_word(w, g[half], out);
  }
};

template <int GS>
struct Groups<F_MX, GS> {
  MxBlock b[2];
  __device__ __forceinline__ void load(uint32_t meta_row, uint32_t /*zero_row*/, int c, int /*ch*/) {
    unsigned short s;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s) : "r"(meta_row + 2 * c));
    b[0] = mx_block((uint32_t)s & 0xFFu);
    b[1] = mx_block((uint32_t)s >> 8);
  }
  __device__ __forceinline__ void decode(uint32_t w, int half, __half2 out[4]) const {
    dq_mx_word(w, b[half], out);
  }
};

__device__ __forceinline__ uint32_t word_of(const uint4& a, const uint4& b, int i) {
  switch (i) {
    case 0: return a.x;
    case 1: return a.y;
    case 2: return a.z;
    case 3: return a.w;
    case 4: return b.x;
    case 5: return b.y;
    case 6: return b.z;
    default: return b.w;
  }
}

template <int FMT, int GS, int MT, bool HOOK>
__global__ void __launch_bounds__(SK_THREADS, 1)
    stream_gemm_kernel(const __grid_constant__ CUtensorMap tmap, const StreamParams a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int stages = a.stages;
  const uint32_t sm_q = (smem_u32(smem) + 1023u) & ~1023u;  // the swizzle pattern repeats every 1024 bytes
  const uint32_t sm_meta = sm_q + (uint32_t)stages * SK_STAGE_Q;
  const uint32_t sm_x = sm_meta + (uint32_t)stages * SK_META;
  const uint32_t sm_bar = sm_x + (uint32_t)a.xrows * (uint32_t)a.xpitch;
  auto full_bar = [&](int s) { return sm_bar + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return sm_bar + 8u * (uint32_t)(stages + s); };

  const int grid = (int)gridDim.x;
  const int m0 = (int)blockIdx.y * a.xrows;          // first activation row of this pass
  const int mrows = min(a.xrows, a.M - m0);            // rows of this pass (the last may be short)
  const int C = a.C;
  const long long u0 = unit_begin(a.U, (int)blockIdx.x, grid);
  const long long u1 = unit_begin(a.U, (int)blockIdx.x + 1, grid);

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 33);  // lane 0's expect_tx arrive + one cp.async arrive per producer lane
      mbar_init(empty_bar(s), SK_CONSUMERS);
    }
    mbar_init_fence();
    tma_prefetch_desc(&tmap);
  }
  __syncthreads();

  if (wid == SK_CONSUMERS) {
    // ------------------------------ producer ------------------------------
    constexpr int NGU = FMT == F_MX ? 8 : SK_KC / GS;  // scales per row per unit
    const int wG = words(a.G);
    int s = 0;
    uint32_t ph = 0;
    int p = (int)(u0 / C), ch = (int)(u0 % C);
    for (long long u = u0; u < u1; ++u) {
      if (!mbar_wait(empty_bar(s), ph ^ 1u, a.status, ST_STREAM_EMPTY_TIMEOUT)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(full_bar(s), SK_STAGE_Q);
        tma_load_2d(sm_q + (uint32_t)s * SK_STAGE_Q, &tmap, ch * (SK_KC / 8), p * SK_ROWS, full_bar(s));
      }
      const uint32_t meta = sm_meta + (uint32_t)s * SK_META;
#pragma unroll
      for (int rr = 0; rr < SK_ROWS / 32; ++rr) {
        const int r = lane + 32 * rr;
        const int n = min(p * SK_ROWS + r, a.N - 1);  // rows past N: any valid row, never used
        if (FMT == F_MX) {
          cp_async<8>(meta + r * 16, (const uint8_t*)a.scales + (size_t)n * a.G + (size_t)ch * 8);
        } else {
          cp_async<NGU * 2>(meta + r * 16, (const __half*)a.scales + (size_t)n * a.G + (size_t)ch * NGU);
          if (FMT == F_W4_ASYM)
            cp_async<4>(meta + SK_META_SCALES + r * 4, a.zeros + (size_t)n * wG + (size_t)((ch * NGU) >> 3));
        }
      }
      cp_async_arrive_noinc(full_bar(s));
      if (++s == stages) {
        s = 0;
        ph ^= 1u;
      }
      if (++ch == C) {
        ch = 0;
        ++p;
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  // Activations of this pass: rows m0 .. m0+xrows-1, FP16, each row re-ordered so
  // that the 16 bytes a lane needs for word slot i of unit `ch` are
  //   chunk (ch*32 + i*4 + c) = halves (h0,h4,h1,h5,h2,h6,h3,h7) of natural word (ch*32 + c*8 + i).
  {
    const int cpr = a.K >> 3;  // 16-byte chunks per activation row
    const int total = mrows * cpr;
    for (int idx = tid; idx < total; idx += 32 * SK_CONSUMERS) {
      const int m = idx / cpr, widx = idx - m * cpr;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.x + (size_t)(m0 + m) * a.K) + widx);
      const int ub = widx >> 5, wi = widx & 31;
      const int dst = (ub << 5) + ((wi & 7) << 2) + (wi >> 3);
      sts128(sm_x + (uint32_t)m * (uint32_t)a.xpitch + ((uint32_t)dst << 4), pair_permute(v));
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * SK_CONSUMERS) : "memory");
  }

  const int g = lane >> 2, c = lane & 3;
  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;

  const int p_first = (int)(u0 / C);
  int p = p_first, ch = (int)(u0 % C), ch_begin = ch;
  int s = 0;
  uint32_t ph = 0;

  // x rows this lane supplies as B-fragment column g (and g + 8 for the second m-tile)
  uint32_t xrow[MT];
  bool xok[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    xok[mt] = (g + 8 * mt) < mrows;
    xrow[mt] = sm_x + (uint32_t)(xok[mt] ? g + 8 * mt : 0) * (uint32_t)a.xpitch + ((uint32_t)c << 4);
  }

  for (long long u = u0; u < u1; ++u) {
    if (!mbar_wait(full_bar(s), ph, a.status, ST_STREAM_FULL_TIMEOUT)) return;
    const int tile_row0 = p * SK_ROWS + wid * 16;
    if (tile_row0 < a.N) {  // warp-uniform
      const uint32_t qs = sm_q + (uint32_t)s * SK_STAGE_Q;
      const uint32_t ra = (uint32_t)(wid * 16 + g);  // row inside the box; ra & 7 == g
      const uint32_t offa = qs + ra * 128u, offb = offa + 8u * 128u;
      const uint32_t c0 = ((uint32_t)(2 * c) ^ (uint32_t)g) << 4, c1 = ((uint32_t)(2 * c + 1) ^ (uint32_t)g) << 4;
      const uint4 qa0 = lds128(offa + c0), qa1 = lds128(offa + c1);
      const uint4 qb0 = lds128(offb + c0), qb1 = lds128(offb + c1);
      const uint32_t meta = sm_meta + (uint32_t)s * SK_META;
      Groups<FMT, GS> ga, gb;
      ga.load(meta + ra * 16u, meta + SK_META_SCALES + ra * 4u, c, ch);
      gb.load(meta + (ra + 8u) * 16u, meta + SK_META_SCALES + (ra + 8u) * 4u, c, ch);
      const uint32_t xoff = (uint32_t)ch << 9;  // 32 chunks of 16 bytes per unit
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        __half2 pa[4], pb[4];
        ga.decode(word_of(qa0, qa1, i), i >> 2, pa);
        gb.decode(word_of(qb0, qb1, i), i >> 2, pb);
        if (HOOK && blockIdx.y == 0) {  // every pass decodes the same weights; one writes them
          const int k = ch * SK_KC + 64 * c + 8 * i;
          const int na = tile_row0 + g, nb = na + 8;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (na < a.N) {
              a.w_out[(size_t)na * a.K + k + j] = __low2half(pa[j]);
              a.w_out[(size_t)na * a.K + k + j + 4] = __high2half(pa[j]);
            }
            if (nb < a.N) {
              a.w_out[(size_t)nb * a.K + k + j] = __low2half(pb[j]);
              a.w_out[(size_t)nb * a.K + k + j + 4] = __high2half(pb[j]);
            }
          }
        }
        const uint32_t f0[4] = {h2_as_u32(pa[0]), h2_as_u32(pb[0]), h2_as_u32(pa[1]), h2_as_u32(pb[1])};
        const uint32_t f1[4] = {h2_as_u32(pa[2]), h2_as_u32(pb[2]), h2_as_u32(pa[3]), h2_as_u32(pb[3])};
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint4 xv = make_uint4(0u, 0u, 0u, 0u);
          if (xok[mt]) xv = lds128(xrow[mt] + xoff + ((uint32_t)i << 6));
          mma_16816(acc[mt], f0, xv.x, xv.y);
          mma_16816(acc[mt], f1, xv.z, xv.w);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(s));
    if (++s == stages) {
      s = 0;
      ph ^= 1u;
    }
    ++ch;
    if (ch == C || u + 1 == u1) {
      // ---- the CTA leaves panel p having covered chunks [ch_begin, ch) ----
      if (tile_row0 < a.N) {
        const bool whole = (ch_begin == 0 && ch == C);
        float out[MT][4];
        bool write = whole;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int i = 0; i < 4; ++i) out[mt][i] = acc[mt][i];
        if (!whole) {
          const int slot = (p == p_first) ? 0 : 1;
          const size_t cta = (size_t)blockIdx.y * grid + blockIdx.x;
          float4* mine = reinterpret_cast<float4*>(a.ws) + (((cta * 2 + slot) * SK_CONSUMERS + wid) * MT) * 32;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            mine[mt * 32 + lane] = make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
          __threadfence();
          __syncwarp();
          const int b_first = unit_owner(a.U, (long long)p * C, grid);
          const int b_last = unit_owner(a.U, (long long)(p + 1) * C - 1, grid);
          int* cnt = a.counters + ((size_t)blockIdx.y * a.P + p) * SK_CONSUMERS + wid;
          int old = 0;
          if (lane == 0) old = atomicAdd(cnt, 1);
          old = __shfl_sync(0xffffffffu, old, 0);
          if (old == b_last - b_first) {  // last of (b_last - b_first + 1) contributors
            __threadfence();
            write = true;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
              for (int i = 0; i < 4; ++i) out[mt][i] = 0.0f;
            for (int b = b_first; b <= b_last; ++b) {  // fixed order: by CTA, not by arrival
              const int sl = ((int)(unit_begin(a.U, b, grid) / C) == p) ? 0 : 1;
              const size_t ob = (size_t)blockIdx.y * grid + b;
              const float4* theirs =
                  reinterpret_cast<const float4*>(a.ws) + (((ob * 2 + sl) * SK_CONSUMERS + wid) * MT) * 32;
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                const float4 v = __ldcg(theirs + mt * 32 + lane);
                out[mt][0] += v.x;
                out[mt][1] += v.y;
                out[mt][2] += v.z;
                out[mt][3] += v.w;
              }
            }
            if (lane == 0) *cnt = 0;  // ready for the next launch
          }
        }
        if (write) {
          const int na = tile_row0 + g, nb = na + 8;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const int col = 8 * mt + 2 * c;  // activation row within this pass
            const int m = m0 + col;
            if (col < mrows) {
              if (na < a.N) a.c[(size_t)m * a.N + na] = __float2half_rn(out[mt][0]);
              if (nb < a.N) a.c[(size_t)m * a.N + nb] = __float2half_rn(out[mt][2]);
            }
            if (col + 1 < mrows) {
              if (na < a.N) a.c[(size_t)(m + 1) * a.N + na] = __float2half_rn(out[mt][1]);
              if (nb < a.N) a.c[(size_t)(m + 1) * a.N + nb] = __float2half_rn(out[mt][3]);
            }
          }
        }
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
      if (ch == C) {
        ch = 0;
        ++p;
      }
      ch_begin = ch;
    }
  }
}

// ------------------------------ host side ---------------------------------

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

template <int FMT, int GS, int MT, bool HOOK>
cudaError_t launch_one(const CUtensorMap& tmap, const StreamParams& sp, dim3 grid, size_t smem,
                       cudaStream_t stream) {
  auto kern = stream_gemm_kernel<FMT, GS, MT, HOOK>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  kern<<<grid, SK_THREADS, smem, stream>>>(tmap, sp);
  return cudaGetLastError();
}

template <int FMT, int GS>
cudaError_t launch_fmt(const CUtensorMap& tmap, const StreamParams& sp, int mt, dim3 grid, size_t smem,
                       cudaStream_t stream) {
  const bool hook = sp.w_out != nullptr;
  if (mt == 1)
    return hook ? launch_one<FMT, GS, 1, true>(tmap, sp, grid, smem, stream)
                : launch_one<FMT, GS, 1, false>(tmap, sp, grid, smem, stream);
  return hook ? launch_one<FMT, GS, 2, true>(tmap, sp, grid, smem, stream)
              : launch_one<FMT, GS, 2, false>(tmap, sp, grid, smem, stream);
}

}  // namespace

namespace {
constexpr int kSmemBudget = 232448 - 1024 /* alignment slack */ - 2 * 8 * SK_MAX_STAGES /* barriers */;
int stages_for(int rows, int K) { return (kSmemBudget - rows * (K * 2 + 64)) / (SK_STAGE_Q + SK_META); }
}  // namespace

bool stream_gemm_supported(int N, int K, int gs_or_0_for_mx, const void* q, const void* scales,
                           const void* x) {
  if (N < SK_ROWS || K < SK_KC || K % SK_KC != 0) return false;
  if (gs_or_0_for_mx != 0 && gs_or_0_for_mx != 32 && gs_or_0_for_mx != 64 && gs_or_0_for_mx != 128)
    return false;
  if (((uintptr_t)q | (uintptr_t)scales | (uintptr_t)x) & 15u) return false;
  if (K > 65536 || stages_for(1, K) < 4) return false;  // one activation row must fit beside a 4-stage ring
  return encode_tiled() != nullptr;
}

void stream_gemm_plan(int N, int K, int M, int sm_count, StreamPlan* plan) {
  const int xpitch = K * 2 + 64;
  // activation rows per pass: 16 if they leave room for a 4-stage ring, else 8, else fewer
  int rows = M < 16 ? M : 16;
  if (rows > 8 && stages_for(rows, K) < 4) rows = 8;
  while (rows > 1 && stages_for(rows, K) < 4) --rows;
  plan->rows_per_pass = rows;
  plan->mt = rows > 8 ? 2 : 1;
  plan->passes = (M + rows - 1) / rows;
  const int st = stages_for(rows, K);
  plan->stages = st > SK_MAX_STAGES ? SK_MAX_STAGES : st;
  plan->P = (N + SK_ROWS - 1) / SK_ROWS;
  plan->C = K / SK_KC;
  plan->U = (long long)plan->P * plan->C;
  plan->grid_x = (int)(plan->U < sm_count ? plan->U : sm_count);
  plan->xpitch = xpitch;
  plan->smem = 1024 + (size_t)plan->stages * (SK_STAGE_Q + SK_META) + (size_t)rows * xpitch + 2 * 8 * SK_MAX_STAGES;
  plan->ws_bytes = (size_t)plan->passes * plan->grid_x * 2 * SK_CONSUMERS * plan->mt * 32 * sizeof(float4);
  plan->counter_ints = (size_t)plan->passes * plan->P * SK_CONSUMERS;
}

// Launches the stream GEMM. `fmt`: 0 = W4 symmetric, 1 = W4 asymmetric, 2 = MXFP4.
// The caller has checked stream_gemm_supported and sized ws / counters by the plan;
// counters are all zero between launches.
cudaError_t stream_gemm_launch(int fmt, int gs, const uint32_t* q, const void* scales, const uint32_t* zeros,
                               int N, int K, int G, const __half* x, __half* c, int M, __half* w_out,
                               const StreamPlan& plan, float* ws, int* counters, int* status,
                               cudaStream_t stream) {
  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {(cuuint64_t)(K / 8), (cuuint64_t)N};
  const cuuint64_t gstride[1] = {(cuuint64_t)(K / 8) * 4};
  const cuuint32_t box[2] = {SK_KC / 8, SK_ROWS};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode_tiled()(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)q, gdim, gstride, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;

  StreamParams sp;
  sp.q = q;
  sp.scales = scales;
  sp.zeros = zeros;
  sp.x = x;
  sp.c = c;
  sp.w_out = w_out;
  sp.N = N;
  sp.K = K;
  sp.M = M;
  sp.G = G;
  sp.C = plan.C;
  sp.P = plan.P;
  sp.U = plan.U;
  sp.stages = plan.stages;
  sp.xpitch = plan.xpitch;
  sp.ws = ws;
  sp.counters = counters;
  sp.status = status;

  sp.xrows = plan.rows_per_pass;
  const dim3 grid((unsigned)plan.grid_x, (unsigned)plan.passes);  // pass y = activation rows y*rows_per_pass ...
  switch (fmt) {
    case F_W4_SYM:
      if (gs == 32) return launch_fmt<F_W4_SYM, 32>(tmap, sp, plan.mt, grid, plan.smem, stream);
      if (gs == 64) return launch_fmt<F_W4_SYM, 64>(tmap, sp, plan.mt, grid, plan.smem, stream);
      return launch_fmt<F_W4_SYM, 128>(tmap, sp, plan.mt, grid, plan.smem, stream);
    case F_W4_ASYM:
      if (gs == 32) return launch_fmt<F_W4_ASYM, 32>(tmap, sp, plan.mt, grid, plan.smem, stream);
      if (gs == 64) return launch_fmt<F_W4_ASYM, 64>(tmap, sp, plan.mt, grid, plan.smem, stream);
      return launch_fmt<F_W4_ASYM, 128>(tmap, sp, plan.mt, grid, plan.smem, stream);
    default:
      return launch_fmt<F_MX, 32>(tmap, sp, plan.mt, grid, plan.smem, stream);
  }
}

}  // namespace w4b
