// HBM-streaming fused dequant GEMM for decode-sized M (the replacement of the
// reference's SIMT kernels fused_kernel / fused_kernel_mx,
// include/w4/fused.cuh:68-170 and include/w4/mxfused.cuh:74-164).
//
// The packed weights are the whole cost: every byte of q / scales / zeros is
// read from HBM exactly once, and the kernel is organised so that this stream
// never stalls and nothing else sits on the critical path.
//
//  * Work unit = 64 rows x 512 k of packed codes = 16 KB, fetched as two 2-D
//    TMA boxes of 64 rows x 128 bytes (cp.async.bulk.tensor, 128-byte swizzle,
//    no multicast). A "panel" is the C = ceil(K/512) units of 64 rows. The
//    units of the whole matrix are numbered panel-major / chunk-fastest and cut
//    into equal contiguous ranges, one per persistent CTA (one CTA per SM), so
//    all SMs finish together whatever N and K are ("stream-K"). Panels are
//    kept short (64 rows) so that a CTA's range is longer than a panel for the
//    usual K: the parts of panels that CTAs share are then done long before
//    their owner needs them.
//  * One warp is the loader: per unit it waits for a free ring stage,
//    issues the two boxes and copies the unit's scales / zero words beside them
//    (cp.async, a few bytes per row); full/empty mbarriers hand the stages
//    over. It touches nothing but the packed weights, so it runs ahead of
//    the previous kernel of the stream (see "launch overlap" below).
//  * The other eight warps are consumers: warp w owns the 16-row tile w & 3 and
//    the 256-k half w >> 2 of every unit. A lane decodes packed
//    words in registers (w4b_common.cuh: no tables, no local memory) into
//    mma.sync m16n8k16 A fragments; the activations sit in shared memory,
//    arranged once per CTA in the decoder's pairing, and are the B fragments;
//    FP32 accumulators stay in registers across the units of a panel. On B200
//    the packed-half pipe issues 64 lanes per clock per SM, so the half2
//    operations of the decode already cost most of the issue budget: there is
//    no room for per-weight FP32 FMAs, and the contraction rides the tensor
//    pipe although the kernel is bandwidth-bound.
//  * Leaving a panel, the warp of the upper k half hands its fragment to the
//    warp of the lower half through shared memory (it never waits for it).
//    A panel whose K range is shared by several CTAs is finished by the CTA
//    that owns the panel's END: the others park their FP32 fragment in a
//    workspace slot, and the CTA's hand-off warp publishes them (fence, counter)
//    and, in the owner, waits (bounded) for the counters and adds the slots in
//    CTA order into shared memory - no consumer warp and no load ever waits for
//    a round trip to L2. Every CTA
//    walks its range as [tail part, whole panels, head part], so what others
//    wait for is produced first and what a CTA waits for is consumed last: in
//    the common case nobody waits, and the order of the additions never depends
//    on timing - outputs are bit-identical from run to run.
//  * Launch overlap (programmatic dependent launch, opt-in by the caller): the
//    CTA uses at most half an SM's shared memory where a useful ring fits in it,
//    so the next launch's CTA becomes resident beside this one and fills its
//    ring with weights while this grid is still computing; its consumers wait
//    for this grid to complete before they read activations or touch c /
//    scratch.
//
// Shapes served: K % 512 == 0, N >= 64, W4 group size 32 / 64 / 128 (MXFP4:
// its fixed 32-element blocks), 16-byte aligned q / scales / x. Anything else
// is routed to the generic kernel by the dispatcher.
#include <cuda.h>

#include <string.h>

#include <atomic>

#include <type_traits>

#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {

namespace {

constexpr int SK_ROWS = 64;                      // rows per unit: 4 tiles of 16
constexpr int SK_KC = 256;                       // k per box (one warp's share of a unit)
constexpr int SK_KU = 2 * SK_KC;                 // k per unit: two boxes side by side
constexpr int SK_BOX = SK_ROWS * SK_KC / 2;      // 8192 bytes of codes per box
constexpr int SK_STAGE_Q = 2 * SK_BOX;           // 16384 bytes of codes per unit
// Scales per row and unit: 512 / gs FP16 values (8, 16 or 32 bytes) or 16 E8M0 bytes; then 8 bytes of zero words.
__host__ __device__ constexpr int sk_meta_row(int fmt, int gs) { return fmt == 2 ? 16 : 2 * (512 / gs); }
__host__ __device__ constexpr int sk_meta(int fmt, int gs) { return SK_ROWS * (sk_meta_row(fmt, gs) + 8); }
__host__ __device__ constexpr int sk_stage(int fmt, int gs) { return SK_STAGE_Q + sk_meta(fmt, gs); }
constexpr int SK_TILES = 4;                      // 16-row tiles per unit
constexpr int SK_CONSUMERS = 2 * SK_TILES;       // consumer warps: tile x k half
constexpr int SK_LOADER = SK_CONSUMERS;          // warp that issues the loads
constexpr int SK_HANDOFF = SK_CONSUMERS + 1;     // warp that exchanges fragments with other CTAs
constexpr int SK_THREADS = 32 * (SK_CONSUMERS + 2);
constexpr int SK_MAX_STAGES = 12;
constexpr int SK_BAR_BYTES = 8 * (2 * SK_MAX_STAGES + 4);  // ring barriers + "parked" + "collected" + "peers_ok" + a counter
constexpr int SK_RED_BYTES_PER_MT = SK_TILES * 32 * 16;      // the upper k half's fragments, one per tile
constexpr int SK_COLLECT_BYTES_PER_MT = SK_TILES * 32 * 16;  // other CTAs' fragments, summed
constexpr int SK_XROW = 1024 + 64;  // streamed activations: bytes per row of a unit's block (== 64 mod 128)
constexpr int SK_XS_BYTES = 256;    // then the sums of the unit's 4 groups x 16 rows (FP32)
__host__ __device__ constexpr int sk_xblock(int mt) { return 8 * mt * SK_XROW + SK_XS_BYTES; }
constexpr int SK_ZERO_BYTES = 512;  // one unit's worth of 16-byte chunks for the four lanes of a column
constexpr int kSmemOptIn = 232448;  // dynamic shared memory a CTA may ask for (227 KB)
// With at most this much per CTA two CTAs fit on an SM (228 KB, 1 KB reserved per CTA): the CTA of the next
// launch becomes resident beside this launch's and pre-loads its ring (programmatic dependent launch).
constexpr int kSmemHalf = (233472 - 2 * 1024) / 2;
constexpr int kMaxDevices = 64;

enum : int { F_W4_SYM = 0, F_W4_ASYM = 1, F_MX = 2 };
// W4 with 128-element groups takes scale and zero point out of the contraction. A masked code is used as the
// FP16 bit pattern it is: 0x000q is the (subnormal) half q * 2^-24, 0x00q0 is q * 2^-20, both exact, so the
// tensor pipe sums x * q over the 128 k of one group straight from the packed word (one shift and four ANDs per
// 8 weights; activations that meet the 2^-20 codes are stored divided by 16) with FP32 accumulation, and the
// group then contributes  s * (2^24 * sum(x q) - z * sum(x))  in FP32, sum(x) per group being worked out once
// per CTA. That is the same number as sum x * (s * (q - z)) without rounding every weight to FP16 first (rel L2
// against the FP64 reference GEMM 2.8e-4 instead of 2.1e-4, gate 1e-3) at less than half the instructions per packed
// word. The w_out hook still emits rn16(s * (q - z)), bit-identical to dequant_one.
__host__ __device__ constexpr bool sk_fold(int fmt, int gs) { return fmt != F_MX && gs == 128; }

struct StreamParams {
  const uint32_t* q;
  const void* scales;
  const uint32_t* zeros;
  const __half* x;
  __half* c;
  __half* w_out;
  int N, K, M;
  int G, wG;    // scales per row: groups (W4) or 32-blocks (MX); zero words per row
  int C, P;     // 512-k units per panel (the last may be half empty), 64-row panels
  int U;        // units = P * C  (U * grid < 2^31: all unit arithmetic is 32-bit)
  int stages;
  int xrows;    // activation rows per pass (<= 8*MT); pass y covers rows y*xrows ...
  int xpitch;   // bytes between activation rows in shared memory (== 64 mod 128)
  const uint8_t* xa;  // streamed activations: one arranged block per (pass, unit), written by x_arrange_kernel
  float* ws;
  int* counters;
  int* status;
  StreamPeers peers;  // world == 0: no exchange
};

// Unit arithmetic is unsigned 32-bit (the launcher guarantees U * grid < 2^31): 64-bit
// divisions would cost every warp microseconds per launch.
__host__ __device__ __forceinline__ int unit_begin(int U, int b, int grid) {
  return (int)((unsigned)U * (unsigned)b / (unsigned)grid);
}
// The CTA whose range holds unit t (ranges are [U*b/grid, U*(b+1)/grid)).
__device__ __forceinline__ int unit_owner(int U, int t, int grid) {
  return (int)((((unsigned)t + 1u) * (unsigned)grid + (unsigned)U - 1u) / (unsigned)U) - 1;
}

// The order in which a CTA walks its range [u0, u1): the part of the last panel
// (whose end another CTA owns) first, then the whole panels, then the part of
// the first panel (whose end this CTA owns). A range inside one panel is one
// segment.
struct Walk {
  int u0, u1, pb, pe;
  int len_tail, n_full, len_head, nseg;
  int p_tail, p_full, p_head, ch_head;  // panels of the tail / first whole / head segment, first chunk of the head
  bool single;
  __device__ Walk(int a, int b, int C) : u0(a), u1(b) {
    p_head = u0 / C;
    ch_head = u0 - p_head * C;
    p_full = ch_head == 0 ? p_head : p_head + 1;
    p_tail = u1 / C;
    pb = p_full * C;  // first panel boundary at or after u0
    pe = p_tail * C;  // last panel boundary at or before u1
    single = pb > pe;  // no boundary inside [u0, u1]: the range lies within one panel
    if (single) {
      len_tail = n_full = 0;
      len_head = u1 - u0;
      nseg = 1;
    } else {
      len_tail = u1 - pe;
      n_full = (pe - pb) / C;
      len_head = pb - u0;
      nseg = (len_tail > 0) + n_full + (len_head > 0);
    }
  }
  // segment i -> panel, first chunk and length, without a division
  __device__ void segment_pc(int i, int C, int* p, int* ch0, int* len) const {
    if (!single) {
      if (len_tail > 0) {
        if (i == 0) {
          *p = p_tail;
          *ch0 = 0;
          *len = len_tail;
          return;
        }
        --i;
      }
      if (i < n_full) {
        *p = p_full + i;
        *ch0 = 0;
        *len = C;
        return;
      }
    }
    *p = p_head;
    *ch0 = ch_head;
    *len = len_head;
  }
  // segment i -> first unit and length (all units of a segment lie in one panel)
  __device__ void segment(int i, int C, int* ua, int* len) const {
    if (single) {
      *ua = u0;
      *len = len_head;
      return;
    }
    if (len_tail > 0) {
      if (i == 0) {
        *ua = pe;
        *len = len_tail;
        return;
      }
      --i;
    }
    if (i < n_full) {
      *ua = pb + i * C;
      *len = C;
      return;
    }
    *ua = u0;
    *len = len_head;
  }
};

// Position in the walk: unit (panel p, chunk ch), the r-th of its segment.
struct Cursor {
  int seg, r, len, p, ch;
  __device__ void start(const Walk& w, int C) {
    seg = r = 0;
    w.segment_pc(0, C, &p, &ch, &len);
  }
  __device__ void next(const Walk& w, int C) {
    ++ch;
    if (++r == len && seg + 1 < w.nseg) {
      w.segment_pc(++seg, C, &p, &ch, &len);
      r = 0;
    }
  }
};

// What a CTA does with panels it covers only in part. It parks at most one fragment per
// tile (the panel whose end another CTA owns) and completes at most one panel (the one
// whose end it owns); panels it covers whole are written directly.
struct Handoff {
  int park_panel, own_panel;  // -1: none
  int b_first, b_last;        // CTAs contributing to own_panel (this CTA is b_last)
  __device__ Handoff() : park_panel(-1), own_panel(-1), b_first(0), b_last(0) {}
  __device__ Handoff(const Walk& w, int U, int C, int grid, int me) : park_panel(-1), own_panel(-1), b_first(0), b_last(0) {
    // only the first and the last segment of a walk can be partial panels
    for (int i = 0; i < w.nseg; i += (w.nseg > 1 ? w.nseg - 1 : 1)) {
      int ua, len;
      w.segment(i, C, &ua, &len);
      const int p = ua / C, ch0 = ua - p * C;
      if (ch0 == 0 && len == C) continue;  // whole panel
      const int last = unit_owner(U, (p + 1) * C - 1, grid);
      if (last == me) {
        own_panel = p;
        b_first = unit_owner(U, p * C, grid);
        b_last = last;
      } else {
        park_panel = p;
      }
    }
  }
};

template <int FMT, int GS>
struct Groups;  // per-row decode constants of one unit (unfolded formats): [0] for words 0-3, [1] for words 4-7

// A unit's row holds 512 / GS scales (and their zero nibbles: one word for 64-element groups, two for
// 32-element groups). The warp of k half kh decodes the half's 256 k, of which lane c owns words 8c..8c+7
// (k = 64c .. 64c+63): with 64-element groups that is group 4kh + c of the unit, with 32-element groups the
// groups 8kh + 2c and 8kh + 2c + 1.
template <int GS>
struct Groups<F_W4_SYM, GS> {
  W4Group g[2];
  __device__ __forceinline__ void load(const uint8_t* meta_row, const uint8_t* /*zero_row*/, int c, int kh) {
    const __half* sc = reinterpret_cast<const __half*>(meta_row);
    const int gi = GS == 64 ? 4 * kh + c : 8 * kh + 2 * c;
    g[0] = w4_group(sc[gi], 8u);
    g[1] = GS == 32 ? w4_group(sc[gi + (GS == 32 ? 1 : 0)], 8u) : g[0];
  }
  __device__ __forceinline__ void decode(uint32_t w, int half, const W4Consts& k, __half2 out[4]) const {
    dq_w4_word(w, g[half], k, out);
  }
  __device__ __forceinline__ bool all_fast() const { return false; }
  __device__ __forceinline__ void decode_fast(uint32_t w, int half, const W4Consts& k, __half2 out[4]) const {
    dq_w4_word(w, g[half], k, out);
  }
};

template <int GS>
struct Groups<F_W4_ASYM, GS> {
  W4Group g[2];
  __device__ __forceinline__ void load(const uint8_t* meta_row, const uint8_t* zero_row, int c, int kh) {
    const __half* sc = reinterpret_cast<const __half*>(meta_row);
    const int gi = GS == 64 ? 4 * kh + c : 8 * kh + 2 * c;
    // 64-element groups: the unit's 8 groups are the 8 nibbles of one word; 32-element groups: word kh of two
    const uint32_t zw = reinterpret_cast<const uint32_t*>(zero_row)[GS == 32 ? kh : 0];
    const int nib = GS == 32 ? 2 * c : gi;
    g[0] = w4_group(sc[gi], (zw >> (4 * nib)) & 0xFu);
    g[1] = GS == 32 ? w4_group(sc[gi + (GS == 32 ? 1 : 0)], (zw >> (4 * nib + 4)) & 0xFu) : g[0];
  }
  __device__ __forceinline__ void decode(uint32_t w, int half, const W4Consts& k, __half2 out[4]) const {
    dq_w4_word(w, g[half], k, out);
  }
  __device__ __forceinline__ bool all_fast() const { return false; }
  __device__ __forceinline__ void decode_fast(uint32_t w, int half, const W4Consts& k, __half2 out[4]) const {
    dq_w4_word(w, g[half], k, out);
  }
};

template <int GS>
struct Groups<F_MX, GS> {
  MxBlock b[2];
  __device__ __forceinline__ void load(const uint8_t* meta_row, const uint8_t* /*zero_row*/, int c, int kh) {
    b[0] = mx_block(meta_row[8 * kh + 2 * c]);
    b[1] = mx_block(meta_row[8 * kh + 2 * c + 1]);
  }
  __device__ __forceinline__ void decode(uint32_t w, int half, const W4Consts&, __half2 out[4]) const {
    dq_mx_word(w, b[half], out);
  }
  // Both blocks in the range of the bit-placement decode: a warp that finds this true for all its lanes decodes
  // the chunk without the per-word choice of the form.
  __device__ __forceinline__ bool all_fast() const { return b[0].fast && b[1].fast; }
  __device__ __forceinline__ void decode_fast(uint32_t w, int half, const W4Consts&, __half2 out[4]) const {
    dq_mx_word_fast(w, b[half], out);
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

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Signals the barrier without waiting for it (the producer half of a producer/consumer pair).
__device__ __forceinline__ void named_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
constexpr int BAR_HANDED = 1;  // +tile: the upper k half has written its fragment (the lower half waits)
constexpr int BAR_TAKEN = 5;   // +tile: the lower half has read it (the upper half waits before rewriting)
constexpr int BAR_XFILL = 9;   // all consumer warps: the activations are in shared memory
constexpr int BAR_DONE = 10;   // all consumer warps: exchange form, end of the CTA's work

// The word slot of a 256-k box that holds natural word wi (0..31) of an activation row: the chunks the four lanes of
// a column read together are adjacent.
//   unfolded: lane c owns words 8c..8c+7, word slot i -> chunk i*4 + c;
//   folded:   lane c owns words 4c..4c+3 of each 128-k half j, slot (j, i) -> chunk (j*4 + i)*4 + c.
__device__ __forceinline__ int x_slot(bool fold, int wi) {
  return fold ? ((wi & 16) | ((wi & 3) << 2) | ((wi >> 2) & 3)) : (((wi & 7) << 2) + (wi >> 3));
}

// Arranges 8 consecutive activations for the decoder: the pairing (h0,h4,h1,h5,h2,h6,h3,h7); for the folded
// formats the pairs (h1,h5) and (h3,h7), which meet codes that carry 2^-20 instead of 2^-24, are divided by 16,
// and *sum8 receives the sum of the 8 values.
__device__ __forceinline__ uint4 x_arrange8(bool fold, uint4 v, float* sum8) {
  uint4 pv = pair_permute(v);
  if (fold) {
    const __half2 sixteenth = u32_as_h2(0x2C002C00u);
    pv.y = h2_as_u32(__hmul2_rn(u32_as_h2(pv.y), sixteenth));
    pv.w = h2_as_u32(__hmul2_rn(u32_as_h2(pv.w), sixteenth));
    const float2 f0 = __half22float2(u32_as_h2(v.x)), f1 = __half22float2(u32_as_h2(v.y));
    const float2 f2 = __half22float2(u32_as_h2(v.z)), f3 = __half22float2(u32_as_h2(v.w));
    *sum8 = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
  }
  return pv;
}

// Pre-pass of the streamed-activation form (the counterpart of the reference's x_to_f32_kernel,
// include/w4/fused.cuh:45-49): writes, for every (pass, 512-k unit), one contiguous block holding the unit's
// activations of the pass's rows in the arrangement the consumers read (rows padded with zeros to 8 * MT) and,
// for the folded formats, the FP32 sum of each row over each of the unit's four groups. The GEMM's loader then
// brings a unit's block in with one bulk copy beside the unit's weights.
constexpr int XA_THREADS = 512;  // one or two chunks per thread: with 64 threads a CTA walked 16 dependent loads, ~10 us per launch
__global__ void __launch_bounds__(XA_THREADS)
    x_arrange_kernel(const __half* __restrict__ x, uint8_t* __restrict__ xa, int M, int K, int C, int xrows, int mt,
                     int fold) {
  pdl_launch_dependents();
  pdl_wait();  // x may be the previous kernel's output; the blocks may still be read by the previous GEMM
  const int ch = (int)blockIdx.x, y = (int)blockIdx.y, lane = threadIdx.x & 31;
  const int m0 = y * xrows, mrows = min(xrows, M - m0), prow = 8 * mt;
  uint8_t* blk = xa + ((size_t)y * C + ch) * sk_xblock(mt);
  float* xs = reinterpret_cast<float*>(blk + (size_t)prow * SK_XROW);
  for (int idx = threadIdx.x; idx < prow * 64; idx += XA_THREADS) {  // (row r, 16-byte chunk widx of the unit)
    const int r = idx >> 6, widx = idx & 63;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < mrows) v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(m0 + r) * K + (size_t)ch * SK_KU) + widx);
    float xsum = 0.0f;
    const uint4 pv = x_arrange8(fold != 0, v, &xsum);
    if (fold) {  // 16 adjacent lanes hold the 16 chunks of one group of one row
#pragma unroll
      for (int d = 1; d < 16; d <<= 1) xsum += __shfl_xor_sync(0xffffffffu, xsum, d);
      if ((lane & 15) == 0) xs[(widx >> 4) * prow + r] = xsum;
    }
    const int dst = (widx & 32) + x_slot(fold != 0, widx & 31);
    *reinterpret_cast<uint4*>(blk + (size_t)r * SK_XROW + ((size_t)dst << 4)) = pv;
  }
}

template <int FMT, int GS, int MT, bool HOOK, bool XS>
__global__ void __launch_bounds__(SK_THREADS, 2)
    stream_gemm_kernel(const __grid_constant__ CUtensorMap tmap, const StreamParams a) {
  constexpr bool FOLD = sk_fold(FMT, GS);
  constexpr int XBLOCK = sk_xblock(MT);
  constexpr int SK_META_ROW = sk_meta_row(FMT, GS), SK_META_ZOFF = SK_ROWS * SK_META_ROW, SK_META = sk_meta(FMT, GS);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int stages = a.stages;
  // the swizzle pattern repeats every 1024 bytes: align the ring to it
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sm_q = smem;
  uint8_t* sm_meta = sm_q + (size_t)stages * SK_STAGE_Q;
  // activations: streamed form - one arranged block per stage; resident form - the pass's rows, a zero area for
  // absent rows and, for the folded formats, the sum of row m over group gidx at [gidx][8 * MT] (FP32)
  uint8_t* sm_x = sm_meta + (size_t)stages * SK_META;
  uint8_t* sm_zero = sm_x + (XS ? (size_t)stages * XBLOCK : (size_t)a.xrows * a.xpitch);
  float* sm_xs = reinterpret_cast<float*>(sm_zero + (XS ? 0 : SK_ZERO_BYTES));
  uint8_t* sm_red = reinterpret_cast<uint8_t*>(sm_xs) + ((FOLD && !XS) ? (size_t)(a.K >> 7) * 8 * MT * 4 : 0);
  uint8_t* sm_collect = sm_red + MT * SK_RED_BYTES_PER_MT;
  const uint32_t sm_bar = smem_u32(sm_collect + MT * SK_COLLECT_BYTES_PER_MT);
  auto full_bar = [&](int s) { return sm_bar + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return sm_bar + 8u * (uint32_t)(stages + s); };
  const uint32_t parked_bar = sm_bar + 8u * (uint32_t)(2 * stages);  // the 4 tiles' fragments are in the workspace
  const uint32_t collected_bar = parked_bar + 8u;                    // the other CTAs' fragments are summed
  const uint32_t peers_bar = collected_bar + 8u;  // exchange form: the peers have this rank's previous slice
  const uint32_t cta_done = peers_bar + 8u;       // exchange form: whether this CTA finished last

  const int grid = (int)gridDim.x;
  const int m0 = (int)blockIdx.y * a.xrows;  // first activation row of this pass
  const int mrows = min(a.xrows, a.M - m0);   // rows of this pass (the last may be short)
  const int C = a.C;
  const Walk walk(unit_begin(a.U, (int)blockIdx.x, grid), unit_begin(a.U, (int)blockIdx.x + 1, grid), C);
  const int total = walk.u1 - walk.u0;

  // Programmatic dependent launch (no-ops unless the launch carries the attribute): the next launch in the
  // stream may start now - its producer fills its ring with weights while this grid is still running - and
  // everything of THIS grid that reads the activations or touches c / scratch first waits for the previous
  // grid to have completed (pdl_wait below).
  pdl_launch_dependents();
  if (tid < stages) {
    mbar_init(full_bar(tid), 33);  // lane 0's expect_tx arrive + one cp.async arrive per producer lane
    mbar_init(empty_bar(tid), SK_CONSUMERS);  // every consumer warp hands the stage back
    if (tid == 0) {
      mbar_init(parked_bar, SK_TILES);
      mbar_init(collected_bar, 1);
      mbar_init(peers_bar, 1);
    }
    mbar_init_fence();
  }
  if (tid == 32 * SK_LOADER) tma_prefetch_desc(&tmap);
  __syncthreads();

  // parked fragment of (CTA, slot, tile): slot 0 when the panel is the CTA's first one
  auto slot_of = [&](int which_cta, int tile_, int panel) {
    const int slot = (unit_begin(a.U, which_cta, grid) / C == panel) ? 0 : 1;
    return reinterpret_cast<float4*>(a.ws) +
           ((((size_t)blockIdx.y * grid + which_cta) * 2 + slot) * SK_TILES + tile_) * MT * 32;
  };

  if (wid == SK_LOADER) {
    // ------------------------------ loader ------------------------------
    // The weights are read without waiting for the previous grid; in the streamed form the activation blocks,
    // which the arrange kernel before this grid writes, follow once that kernel has completed.
    constexpr int NGU = FMT == F_MX ? SK_KU / 32 : SK_KU / GS;  // scales per row and unit
    constexpr int SBYTES = FMT == F_MX ? NGU : 2 * NGU;        // 8 (gs 128), 16 (gs 64, MX) or 32 (gs 32) bytes
    constexpr int ZBYTES = NGU > 8 ? 8 : 4;                    // zero words of the unit's groups
    // One unit's weights: two boxes + the rows' scales / zero words; the stage's full barrier then expects the
    // boxes' bytes (and, in the streamed form, the activation block's, which issue_x brings).
    auto issue_w = [&](int s, int p, int ch) {
      if (lane == 0) {
        const uint32_t dst = smem_u32(sm_q) + (uint32_t)s * SK_STAGE_Q;
        mbar_arrive_expect_tx(full_bar(s), SK_STAGE_Q + (XS ? XBLOCK : 0));
        tma_load_2d(dst, &tmap, ch * (SK_KU / 8), p * SK_ROWS, full_bar(s));
        tma_load_2d(dst + SK_BOX, &tmap, ch * (SK_KU / 8) + SK_KC / 8, p * SK_ROWS, full_bar(s));
      }
      const uint32_t meta = smem_u32(sm_meta) + (uint32_t)s * SK_META;
      const int g0 = ch * NGU;  // the unit's first group (or MX block) within the row
#pragma unroll
      for (int rr = 0; rr < SK_ROWS / 32; ++rr) {
        const int row = lane + 32 * rr;
        const int n = min(p * SK_ROWS + row, a.N - 1);  // rows past N: any valid row, never used
        const uint8_t* src = (const uint8_t*)a.scales + ((size_t)n * a.G + g0) * (FMT == F_MX ? 1 : 2);
        if constexpr (SBYTES == 32) {
          cp_async<16>(meta + row * SK_META_ROW, src);
          cp_async<16>(meta + row * SK_META_ROW + 16, src + 16);
        } else {
          cp_async<SBYTES>(meta + row * SK_META_ROW, src);
        }
        if (FMT == F_W4_ASYM)
          cp_async<ZBYTES>(meta + SK_META_ZOFF + row * 8, a.zeros + (size_t)n * a.wG + (size_t)((g0 >> 3) & ~(ZBYTES / 4 - 1)));
      }
      cp_async_arrive_noinc(full_bar(s));
    };
    // The unit's arranged activations (streamed form): one bulk copy of the (pass, unit) block.
    auto issue_x = [&](int s, int ch) {
      if (XS && lane == 0)
        bulk_load_1d(smem_u32(sm_x) + (uint32_t)s * XBLOCK, a.xa + ((size_t)blockIdx.y * C + ch) * XBLOCK, XBLOCK,
                     full_bar(s));
    };
    Cursor cur;
    cur.start(walk, C);
    // The first ring fill needs no free-stage wait. Weights go out at once; the activation blocks are written by
    // the arrange kernel that precedes this grid, so they follow once that kernel has completed.
    const int first = min(stages, total);
    Cursor cx = cur;
    for (int j = 0; j < first; ++j) {
      issue_w(j, cur.p, cur.ch);
      cur.next(walk, C);
    }
    if (XS) {
      pdl_wait();
      for (int j = 0; j < first; ++j) {
        issue_x(j, cx.ch);
        cx.next(walk, C);
      }
    }
    int s = first == stages ? 0 : first;
    uint32_t ph = first == stages ? 1u : 0u;
    for (int j = first; j < total; ++j) {
      if (!mbar_wait(empty_bar(s), ph ^ 1u, a.status, ST_STREAM_EMPTY_TIMEOUT)) return;
      issue_w(s, cur.p, cur.ch);
      issue_x(s, cur.ch);
      if (++s == stages) {
        s = 0;
        ph ^= 1u;
      }
      cur.next(walk, C);
    }
    return;
  }

  if (wid == SK_HANDOFF) {
    // ------------------------------ hand-offs ------------------------------
    // This warp does the CTA's exchanges with other CTAs, so that neither a consumer warp nor the loader ever
    // waits for a round trip to L2: (1) once the four tile warps have parked their fragment it fences and
    // bumps the tiles' counters; (2) for the panel this CTA completes it waits for the other CTAs' counters,
    // adds their fragments in CTA order into shared memory and signals `collected`.
    const Handoff hand(walk, a.U, C, grid, (int)blockIdx.x);
    auto tile_live = [&](int panel, int t) { return panel * SK_ROWS + t * 16 < a.N; };
    if (a.peers.world && a.peers.carry) {
      // Carry form: while the CTA's other warps stream this step's weights, this warp - which has nothing to do
      // until the first fragments are parked, and whose hand-offs are only consumed at the other end of the
      // grid's run - delivers its share of the PREVIOUS step's slice to every peer. Flow control as in the
      // exchange kernel: rank p must have posted the step before the previous one (with three slice buffers
      // nothing it may still read is then overwritten). Each warp makes its stores visible system-wide and
      // counts itself; the warp that completes the count posts the step to every peer.
      pdl_wait();  // the previous grid wrote the slice
      if (a.peers.prev_bytes) {
        if (lane < a.peers.world && lane != a.peers.rank) {
          const volatile unsigned long long* flag = reinterpret_cast<const volatile unsigned long long*>(a.peers.flags_local) + lane;
          const unsigned long long sent = *(reinterpret_cast<const volatile unsigned long long*>(a.peers.counters) + lane);
          const long long t0 = clock64();
          while (sent >= 2 && *flag + 1 < sent) {  // this delivery is step sent + 1: rank `lane` has posted sent - 1
            __nanosleep(100);
            if (clock64() - t0 > kWaitLimitCycles) {
              atomicExch(a.status, ST_PEER_TIMEOUT);
              break;
            }
          }
        }
        __syncwarp();
        const size_t n16 = a.peers.prev_bytes >> 4;
        const uint4* src = reinterpret_cast<const uint4*>(a.peers.prev_src);
        const size_t nw = (size_t)gridDim.x * gridDim.y, me = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
        for (size_t i = me * 32 + lane; i < n16; i += nw * 32) {
          const uint4 v = __ldcg(src + i);
          for (int pr = 0; pr < a.peers.world; ++pr)
            if (pr != a.peers.rank) reinterpret_cast<uint4*>(a.peers.c_peer[pr])[i] = v;
        }
        if (me == 0)  // a tail shorter than 16 bytes
          for (size_t b = (n16 << 4) + 2 * lane; b < a.peers.prev_bytes; b += 64)
            for (int pr = 0; pr < a.peers.world; ++pr)
              if (pr != a.peers.rank)
                *reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(a.peers.c_peer[pr]) + b) =
                    *reinterpret_cast<const volatile __half*>(reinterpret_cast<const uint8_t*>(src) + b);
        // Visibility, by the scoped memory model's causality order: this warp's copies precede its count at device
        // scope (fence + atomic), the counting chain reaches the warp that completes it (atomic + fence), and that
        // warp's system-scope releases of the flags carry everything that precedes them to the peers. The
        // per-warp fences at device scope keep the 148 warps from each paying a system-scope fence (1.6 us on
        // the kernel); the releases go out side by side, one lane per peer (one after the other they took
        // 10 us for seven peers).
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(a.peers.done, 1) == (int)nw - 1 ? 1 : 0;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          if (lane == 0) *a.peers.done = 0;  // ready for the next launch
          if (lane < a.peers.world && lane != a.peers.rank) {
            const unsigned long long step = a.peers.counters[lane] + 1ull;
            asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.peers.flag_dst[lane]), "l"(step) : "memory");
            a.peers.counters[lane] = step;
          }
        }
        __syncwarp();
      }
    } else if (a.peers.world) {
      // Exchange form: before this grid stores into the peers' arenas, every peer's slice of the previous step
      // must have arrived here - then no peer is more than one step behind and, with three slice buffers in
      // rotation, nothing a peer may still read is overwritten. In steady state the flags are long there.
      pdl_wait();
      if (lane < a.peers.world && lane != a.peers.rank) {
        const volatile unsigned long long* flag = reinterpret_cast<const volatile unsigned long long*>(a.peers.flags_local) + lane;
        const unsigned long long want = *(reinterpret_cast<const volatile unsigned long long*>(a.peers.counters) + lane);
        const long long t0 = clock64();
        while (*flag < want) {
          __nanosleep(100);
          if (clock64() - t0 > kWaitLimitCycles) {
            atomicExch(a.status, ST_PEER_TIMEOUT);
            break;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(peers_bar);
    }
    if (hand.park_panel >= 0) {
      // (the consumers park after they have waited for the previous grid)
      if (!mbar_wait(parked_bar, 0u, a.status, ST_STREAM_PANEL_TIMEOUT)) return;
      __threadfence();  // the parked fragments are visible before the counters move
      if (lane < SK_TILES && tile_live(hand.park_panel, lane))
        atomicAdd(a.counters + ((size_t)blockIdx.y * a.P + hand.park_panel) * SK_TILES + lane, 1);
    }
    if (hand.own_panel < 0) return;
    pdl_wait();  // the counters of shared panels belong to the previous grid until it is done
    int* cnt = a.counters + ((size_t)blockIdx.y * a.P + hand.own_panel) * SK_TILES;
    {
      const long long t0 = clock64();
      for (;;) {
        bool ready = true;
        if (lane < SK_TILES && tile_live(hand.own_panel, lane))
          ready = *reinterpret_cast<volatile int*>(cnt + lane) >= hand.b_last - hand.b_first;
        if (__all_sync(0xffffffffu, ready)) break;
        __nanosleep(100);
        if (clock64() - t0 > kWaitLimitCycles) {
          if (lane == 0) atomicExch(a.status, ST_STREAM_PANEL_TIMEOUT);
          return;
        }
      }
    }
    __threadfence();
    constexpr int TB = MT == 1 ? SK_TILES : 2;  // tiles whose fragments are in flight together
#pragma unroll 1
    for (int t0 = 0; t0 < SK_TILES; t0 += TB) {
      float4 sum[TB][MT];
#pragma unroll
      for (int t = 0; t < TB; ++t)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) sum[t][mt] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int b = hand.b_first; b < hand.b_last; ++b) {  // fixed order: by CTA, never by arrival
        float4 v[TB][MT];
#pragma unroll
        for (int t = 0; t < TB; ++t) {
          const float4* theirs = slot_of(b, t0 + t, hand.own_panel);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            v[t][mt] = tile_live(hand.own_panel, t0 + t) ? __ldcg(theirs + mt * 32 + lane)
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int t = 0; t < TB; ++t)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            sum[t][mt].x += v[t][mt].x;
            sum[t][mt].y += v[t][mt].y;
            sum[t][mt].z += v[t][mt].z;
            sum[t][mt].w += v[t][mt].w;
          }
      }
#pragma unroll
      for (int t = 0; t < TB; ++t)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          reinterpret_cast<float4*>(sm_collect)[((t0 + t) * MT + mt) * 32 + lane] = sum[t][mt];
    }
    if (lane < SK_TILES) cnt[lane] = 0;  // ready for the next launch
    __syncwarp();
    if (lane == 0) mbar_arrive(collected_bar);
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int tile = wid & (SK_TILES - 1), kh = wid >> 2;  // 16-row tile, 256-k half of every unit
  const int g = lane >> 2, c = lane & 3;
  // MMA row g (and g + 8) of the tile is box row rg (and rg + 8). Unfolded: rg = g, and a lane reads the
  // 16-byte chunks 2c, 2c+1 of its rows. Folded: a lane reads chunks c and c + 4 (so that the four lanes of
  // an MMA stay inside one 128-k group), and rg interleaves the rows (0,4,1,5,2,6,3,7) so that the two rows
  // that share a shared-memory wavefront differ in swizzle bit 2: no bank conflicts either way.
  const int rg = FOLD ? (((g & 1) << 2) | (g >> 1)) : g;
  const int ra = tile * 16 + rg;  // row inside the box; ra & 7 == rg
  const uint32_t sw0 = FOLD ? ((uint32_t)c ^ (uint32_t)rg) << 4 : ((uint32_t)(2 * c) ^ (uint32_t)rg) << 4;
  const uint32_t sw1 = FOLD ? ((uint32_t)(c + 4) ^ (uint32_t)rg) << 4 : ((uint32_t)(2 * c + 1) ^ (uint32_t)rg) << 4;

  pdl_wait();  // the activations may be the previous grid's output
  if constexpr (!XS) {
  // Activations of this pass: rows m0 .. m0+mrows-1, FP16, each row re-ordered so that the 16 bytes a lane
  // needs for one packed word are one chunk in the decoder's pairing (h0,h4,h1,h5,h2,h6,h3,h7), and the chunks
  // the four lanes of a column read together are adjacent:
  //   unfolded: lane c owns words 8c..8c+7, word slot i -> chunk i*4 + c;
  //   folded:   lane c owns words 4c..4c+3 of each 128-k half j, slot (j, i) -> chunk (j*4 + i)*4 + c.
  {
    const int cpr = a.K >> 3;  // 16-byte chunks per activation row
    for (int m = 0; m < mrows; ++m) {
      const uint4* src = reinterpret_cast<const uint4*>(a.x + (size_t)(m0 + m) * a.K);
      uint8_t* dst_row = sm_x + (size_t)m * a.xpitch;
      for (int w0 = tid; w0 < cpr; w0 += 4 * 32 * SK_CONSUMERS) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int widx = w0 + u * 32 * SK_CONSUMERS;
          if (widx < cpr) v[u] = __ldg(src + widx);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int widx = w0 + u * 32 * SK_CONSUMERS;
          if (widx < cpr) {
            const int ub = widx >> 5, wi = widx & 31;
            const int dst = (ub << 5) + (FOLD ? ((wi & 16) | ((wi & 3) << 2) | ((wi >> 2) & 3)) : (((wi & 7) << 2) + (wi >> 3)));
            uint4 pv = pair_permute(v[u]);
            if (FOLD) {
              // the pairs (h1,h5) and (h3,h7) meet codes that carry 2^-20 instead of 2^-24
              const __half2 sixteenth = u32_as_h2(0x2C002C00u);
              pv.y = h2_as_u32(__hmul2_rn(u32_as_h2(pv.y), sixteenth));
              pv.w = h2_as_u32(__hmul2_rn(u32_as_h2(pv.w), sixteenth));
              // sum of the 8 activations, then of the 16 chunks of the group (16 adjacent lanes), fixed order
              const float2 f0 = __half22float2(u32_as_h2(v[u].x)), f1 = __half22float2(u32_as_h2(v[u].y));
              const float2 f2 = __half22float2(u32_as_h2(v[u].z)), f3 = __half22float2(u32_as_h2(v[u].w));
              float xsum = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
#pragma unroll
              for (int d = 1; d < 16; d <<= 1) xsum += __shfl_xor_sync(0xffffffffu, xsum, d);
              if ((lane & 15) == 0) sm_xs[(size_t)(widx >> 4) * (8 * MT) + m] = xsum;
            }
            *reinterpret_cast<uint4*>(dst_row + ((size_t)dst << 4)) = pv;
          }
        }
      }
    }
    if (tid < SK_ZERO_BYTES / 16) reinterpret_cast<uint4*>(sm_zero)[tid] = make_uint4(0u, 0u, 0u, 0u);
    named_barrier(BAR_XFILL, 32 * SK_CONSUMERS);
  }
  }

  // x rows this lane supplies as B-fragment column g (and g + 8 for the second m-tile). Lanes whose
  // column has no activation row read the zero area instead (plain loads that the compiler is free to
  // schedule among the decode instructions).
  const uint8_t* xrow[MT];
  bool xok[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    if (XS) {  // the stage's block holds 8 * MT rows (absent ones as zeros); this warp reads its k half
      xok[mt] = false;
      xrow[mt] = sm_x + (size_t)(g + 8 * mt) * SK_XROW + (kh << 9) + (c << 4);
    } else {
      xok[mt] = (g + 8 * mt) < mrows;
      xrow[mt] = (xok[mt] ? sm_x + (size_t)(g + 8 * mt) * a.xpitch : sm_zero) + (c << 4);
    }
  }
  const W4Consts kc = w4_consts();
  int s = 0;        // ring slot of the next unit
  uint32_t ph = 0;  // phase parity of that slot's full barrier
  // A warp whose bounded wait ran out stops waiting and computing but keeps handing stages back, so that
  // the CTA ends instead of hanging.
  bool alive = true;
  bool peers_ok = false;
  for (int seg = 0; seg < walk.nseg; ++seg) {
    int p, ch0, len;
    walk.segment_pc(seg, C, &p, &ch0, &len);
    const int tile_row0 = p * SK_ROWS + tile * 16;
    const bool live = tile_row0 < a.N;  // warp-uniform

    float acc[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][h][i] = 0.0f;

    for (int r = 0; r < len; ++r) {
      const int s_now = s;
      const uint32_t ph_now = ph;
      if (++s == stages) {
        s = 0;
        ph ^= 1u;
      }
      if (alive && !mbar_wait(full_bar(s_now), ph_now, a.status, ST_STREAM_FULL_TIMEOUT)) alive = false;
      const int ch = 2 * (ch0 + r) + kh;  // this warp's 256-k chunk of the row
      if (live && alive) {
        const uint8_t* qs = sm_q + (size_t)s_now * SK_STAGE_Q + (size_t)kh * SK_BOX + (size_t)ra * 128;
        const uint8_t* meta = sm_meta + (size_t)s_now * SK_META;
        const uint4 qa0 = *reinterpret_cast<const uint4*>(qs + sw0);
        const uint4 qa1 = *reinterpret_cast<const uint4*>(qs + sw1);
        const uint4 qb0 = *reinterpret_cast<const uint4*>(qs + 8 * 128 + sw0);
        const uint4 qb1 = *reinterpret_cast<const uint4*>(qs + 8 * 128 + sw1);
        const uint8_t* xu[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)  // resident: 32 chunks of 16 bytes per 256 k of the row; streamed: the stage's block
          xu[mt] = xrow[mt] + (XS ? (size_t)s_now * XBLOCK : (xok[mt] ? ((size_t)ch << 9) : 0));
        if constexpr (FOLD) {
          // the unit holds 4 groups per row (8 bytes of scales, one zero word); this warp's half has two
          const uint32_t sa2 = *reinterpret_cast<const uint32_t*>(meta + ra * SK_META_ROW + 4 * kh);
          const uint32_t sb2 = *reinterpret_cast<const uint32_t*>(meta + (ra + 8) * SK_META_ROW + 4 * kh);
          uint32_t zza = 0x88u, zzb = 0x88u;  // symmetric: z = 8 for both groups
          if (FMT == F_W4_ASYM) {
            const int shb = (ch & 3) << 3;  // groups 2ch, 2ch+1 -> nibbles (2ch & 7), +1 of the zero word
            zza = *reinterpret_cast<const uint32_t*>(meta + SK_META_ZOFF + ra * 8) >> shb;
            zzb = *reinterpret_cast<const uint32_t*>(meta + SK_META_ZOFF + (ra + 8) * 8) >> shb;
          }
          float ga_[2][MT][4];  // per group j: 2^-24 * sum of x * q over the group's 128 k
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
              for (int e = 0; e < 4; ++e) ga_[j][mt][e] = 0.0f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const uint32_t wa = word_of(qa0, qa1, 4 * j + i), wb = word_of(qb0, qb1, 4 * j + i);
              const uint32_t ha = wa >> 8, hb = wb >> 8;
              // codes as FP16 bit patterns, rows a / b: (k0,k4) (k1,k5)/16 | (k2,k6) (k3,k7)/16 of the word
              const uint32_t f0[4] = {wa & kc.lo, wb & kc.lo, wa & kc.hi, wb & kc.hi};
              const uint32_t f1[4] = {ha & kc.lo, hb & kc.lo, ha & kc.hi, hb & kc.hi};
              if (HOOK && blockIdx.y == 0) {  // every pass decodes the same weights; one writes them
                const W4Group wga = w4_group(__ushort_as_half((unsigned short)(sa2 >> (16 * j))), (zza >> (4 * j)) & 0xFu);
                const W4Group wgb = w4_group(__ushort_as_half((unsigned short)(sb2 >> (16 * j))), (zzb >> (4 * j)) & 0xFu);
                __half2 pa[4], pb[4];
                dq_w4_word(wa, wga, kc, pa);
                dq_w4_word(wb, wgb, kc, pb);
                const int k = ch * SK_KC + 128 * j + 32 * c + 8 * i;
                const int na = tile_row0 + rg, nb = na + 8;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                  if (na < a.N) {
                    a.w_out[(size_t)na * a.K + k + jj] = __low2half(pa[jj]);
                    a.w_out[(size_t)na * a.K + k + jj + 4] = __high2half(pa[jj]);
                  }
                  if (nb < a.N) {
                    a.w_out[(size_t)nb * a.K + k + jj] = __low2half(pb[jj]);
                    a.w_out[(size_t)nb * a.K + k + jj + 4] = __high2half(pb[jj]);
                  }
                }
              }
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xu[mt] + ((4 * j + i) << 6));
                mma_16816(ga_[j][mt], f0, xv.x, xv.y);
                mma_16816(ga_[j][mt], f1, xv.z, xv.w);
              }
            }
          }
          // group j adds  s * (2^24 * ga - z * sum(x))  to the rows' sums
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float sa = __half2float(__ushort_as_half((unsigned short)(sa2 >> (16 * j))));
            const float sb = __half2float(__ushort_as_half((unsigned short)(sb2 >> (16 * j))));
            // z as a float: 2^23 + z has z in its low mantissa bits
            const float fza = __uint_as_float(0x4B000000u | ((zza >> (4 * j)) & 0xFu)) - 8388608.0f;
            const float fzb = __uint_as_float(0x4B000000u | ((zzb >> (4 * j)) & 0xFu)) - 8388608.0f;
            const float sa24 = sa * 16777216.0f, sb24 = sb * 16777216.0f;
            const float nza = -(sa * fza), nzb = -(sb * fzb);
            const float* xs = XS ? reinterpret_cast<const float*>(sm_x + (size_t)s_now * XBLOCK + 8 * MT * SK_XROW) +
                                       (2 * kh + j) * (8 * MT) + 2 * c
                                 : sm_xs + (size_t)(2 * ch + j) * (8 * MT) + 2 * c;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const float2 xs2 = *reinterpret_cast<const float2*>(xs + 8 * mt);
              acc[mt][0][0] = fmaf(nza, xs2.x, fmaf(sa24, ga_[j][mt][0], acc[mt][0][0]));
              acc[mt][0][1] = fmaf(nza, xs2.y, fmaf(sa24, ga_[j][mt][1], acc[mt][0][1]));
              acc[mt][0][2] = fmaf(nzb, xs2.x, fmaf(sb24, ga_[j][mt][2], acc[mt][0][2]));
              acc[mt][0][3] = fmaf(nzb, xs2.y, fmaf(sb24, ga_[j][mt][3], acc[mt][0][3]));
            }
          }
        } else {
          Groups<FMT, GS> ga, gb;
          ga.load(meta + ra * SK_META_ROW, meta + SK_META_ZOFF + ra * 8, c, kh);
          gb.load(meta + (ra + 8) * SK_META_ROW, meta + SK_META_ZOFF + (ra + 8) * 8, c, kh);
          // MXFP4: one vote per chunk instead of a choice of the decode form per word
          bool uniform_fast = false;
          if constexpr (FMT == F_MX) uniform_fast = __all_sync(__activemask(), ga.all_fast() && gb.all_fast()) != 0;
          auto step = [&](int i, auto fast_form) {
            __half2 pa[4], pb[4];
            if constexpr (decltype(fast_form)::value) {
              ga.decode_fast(word_of(qa0, qa1, i), i >> 2, kc, pa);
              gb.decode_fast(word_of(qb0, qb1, i), i >> 2, kc, pb);
            } else {
              ga.decode(word_of(qa0, qa1, i), i >> 2, kc, pa);
              gb.decode(word_of(qb0, qb1, i), i >> 2, kc, pb);
            }
            if (HOOK && blockIdx.y == 0) {  // every pass decodes the same weights; one writes them
              const int k = ch * SK_KC + 64 * c + 8 * i;
              const int na = tile_row0 + rg, nb = na + 8;
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) {
                if (na < a.N) {
                  a.w_out[(size_t)na * a.K + k + jj] = __low2half(pa[jj]);
                  a.w_out[(size_t)na * a.K + k + jj + 4] = __high2half(pa[jj]);
                }
                if (nb < a.N) {
                  a.w_out[(size_t)nb * a.K + k + jj] = __low2half(pb[jj]);
                  a.w_out[(size_t)nb * a.K + k + jj + 4] = __high2half(pb[jj]);
                }
              }
            }
            const uint32_t f0[4] = {h2_as_u32(pa[0]), h2_as_u32(pb[0]), h2_as_u32(pa[1]), h2_as_u32(pb[1])};
            const uint32_t f1[4] = {h2_as_u32(pa[2]), h2_as_u32(pb[2]), h2_as_u32(pa[3]), h2_as_u32(pb[3])};
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint4 xv = *reinterpret_cast<const uint4*>(xu[mt] + (i << 6));
              mma_16816(acc[mt][0], f0, xv.x, xv.y);
              mma_16816(acc[mt][1], f1, xv.z, xv.w);
            }
          };
          if (FMT == F_MX && uniform_fast) {
#pragma unroll
            for (int i = 0; i < 8; ++i) step(i, std::true_type{});
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) step(i, std::false_type{});
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(s_now));
    }

    // ---- the CTA leaves panel p having covered chunks [ch0, ch0 + len) ----
    float out[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) out[mt][i] = acc[mt][0][i] + acc[mt][1][i];
    // The two k halves of the tile: the upper hands its fragment to the lower. It writes, signals and goes on
    // to the next segment; it only waits if the lower half has not yet read the previous segment's fragment.
    // Every segment runs this protocol, dead tiles and timed-out warps included, so the barriers always pair up.
    float4* red = reinterpret_cast<float4*>(sm_red) + (size_t)tile * MT * 32;
    if (kh == 1) {
      if (seg > 0) named_barrier(BAR_TAKEN + tile, 64);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) red[mt * 32 + lane] = make_float4(out[mt][0], out[mt][1], out[mt][2], out[mt][3]);
      named_arrive(BAR_HANDED + tile, 64);
      continue;
    }
    named_barrier(BAR_HANDED + tile, 64);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const float4 v = red[mt * 32 + lane];
      out[mt][0] += v.x;
      out[mt][1] += v.y;
      out[mt][2] += v.z;
      out[mt][3] += v.w;
    }
    if (seg + 1 < walk.nseg) named_arrive(BAR_TAKEN + tile, 64);
    // (only the lower-half warps get here, with the tile's complete fragment for this segment)
    const bool whole = (ch0 == 0 && len == C);  // the whole K range was ours
    const bool owner = !whole && unit_owner(a.U, (p + 1) * C - 1, grid) == (int)blockIdx.x;
    if (!whole && !owner) {
      // park the fragment; the producer warp publishes it, the panel's owner collects it
      if (live && alive) {
        float4* mine = slot_of((int)blockIdx.x, tile, p);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          __stcg(mine + mt * 32 + lane, make_float4(out[mt][0], out[mt][1], out[mt][2], out[mt][3]));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(parked_bar);  // the count covers all four tiles, dead or alive
      continue;
    }
    if (!live || !alive) continue;
    if (owner) {
      // this CTA completes the panel: the producer warp has summed the others' fragments
      if (!mbar_wait(collected_bar, 0u, a.status, ST_STREAM_PANEL_TIMEOUT)) {
        alive = false;
        continue;
      }
      const float4* others = reinterpret_cast<const float4*>(sm_collect) + (size_t)tile * MT * 32;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const float4 v = others[mt * 32 + lane];
        out[mt][0] = v.x + out[mt][0];
        out[mt][1] = v.y + out[mt][1];
        out[mt][2] = v.z + out[mt][2];
        out[mt][3] = v.w + out[mt][3];
      }
    }
    {
      const int na = tile_row0 + rg, nb = na + 8;
      auto put = [&](size_t idx, float v) { a.c[idx] = __float2half_rn(v); };
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int col = 8 * mt + 2 * c;  // activation row within this pass
        const int m = m0 + col;
        if (col < mrows) {
          if (na < a.N) put((size_t)m * a.N + na, out[mt][0]);
          if (nb < a.N) put((size_t)m * a.N + nb, out[mt][2]);
        }
        if (col + 1 < mrows) {
          if (na < a.N) put((size_t)(m + 1) * a.N + na, out[mt][1]);
          if (nb < a.N) put((size_t)(m + 1) * a.N + nb, out[mt][3]);
        }
      }
    }
  }
  if (a.peers.world && !a.peers.carry) {
    // Exchange form: the CTA that finishes last sends the finished slice to every peer and posts the step. Every
    // consumer warp makes its part of c visible on this GPU; the CTA then counts itself at the grid's counter.
    // The CTA that completes the count sees the whole slice: its 256 consumer threads copy it into the peers'
    // arenas (plain 16-byte peer stores, every piece in flight at once), make the copies visible system-wide, and
    // one thread releases the flags.
    __threadfence();
    named_barrier(BAR_DONE, 32 * SK_CONSUMERS);
    if (tid == 0) {
      const uint32_t last = atomicAdd(a.peers.done, 1) == (int)(gridDim.x * gridDim.y) - 1 ? 1u : 0u;
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(cta_done), "r"(last) : "memory");
    }
    named_barrier(BAR_DONE, 32 * SK_CONSUMERS);
    uint32_t last;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(last) : "r"(cta_done) : "memory");
    if (last) {
      __threadfence();
      (void)peers_ok;
      mbar_wait(peers_bar, 0u, a.status, ST_PEER_TIMEOUT);  // the peers have taken the previous step (long ago)
      const size_t bytes = (size_t)a.M * a.N * sizeof(__half);
      const size_t n16 = bytes >> 4;
      const uint4* src = reinterpret_cast<const uint4*>(a.c);
      constexpr int NT = 32 * SK_CONSUMERS;
      for (size_t i0 = 0; i0 < n16; i0 += 8 * NT) {  // batches of 8 pieces per thread, in flight together
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const size_t i = i0 + (size_t)u * NT + tid;
          if (i < n16) v[u] = __ldcg(src + i);
        }
        for (int pr = 0; pr < a.peers.world; ++pr) {
          if (pr == a.peers.rank) continue;
          uint4* dst = reinterpret_cast<uint4*>(a.peers.c_peer[pr]);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const size_t i = i0 + (size_t)u * NT + tid;
            if (i < n16) dst[i] = v[u];
          }
        }
      }
      for (int pr = 0; pr < a.peers.world; ++pr) {  // a tail shorter than 16 bytes
        if (pr == a.peers.rank) continue;
        for (size_t b = (n16 << 4) + 2 * tid; b < bytes; b += 2 * NT)
          *reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(a.peers.c_peer[pr]) + b) =
              *reinterpret_cast<const volatile __half*>(reinterpret_cast<const uint8_t*>(src) + b);
      }
      __threadfence_system();
      named_barrier(BAR_DONE, 32 * SK_CONSUMERS);
      if (tid == 0) *a.peers.done = 0;  // ready for the next launch
      if (tid < a.peers.world && tid != a.peers.rank) {  // one thread per peer: the releases' fences side by side
        const unsigned long long step = a.peers.counters[tid] + 1ull;
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.peers.flag_dst[tid]), "l"(step) : "memory");
        a.peers.counters[tid] = step;
      }
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

template <int FMT, int GS, int MT, bool HOOK, bool XS>
cudaError_t launch_one(const CUtensorMap& tmap, const StreamParams& sp, dim3 grid, size_t smem, bool overlap,
                       cudaStream_t stream) {
  auto kern = stream_gemm_kernel<FMT, GS, MT, HOOK, XS>;
  // The shared-memory opt-in is a per-device attribute of the function: set it once on every device used.
  static std::atomic<bool> configured[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (!configured[dev].load(std::memory_order_acquire)) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemOptIn);
    if (e != cudaSuccess) return e;
    configured[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(SK_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, tmap, sp);
}

template <int FMT, int GS, bool XS>
cudaError_t launch_mt(const CUtensorMap& tmap, const StreamParams& sp, int mt, dim3 grid, size_t smem,
                      bool overlap, cudaStream_t stream) {
  const bool hook = sp.w_out != nullptr;
  if (mt == 1)
    return hook ? launch_one<FMT, GS, 1, true, XS>(tmap, sp, grid, smem, overlap, stream)
                : launch_one<FMT, GS, 1, false, XS>(tmap, sp, grid, smem, overlap, stream);
  return hook ? launch_one<FMT, GS, 2, true, XS>(tmap, sp, grid, smem, overlap, stream)
              : launch_one<FMT, GS, 2, false, XS>(tmap, sp, grid, smem, overlap, stream);
}

template <int FMT, int GS>
cudaError_t launch_fmt(const CUtensorMap& tmap, const StreamParams& sp, int mt, dim3 grid, size_t smem,
                       bool overlap, cudaStream_t stream) {
  return sp.xa ? launch_mt<FMT, GS, true>(tmap, sp, mt, grid, smem, overlap, stream)
               : launch_mt<FMT, GS, false>(tmap, sp, mt, grid, smem, overlap, stream);
}

// Shared memory of one CTA without the ring, resident form: alignment slack, barriers, `rows` activation rows,
// zero area, group sums (folded formats), exchange areas.
size_t fixed_smem(int rows, int K) {
  const int mt = rows > 8 ? 2 : 1;
  return 1024 + SK_BAR_BYTES + (size_t)rows * (K * 2 + 64) + SK_ZERO_BYTES + (size_t)(K / 128) * 8 * mt * 4 +
         (size_t)mt * (SK_RED_BYTES_PER_MT + SK_COLLECT_BYTES_PER_MT);
}
// Ring depth that fits beside `rows` resident activation rows within `budget` bytes per CTA.
constexpr int kMinStagesHalf = 5;  // a ring worth confining to half an SM
int stages_for(int rows, int K, int stage_bytes, int budget) {
  const long long room = (long long)budget - (long long)fixed_smem(rows, K);
  return room <= 0 ? 0 : (int)(room / stage_bytes);
}
// Streamed form: the activations travel with the units, a stage also holds the unit's arranged block.
size_t fixed_smem_xs(int mt) {
  return 1024 + SK_BAR_BYTES + (size_t)mt * (SK_RED_BYTES_PER_MT + SK_COLLECT_BYTES_PER_MT);
}
int stages_for_xs(int mt, int stage_bytes, int budget) {
  return (int)(((long long)budget - (long long)fixed_smem_xs(mt)) / (stage_bytes + sk_xblock(mt)));
}

}  // namespace

bool stream_gemm_supported(int N, int K, int gs_or_0_for_mx, const void* q, const void* scales,
                           const void* x) {
  if (N < SK_ROWS || K < SK_KU || K % SK_KU != 0) return false;
  if (gs_or_0_for_mx != 0 && gs_or_0_for_mx != 32 && gs_or_0_for_mx != 64 && gs_or_0_for_mx != 128)
    return false;
  if (((uintptr_t)q | (uintptr_t)scales | (uintptr_t)x) & 15u) return false;
  if (K > (1 << 20)) return false;
  // 32-bit unit arithmetic: units * CTAs below 2^31 (>= 100 GB of packed weights on 148 SMs)
  if ((long long)((N + SK_ROWS - 1) / SK_ROWS) * (K / SK_KU) * 1024 >= (1LL << 31)) return false;
  return encode_tiled() != nullptr;
}

void stream_gemm_plan(int N, int K, int M, int gs_or_0_for_mx, int sm_count, StreamPlan* plan) {
  const int xpitch = K * 2 + 64;
  const int stage = gs_or_0_for_mx == 0 ? sk_stage(F_MX, 32) : sk_stage(F_W4_SYM, gs_or_0_for_mx);
  plan->P = (N + SK_ROWS - 1) / SK_ROWS;
  plan->C = K / SK_KU;
  plan->U = (long long)plan->P * plan->C;
  plan->grid_x = (int)(plan->U < sm_count ? plan->U : sm_count);
  plan->xpitch = xpitch;
  // Resident form: the activation rows stay in shared memory, re-arranged once per CTA. It is used while they
  // leave a ring of kMinStagesHalf stages in HALF an SM's shared memory (one or two rows of 4K activations), so
  // that the next launch's CTA sits beside this one; beyond that the streamed form is faster (measured at
  // N = 14336, K = 4096: M = 2 10.3 against 11.0 us, M = 3 11.7 against 10.9 us, M = 4 12.2 against 10.9 us).
  // MXFP4 always takes the streamed form: its per-weight decode is the limit, a second CTA on the SM only competes
  // for issue slots (measured, M = 1: 8192 x 8192 25.4 against 21.9 us, N = 14336, K = 4096 21.8 against 19.3 us).
  if (gs_or_0_for_mx != 0 && M <= 8 && stages_for(M, K, stage, kSmemHalf) >= kMinStagesHalf) {
    plan->streamed = 0;
    plan->rows_per_pass = M;
    plan->mt = 1;
    plan->passes = 1;
    const int st = stages_for(M, K, stage, kSmemHalf);
    plan->stages = st > SK_MAX_STAGES ? SK_MAX_STAGES : st;
    plan->smem = fixed_smem(M, K) + (size_t)plan->stages * stage;
    plan->xa_bytes = 0;
  } else {
    // Streamed form: a pre-pass arranges the activations per 512-k unit and the loader brings each unit's block
    // in beside its weights, so shared memory does not grow with K and up to 16 rows go through in one pass.
    const int rows = M < 16 ? M : 16;
    plan->streamed = 1;
    plan->rows_per_pass = rows;
    plan->mt = rows > 8 ? 2 : 1;
    plan->passes = (M + rows - 1) / rows;
    // Measured on B200 (N = 14336, K = 4096, M = 8 / 16, launches overlapped): rings of 4 / 3 stages are as fast
    // as deeper ones (12.4 / 17.7 us), and two consecutive launches sharing an SM cost 4 us (the arrange kernel
    // sits between them in the stream) - so the request is kept above half an SM's shared memory.
    const int st = stages_for_xs(plan->mt, stage, kSmemOptIn);
    const int want = plan->mt == 1 ? 5 : 4;
    plan->stages = st > want ? want : st;
    plan->smem = fixed_smem_xs(plan->mt) + (size_t)plan->stages * (stage + sk_xblock(plan->mt));
    if (plan->smem <= (size_t)kSmemHalf) plan->smem = (size_t)kSmemHalf + 1024;
    plan->xa_bytes = (size_t)plan->passes * plan->C * sk_xblock(plan->mt);
  }
  plan->ws_bytes = (size_t)plan->passes * plan->grid_x * 2 * SK_TILES * plan->mt * 32 * sizeof(float4);
  plan->counter_ints = (size_t)plan->passes * plan->P * SK_TILES;
}

// Launches the stream GEMM. `fmt`: 0 = W4 symmetric, 1 = W4 asymmetric, 2 = MXFP4.
// The caller has checked stream_gemm_supported and sized ws / counters by the plan;
// counters are all zero between launches. `overlap` launches with programmatic stream
// serialization: the grid may start while the previous kernel of the stream is still running
// and reads the packed weights (q / scales / zeros) before that kernel has completed - the
// caller promises that the previous kernel does not write them. Activations, outputs and
// scratch are only touched after the previous kernel has completed. `xa` (plan.xa_bytes, 16-byte aligned) holds
// the arranged activations of the streamed form; it is written by a pre-pass launched here.
cudaError_t stream_gemm_launch(int fmt, int gs, const uint32_t* q, const void* scales, const uint32_t* zeros,
                               int N, int K, int G, const __half* x, __half* c, int M, __half* w_out,
                               const StreamPlan& plan, float* ws, int* counters, void* xa, int* status,
                               bool overlap, cudaStream_t stream, int* launches, const StreamPeers* peers) {
  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {(cuuint64_t)(K / 8), (cuuint64_t)N};
  const cuuint64_t gstride[1] = {(cuuint64_t)(K / 8) * 4};
  const cuuint32_t box[2] = {SK_KC / 8, SK_ROWS};  // 32 words = 128 bytes wide: the swizzle span
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
  sp.wG = words(G);
  sp.C = plan.C;
  sp.P = plan.P;
  sp.U = (int)plan.U;
  sp.stages = plan.stages;
  sp.xpitch = plan.xpitch;
  sp.ws = ws;
  sp.counters = counters;
  sp.status = status;
  sp.xrows = plan.rows_per_pass;
  sp.xa = plan.streamed ? (const uint8_t*)xa : nullptr;
  if (peers) {
    sp.peers = *peers;
  } else {
    memset(&sp.peers, 0, sizeof(sp.peers));
  }
  if (launches) *launches = plan.streamed ? 2 : 1;
  if (plan.streamed) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)plan.C, (unsigned)plan.passes);
    cfg.blockDim = dim3(XA_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, x_arrange_kernel, x, (uint8_t*)xa, M, K, plan.C, plan.rows_per_pass,
                                             plan.mt, (int)sk_fold(fmt, gs));
    if (e != cudaSuccess) return e;
  }
  const dim3 grid((unsigned)plan.grid_x, (unsigned)plan.passes);  // pass y = activation rows y*rows_per_pass ...
  switch (fmt) {
    case F_W4_SYM:
      if (gs == 32) return launch_fmt<F_W4_SYM, 32>(tmap, sp, plan.mt, grid, plan.smem, overlap, stream);
      if (gs == 64) return launch_fmt<F_W4_SYM, 64>(tmap, sp, plan.mt, grid, plan.smem, overlap, stream);
      return launch_fmt<F_W4_SYM, 128>(tmap, sp, plan.mt, grid, plan.smem, overlap, stream);
    case F_W4_ASYM:
      if (gs == 32) return launch_fmt<F_W4_ASYM, 32>(tmap, sp, plan.mt, grid, plan.smem, overlap, stream);
      if (gs == 64) return launch_fmt<F_W4_ASYM, 64>(tmap, sp, plan.mt, grid, plan.smem, overlap, stream);
      return launch_fmt<F_W4_ASYM, 128>(tmap, sp, plan.mt, grid, plan.smem, overlap, stream);
    default:
      return launch_fmt<F_MX, 32>(tmap, sp, plan.mt, grid, plan.smem, overlap, stream);
  }
}

}  // namespace w4b
