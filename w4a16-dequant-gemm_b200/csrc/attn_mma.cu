// Split-S decode attention on the tensor pipe for the common head sizes
// (D = 64 or 128; W4 / FP8 group size 32, 64 or 128; FP16): the fast form of
// the reference's flash_*_phase1 kernels (include/w4/kvflash.cuh:73-199,
// 202-288, 459-570, 598-723). attn_flash.cu keeps every other shape.
//
// grid = (heads, splits); a CTA owns a contiguous slice of one head's positions
// and each of its 4 warps walks blocks of 16 positions with an online softmax.
// Per block and warp:
//
//   scores = K q   mma.m16n8k16 with A = K (16 positions x 16 d per step), B = q in
//                  every column. Lane (g, c) decodes the quarter c of rows g and
//                  g + 8 in registers straight into A fragments - the k slots of a
//                  step may hold any d as long as q is arranged the same way, so a
//                  packed W4 word is used exactly as the decoder emits it.
//   out^T += V^T p mma.m16n8k16 with A = V^T (16 d x 16 positions), B = p in every
//                  column. A fragment registers pair two POSITIONS of one d; lane
//                  (g, c) therefore loads positions 2c, 2c+1, 2c+8, 2c+9 of the d range
//                  of g, interleaves the codes of two positions with one byte
//                  permute per word and decodes both positions in each half2
//                  operation (two scales / zero points per instruction). No shared
//                  memory, no transposes, every cache byte is loaded once.
//
// Batched paged form with shared pages (MULTI): a CTA serves up to eight sequences of one head at a time, sequence
// j in column j of both products - B = the eight queries, resp. the eight weight vectors. A block whose page is
// the same for all of them (a shared prefix) is loaded and decoded ONCE for the eight; a block with different
// pages runs once per sequence with only that sequence's column live. Columns of an MMA are independent dot
// products and a sequence's slices, block order and merge order depend on its own length only, so its output
// does not depend on the company it has in the call (with one sequence per call: the bits of the
// single-sequence entry); only the work is shared.
//
// Dequantised values are bit-identical to the host formats (the same decoders as
// the GEMM kernels; FP8: the byte placed in a half is code * 2^-8, times 256 is
// exact, times the scale rounds once). Sums are formed in a fixed order: lanes,
// then warps, then splits - the same call gives the same bits, with or without the
// dequantisation hooks, paged or contiguous.
#include <math_constants.h>

#include <atomic>

#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {
namespace {

constexpr int MA_WARPS = 4;
constexpr int MA_THREADS = 32 * MA_WARPS;
constexpr int MA_BLOCK = 16;  // positions per warp step

struct MmaParams {
  AttnSource src;
  const __half* q;
  __half* out;
  float* ws;
  __half* k_out;
  __half* v_out;
  int H, S, splits;
  int gshift;  // log2(group size)
  int wide;    // the hooks may be written 16 bytes at a time
  // batched paged form: grid.x = nseq * H; sequence i has seq_lens[i] positions and the block table
  // bt + i * bt_stride; its slices are cut for attn_batched_rows(nseq, H) rows
  int nseq;             // 0: single sequence
  const int* seq_lens;  // device, nseq entries
  int bt_stride;
  int sm_count;
  int pshift;  // log2(page) when the page is a power of two >= 16, else -1
};

// The arrays of one head (rows are then indexed with 32-bit multiplies by constant strides).
struct HeadBase {
  const uint8_t* k;
  const uint8_t* v;
  const __half* sk;
  const __half* sv;
  const uint32_t* zk;
  const uint32_t* zv;
  int G, wG;
};

// Decode constants for two rows at once: low half = first row, high half = second row.
__device__ __forceinline__ W4Group w4_group2(__half s1, uint32_t z1, __half s2, uint32_t z2) {
  W4Group g;
  g.s2 = __halves2half2(s1, s2);
  const uint32_t z = z1 | (z2 << 16);
  g.za = u32_as_h2(z + 0x64006400u);         // 1024 + z
  g.zb = u32_as_h2((z << 4) + 0xD400D400u);  // -(64 + z)
  return g;
}

// FP8 E4M3 pair sitting in bits 15..8 and 31..24 of x (other bits arbitrary) -> the two
// dequantised halves, each times its scale in s2.
__device__ __forceinline__ __half2 dq_f8_pair(uint32_t x, __half2 s2) {
  const uint32_t mag = (x >> 1) & 0x3F803F80u;
  const uint32_t bits = and_or(x, 0x80008000u, mag);  // sign | exponent, mantissa: code * 2^-8
  const __half2 v = __hmul2_rn(u32_as_h2(bits), u32_as_h2(0x5C005C00u));  // * 256, exact
  return __hmul2_rn(v, s2);
}

__device__ __forceinline__ __half ldg_half(const __half* p) {
  return __ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p)));
}

// ---------------------------------------------------------------------------
// Raw data of one block of 16 positions, as loaded by one lane.
//   K side: rows g and g + 8, elements [E*c, E*c + E) with E = D/4.
//   V side: rows 2c, 2c+1, 2c+8, 2c+9, elements [EV*g, EV*g + EV) with EV = D/8.
// ---------------------------------------------------------------------------
template <int FMT, int D>
struct BlockData;

template <int D>
struct BlockData<ATTN_FP16, D> {
  static constexpr int KU = D / 32, VU = D / 64;  // uint4 per row
  uint4 k[2][KU];
  uint4 v[4][VU];
  __device__ __forceinline__ void load(const HeadBase& s, const int rk[2], const int rv[4], int g, int c,
                                       int /*gshift*/) {
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int i = 0; i < KU; ++i)
        k[r][i] = __ldg(reinterpret_cast<const uint4*>(s.k + (size_t)(unsigned)rk[r] * (2 * D) + (D / 2) * c) + i);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int i = 0; i < VU; ++i)
        v[r][i] = __ldg(reinterpret_cast<const uint4*>(s.v + (size_t)(unsigned)rv[r] * (2 * D) + (D / 4) * g) + i);
  }
};

template <int D>
struct BlockData<ATTN_F8, D> {
  static constexpr int KW = D / 16, VW = D / 32;  // 32-bit words per row
  uint32_t k[2][KW];
  uint32_t v[4][VW];
  __half ks[2], vs[4];
  __device__ __forceinline__ void load(const HeadBase& s, const int rk[2], const int rv[4], int g, int c,
                                       int gshift) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint8_t* p = s.k + (size_t)(unsigned)rk[r] * D + (D / 4) * c;
      if (KW == 8) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(p)), b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
        k[r][0] = a.x, k[r][1] = a.y, k[r][2] = a.z, k[r][3] = a.w;
        k[r][4 % KW] = b.x, k[r][5 % KW] = b.y, k[r][6 % KW] = b.z, k[r][7 % KW] = b.w;
      } else {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
        k[r][0] = a.x, k[r][1] = a.y, k[r][2] = a.z, k[r][3] = a.w;
      }
      ks[r] = ldg_half(s.sk + (size_t)(unsigned)(rk[r] * s.G + (((D / 4) * c) >> gshift)));
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint8_t* p = s.v + (size_t)(unsigned)rv[r] * D + (D / 8) * g;
      if (VW == 4) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
        v[r][0] = a.x, v[r][1] = a.y, v[r][2 % VW] = a.z, v[r][3 % VW] = a.w;
      } else {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(p));
        v[r][0] = a.x, v[r][1] = a.y;
      }
      vs[r] = ldg_half(s.sv + (size_t)(unsigned)(rv[r] * s.G + (((D / 8) * g) >> gshift)));
    }
  }
};

template <int D, bool ASYM>
struct W4Ring;

template <int FMT, int D>
struct BlockDataW4 {
  static constexpr int KW = D / 32, VW = D / 64;  // packed words per row
  static constexpr int WD = D / 8;                // words per cache row
  uint32_t k[2][KW];
  uint32_t v[4][VW];
  __half ks[2], vs[4];
  uint32_t kz[2], vz[4];  // zero points
  // from a stage of the lane-private ring
  __device__ __forceinline__ void collect(uint32_t st, int lane, int g, int c, int gshift, int G) {
    using R = W4Ring<D, FMT == ATTN_W4_ASYM>;
    R::collect_codes(*this, st, lane);
    const int gk = ((D / 4) * c) >> gshift, gv = ((D / 8) * g) >> gshift;
#pragma unroll
    for (int r = 0; r < 2; ++r) ks[r] = R::k_scale(st, r, lane, gk), kz[r] = R::k_zero(st, r, lane, gk);
#pragma unroll
    for (int r = 0; r < 4; ++r) vs[r] = R::v_scale(st, r, lane, gv), vz[r] = R::v_zero(st, r, lane, gv);
    (void)G;
  }
  __device__ __forceinline__ void load(const HeadBase& s, const int rk[2], const int rv[4], int g, int c,
                                       int gshift) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint32_t* p = reinterpret_cast<const uint32_t*>(s.k + (size_t)(unsigned)rk[r] * (WD * 4)) + KW * c;
      if (KW == 4) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
        k[r][0] = a.x, k[r][1] = a.y, k[r][2 % KW] = a.z, k[r][3 % KW] = a.w;
      } else {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(p));
        k[r][0] = a.x, k[r][1] = a.y;
      }
      const int grp = ((D / 4) * c) >> gshift;
      ks[r] = ldg_half(s.sk + (size_t)(unsigned)(rk[r] * s.G + grp));
      kz[r] = FMT == ATTN_W4_ASYM ? ((__ldg(s.zk + (size_t)(unsigned)(rk[r] * s.wG + (grp >> 3))) >> (4 * (grp & 7))) & 0xFu)
                                  : 8u;
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint32_t* p = reinterpret_cast<const uint32_t*>(s.v + (size_t)(unsigned)rv[r] * (WD * 4)) + VW * g;
      if (VW == 2) {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(p));
        v[r][0] = a.x, v[r][1 % VW] = a.y;
      } else {
        v[r][0] = __ldg(p);
      }
      const int grp = ((D / 8) * g) >> gshift;
      vs[r] = ldg_half(s.sv + (size_t)(unsigned)(rv[r] * s.G + grp));
      vz[r] = FMT == ATTN_W4_ASYM ? ((__ldg(s.zv + (size_t)(unsigned)(rv[r] * s.wG + (grp >> 3))) >> (4 * (grp & 7))) & 0xFu)
                                  : 8u;
    }
  }
};
template <int D>
struct BlockData<ATTN_W4_SYM, D> : BlockDataW4<ATTN_W4_SYM, D> {};
template <int D>
struct BlockData<ATTN_W4_ASYM, D> : BlockDataW4<ATTN_W4_ASYM, D> {};

// W4 block of the single-sequence form, whose products take the scales OUT of the contraction (see the kernel):
// the same words, but the K scales of the two quarters whose partial scores this lane finishes (quarters 2c and
// 2c + 1 of rows g and g + 8; lanes c >= 2 finish nothing and load what lanes c - 2 load) and the V scales of the
// group that is this lane's COLUMN of the second product (group g; none for g >= G). With hooks the scales of
// the lane's own words come along for the exact decode.
template <int FMT, int D, bool HOOK>
struct BlockDataW4Fold {
  static constexpr int KW = D / 32, VW = D / 64, WD = D / 8, E = D / 4;
  uint32_t k[2][KW];
  uint32_t v[4][VW];
  __half ks[2][2], vs[4];
  uint32_t kz[2][2], vz[4];
  __half ks_own[HOOK ? 2 : 1], vs_own[HOOK ? 4 : 1];
  uint32_t kz_own[HOOK ? 2 : 1];
  // from a stage of the lane-private ring (never with hooks)
  __device__ __forceinline__ void collect(uint32_t st, int lane, int g, int c, int gshift, int G) {
    using R = W4Ring<D, FMT == ATTN_W4_ASYM>;
    R::collect_codes(*this, st, lane);
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int grp = (E * ((2 * c + x) & 3)) >> gshift;
        ks[r][x] = R::k_scale(st, r, lane, grp), kz[r][x] = R::k_zero(st, r, lane, grp);
      }
    const int col = min(g, G - 1), gv = ((D / 8) * g) >> gshift;
#pragma unroll
    for (int r = 0; r < 4; ++r) vs[r] = R::v_scale(st, r, lane, col), vz[r] = R::v_zero(st, r, lane, gv);
  }
  __device__ __forceinline__ static uint32_t zero_of(const uint32_t* z, int row, int wG, int grp) {
    return FMT == ATTN_W4_ASYM ? ((__ldg(z + (size_t)(unsigned)(row * wG + (grp >> 3))) >> (4 * (grp & 7))) & 0xFu) : 8u;
  }
  __device__ __forceinline__ void load(const HeadBase& s, const int rk[2], const int rv[4], int g, int c, int gshift) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint32_t* p = reinterpret_cast<const uint32_t*>(s.k + (size_t)(unsigned)rk[r] * (WD * 4)) + KW * c;
      if (KW == 4) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
        k[r][0] = a.x, k[r][1] = a.y, k[r][2 % KW] = a.z, k[r][3 % KW] = a.w;
      } else {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(p));
        k[r][0] = a.x, k[r][1] = a.y;
      }
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int grp = (E * ((2 * c + x) & 3)) >> gshift;
        ks[r][x] = ldg_half(s.sk + (size_t)(unsigned)(rk[r] * s.G + grp));
        kz[r][x] = zero_of(s.zk, rk[r], s.wG, grp);
      }
      if (HOOK) {
        const int grp = (E * c) >> gshift;
        ks_own[r % (HOOK ? 2 : 1)] = ldg_half(s.sk + (size_t)(unsigned)(rk[r] * s.G + grp));
        kz_own[r % (HOOK ? 2 : 1)] = zero_of(s.zk, rk[r], s.wG, grp);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint32_t* p = reinterpret_cast<const uint32_t*>(s.v + (size_t)(unsigned)rv[r] * (WD * 4)) + VW * g;
      if (VW == 2) {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(p));
        v[r][0] = a.x, v[r][1 % VW] = a.y;
      } else {
        v[r][0] = __ldg(p);
      }
      const int col = min(g, s.G - 1);
      const int grp = ((D / 8) * g) >> gshift;  // the group of this lane's own rows of V^T
      vs[r] = ldg_half(s.sv + (size_t)(unsigned)(rv[r] * s.G + col));
      vz[r] = zero_of(s.zv, rv[r], s.wG, grp);
      if (HOOK) vs_own[r % (HOOK ? 4 : 1)] = ldg_half(s.sv + (size_t)(unsigned)(rv[r] * s.G + grp));
    }
  }
};

// ---------------------------------------------------------------------------
// Lane-private shared-memory ring for the W4 forms (ASYNC): instead of holding the next block in registers, a
// lane cp.async's exactly the pieces it will consume itself - its two K row quarters, its four V row eighths
// and the scale (and zero-point) rows that belong to them - into its own slots of a stage, up to two blocks
// ahead, and reads them back with shared-memory loads when the block's turn comes. No lane reads another
// lane's slots, so cp.async.wait_group is the only synchronisation. Pieces are laid out [piece][lane] so that
// a warp's load of one piece is conflict-free. Needs scale rows of at least four bytes (G >= 2).
// ---------------------------------------------------------------------------
template <int D, bool ASYM>
struct W4Ring {
  static constexpr int KB = D / 8, VB = D / 16;  // bytes per lane of a K row quarter / a V row eighth
  static constexpr int OFF_V = 2 * 32 * KB;
  static constexpr int OFF_SK = OFF_V + 4 * 32 * VB;
  static constexpr int OFF_SV = OFF_SK + 2 * 32 * 8;
  static constexpr int OFF_ZK = OFF_SV + 4 * 32 * 8;
  static constexpr int OFF_ZV = OFF_ZK + 2 * 32 * 4;
  static constexpr int STAGE = ASYM ? OFF_ZV + 4 * 32 * 4 : OFF_ZK;
  static constexpr int DEPTH = 3;

  __device__ __forceinline__ static void issue(uint32_t st, const HeadBase& s, const int rk[2], const int rv[4], int lane,
                                               int g, int c) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      cp_async<KB>(st + r * 32 * KB + lane * KB, s.k + (size_t)(unsigned)rk[r] * (D / 2) + KB * c);
      const __half* sp = s.sk + (size_t)(unsigned)(rk[r] * s.G);
      if (s.G == 4)
        cp_async<8>(st + OFF_SK + r * 256 + lane * 8, sp);
      else
        cp_async<4>(st + OFF_SK + r * 256 + lane * 8, sp);
      if (ASYM) cp_async<4>(st + OFF_ZK + r * 128 + lane * 4, s.zk + (size_t)(unsigned)(rk[r] * s.wG));
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      cp_async<VB>(st + OFF_V + r * 32 * VB + lane * VB, s.v + (size_t)(unsigned)rv[r] * (D / 2) + VB * g);
      const __half* sp = s.sv + (size_t)(unsigned)(rv[r] * s.G);
      if (s.G == 4)
        cp_async<8>(st + OFF_SV + r * 256 + lane * 8, sp);
      else
        cp_async<4>(st + OFF_SV + r * 256 + lane * 8, sp);
      if (ASYM) cp_async<4>(st + OFF_ZV + r * 128 + lane * 4, s.zv + (size_t)(unsigned)(rv[r] * s.wG));
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // the pieces every W4 block type shares
  template <typename B>
  __device__ __forceinline__ static void collect_codes(B& b, uint32_t st, int lane) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (KB == 16) {
        const uint4 a = lds128(st + r * 32 * KB + lane * KB);
        b.k[r][0] = a.x, b.k[r][1] = a.y, b.k[r][2 % B::KW] = a.z, b.k[r][3 % B::KW] = a.w;
      } else {
        const uint2 a = lds64(st + r * 32 * KB + lane * KB);
        b.k[r][0] = a.x, b.k[r][1] = a.y;
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (VB == 8) {
        const uint2 a = lds64(st + OFF_V + r * 32 * VB + lane * VB);
        b.v[r][0] = a.x, b.v[r][1 % B::VW] = a.y;
      } else {
        b.v[r][0] = lds32(st + OFF_V + r * 32 * VB + lane * VB);
      }
    }
  }
  __device__ __forceinline__ static __half k_scale(uint32_t st, int r, int lane, int grp) {
    return __ushort_as_half(lds16(st + OFF_SK + r * 256 + lane * 8 + 2 * grp));
  }
  __device__ __forceinline__ static __half v_scale(uint32_t st, int r, int lane, int grp) {
    return __ushort_as_half(lds16(st + OFF_SV + r * 256 + lane * 8 + 2 * grp));
  }
  __device__ __forceinline__ static uint32_t k_zero(uint32_t st, int r, int lane, int grp) {
    return ASYM ? (lds32(st + OFF_ZK + r * 128 + lane * 4) >> (4 * grp)) & 0xFu : 8u;
  }
  __device__ __forceinline__ static uint32_t v_zero(uint32_t st, int r, int lane, int grp) {
    return ASYM ? (lds32(st + OFF_ZV + r * 128 + lane * 4) >> (4 * grp)) & 0xFu : 8u;
  }
};

template <int FMT, int D, bool FOLD, bool HOOK>
struct BlockSel {
  using type = BlockData<FMT, D>;
};
template <int FMT, int D, bool HOOK>
struct BlockSel<FMT, D, true, HOOK> {
  using type = BlockDataW4Fold<FMT, D, HOOK>;
};

// The eight codes of a packed word as FP16 bit patterns, no arithmetic: out[0] = codes (0, 4) and out[2] = codes
// (2, 6) are code * 2^-24 (a code in the low nibble of a half is that subnormal), out[1] = codes (1, 5) and
// out[3] = codes (3, 7) are code * 2^-20 (the nibble above). 1 shift + 4 AND.
__device__ __forceinline__ void w4_raw_codes(uint32_t qw, const W4Consts& k, uint32_t out[4]) {
  const uint32_t hi = qw >> 8;
  out[0] = qw & k.lo;
  out[1] = qw & k.hi;
  out[2] = hi & k.lo;
  out[3] = hi & k.hi;
}

__device__ __forceinline__ uint4 unpair4(const __half2 p[4]) {  // (e, e+4) pairs -> 8 halves in order
  uint4 r;
  r.x = __byte_perm(h2_as_u32(p[0]), h2_as_u32(p[1]), 0x5410);
  r.y = __byte_perm(h2_as_u32(p[2]), h2_as_u32(p[3]), 0x5410);
  r.z = __byte_perm(h2_as_u32(p[0]), h2_as_u32(p[1]), 0x7632);
  r.w = __byte_perm(h2_as_u32(p[2]), h2_as_u32(p[3]), 0x7632);
  return r;
}

// Eight halves to dst (16-byte store when allowed).
__device__ __forceinline__ void store8(__half* dst, uint4 v, bool wide) {
  if (wide) {
    *reinterpret_cast<uint4*>(dst) = v;
  } else {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      dst[2 * i] = __ushort_as_half((unsigned short)(w[i] & 0xFFFFu));
      dst[2 * i + 1] = __ushort_as_half((unsigned short)(w[i] >> 16));
    }
  }
}

template <int FMT, int D, bool HOOK, bool MULTI, bool ASYNC>
__global__ void __launch_bounds__(MA_THREADS, (HOOK || FMT == ATTN_FP16) ? 2 : (FMT == ATTN_F8 ? 3 : 4)) attn_mma_kernel(const MmaParams p) {
  constexpr int E = D / 4;    // K elements per lane per row
  constexpr int EV = D / 8;   // V elements per lane per row
  constexpr int NQ = E / 8;   // q fragments (8 elements each) per lane
  constexpr int NT = EV / 2;  // output tiles (16 d each... per lane: rows g and g+8)
  constexpr bool IS_W4 = FMT == ATTN_W4_SYM || FMT == ATTN_W4_ASYM;
  // Single-sequence W4: the scales are taken out of both contractions. The A operands are the raw codes (exact
  // FP16 subnormals, five instructions per word instead of thirteen) and the spare columns of the products keep
  // apart what needs different scales: in scores = K q, B holds q in column n only for the k slots of lane n, so
  // column n is the partial score of quarter n of the head dimension and is scaled afterwards in FP32
  // (s * (2^24 * sum - z * sum of q)); in out^T = V^T p, column n of B is p * scale of group n (rounded to FP16 as
  // p alone was), row d reads its own group's column, and one more MMA with an all-ones A gives the sums that
  // carry the zero points. With hooks the same arithmetic runs and the exact decode is done beside it for the
  // stores, so the output bits do not depend on the hooks. (MULTI needs the columns for the sequences.)
  constexpr bool FOLD = IS_W4 && !MULTI;
  using Blk = typename BlockSel<FMT, D, FOLD, HOOK>::type;
  constexpr int COLS = MULTI ? 8 : 1;  // sequences per CTA (columns of the products that carry distinct data)
  constexpr int NC = MULTI ? 2 : 1;    // columns whose softmax state a lane keeps (2c, 2c + 1)
  using Ring = W4Ring<D, FMT == ATTN_W4_ASYM>;
  extern __shared__ __align__(16) uint8_t sm_dyn[];  // ASYNC: the warps' rings; the merge reuses it afterwards
  __shared__ float sm_ml[MA_WARPS][COLS][2];
  __shared__ float sm_acc_static[ASYNC ? 1 : MA_WARPS][ASYNC ? 1 : COLS][ASYNC ? 1 : D];
  float(*sm_acc)[COLS][D] = ASYNC ? reinterpret_cast<float(*)[COLS][D]>(sm_dyn)
                                  : reinterpret_cast<float(*)[COLS][D]>(&sm_acc_static[0][0][0]);
  // MULTI: the last slices first - those past a shared prefix run once per sequence and take the longest
  const int sp = MULTI ? (int)(gridDim.y - 1 - blockIdx.y) : (int)blockIdx.y;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const AttnSource& s = p.src;
  const W4Consts kc = w4_consts();
  const uint32_t ring = ASYNC ? smem_u32(sm_dyn) + (uint32_t)wid * (Ring::DEPTH * Ring::STAGE) : 0u;
  // MULTI: blockIdx.x = group * H + head, a group = eight consecutive sequences (fewer at the end). When their
  // lengths are equal they share one pass; otherwise each sequence gets a pass of its own with one live column.
  const int h = MULTI ? (int)(blockIdx.x % p.H) : (p.nseq ? (int)(blockIdx.x % p.H) : (int)blockIdx.x);
  const int seq0 = MULTI ? 8 * (int)(blockIdx.x / p.H) : 0;
  const int count = MULTI ? min(8, p.nseq - seq0) : 1;
  int npass = 1, my_len = 0;
  if constexpr (MULTI) {
    my_len = __ldg(p.seq_lens + seq0 + min(lane, count - 1));
    npass = __all_sync(0xffffffffu, my_len == __shfl_sync(0xffffffffu, my_len, 0)) ? 1 : count;
  }
  HeadBase hb;
  {
    const size_t slab = (size_t)h * (size_t)s.slab_rows;
    const size_t row_bytes = FMT == ATTN_FP16 ? 2 * D : (FMT == ATTN_F8 ? D : D / 2);
    hb.k = reinterpret_cast<const uint8_t*>(s.k) + slab * row_bytes;
    hb.v = reinterpret_cast<const uint8_t*>(s.v) + slab * row_bytes;
    hb.G = s.G;
    hb.wG = words(s.G);
    hb.sk = s.s_k ? s.s_k + slab * s.G : nullptr;
    hb.sv = s.s_v ? s.s_v + slab * s.G : nullptr;
    hb.zk = s.z_k ? s.z_k + slab * hb.wG : nullptr;
    hb.zv = s.z_v ? s.z_v + slab * hb.wG : nullptr;
  }
  const float scale = rsqrtf((float)D);

#pragma unroll 1
  for (int pass = 0; pass < npass; ++pass) {
  // live columns of this pass, the sequence whose geometry it uses, and the row of q / out of column 0
  const uint32_t colmask = MULTI ? (npass == 1 ? (1u << count) - 1u : 1u << pass) : 1u;
  const int firstcol = MULTI ? (npass == 1 ? 0 : pass) : 0;
  const int hx = MULTI ? (seq0 * p.H + h) : (int)blockIdx.x;  // hx: row of q / out (sequence-major in the batched form)
  const int S = MULTI ? __shfl_sync(0xffffffffu, my_len, firstcol) : (p.nseq ? __ldg(p.seq_lens + hx / p.H) : p.S);
  const int splits = p.nseq ? attn_flash_splits(attn_batched_rows(p.nseq, p.H), S, p.sm_count) : p.splits;
  if (sp >= splits) continue;  // (batched: the grid is sized for the longest sequence)
  const int* bt = p.src.bt ? p.src.bt + (p.nseq ? (size_t)(MULTI ? seq0 : hx / p.H) * p.bt_stride : 0) : nullptr;
  // slices are cut at multiples of 64 positions: the four warps of a CTA get the same number of blocks
  const int units = (S + MA_WARPS * MA_BLOCK - 1) / (MA_WARPS * MA_BLOCK);
  const int t0 = MA_WARPS * MA_BLOCK * (int)((long long)units * sp / splits);
  const int t1 = min(S, MA_WARPS * MA_BLOCK * (int)((long long)units * (sp + 1) / splits));
  // q of this lane's K quarter, in the pairing its K fragments use (MULTI: the query of sequence g, column g)
  uint4 qf[NQ];
#pragma unroll
  for (int i = 0; i < NQ; ++i) {
    const size_t qrow = MULTI ? (size_t)hx + (size_t)min(g, count - 1) * p.H : (size_t)hx;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.q + qrow * D + E * c) + i);
    qf[i] = (FMT == ATTN_W4_SYM || FMT == ATTN_W4_ASYM) ? pair_permute(v) : v;
  }

  // FOLD: sums of q over the two quarters whose partial scores this lane finishes, times the symmetric zero
  // point; q itself only in the column that is this lane's own quarter, the hi-nibble pairs divided by 16
  float zq[2] = {0.0f, 0.0f};
  float c1[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // FOLD: 2^-24 * sum over positions of p * scale * zero point, per column
  if constexpr (FOLD) {
    float qs = 0.0f;
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
      const uint32_t w[4] = {qf[i].x, qf[i].y, qf[i].z, qf[i].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(u32_as_h2(w[e]));
        qs += f.x + f.y;
      }
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) zq[x] = __shfl_sync(0xffffffffu, qs, (lane & ~3) | ((2 * c + x) & 3));
    const __half2 sixteenth = u32_as_h2(0x2C002C00u);
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
      qf[i].y = h2_as_u32(__hmul2_rn(u32_as_h2(qf[i].y), sixteenth));
      qf[i].w = h2_as_u32(__hmul2_rn(u32_as_h2(qf[i].w), sixteenth));
      if (g != c) qf[i] = make_uint4(0u, 0u, 0u, 0u);
    }
  }

  float m[NC], l[NC];
#pragma unroll
  for (int x = 0; x < NC; ++x) m[x] = -CUDART_INF_F, l[x] = 0.0f;
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;

  // rows of a block: K rows g, g + 8 and V rows 2c, 2c+1, 2c+8, 2c+9 of the 16 positions from tb
  auto rows_of = [&](int tb, int page_id, int rk[2], int rv[4]) {
    const int last = t1 - 1;  // positions past the slice read a valid row and get weight 0
    if (MULTI || bt == nullptr || p.pshift >= 0) {
      // contiguous cache, or pages that are a power of two >= 16: the block's 16 positions (tb is a multiple of
      // 16) lie in one page, so one table entry serves the block (MULTI: the caller has looked it up)
      // (MULTI: a table entry outside the pool is clamped rather than followed)
      const int pg = MULTI ? min(max(page_id, 0), (int)(s.slab_rows >> p.pshift) - 1)
                           : (bt == nullptr ? 0 : __ldg(bt + (tb >> p.pshift)));
      const int base = bt == nullptr ? tb : (pg << p.pshift) + (tb & ((1 << p.pshift) - 1));
      const int lim = last - tb;
      rk[0] = base + min(g, lim);
      rk[1] = base + min(g + 8, lim);
      rv[0] = base + min(2 * c, lim);
      rv[1] = base + min(2 * c + 1, lim);
      rv[2] = base + min(2 * c + 8, lim);
      rv[3] = base + min(2 * c + 9, lim);
    } else {
      auto row = [&](int t) { return __ldg(bt + t / s.page) * s.page + (t % s.page); };
      rk[0] = row(min(tb + g, last));
      rk[1] = row(min(tb + g + 8, last));
      rv[0] = row(min(tb + 2 * c, last));
      rv[1] = row(min(tb + 2 * c + 1, last));
      rv[2] = row(min(tb + 2 * c + 8, last));
      rv[3] = row(min(tb + 2 * c + 9, last));
    }
  };
  auto fetch = [&](Blk& blk, int tb, int page_id) {
    int rk[2], rv[4];
    rows_of(tb, page_id, rk, rv);
    blk.load(hb, rk, rv, g, c, p.gshift);
  };
  // ASYNC: the same block into stage `slot` of this warp's ring (one cp.async group), and out of it
  auto issue = [&](int slot, int tb, int page_id) {
    int rk[2], rv[4];
    rows_of(tb, page_id, rk, rv);
    if constexpr (IS_W4) Ring::issue(ring + (uint32_t)slot * Ring::STAGE, hb, rk, rv, lane, g, c);
  };
  auto collect = [&](Blk& blk, int slot) {
    if constexpr (ASYNC) blk.collect(ring + (uint32_t)slot * Ring::STAGE, lane, g, c, p.gshift, hb.G);
  };
  auto empty_group = [&]() { asm volatile("cp.async.commit_group;" ::: "memory"); };
  auto wait_oldest = [&]() { asm volatile("cp.async.wait_group %0;" ::"n"(Ring::DEPTH - 1) : "memory"); };

  // Hook stores of four V rows from (row 2c | row 2c+1) and (row 2c+8 | row 2c+9) pairs of halves
  auto store_v_rows_at = [&](const uint32_t* a12, const uint32_t* a34, int tb) {
#pragma unroll
      for (int e0 = 0; e0 < EV; e0 += 8) {
        uint4 a, b, cc, d;
        a.x = __byte_perm(a12[e0], a12[e0 + 1], 0x5410), a.y = __byte_perm(a12[e0 + 2], a12[e0 + 3], 0x5410);
        a.z = __byte_perm(a12[e0 + 4], a12[e0 + 5], 0x5410), a.w = __byte_perm(a12[e0 + 6], a12[e0 + 7], 0x5410);
        b.x = __byte_perm(a12[e0], a12[e0 + 1], 0x7632), b.y = __byte_perm(a12[e0 + 2], a12[e0 + 3], 0x7632);
        b.z = __byte_perm(a12[e0 + 4], a12[e0 + 5], 0x7632), b.w = __byte_perm(a12[e0 + 6], a12[e0 + 7], 0x7632);
        cc.x = __byte_perm(a34[e0], a34[e0 + 1], 0x5410), cc.y = __byte_perm(a34[e0 + 2], a34[e0 + 3], 0x5410);
        cc.z = __byte_perm(a34[e0 + 4], a34[e0 + 5], 0x5410), cc.w = __byte_perm(a34[e0 + 6], a34[e0 + 7], 0x5410);
        d.x = __byte_perm(a34[e0], a34[e0 + 1], 0x7632), d.y = __byte_perm(a34[e0 + 2], a34[e0 + 3], 0x7632);
        d.z = __byte_perm(a34[e0 + 4], a34[e0 + 5], 0x7632), d.w = __byte_perm(a34[e0 + 6], a34[e0 + 7], 0x7632);
        const int d0 = EV * g + e0;
        const size_t base = ((size_t)h * p.S + tb) * D + d0;
        if (tb + 2 * c < t1) store8(p.v_out + base + (size_t)(2 * c) * D, a, p.wide);
        if (tb + 2 * c + 1 < t1) store8(p.v_out + base + (size_t)(2 * c + 1) * D, b, p.wide);
        if (tb + 2 * c + 8 < t1) store8(p.v_out + base + (size_t)(2 * c + 8) * D, cc, p.wide);
        if (tb + 2 * c + 9 < t1) store8(p.v_out + base + (size_t)(2 * c + 9) * D, d, p.wide);
      }
  };

  auto compute = [&](const Blk& cur, int tb, int ucol) {
    auto store_v_rows = [&](const uint32_t* a12, const uint32_t* a34) { store_v_rows_at(a12, a34, tb); };

    // ---------------- scores of rows g and g + 8 ----------------
    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
    if constexpr (FMT == ATTN_FP16) {
#pragma unroll
      for (int i = 0; i < NQ; ++i) {
        const uint32_t f0[4] = {cur.k[0][i].x, cur.k[1][i].x, cur.k[0][i].y, cur.k[1][i].y};
        const uint32_t f1[4] = {cur.k[0][i].z, cur.k[1][i].z, cur.k[0][i].w, cur.k[1][i].w};
        mma_16816(sa, f0, qf[i].x, qf[i].y);
        mma_16816(sb, f1, qf[i].z, qf[i].w);
      }
    } else if constexpr (FMT == ATTN_F8) {
      const __half2 s0 = __half2half2(cur.ks[0]), s1 = __half2half2(cur.ks[1]);
#pragma unroll
      for (int i = 0; i < NQ; ++i) {  // 8 bytes = 2 words per row per fragment
        __half2 a[4], b[4];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          const uint32_t x0 = cur.k[0][2 * i + w], x1 = cur.k[1][2 * i + w];
          a[2 * w] = dq_f8_pair(__byte_perm(x0, 0, 0x1404), s0);      // bytes 0, 1
          a[2 * w + 1] = dq_f8_pair(__byte_perm(x0, 0, 0x3424), s0);  // bytes 2, 3
          b[2 * w] = dq_f8_pair(__byte_perm(x1, 0, 0x1404), s1);
          b[2 * w + 1] = dq_f8_pair(__byte_perm(x1, 0, 0x3424), s1);
        }
        if (HOOK && p.k_out) {
          const int d0 = E * c + 8 * i;
          uint4 ua, ub;
          ua.x = h2_as_u32(a[0]), ua.y = h2_as_u32(a[1]), ua.z = h2_as_u32(a[2]), ua.w = h2_as_u32(a[3]);
          ub.x = h2_as_u32(b[0]), ub.y = h2_as_u32(b[1]), ub.z = h2_as_u32(b[2]), ub.w = h2_as_u32(b[3]);
          if (tb + g < t1) store8(p.k_out + ((size_t)h * p.S + tb + g) * D + d0, ua, p.wide);
          if (tb + g + 8 < t1) store8(p.k_out + ((size_t)h * p.S + tb + g + 8) * D + d0, ub, p.wide);
        }
        const uint32_t f0[4] = {h2_as_u32(a[0]), h2_as_u32(b[0]), h2_as_u32(a[1]), h2_as_u32(b[1])};
        const uint32_t f1[4] = {h2_as_u32(a[2]), h2_as_u32(b[2]), h2_as_u32(a[3]), h2_as_u32(b[3])};
        mma_16816(sa, f0, qf[i].x, qf[i].y);
        mma_16816(sb, f1, qf[i].z, qf[i].w);
      }
    } else if constexpr (FOLD) {
#pragma unroll
      for (int i = 0; i < NQ; ++i) {
        uint32_t a[4], b[4];
        w4_raw_codes(cur.k[0][i], kc, a);
        w4_raw_codes(cur.k[1][i], kc, b);
        if (HOOK && p.k_out) {
          __half2 ea[4], eb[4];
          dq_w4_word(cur.k[0][i], w4_group(cur.ks_own[0], cur.kz_own[0]), kc, ea);
          dq_w4_word(cur.k[1][i], w4_group(cur.ks_own[HOOK ? 1 : 0], cur.kz_own[HOOK ? 1 : 0]), kc, eb);
          const int d0 = E * c + 8 * i;
          if (tb + g < t1) store8(p.k_out + ((size_t)h * p.S + tb + g) * D + d0, unpair4(ea), p.wide);
          if (tb + g + 8 < t1) store8(p.k_out + ((size_t)h * p.S + tb + g + 8) * D + d0, unpair4(eb), p.wide);
        }
        const uint32_t f0[4] = {a[0], b[0], a[1], b[1]};
        const uint32_t f1[4] = {a[2], b[2], a[3], b[3]};
        mma_16816(sa, f0, qf[i].x, qf[i].y);
        mma_16816(sb, f1, qf[i].z, qf[i].w);
      }
      // columns 2c, 2c + 1 (c < 2) are the code sums of quarters 2c, 2c + 1: scale them, add the four quarters
      // of a row within the quad, and leave the row's score in every column as the plain form does
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float part = 0.0f;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const float zt = FMT == ATTN_W4_ASYM ? (float)cur.kz[r][x] * zq[x] : 8.0f * zq[x];
          part = fmaf(__half2float(cur.ks[r][x]), fmaf(sa[2 * r + x] + sb[2 * r + x], 16777216.0f, -zt), part);
        }
        part = c < 2 ? part : 0.0f;
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        sa[2 * r] = part;
        sb[2 * r] = 0.0f;
      }
    } else {
      const W4Group ga = w4_group(cur.ks[0], cur.kz[0]), gb = w4_group(cur.ks[1], cur.kz[1]);
#pragma unroll
      for (int i = 0; i < NQ; ++i) {
        __half2 a[4], b[4];
        dq_w4_word(cur.k[0][i], ga, kc, a);
        dq_w4_word(cur.k[1][i], gb, kc, b);
        const uint32_t f0[4] = {h2_as_u32(a[0]), h2_as_u32(b[0]), h2_as_u32(a[1]), h2_as_u32(b[1])};
        const uint32_t f1[4] = {h2_as_u32(a[2]), h2_as_u32(b[2]), h2_as_u32(a[3]), h2_as_u32(b[3])};
        mma_16816(sa, f0, qf[i].x, qf[i].y);
        mma_16816(sb, f1, qf[i].z, qf[i].w);
      }
    }
    uint32_t pb0, pb1;
    if constexpr (!MULTI) {
    // the MMA has summed the four lanes' quarters; every column of the product holds the score
    float s0 = sa[0] + sb[0], s1 = sa[2] + sb[2];
    s0 = (tb + g < t1) ? s0 * scale : -CUDART_INF_F;
    s1 = (tb + g + 8 < t1) ? s1 * scale : -CUDART_INF_F;

    // ---------------- online softmax over the block ----------------
    float bm = fmaxf(s0, s1);
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 8));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 16));
    // A new running maximum (the same decision in every lane; rare after the first blocks). Only columns 0 of
    // the accumulators are ever read in the plain form (every column holds the same sums), so only those are
    // rescaled there.
#pragma unroll 1
    // The trip count (0 or 1) comes out of a vote so that the compiler sees a loop and not an `if` it may turn into
    // predicated multiplications that cost every block their issue slots.
    for (int again = __popc(__ballot_sync(0xffffffffu, bm > m[0])) >> 5; again > 0; --again) {
      const float corr = __expf(m[0] - bm);  // m = -inf on the first block: 0
      l[0] *= corr;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        acc[j][0] *= corr;
        acc[j][2] *= corr;
        if (FOLD) {  // (a row's sum sits in its group's column)
          acc[j][1] *= corr;
          acc[j][3] *= corr;
        }
      }
      if (FOLD) {
#pragma unroll
        for (int i = 0; i < 4; ++i) c1[i] *= corr;
      }
      m[0] = bm;
    }
    // weights as FP16 (the MMA's input type); the denominator adds the same rounded values
    const __half2 pp = __floats2half2_rn(__expf(s0 - m[0]), __expf(s1 - m[0]));  // (p[g], p[g+8])
    float ps = __low2float(pp) + __high2float(pp);
    ps += __shfl_xor_sync(0xffffffffu, ps, 4);
    ps += __shfl_xor_sync(0xffffffffu, ps, 8);
    ps += __shfl_xor_sync(0xffffffffu, ps, 16);
    l[0] += ps;
    const uint32_t pu = __shfl_sync(0xffffffffu, h2_as_u32(pp), 8 * c);      // positions 2c, 2c+8
    const uint32_t pv = __shfl_sync(0xffffffffu, h2_as_u32(pp), 8 * c + 4);  // positions 2c+1, 2c+9
    pb0 = __byte_perm(pu, pv, 0x5410);                                       // (p[2c], p[2c+1])
    pb1 = __byte_perm(pu, pv, 0x7632);                                       // (p[2c+8], p[2c+9])
    } else {
    // Column n of the product is sequence n: this lane holds the scores of positions g, g + 8 for the
    // sequences 2c and 2c + 1. Each column runs the single-sequence arithmetic above on its own values.
    uint32_t ppu[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const int col = 2 * c + x;
      const bool live = ucol < 0 ? ((colmask >> col) & 1u) != 0 : col == ucol;
      float s0 = sa[x] + sb[x], s1 = sa[2 + x] + sb[2 + x];
      s0 = (live && tb + g < t1) ? s0 * scale : -CUDART_INF_F;
      s1 = (live && tb + g + 8 < t1) ? s1 * scale : -CUDART_INF_F;
      float bm = fmaxf(s0, s1);
      bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
      bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 8));
      bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 16));
      // The reference point of a column's exponentials only moves when the block's maximum exceeds it by more
      // than 8 (weights then stay below e^8, well inside FP16): with eight columns and slices of a few blocks a
      // plain running maximum would rescale the accumulators on almost every item. A vote first, so that the
      // rescale is a warp-uniform branch and not predicated multiplications on every item.
      if (__any_sync(0xffffffffu, bm > m[x] + 8.0f)) {
        const float corr = bm > m[x] + 8.0f ? __expf(m[x] - bm) : 1.0f;
        l[x] *= corr;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          acc[j][x] *= corr;
          acc[j][2 + x] *= corr;
        }
        m[x] = bm > m[x] + 8.0f ? bm : m[x];
      }
      // a column that is not live gets weight 0 (its maximum may still be -inf)
      const __half2 pp = live ? __floats2half2_rn(__expf(s0 - m[x]), __expf(s1 - m[x])) : __floats2half2_rn(0.0f, 0.0f);
      float ps = __low2float(pp) + __high2float(pp);
      ps += __shfl_xor_sync(0xffffffffu, ps, 4);
      ps += __shfl_xor_sync(0xffffffffu, ps, 8);
      ps += __shfl_xor_sync(0xffffffffu, ps, 16);
      l[x] += ps;
      ppu[x] = h2_as_u32(pp);
    }
    // B of the second product: this lane needs positions 2c, 2c+1, 2c+8, 2c+9 of sequence g; the lanes
    // (2c, g / 2) and (2c + 1, g / 2) hold them in their column g % 2
    const int src = 8 * c + (g >> 1);
    const uint32_t u0 = __shfl_sync(0xffffffffu, ppu[0], src), u1 = __shfl_sync(0xffffffffu, ppu[1], src);
    const uint32_t v0 = __shfl_sync(0xffffffffu, ppu[0], src + 4), v1 = __shfl_sync(0xffffffffu, ppu[1], src + 4);
    const uint32_t pu = (g & 1) ? u1 : u0, pv = (g & 1) ? v1 : v0;
    pb0 = __byte_perm(pu, pv, 0x5410);
    pb1 = __byte_perm(pu, pv, 0x7632);
    }

    // ---------------- V^T fragments: element e of rows (2c, 2c+1) and of rows (2c+8, 2c+9) ----------------
    uint32_t v12[EV], v34[EV];
    if constexpr (FMT == ATTN_FP16) {
#pragma unroll
      for (int e = 0; e < EV; e += 2) {
        const uint4& r0 = cur.v[0][e / 8];
        const uint4& r1 = cur.v[1][e / 8];
        const uint4& r2 = cur.v[2][e / 8];
        const uint4& r3 = cur.v[3][e / 8];
        const int w = (e / 2) & 3;
        const uint32_t x0 = w == 0 ? r0.x : (w == 1 ? r0.y : (w == 2 ? r0.z : r0.w));
        const uint32_t x1 = w == 0 ? r1.x : (w == 1 ? r1.y : (w == 2 ? r1.z : r1.w));
        const uint32_t x2 = w == 0 ? r2.x : (w == 1 ? r2.y : (w == 2 ? r2.z : r2.w));
        const uint32_t x3 = w == 0 ? r3.x : (w == 1 ? r3.y : (w == 2 ? r3.z : r3.w));
        v12[e] = __byte_perm(x0, x1, 0x5410);
        v12[e + 1] = __byte_perm(x0, x1, 0x7632);
        v34[e] = __byte_perm(x2, x3, 0x5410);
        v34[e + 1] = __byte_perm(x2, x3, 0x7632);
      }
    } else if constexpr (FMT == ATTN_F8) {
      const __half2 s12 = __halves2half2(cur.vs[0], cur.vs[1]), s34 = __halves2half2(cur.vs[2], cur.vs[3]);
#pragma unroll
      for (int e = 0; e < EV; ++e) {
        const int w = e >> 2, b = e & 3;
        // byte b of the first row to byte 1, byte b of the second row to byte 3
        const uint32_t sel = b == 0 ? 0x4000u : (b == 1 ? 0x5010u : (b == 2 ? 0x6020u : 0x7030u));
        v12[e] = h2_as_u32(dq_f8_pair(__byte_perm(cur.v[0][w], cur.v[1][w], sel), s12));
        v34[e] = h2_as_u32(dq_f8_pair(__byte_perm(cur.v[2][w], cur.v[3][w], sel), s34));
      }
    } else if constexpr (FOLD) {
      // B of this product: column g = p times the scale of group g (nothing for g >= G). The zero points ride a
      // second A operand: rows d hold the zero point of their own group at each position (as the codes are held),
      // so that column's sum is the exact counterpart of the code sums - same B, same products.
      {
        const bool live = g < hb.G;
        __half2 s01 = __halves2half2(cur.vs[0], cur.vs[1]), s23 = __halves2half2(cur.vs[2], cur.vs[3]);
        if (!live) s01 = s23 = u32_as_h2(0u);
        pb0 = h2_as_u32(__hmul2_rn(u32_as_h2(pb0), s01));
        pb1 = h2_as_u32(__hmul2_rn(u32_as_h2(pb1), s23));
        const uint32_t za = cur.vz[0] | (cur.vz[1] << 16), zb = cur.vz[2] | (cur.vz[3] << 16);  // z * 2^-24
        const uint32_t zf[4] = {za, za, zb, zb};
        mma_16816(c1, zf, pb0, pb1);
      }
#pragma unroll
      for (int w = 0; w < EV / 8; ++w) {
        uint32_t lo[4], hi[4];
        w4_raw_codes(__byte_perm(cur.v[0][w], cur.v[1][w], 0x5410), kc, lo);  // codes 0..3 of both rows
        w4_raw_codes(__byte_perm(cur.v[0][w], cur.v[1][w], 0x7632), kc, hi);  // codes 4..7
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v12[8 * w + i] = lo[i];
          v12[8 * w + 4 + i] = hi[i];
        }
        w4_raw_codes(__byte_perm(cur.v[2][w], cur.v[3][w], 0x5410), kc, lo);
        w4_raw_codes(__byte_perm(cur.v[2][w], cur.v[3][w], 0x7632), kc, hi);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v34[8 * w + i] = lo[i];
          v34[8 * w + 4 + i] = hi[i];
        }
      }
      if (HOOK && p.v_out) {  // the exact values, for the stores only
        const W4Group g12 = w4_group2(cur.vs_own[0], cur.vz[0], cur.vs_own[HOOK ? 1 : 0], cur.vz[1]);
        const W4Group g34 = w4_group2(cur.vs_own[HOOK ? 2 : 0], cur.vz[2], cur.vs_own[HOOK ? 3 : 0], cur.vz[3]);
        uint32_t e12[EV], e34[EV];
#pragma unroll
        for (int w = 0; w < EV / 8; ++w) {
          __half2 lo[4], hi[4];
          dq_w4_word(__byte_perm(cur.v[0][w], cur.v[1][w], 0x5410), g12, kc, lo);
          dq_w4_word(__byte_perm(cur.v[0][w], cur.v[1][w], 0x7632), g12, kc, hi);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            e12[8 * w + i] = h2_as_u32(lo[i]);
            e12[8 * w + 4 + i] = h2_as_u32(hi[i]);
          }
          dq_w4_word(__byte_perm(cur.v[2][w], cur.v[3][w], 0x5410), g34, kc, lo);
          dq_w4_word(__byte_perm(cur.v[2][w], cur.v[3][w], 0x7632), g34, kc, hi);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            e34[8 * w + i] = h2_as_u32(lo[i]);
            e34[8 * w + 4 + i] = h2_as_u32(hi[i]);
          }
        }
        store_v_rows(e12, e34);
      }
    } else {
      const W4Group g12 = w4_group2(cur.vs[0], cur.vz[0], cur.vs[1], cur.vz[1]);
      const W4Group g34 = w4_group2(cur.vs[2], cur.vz[2], cur.vs[3], cur.vz[3]);
#pragma unroll
      for (int w = 0; w < EV / 8; ++w) {
        __half2 lo[4], hi[4];
        dq_w4_word(__byte_perm(cur.v[0][w], cur.v[1][w], 0x5410), g12, kc, lo);
        dq_w4_word(__byte_perm(cur.v[0][w], cur.v[1][w], 0x7632), g12, kc, hi);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v12[8 * w + i] = h2_as_u32(lo[i]);
          v12[8 * w + 4 + i] = h2_as_u32(hi[i]);
        }
        dq_w4_word(__byte_perm(cur.v[2][w], cur.v[3][w], 0x5410), g34, kc, lo);
        dq_w4_word(__byte_perm(cur.v[2][w], cur.v[3][w], 0x7632), g34, kc, hi);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v34[8 * w + i] = h2_as_u32(lo[i]);
          v34[8 * w + 4 + i] = h2_as_u32(hi[i]);
        }
      }
    }
    if (HOOK && p.v_out && FMT != ATTN_FP16 && !FOLD) store_v_rows(v12, v34);
    // out^T tile j: row g <-> d = EV*g + j, row g + 8 <-> d = EV*g + NT + j
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const uint32_t f[4] = {v12[j], v12[j + NT], v34[j], v34[j + NT]};
      mma_16816(acc[j], f, pb0, pb1);
    }
  };

  // Two buffers in turn: the next block's loads fly while this one is computed.
  const int step = MA_WARPS * MA_BLOCK;
  int tb = t0 + wid * MA_BLOCK;
  if constexpr (ASYNC && !MULTI) {
    // blocks tb, tb + step, ... of this warp; DEPTH - 1 of them in flight ahead of the one being computed
    Blk blk;
    int ti = tb, slot = 0;
#pragma unroll
    for (int k = 0; k < Ring::DEPTH - 1; ++k) {
      if (ti < t1) {
        issue(k, ti, 0);
        ti += step;
      } else {
        empty_group();
      }
    }
    while (tb < t1) {
      const int ahead = slot == 0 ? Ring::DEPTH - 1 : slot - 1;  // the stage freed by the previous block
      if (ti < t1) {
        issue(ahead, ti, 0);
        ti += step;
      } else {
        empty_group();
      }
      wait_oldest();
      collect(blk, slot);
      compute(blk, tb, -1);
      tb += step;
      slot = slot == Ring::DEPTH - 1 ? 0 : slot + 1;
    }
  } else if constexpr (!MULTI) {
    Blk bufa, bufb;
    if (tb < t1) fetch(bufa, tb, 0);
    while (tb < t1) {
      if (tb + step < t1) fetch(bufb, tb + step, 0);
      compute(bufa, tb, -1);
      tb += step;
      if (tb >= t1) break;
      if (tb + step < t1) fetch(bufa, tb + step, 0);
      compute(bufb, tb, -1);
      tb += step;
    }
  } else {
    // Items: a block whose page is common to the live sequences is one item for all columns (ucol = -1);
    // otherwise one item per live sequence. Lane j keeps the page of sequence j for the block at hand.
    int pages = 0;
    auto classify = [&](int t) -> int {  // loads the block's pages; returns the first item's column
      pages = __ldg(bt + (size_t)min(lane, count - 1) * p.bt_stride + (t >> p.pshift));
      const int first = __shfl_sync(0xffffffffu, pages, firstcol);  // (every lane takes part in the shuffle)
      const bool same = !((colmask >> lane) & 1u) || pages == first;
      return __all_sync(0xffffffffu, same) ? -1 : firstcol;
    };
    // the item after (t, u): false when the slice is done
    auto advance = [&](int& t, int& u) -> bool {
      if (u >= 0) {
        const uint32_t rest = colmask >> (u + 1);
        if (rest) {
          u += __ffs(rest);
          return true;
        }
      }
      t += step;
      if (t >= t1) return false;
      u = classify(t);
      return true;
    };
    auto page_of = [&](int u) { return __shfl_sync(0xffffffffu, pages, u < 0 ? firstcol : u); };
    if constexpr (ASYNC) {
      // the item cursor (ti, ui) runs DEPTH - 1 items ahead of the item being computed
      static_assert(Ring::DEPTH == 3, "two items in flight");
      Blk blk;
      int ti = tb, ui = 0, slot = 0;
      bool more = tb < t1;
      int t0q = 0, u0q = 0, t1q = 0, u1q = 0;  // the items in stages slot and slot + 1
      bool have0 = false, have1 = false;
      if (more) {
        ui = classify(ti);
        issue(0, ti, page_of(ui));
        t0q = ti, u0q = ui, have0 = true;
        more = advance(ti, ui);
      } else {
        empty_group();
      }
      if (more) {
        issue(1, ti, page_of(ui));
        t1q = ti, u1q = ui, have1 = true;
        more = advance(ti, ui);
      } else {
        empty_group();
      }
      while (have0) {
        const int ahead = slot == 0 ? 2 : slot - 1;
        int t2q = 0, u2q = 0;
        const bool have2 = more;
        if (more) {
          issue(ahead, ti, page_of(ui));
          t2q = ti, u2q = ui;
          more = advance(ti, ui);
        } else {
          empty_group();
        }
        wait_oldest();
        collect(blk, slot);
        compute(blk, t0q, u0q);
        t0q = t1q, u0q = u1q, have0 = have1;
        t1q = t2q, u1q = u2q, have1 = have2;
        slot = slot == 2 ? 0 : slot + 1;
      }
    } else {
    Blk bufa, bufb;
    int ucur = 0;
    bool have = tb < t1;
    if (have) {
      ucur = classify(tb);
      fetch(bufa, tb, page_of(ucur));
    }
    while (have) {
      int tn = tb, un = ucur;
      have = advance(tn, un);
      if (have) fetch(bufb, tn, page_of(un));
      compute(bufa, tb, ucur);
      if (!have) break;
      tb = tn, ucur = un;
      have = advance(tn, un);
      if (have) fetch(bufa, tn, page_of(un));
      compute(bufb, tb, ucur);
      tb = tn, ucur = un;
    }
    }
  }
  if constexpr (ASYNC) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // every warp is done with its ring: the merge buffer lives there
  }

  // ---- warps of the CTA, merged in warp order (single form: every column of acc holds the same value) ----
  if (pass > 0) __syncthreads();  // the previous pass's readers are done
  if constexpr (!MULTI) {
    if (lane == 0) {
      sm_ml[wid][0][0] = m[0];
      sm_ml[wid][0][1] = l[0];
    }
    if constexpr (FOLD) {
      // rows g and g + 8 of every tile belong to group nv: their sums sit in column nv (lane nv / 2, element
      // nv % 2); tiles with odd j were fed the nibbles that carry a factor 16
      const int nv = (EV * g) >> p.gshift;
      if (c == (nv >> 1)) {
        const bool odd = (nv & 1) != 0;
        const float zt = odd ? c1[1] : c1[0];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const float fj = (j & 1) ? 0.0625f : 1.0f;
          sm_acc[wid][0][EV * g + j] = 16777216.0f * ((odd ? acc[j][1] : acc[j][0]) * fj - zt);
          sm_acc[wid][0][EV * g + NT + j] = 16777216.0f * ((odd ? acc[j][3] : acc[j][2]) * fj - zt);
        }
      }
    } else if (c == 0) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        sm_acc[wid][0][EV * g + j] = acc[j][0];
        sm_acc[wid][0][EV * g + NT + j] = acc[j][2];
      }
    }
  } else {
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      if (g == 0) {
        sm_ml[wid][2 * c + x][0] = m[x];
        sm_ml[wid][2 * c + x][1] = l[x];
      }
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        sm_acc[wid][2 * c + x][EV * g + j] = acc[j][x];
        sm_acc[wid][2 * c + x][EV * g + NT + j] = acc[j][2 + x];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < COLS * D; idx += MA_THREADS) {
    const int col = idx / D, d = idx - col * D;
    if (MULTI && !((colmask >> col) & 1u)) continue;
    float mm = sm_ml[0][col][0], ll = sm_ml[0][col][1], a = sm_acc[0][col][d];
#pragma unroll
    for (int w = 1; w < MA_WARPS; ++w) {
      const float m2 = sm_ml[w][col][0], l2 = sm_ml[w][col][1], a2 = sm_acc[w][col][d];
      const float mn = fmaxf(mm, m2);
      const float fa = (mm == -CUDART_INF_F) ? 0.0f : __expf(mm - mn);
      const float fb = (m2 == -CUDART_INF_F) ? 0.0f : __expf(m2 - mn);
      ll = ll * fa + l2 * fb;
      a = a * fa + a2 * fb;
      mm = mn;
    }
    const size_t row = (size_t)hx + (size_t)col * p.H;  // (col is 0 in the single form)
    if (splits == 1) {
      p.out[row * D + d] = __float2half_rn(a / ll);
    } else {
      float* part = p.ws + (row * (p.nseq ? p.splits : splits) + sp) * (size_t)(D + 2);
      if (d == 0) {
        part[0] = mm;
        part[1] = ll;
      }
      part[2 + d] = a;
    }
  }
  if (ASYNC && MULTI) __syncthreads();  // the next pass's ring reuses the merge buffer
  }  // pass
}

// The lane-private ring needs scale rows of at least four bytes at four-byte boundaries.
static bool ring_ok(const MmaParams& p) {
  const AttnSource& s = p.src;
  if (s.G != 2 && s.G != 4) return false;
  const uintptr_t need = s.G == 4 ? 7u : 3u;
  return ((((uintptr_t)s.s_k | (uintptr_t)s.s_v) & need) == 0);
}

// (one instantiation per kernel: the shared-memory opt-in is a per-device attribute of the function, set once)
template <int FMT, int D, bool MULTI>
cudaError_t launch_ring(dim3 grid, size_t smem, const MmaParams& p, cudaStream_t stream) {
  auto kern = attn_mma_kernel<FMT, D, false, MULTI, true>;
  static std::atomic<bool> configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev].load(std::memory_order_acquire)) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return e;
    configured[dev].store(true, std::memory_order_release);
  }
  kern<<<grid, MA_THREADS, smem, stream>>>(p);
  return cudaGetLastError();
}

template <int FMT, int D>
cudaError_t launch_d(const MmaParams& p, cudaStream_t stream) {
  const dim3 grid((unsigned)(p.nseq ? p.nseq * p.H : p.H), (unsigned)p.splits);
  if constexpr (FMT == ATTN_W4_SYM || FMT == ATTN_W4_ASYM) {
    using Ring = W4Ring<D, FMT == ATTN_W4_ASYM>;
    const bool ring = ring_ok(p) && !(p.k_out || p.v_out);
    const size_t ring_bytes = (size_t)MA_WARPS * Ring::DEPTH * Ring::STAGE;
    if (p.nseq > 1 && p.pshift >= 0) {  // sequences of one pool, eight to a CTA: shared pages are decoded once
      const dim3 ggrid((unsigned)(((p.nseq + 7) / 8) * p.H), (unsigned)p.splits);
      if (ring) {
        const size_t merge_bytes = (size_t)MA_WARPS * 8 * D * sizeof(float);
        return launch_ring<FMT, D, true>(ggrid, ring_bytes > merge_bytes ? ring_bytes : merge_bytes, p, stream);
      }
      attn_mma_kernel<FMT, D, false, true, false><<<ggrid, MA_THREADS, 0, stream>>>(p);
      return cudaGetLastError();
    }
    // single sequence: measured faster with the ring only where zero-point rows add to the loads (asymmetric:
    // 148 -> 135 us at B*H = 256, S = 8192); symmetric caches keep the register prefetch (100 vs 112 us)
    if (ring && FMT == ATTN_W4_ASYM) return launch_ring<FMT, D, false>(grid, ring_bytes, p, stream);
  }
  if (p.k_out || p.v_out)
    attn_mma_kernel<FMT, D, true, false, false><<<grid, MA_THREADS, 0, stream>>>(p);
  else
    attn_mma_kernel<FMT, D, false, false, false><<<grid, MA_THREADS, 0, stream>>>(p);
  return cudaGetLastError();
}

template <int FMT>
cudaError_t launch_fmt(const MmaParams& p, int D, cudaStream_t stream) {
  return D == 128 ? launch_d<FMT, 128>(p, stream) : launch_d<FMT, 64>(p, stream);
}

}  // namespace

bool attn_mma_supported(const AttnSource& src, int D, const void* q, const void* k_out, const void* v_out) {
  if (D != 64 && D != 128) return false;
  if (src.fmt != ATTN_FP16) {
    if (src.gs != 32 && src.gs != 64 && src.gs != 128) return false;
    if (src.gs > D || src.G * src.gs != D) return false;
  }
  if (((uintptr_t)src.k | (uintptr_t)src.v | (uintptr_t)q) & 15u) return false;
  (void)k_out;
  (void)v_out;
  return true;
}

// One pass over the cache: partial (m, l, acc) per (head, split) into ws, or the output itself
// when splits == 1. The caller runs the split combine.
static int page_shift(const AttnSource& src) {
  if (!src.bt) return -1;
  for (int b = 4; b < 31; ++b)
    if (src.page == (1 << b)) return b;
  return -1;
}

static cudaError_t launch_any(MmaParams& p, int D, cudaStream_t stream) {
  const AttnSource& src = p.src;
  p.gshift = src.gs == 128 ? 7 : (src.gs == 64 ? 6 : 5);
  p.wide = ((((uintptr_t)p.k_out | (uintptr_t)p.v_out) & 15u) == 0) ? 1 : 0;
  p.pshift = page_shift(src);
  switch (src.fmt) {
    case ATTN_FP16: return launch_fmt<ATTN_FP16>(p, D, stream);
    case ATTN_W4_SYM: return launch_fmt<ATTN_W4_SYM>(p, D, stream);
    case ATTN_W4_ASYM: return launch_fmt<ATTN_W4_ASYM>(p, D, stream);
    default: return launch_fmt<ATTN_F8>(p, D, stream);
  }
}

cudaError_t attn_mma_launch(const AttnSource& src, const __half* q, __half* out, int H, int S, int D, int splits,
                            float* ws, __half* k_out, __half* v_out, cudaStream_t stream) {
  MmaParams p;
  p.src = src;
  p.q = q;
  p.out = out;
  p.ws = ws;
  p.k_out = k_out;
  p.v_out = v_out;
  p.H = H;
  p.S = S;
  p.splits = splits;
  p.nseq = 0;
  p.seq_lens = nullptr;
  p.bt_stride = 0;
  p.sm_count = 0;
  return launch_any(p, D, stream);
}

// The batched paged form: grid.x = nseq * H rows of q / out, grid.y = the longest sequence's slice count.
cudaError_t attn_mma_batched_launch(const AttnSource& src, const __half* q, __half* out, int H, int D, int nseq,
                                    const int* seq_lens, int bt_stride, int max_splits, int sm_count, float* ws,
                                    cudaStream_t stream) {
  MmaParams p;
  p.src = src;
  p.q = q;
  p.out = out;
  p.ws = ws;
  p.k_out = nullptr;
  p.v_out = nullptr;
  p.H = H;
  p.S = 0;
  p.splits = max_splits;
  p.nseq = nseq;
  p.seq_lens = seq_lens;
  p.bt_stride = bt_stride;
  p.sm_count = sm_count;
  return launch_any(p, D, stream);
}

}  // namespace w4b
