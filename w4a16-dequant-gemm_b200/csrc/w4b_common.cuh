// Device-side building blocks shared by every kernel of libw4b200:
//  * the scalar dequantisation steps, written as the formats define them
//    (one exact float product, one round-to-nearest-even conversion to FP16),
//  * register-level decoders that turn one packed 32-bit word (8 codes) into
//    four half2 pairs with the same bits as the scalar steps,
//  * thin wrappers over the sm_100a PTX used for asynchronous data movement
//    (mbarrier, cp.async, cp.async.bulk.tensor) with bounded waits.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "w4b_kernels.h"

namespace w4b {

// Status codes written to the device status word by a kernel that gave up on
// a bounded wait. The kernel then returns early; its output is undefined.
enum : int {
  ST_OK = 0,
  ST_STREAM_FULL_TIMEOUT = 101,   // stream GEMM: a consumer never saw its stage filled
  ST_STREAM_EMPTY_TIMEOUT = 102,  // stream GEMM: the producer never got a stage back
  ST_STREAM_PANEL_TIMEOUT = 103,  // stream GEMM: a panel owner never saw the other CTAs' fragments
  ST_TENSOR_TIMEOUT = 201,        // tensor GEMM: a pipeline wait ran out
  ST_FLASH_TIMEOUT = 301,         // flash decode: a pipeline wait ran out
  ST_PEER_TIMEOUT = 401,          // peer all-gather: a peer's slice never arrived
  ST_QUANT_INVALID = 501,         // device quantizer: a value or scale the host quantizer would have thrown on
};

// --------------------------------------------------------------------------
// Scalar dequantisation: the definitions (bit-identical to the host formats).
// --------------------------------------------------------------------------

// W4: w = rn_f16(float(s) * float(q - z)); the product of an 11-bit and a
// 5-bit significand is exact in float, so there is exactly one rounding.
__device__ __forceinline__ __half dq_w4_scalar(__half s, int q, int z) {
  return __float2half_rn(__half2float(s) * (float)(q - z));
}

// 2^(se-127) as a float, built from bits (se == 0 is the subnormal 2^-127).
__device__ __forceinline__ float e8m0_to_float(uint32_t se) {
  return __uint_as_float(se == 0 ? 0x00400000u : (se << 23));
}

// MXFP4: E2M1 magnitude {0,.5,1,1.5,2,3,4,6}[code&7], sign = code bit 3 applied
// to the magnitude (code 8 is -0), times 2^(se-127); exact in float, one rounding.
__device__ __forceinline__ __half dq_mx_scalar(uint32_t se, int q) {
  const int e = (q >> 1) & 3, m = q & 1;
  const float mag = e == 0 ? 0.5f * (float)m : (float)(2 + m) * (0.25f * (float)(1 << e));
  const float v = (q & 8) ? -mag : mag;
  return __float2half_rn(e8m0_to_float(se) * v);
}

// FP8 E4M3 decode: e == 0 -> m * 2^-9, else (8 + m) * 2^(e - 10); exact.
__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
  const uint32_t e = (b >> 3) & 0xF, m = b & 7;
  const float mag = e == 0 ? (float)m * 0.001953125f : (float)(8 + m) * __uint_as_float((e + 117u) << 23);
  return (b & 0x80) ? -mag : mag;
}

__device__ __forceinline__ __half dq_f8_scalar(__half s, uint32_t b) {
  return __float2half_rn(__half2float(s) * e4m3_to_float(b));
}

// --------------------------------------------------------------------------
// Word decoders. A packed word holds codes n0..n7 for k = 8w .. 8w+7, low
// nibble first. The decoders return four half2 values
//     out[i] = ( w[8w + i] , w[8w + i + 4] ),  i = 0..3
// (the pairing that falls out of masking both 16-bit halves of the word at
// once). Activations are laid out in the same pairing by the kernels.
// --------------------------------------------------------------------------

__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) {
  return *reinterpret_cast<__half2*>(&v);
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) {
  return *reinterpret_cast<uint32_t*>(&v);
}

// Per-(row, group) constants of the W4 decoder.
struct W4Group {
  __half2 s2;  // (s, s)
  __half2 za;  // (1024 + z, 1024 + z)
  __half2 zb;  // (-(64 + z), -(64 + z))
};

__device__ __forceinline__ W4Group w4_group(__half s, uint32_t z) {
  W4Group g;
  g.s2 = __half2half2(s);
  g.za = u32_as_h2(z * 0x00010001u + 0x64006400u);  // 0x6400 | z  == 1024 + z
  g.zb = u32_as_h2(z * 0x00100010u + 0xD400D400u);  // 0xD400 | z<<4 == -(64 + z)
  return g;
}

// (a & b) | c in one LOP3 (the constants are kept in registers by the assembler).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// (code | 0x6400) is the half 1024 + code; (code<<4 | 0x6400) is 1024 + 16*code.
// Subtracting 1024 + z (or fma by 1/16 and adding -(64+z)) gives the integer
// code - z exactly; the half multiply by s then rounds the exact product once,
// which is what dq_w4_scalar does in float. Subnormal results are kept.
// 13 instructions per word: 1 shift, 4 LOP3, 2 HADD2, 2 HFMA2, 4 HMUL2.
//
// The four constants come from `mov` instructions the compiler cannot see
// through: it then keeps them in registers for the whole kernel instead of
// re-creating them next to every use (which costs an instruction per use).
struct W4Consts {
  uint32_t magic, lo, hi;
  __half2 sixteenth;
};

__device__ __forceinline__ W4Consts w4_consts() {
  W4Consts k;
  uint32_t s;
  asm volatile("mov.b32 %0, 0x64006400;" : "=r"(k.magic));
  asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(k.lo));
  asm volatile("mov.b32 %0, 0x00F000F0;" : "=r"(k.hi));
  asm volatile("mov.b32 %0, 0x2C002C00;" : "=r"(s));  // (1/16, 1/16)
  k.sixteenth = u32_as_h2(s);
  return k;
}

__device__ __forceinline__ void dq_w4_word(uint32_t qw, const W4Group& g, const W4Consts& k, __half2 out[4]) {
  const uint32_t hi = qw >> 8;
  const __half2 t0 = u32_as_h2(and_or(qw, k.lo, k.magic));
  const __half2 t1 = u32_as_h2(and_or(qw, k.hi, k.magic));
  const __half2 t2 = u32_as_h2(and_or(hi, k.lo, k.magic));
  const __half2 t3 = u32_as_h2(and_or(hi, k.hi, k.magic));
  out[0] = __hmul2_rn(__hsub2_rn(t0, g.za), g.s2);
  out[1] = __hmul2_rn(__hfma2(t1, k.sixteenth, g.zb), g.s2);
  out[2] = __hmul2_rn(__hsub2_rn(t2, g.za), g.s2);
  out[3] = __hmul2_rn(__hfma2(t3, k.sixteenth, g.zb), g.s2);
}

// The integer part of the W4 decoder: out = (q - z) as exact FP16 integers, in the same pairing.
// za = (1024 + z, 1024 + z), zb = (-(64 + z), -(64 + z)). 9 instructions per word.
__device__ __forceinline__ void dq_w4_int(uint32_t qw, __half2 za, __half2 zb, const W4Consts& k, __half2 out[4]) {
  const uint32_t hi = qw >> 8;
  const __half2 t0 = u32_as_h2(and_or(qw, k.lo, k.magic));
  const __half2 t1 = u32_as_h2(and_or(qw, k.hi, k.magic));
  const __half2 t2 = u32_as_h2(and_or(hi, k.lo, k.magic));
  const __half2 t3 = u32_as_h2(and_or(hi, k.hi, k.magic));
  out[0] = __hsub2_rn(t0, za);
  out[1] = __hfma2(t1, k.sixteenth, zb);
  out[2] = __hsub2_rn(t2, za);
  out[3] = __hfma2(t3, k.sixteenth, zb);
}

// Convenience form for code that decodes a handful of words.
__device__ __forceinline__ void dq_w4_word(uint32_t qw, const W4Group& g, __half2 out[4]) {
  W4Consts k;
  k.magic = 0x64006400u;
  k.lo = 0x000F000Fu;
  k.hi = 0x00F000F0u;
  k.sixteenth = u32_as_h2(0x2C002C00u);
  dq_w4_word(qw, g, k, out);
}

// MXFP4 block multiplier. An E2M1 code placed as sign -> bit 15 and (e1 e0 m)
// -> bits 11..9 is the half value code * 2^-14 (its e == 0 codes land on half
// subnormals). Multiplying by 2^(se - 113) gives code * 2^(se - 127) with one
// rounding. That power of two is a half only for 89 <= se <= 128; `exact` says
// whether the fast form applies, otherwise the scalar definition is used.
struct MxBlock {
  __half2 h2;
  uint32_t se;
  bool fast;
};

__device__ __forceinline__ MxBlock mx_block(uint32_t se) {
  MxBlock b;
  b.se = se;
  b.fast = (se >= 89u) && (se <= 128u);
  // 2^(se-113): normal half for se >= 99 (biased exponent se - 98), subnormal below.
  const uint32_t bits = se >= 99u ? ((se - 98u) << 10) : (1u << ((se - 89u) & 15u));
  b.h2 = u32_as_h2(bits * 0x00010001u);
  return b;
}

// The fast form alone, for callers that have established b.fast (for a whole warp, say).
__device__ __forceinline__ void dq_mx_word_fast(uint32_t qw, const MxBlock& b, __half2 out[4]) {
  const uint32_t kMag = 0x0E000E00u, kSign = 0x80008000u;
  const uint32_t r0 = and_or(qw << 12, kSign, (qw << 9) & kMag);
  const uint32_t r1 = and_or(qw << 8, kSign, (qw << 5) & kMag);
  const uint32_t r2 = and_or(qw << 4, kSign, (qw << 1) & kMag);
  const uint32_t r3 = and_or(qw, kSign, (qw >> 3) & kMag);
  out[0] = __hmul2_rn(u32_as_h2(r0), b.h2);
  out[1] = __hmul2_rn(u32_as_h2(r1), b.h2);
  out[2] = __hmul2_rn(u32_as_h2(r2), b.h2);
  out[3] = __hmul2_rn(u32_as_h2(r3), b.h2);
}

__device__ __forceinline__ void dq_mx_word(uint32_t qw, const MxBlock& b, __half2 out[4]) {
  if (b.fast) {
    dq_mx_word_fast(qw, b, out);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      out[i] = __halves2half2(dq_mx_scalar(b.se, (int)((qw >> (4 * i)) & 0xF)),
                              dq_mx_scalar(b.se, (int)((qw >> (4 * i + 16)) & 0xF)));
  }
}

// --------------------------------------------------------------------------
// Asynchronous data movement (inline PTX, sm_100a).
// --------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy (TMA).
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

// One try_wait: the hardware may park the thread for a short, implementation-defined time
// while the phase is incomplete. (Giving it an explicit suspend-time hint made waiters
// oversleep by microseconds here: the wake-ups then follow a growing sleep interval.)
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking test of a barrier phase.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// About one second at B200 clocks; a wait that long is a lost signal.
constexpr long long kWaitLimitCycles = 2000000000LL;

// Bounded wait: returns false (after recording `code` in *status) instead of
// spinning for ever, so a protocol error ends the kernel rather than the GPU.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitLimitCycles) {
      if (status) atomicExch(status, code);
      return false;
    }
  }
  return true;
}

// 4/8/16-byte asynchronous global->shared copy (non-bulk), tracked by
// cp_async_arrive_noinc on an mbarrier whose expected count includes the
// issuing thread.
template <int BYTES>
__device__ __forceinline__ void cp_async(uint32_t dst, const void* src) {
  static_assert(BYTES == 4 || BYTES == 8 || BYTES == 16, "cp.async size");
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(src), "n"(BYTES)
               : "memory");
}

__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// One 2-D TMA tile load (no multicast) completing on `bar`. x is the inner
// coordinate in elements; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// Untiled bulk copy global -> shared; both addresses and the size 16-byte aligned.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// Programmatic dependent launch. Both are no-ops in a grid that was launched without the
// programmatic-stream-serialization attribute.
//  launch_dependents: the next grid in the stream may be scheduled once every CTA of this grid
//    has executed it (or exited);
//  wait: blocks until the grid this one depends on has completed and its memory is visible.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_16816(float d[4], const uint32_t a[4], uint32_t b0,
                                          uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}

// 16-byte shared load executed only where `on` is set; elsewhere v keeps its value
// and the lane generates no shared-memory traffic.
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ unsigned short lds16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ void lds128_if(uint4& v, uint32_t addr, bool on) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.u32 p, %5, 0;\n"
      "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
      "}\n"
      : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
      : "r"(addr), "r"((uint32_t)on)
      : "memory");
}

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Reorders eight consecutive halves (h0..h7) into the decoder's pairing:
// (h0,h4) (h1,h5) (h2,h6) (h3,h7).
__device__ __forceinline__ uint4 pair_permute(uint4 v) {
  uint4 r;
  r.x = __byte_perm(v.x, v.z, 0x5410);
  r.y = __byte_perm(v.x, v.z, 0x7632);
  r.z = __byte_perm(v.y, v.w, 0x5410);
  r.w = __byte_perm(v.y, v.w, 0x7632);
  return r;
}

}  // namespace w4b
