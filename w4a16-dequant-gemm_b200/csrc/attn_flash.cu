// Split-S ("flash-decoding") decode attention, one query token per head, over
// FP16, W4, FP8-E4M3 and paged-W4 KV caches with dequantisation at load; the
// replacement of the reference's flash_*_phase1 / flash_phase2 kernels
// (include/w4/kvflash.cuh:73-199,202-288,294-348,459-570,598-723) and, through
// the same code, of its single-block kernels (include/w4/kvattention.cuh:113-224).
//
// grid = (heads, splits). A CTA walks a contiguous slice of one head's positions
// exactly once: K and V of a position are read together, scores go through an
// online softmax (running max m, running sum l, running sum_t p_t v_t), so no
// per-position state is kept and S is unbounded. A position is served by
// LPP = 2^ceil(log2(words(D))) lanes (8 elements each), so a warp covers 32/LPP
// positions per step. Sub-groups, warps and finally splits are merged with the
// usual (m, l, acc) rescaling in a FIXED order; with a paged cache only the
// row address changes. Paged and contiguous calls over the same logical cache
// therefore produce identical bits, and every call is reproducible.
#include <math_constants.h>

#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {
namespace {

constexpr int FA_WARPS = 4;
constexpr int FA_THREADS = 32 * FA_WARPS;
constexpr int FA_MIN_SPLIT = 64;  // positions; shorter slices are not worth a CTA

struct FlashParams {
  AttnSource src;
  const __half* q;
  __half* out;
  float* ws;
  __half* k_out;
  __half* v_out;
  int H, S, D, splits;
  int wd;   // 8-element granules per row
  int lpp;  // lanes per position (power of two, <= 32)
};

struct Online {
  float m, l;
};

__device__ __forceinline__ long long row_of(const AttnSource& s, int h, int t) {
  const long long r = s.bt ? (long long)s.bt[t / s.page] * s.page + (t % s.page) : (long long)t;
  return (long long)h * s.slab_rows + r;
}

// Eight consecutive elements [8j, 8j+8) of one cache row as floats (natural order).
// `hook`, when non-null, receives the FP16 values (elements past D are skipped).
template <int FMT>
__device__ __forceinline__ void load_granule(const AttnSource& s, bool vside, long long row, int j, int D,
                                             float out[8], __half* hook) {
  __half h8[8];
  const int d0 = 8 * j;
  if (FMT == ATTN_FP16) {
    const __half* base = (const __half*)(vside ? s.v : s.k) + row * D + d0;
    if ((D & 7) == 0 && (((uintptr_t)base) & 15u) == 0) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(base));
      *reinterpret_cast<uint4*>(h8) = v;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) h8[e] = d0 + e < D ? base[e] : __ushort_as_half((unsigned short)0);
    }
  } else if (FMT == ATTN_F8) {
    const uint8_t* base = (const uint8_t*)(vside ? s.v : s.k) + row * D + d0;  // 4-byte aligned: D % 4 == 0
    const __half sc = (vside ? s.s_v : s.s_k)[row * s.G + d0 / s.gs];
    const uint32_t w0 = __ldg(reinterpret_cast<const uint32_t*>(base));
    const uint32_t w1 = d0 + 4 < D ? __ldg(reinterpret_cast<const uint32_t*>(base) + 1) : 0u;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      h8[e] = dq_f8_scalar(sc, (w0 >> (8 * e)) & 0xFFu);
      h8[e + 4] = dq_f8_scalar(sc, (w1 >> (8 * e)) & 0xFFu);
    }
  } else {
    const int wdw = words(D);
    const uint32_t qw = __ldg((const uint32_t*)(vside ? s.v : s.k) + row * wdw + j);
    const int grp = d0 / s.gs;
    const __half sc = (vside ? s.s_v : s.s_k)[row * s.G + grp];
    uint32_t z = 8u;
    if (FMT == ATTN_W4_ASYM)
      z = ((vside ? s.z_v : s.z_k)[row * words(s.G) + (grp >> 3)] >> (4 * (grp & 7))) & 0xFu;
    __half2 o[4];
    dq_w4_word(qw, w4_group(sc, z), o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      h8[i] = __low2half(o[i]);
      h8[i + 4] = __high2half(o[i]);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) out[e] = __half2float(h8[e]);
  if (hook) {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (d0 + e < D) hook[d0 + e] = h8[e];
  }
}

// (m, l, acc) <- merge((m, l, acc), (m2, l2, acc2)); an empty side has m = -inf, l = 0.
template <int N>
__device__ __forceinline__ void merge_state(float& m, float& l, float acc[N], float m2, float l2,
                                            const float acc2[N]) {
  const float mn = fmaxf(m, m2);
  const float a = (m == -CUDART_INF_F) ? 0.0f : __expf(m - mn);
  const float b = (m2 == -CUDART_INF_F) ? 0.0f : __expf(m2 - mn);
  l = l * a + l2 * b;
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = acc[i] * a + acc2[i] * b;
  m = mn;
}

template <int FMT, int GPL, bool HOOK>
__global__ void __launch_bounds__(FA_THREADS) flash_decode_kernel(const FlashParams p) {
  __shared__ float sm_ml[FA_WARPS][2];
  __shared__ float sm_acc[FA_WARPS][512];
  const int h = blockIdx.x, sp = blockIdx.y;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int D = p.D, lpp = p.lpp, ppw = 32 / lpp;
  const int sub = lane / lpp, li = lane % lpp;
  const int t0 = (int)((long long)p.S * sp / p.splits), t1 = (int)((long long)p.S * (sp + 1) / p.splits);
  const float inv_sqrt_d = rsqrtf((float)D);

  float qf[GPL][8];
  bool have[GPL];
#pragma unroll
  for (int gi = 0; gi < GPL; ++gi) {
    const int j = li + lpp * gi;
    have[gi] = j < p.wd;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int d = 8 * j + e;
      qf[gi][e] = (have[gi] && d < D) ? __half2float(p.q[(size_t)h * D + d]) : 0.0f;
    }
  }

  float m = -CUDART_INF_F, l = 0.0f;
  float acc[GPL * 8];
#pragma unroll
  for (int i = 0; i < GPL * 8; ++i) acc[i] = 0.0f;

  for (int base = t0 + wid * ppw; base < t1; base += FA_WARPS * ppw) {
    const int t = base + sub;
    const bool active = t < t1;
    long long row = 0;
    if (active) row = row_of(p.src, h, t);
    float dot = 0.0f;
    if (active) {
#pragma unroll
      for (int gi = 0; gi < GPL; ++gi) {
        if (!have[gi]) continue;
        float kf[8];
        load_granule<FMT>(p.src, false, row, li + lpp * gi, D, kf,
                          HOOK && p.k_out ? p.k_out + ((size_t)h * p.S + t) * D : nullptr);
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(qf[gi][e], kf[e], dot);
      }
    }
    for (int off = lpp >> 1; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    if (active) {
      const float s = dot * inv_sqrt_d;
      const float mn = fmaxf(m, s);
      const float corr = __expf(m - mn);  // m = -inf on the first position: exp(-inf) = 0
      const float pw = __expf(s - mn);
      l = l * corr + pw;
      m = mn;
#pragma unroll
      for (int gi = 0; gi < GPL; ++gi) {
        if (!have[gi]) continue;
        float vf[8];
        load_granule<FMT>(p.src, true, row, li + lpp * gi, D, vf,
                          HOOK && p.v_out ? p.v_out + ((size_t)h * p.S + t) * D : nullptr);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[gi * 8 + e] = fmaf(pw, vf[e], acc[gi * 8 + e] * corr);
      }
    }
  }

  // sub-groups of a warp: lane and lane ^ off hold the same granules of different positions
  for (int off = lpp; off < 32; off <<= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, off);
    const float l2 = __shfl_xor_sync(0xffffffffu, l, off);
    float a2[GPL * 8];
#pragma unroll
    for (int i = 0; i < GPL * 8; ++i) a2[i] = __shfl_xor_sync(0xffffffffu, acc[i], off);
    // both partners must apply the merge in the same operand order to agree bit for bit
    if ((lane & off) == 0) {
      merge_state<GPL * 8>(m, l, acc, m2, l2, a2);
    } else {
      float mm = m2, ll = l2;
      merge_state<GPL * 8>(mm, ll, a2, m, l, acc);
      m = mm;
      l = ll;
#pragma unroll
      for (int i = 0; i < GPL * 8; ++i) acc[i] = a2[i];
    }
  }

  // warps of the CTA, merged by warp 0 in warp order
  if (lane < lpp) {
    if (lane == 0) {
      sm_ml[wid][0] = m;
      sm_ml[wid][1] = l;
    }
#pragma unroll
    for (int gi = 0; gi < GPL; ++gi)
      if (have[gi])
#pragma unroll
        for (int e = 0; e < 8; ++e) sm_acc[wid][8 * (li + lpp * gi) + e] = acc[gi * 8 + e];
  }
  __syncthreads();
  if (wid != 0 || lane >= lpp) return;
  for (int w = 1; w < FA_WARPS; ++w) {
    float a2[GPL * 8];
#pragma unroll
    for (int gi = 0; gi < GPL; ++gi)
#pragma unroll
      for (int e = 0; e < 8; ++e) a2[gi * 8 + e] = have[gi] ? sm_acc[w][8 * (li + lpp * gi) + e] : 0.0f;
    merge_state<GPL * 8>(m, l, acc, sm_ml[w][0], sm_ml[w][1], a2);
  }
  if (p.splits == 1) {
    const float inv = 1.0f / l;
#pragma unroll
    for (int gi = 0; gi < GPL; ++gi)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int d = 8 * (li + lpp * gi) + e;
        if (have[gi] && d < D) p.out[(size_t)h * D + d] = __float2half_rn(acc[gi * 8 + e] * inv);
      }
  } else {
    float* part = p.ws + ((size_t)h * p.splits + sp) * (size_t)(D + 2);
    if (lane == 0) {
      part[0] = m;
      part[1] = l;
    }
#pragma unroll
    for (int gi = 0; gi < GPL; ++gi)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int d = 8 * (li + lpp * gi) + e;
        if (have[gi] && d < D) part[2 + d] = acc[gi * 8 + e];
      }
  }
}

// Per head: rescale and add the split partials in split order. Batched form (seq_lens != null): row h of the
// output belongs to sequence h / H, whose slice count follows from its own length; the workspace keeps
// `splits` (the longest sequence's count) slots per row.
constexpr int FC_MAX = 1024;  // splits whose maxima / denominators fit the shared-memory table

__global__ void flash_combine_kernel(const float* __restrict__ ws, __half* __restrict__ out, int splits, int D,
                                     const int* __restrict__ seq_lens, int H, int sm_count) {
  __shared__ float sm_w[FC_MAX], sm_l[FC_MAX];
  __shared__ float sm_max[4];
  const int h = blockIdx.x;
  const float* hb = ws + (size_t)h * splits * (size_t)(D + 2);
  if (seq_lens) splits = attn_flash_splits(attn_batched_rows((int)gridDim.x / H, H), __ldg(seq_lens + h / H), sm_count);
  if (splits == 1 && seq_lens) return;  // the slice pass wrote the output itself
  const size_t pitch = (size_t)(D + 2);
  float mx = -CUDART_INF_F, den = 0.0f;
  if (splits <= FC_MAX) {
    // The slices' maxima and denominators come in with all loads in flight at once (a thread per slice), and
    // the sums over the slices keep eight loads ahead: walked one dependent load after the other, three passes
    // over the slices cost this kernel 10 us beside a slice pass of 55 us. The order of every sum is unchanged.
    float lm = -CUDART_INF_F;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
      const float m = hb[(size_t)s * pitch];
      sm_w[s] = m;
      sm_l[s] = hb[(size_t)s * pitch + 1];
      lm = fmaxf(lm, m);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) lm = fmaxf(lm, __shfl_xor_sync(0xffffffffu, lm, d));
    if ((threadIdx.x & 31) == 0) sm_max[threadIdx.x >> 5] = lm;
    __syncthreads();
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, sm_max[w]);
    for (int s = threadIdx.x; s < splits; s += blockDim.x) sm_w[s] = __expf(sm_w[s] - mx);
    __syncthreads();
    for (int s = 0; s < splits; ++s) den += sm_w[s] * sm_l[s];
    const float inv = 1.0f / den;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float a = 0.0f;
      const float* col = hb + 2 + d;
      int s = 0;
      for (; s + 8 <= splits; s += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = col[(size_t)(s + u) * pitch];
#pragma unroll
        for (int u = 0; u < 8; ++u) a += sm_w[s + u] * v[u];
      }
      for (; s < splits; ++s) a += sm_w[s] * col[(size_t)s * pitch];
      out[(size_t)h * D + d] = __float2half_rn(a * inv);
    }
    return;
  }
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, hb[(size_t)s * (D + 2)]);
  for (int s = 0; s < splits; ++s) den += __expf(hb[(size_t)s * (D + 2)] - mx) * hb[(size_t)s * (D + 2) + 1];
  const float inv = 1.0f / den;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.0f;
    for (int s = 0; s < splits; ++s) {
      const float* pb = hb + (size_t)s * (D + 2);
      a += __expf(pb[0] - mx) * pb[2 + d];
    }
    out[(size_t)h * D + d] = __float2half_rn(a * inv);
  }
}

template <int FMT>
cudaError_t launch_fmt(const FlashParams& p, cudaStream_t stream) {
  const dim3 grid((unsigned)p.H, (unsigned)p.splits);
  const bool hook = p.k_out || p.v_out;
  const bool two = p.wd > 32;
  if (two) {
    if (hook)
      flash_decode_kernel<FMT, 2, true><<<grid, FA_THREADS, 0, stream>>>(p);
    else
      flash_decode_kernel<FMT, 2, false><<<grid, FA_THREADS, 0, stream>>>(p);
  } else {
    if (hook)
      flash_decode_kernel<FMT, 1, true><<<grid, FA_THREADS, 0, stream>>>(p);
    else
      flash_decode_kernel<FMT, 1, false><<<grid, FA_THREADS, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace

size_t attn_flash_ws_bytes(int H, int D, int splits) {
  return (size_t)H * splits * (size_t)(D + 2) * sizeof(float);
}

cudaError_t attn_flash_launch(const AttnSource& src, const __half* q, __half* out, int H, int S, int D, int splits,
                              float* ws, __half* k_out, __half* v_out, cudaStream_t stream, int* launches) {
  FlashParams p;
  p.src = src;
  p.q = q;
  p.out = out;
  p.ws = ws;
  p.k_out = k_out;
  p.v_out = v_out;
  p.H = H;
  p.S = S;
  p.D = D;
  p.splits = splits;
  p.wd = (D + 7) / 8;
  int lpp = 1;
  while (lpp < p.wd && lpp < 32) lpp <<= 1;
  p.lpp = lpp;
  cudaError_t e;
  if (attn_mma_supported(src, D, q, k_out, v_out)) {
    e = attn_mma_launch(src, q, out, H, S, D, splits, ws, k_out, v_out, stream);
    *launches = 1;
    if (e != cudaSuccess || splits == 1) return e;
    flash_combine_kernel<<<H, 128, 0, stream>>>(ws, out, splits, D, nullptr, 0, 0);
    *launches = 2;
    return cudaGetLastError();
  }
  switch (src.fmt) {
    case ATTN_FP16: e = launch_fmt<ATTN_FP16>(p, stream); break;
    case ATTN_W4_SYM: e = launch_fmt<ATTN_W4_SYM>(p, stream); break;
    case ATTN_W4_ASYM: e = launch_fmt<ATTN_W4_ASYM>(p, stream); break;
    default: e = launch_fmt<ATTN_F8>(p, stream); break;
  }
  *launches = 1;
  if (e != cudaSuccess || splits == 1) return e;
  flash_combine_kernel<<<H, 128, 0, stream>>>(ws, out, splits, D, nullptr, 0, 0);
  *launches = 2;
  return cudaGetLastError();
}

// Batched paged decode attention: nseq sequences over one pool, one slice pass and one combine for all of them.
// A sequence of length S is cut into attn_flash_splits(attn_batched_rows(nseq, H), S, sm_count) slices (a function of
// its own length only, so the result does not depend on which sequences share the call with it); `max_splits` is
// that of the longest sequence and ws holds nseq * H * max_splits partials.
cudaError_t attn_flash_batched_launch(const AttnSource& src, const __half* q, __half* out, int H, int D, int nseq,
                                      const int* seq_lens, int bt_stride, int max_splits, int sm_count, float* ws,
                                      cudaStream_t stream, int* launches) {
  cudaError_t e = attn_mma_batched_launch(src, q, out, H, D, nseq, seq_lens, bt_stride, max_splits, sm_count, ws, stream);
  *launches = 1;
  if (e != cudaSuccess || max_splits == 1) return e;
  flash_combine_kernel<<<nseq * H, 128, 0, stream>>>(ws, out, max_splits, D, seq_lens, H, sm_count);
  *launches = 2;
  return cudaGetLastError();
}

}  // namespace w4b
