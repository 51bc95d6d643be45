#pragma once
// Drop-in GPU header: the split-S flash-decode entries of the reference's
// include/w4/kvflash.cuh (FLASH_TILE :35, validate_kv_flash :37-54, attention_w4_flash
// :350-363, attention_fp16_flash :365-384, DeviceKVF8 :390-396, validate_kv_f8 :398-411,
// dequant_f8 :435-457, attention_f8_flash :572-590, attention_w4_flash_paged :725-764)
// over the C ABI of libw4b200. FLASH_TILE keeps its role in the S bound (65535 tiles).
#include "kvattention.cuh"
#include "kvfp8.hpp"

namespace w4::gpu {

constexpr int FLASH_TILE = 256;

inline void validate_kv_flash(const DeviceKVW4& p) {
  if (p.H < 1 || p.S < 1 || p.D < 1) throw std::invalid_argument("kv flash: bad dims");
  if (p.D > KV_MAX_D) throw std::invalid_argument("kv flash: D exceeds the shared-memory bound");
  if (p.gs < 8 || p.gs % 8 != 0) throw std::invalid_argument("kv flash: gs must be a multiple of 8");
  if (p.G != (p.D + p.gs - 1) / p.gs) throw std::invalid_argument("kv flash: G inconsistent with D, gs");
  if (!p.q_k || !p.s_k || !p.q_v || !p.s_v) throw std::invalid_argument("kv flash: null pointer");
  if (!p.symmetric && (!p.z_k || !p.z_v)) throw std::invalid_argument("kv flash: asymmetric without zeros");
  if (p.symmetric && (p.z_k || p.z_v)) throw std::invalid_argument("kv flash: symmetric carries no zeros");
  if (p.S > 65535 * FLASH_TILE) throw std::invalid_argument("kv flash: S exceeds the tile-grid bound");
}

inline void attention_w4_flash(const DeviceKVW4& p, const __half* q, __half* out, cudaStream_t stream = 0,
                               __half* k_out = nullptr, __half* v_out = nullptr) {
  abi_check(w4b_attn_flash_w4(abi(p), q, out, stream, k_out, v_out));
}

inline void attention_fp16_flash(const __half* q, const __half* k16, const __half* v16, __half* out, int H, int S,
                                 int D, cudaStream_t stream = 0) {
  abi_check(w4b_attn_flash_fp16(q, k16, v16, out, H, S, D, stream));
}

struct DeviceKVF8 {
  int H, S, D, gs, G;
  const uint8_t* q_k;
  const __half* s_k;
  const uint8_t* q_v;
  const __half* s_v;
};
static_assert(sizeof(DeviceKVF8) == sizeof(w4b_kv_f8), "descriptor layouts must agree");

inline const w4b_kv_f8* abi(const DeviceKVF8& p) { return reinterpret_cast<const w4b_kv_f8*>(&p); }

inline void validate_kv_f8(const DeviceKVF8& p) {
  if (p.H < 1 || p.S < 1 || p.D < 1) throw std::invalid_argument("kv f8 flash: bad dims");
  if (p.D > KV_MAX_D) throw std::invalid_argument("kv f8 flash: D exceeds the shared bound");
  if (p.gs < 8 || p.gs % 8 != 0) throw std::invalid_argument("kv f8 flash: gs must be a multiple of 8");
  if (p.G != (p.D + p.gs - 1) / p.gs) throw std::invalid_argument("kv f8 flash: G inconsistent with D, gs");
  if (!p.q_k || !p.s_k || !p.q_v || !p.s_v) throw std::invalid_argument("kv f8 flash: null pointer");
  if (p.S > 65535 * FLASH_TILE) throw std::invalid_argument("kv f8 flash: S exceeds the tile-grid bound");
}

inline void dequant_f8(const uint8_t* q, const __half* s, __half* w, int S, int D, int gs, cudaStream_t stream = 0) {
  abi_check(w4b_dequant_f8(q, reinterpret_cast<const uint16_t*>(s), w, S, D, gs, stream));
}

inline void attention_f8_flash(const DeviceKVF8& p, const __half* q, __half* out, cudaStream_t stream = 0,
                               __half* k_out = nullptr, __half* v_out = nullptr) {
  abi_check(w4b_attn_flash_f8(abi(p), q, out, stream, k_out, v_out));
}

inline void attention_w4_flash_paged(const DeviceKVW4& p, const int* bt, int page, int npages, const __half* q,
                                     __half* out, cudaStream_t stream = 0, __half* k_out = nullptr,
                                     __half* v_out = nullptr) {
  abi_check(w4b_attn_flash_w4_paged(abi(p), bt, page, npages, q, out, stream, k_out, v_out));
}

}  // namespace w4::gpu
