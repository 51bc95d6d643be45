#pragma once
// Drop-in host header: the paged W4 KV cache - per head a pool of npages pages of
// `page` positions, a block table mapping logical pages to physical ones - with the
// names and contracts of the reference's include/w4/kvpaged.hpp (KVCacheW4Paged
// :25-34, validate_paged :36-67, paged_from_contiguous :72-134). Paging changes where
// a position lives, never what it contains.
#include <cuda_fp16.h>

#include <stdexcept>
#include <vector>

#include "kvcache.hpp"

namespace w4::kv {

struct KVCacheW4Paged {
  int H = 0, S = 0, D = 0, gs = 0, G = 0;
  int page = 0;    // positions per page
  int npages = 0;  // physical pages in the pool, per head
  bool symmetric = true;
  std::vector<uint32_t> q_k, q_v;  // H slabs of npages*page*words(D)
  std::vector<__half> s_k, s_v;    // H slabs of npages*page*G
  std::vector<uint32_t> z_k, z_v;  // asymmetric only
  std::vector<int> block_table;    // ceil(S/page) entries < npages, no repeats
};

namespace detail {
inline bool table_ok(const std::vector<int>& bt, size_t pool_pages) {
  std::vector<char> seen(pool_pages, 0);
  for (const int b : bt) {
    if (b < 0 || (size_t)b >= pool_pages || seen[(size_t)b]) return false;
    seen[(size_t)b] = 1;
  }
  return true;
}
}  // namespace detail

inline void validate_paged(const KVCacheW4Paged& c) {
  using w4::detail::require;
  require(c.H >= 1 && c.S >= 1 && c.D >= 1, "paged: bad dims");
  require(c.gs >= 8 && c.gs % 8 == 0, "paged: gs must be a multiple of 8");
  require(c.G == (c.D + c.gs - 1) / c.gs, "paged: G inconsistent with D, gs");
  require(c.page >= 1 && c.npages >= 1, "paged: bad page geometry");
  const size_t lpages = ((size_t)c.S + c.page - 1) / c.page;
  require(c.block_table.size() == lpages, "paged: block table size");
  require((size_t)c.npages >= lpages, "paged: pool smaller than table");
  const size_t rows = (size_t)c.H * c.npages * c.page;
  require(c.q_k.size() == rows * words(c.D) && c.q_v.size() == rows * words(c.D), "paged: q size");
  require(c.s_k.size() == rows * c.G && c.s_v.size() == rows * c.G, "paged: scales size");
  if (!c.symmetric)
    require(c.z_k.size() == rows * words(c.G) && c.z_v.size() == rows * words(c.G), "paged: zeros size");
  require(detail::table_ok(c.block_table, (size_t)c.npages), "paged: block table entry out of pool or repeated");
}

// Logical page i of every head lands at physical page bt[i]; the pool has exactly
// bt.size() pages per head; rows past S in the last logical page stay zero.
inline KVCacheW4Paged paged_from_contiguous(const KVCacheW4& c, int page, const std::vector<int>& bt) {
  using w4::detail::require;
  validate_cache(c);
  require(page >= 1, "paged_from: bad page size");
  const size_t lpages = ((size_t)c.S + (size_t)page - 1) / (size_t)page;
  require(bt.size() == lpages, "paged_from: block table size");
  require(detail::table_ok(bt, bt.size()), "paged_from: bad block table");
  KVCacheW4Paged p;
  p.H = c.H;
  p.S = c.S;
  p.D = c.D;
  p.gs = c.gs;
  p.G = c.G;
  p.page = page;
  p.npages = (int)bt.size();
  p.symmetric = c.symmetric;
  p.block_table = bt;
  const size_t pool_rows = (size_t)p.npages * page;
  const auto scatter = [&](const auto& src, auto& dst, size_t per_row) {
    using T = typename std::decay_t<decltype(src)>::value_type;
    dst.assign((size_t)c.H * pool_rows * per_row, T{});
    for (int h = 0; h < c.H; ++h)
      for (int t = 0; t < c.S; ++t) {
        const size_t to = (size_t)h * pool_rows + (size_t)bt[(size_t)t / page] * page + (size_t)t % page;
        std::copy_n(src.begin() + ((size_t)h * c.S + t) * per_row, per_row, dst.begin() + to * per_row);
      }
  };
  scatter(c.q_k, p.q_k, (size_t)words(c.D));
  scatter(c.q_v, p.q_v, (size_t)words(c.D));
  scatter(c.s_k, p.s_k, (size_t)c.G);
  scatter(c.s_v, p.s_v, (size_t)c.G);
  if (!c.symmetric) {
    scatter(c.z_k, p.z_k, (size_t)words(c.G));
    scatter(c.z_v, p.z_v, (size_t)words(c.G));
  }
  return p;
}

}  // namespace w4::kv
