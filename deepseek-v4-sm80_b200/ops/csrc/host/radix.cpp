// Host helpers on the scheduler's hot path.
//
//  * dsv4_first_mismatch: length of the common prefix of two token-id arrays, the
//    radix tree's inner comparison (the reference does this with std::mismatch in
//    python/minisgl/kernel/csrc/src/radix.cpp:19-44).  Here it compares 8 bytes at
//    a time and finishes with a scalar tail.
//  * dsv4_fill_token_locs: expands a list of page ids into token locations
//    page*page_size + offset for a [begin, end) token range of one request row.
//  * dsv4_check_view: validates a tensor view (shape / dtype / contiguity).
#include <cstring>

#include "check.h"

DSV4_HOST_API const char* dsv4_host_last_error() { return dsv4::g_last_error.c_str(); }

DSV4_HOST_API int64_t dsv4_first_mismatch(const void* a, const void* b, int64_t n, int32_t elem_bytes) {
  if (n <= 0) return 0;
  const unsigned char* pa = static_cast<const unsigned char*>(a);
  const unsigned char* pb = static_cast<const unsigned char*>(b);
  const int64_t total = n * elem_bytes;
  int64_t i = 0;
  for (; i + 8 <= total; i += 8) {
    uint64_t x, y;
    std::memcpy(&x, pa + i, 8);
    std::memcpy(&y, pb + i, 8);
    if (x != y) {
      const int byte = __builtin_ctzll(x ^ y) >> 3;
      return (i + byte) / elem_bytes;
    }
  }
  for (; i < total; ++i)
    if (pa[i] != pb[i]) return i / elem_bytes;
  return n;
}

DSV4_HOST_API int32_t dsv4_fill_token_locs(int32_t* row, int64_t row_len, const int32_t* pages, int64_t n_pages,
                                            int64_t begin, int64_t end, int32_t page_size) {
  dsv4::Check c;
  c.require(begin >= 0 && end >= begin && end <= row_len, "token range outside the page-table row");
  c.require(page_size > 0, "page_size must be positive");
  const int64_t first_page = begin / page_size;
  c.require((end + page_size - 1) / page_size - first_page <= n_pages, "not enough pages for the token range");
  if (!c.ok()) return 1;
  for (int64_t t = begin; t < end; ++t) {
    const int64_t p = t / page_size - first_page;
    row[t] = pages[p] * page_size + static_cast<int32_t>(t % page_size);
  }
  return 0;
}

DSV4_HOST_API int32_t dsv4_check_view(const dsv4::TensorView* t, int32_t ndim, int32_t dtype, int32_t need_contig) {
  dsv4::Check c;
  c.dim(*t, ndim, "unexpected tensor rank").dtype(*t, dtype, "unexpected tensor dtype");
  if (need_contig) c.contiguous(*t, "tensor must be contiguous");
  return c.ok() ? 0 : 1;
}
