// Where a row of logits sits on the 16-byte grid.  A row may begin anywhere on the element
// grid (odd vocabulary sizes, views).  Bulk copies and 128-bit loads need 16-byte aligned
// addresses, so they cover the row from its first 16-byte boundary (`head` elements in) to
// its last; the few elements before and after are read with ordinary loads.
#pragma once
#include <stdint.h>

namespace tome {

struct K1RowGeom {
  int64_t head;        // elements before the first 16-byte boundary (0 for an aligned row)
  int64_t bulk_bytes;  // bytes between the first and the last boundary (a multiple of 16)
  int64_t tail_begin;  // first element after them
};

template <typename T>
__device__ __forceinline__ K1RowGeom k1_row_geom(const T* src, int64_t vocab) {
  constexpr int64_t ES = sizeof(T);
  K1RowGeom g;
  const int64_t to_boundary =
      static_cast<int64_t>((16u - (reinterpret_cast<uintptr_t>(src) & 15u)) & 15u) / ES;
  g.head = to_boundary < vocab ? to_boundary : vocab;
  g.bulk_bytes = ((vocab - g.head) * ES) & ~static_cast<int64_t>(15);
  g.tail_begin = g.head + g.bulk_bytes / ES;
  return g;
}

}  // namespace tome
