// A cache entry whose keys and values have different sizes per position and kv head: a page holds `page_size`
// positions of every kv head as [ keys: kv_head, row, key_dim | values: kv_head, row, value_dim ]. With equal sizes
// this is the layout of `KvLayout`.
#pragma once
#include "common.cuh"

struct WideKv {
  void* base;
  const int* page_table;
  int max_pages, page_size, kv_heads, key_dim, value_dim;
};
__device__ __forceinline__ size_t page_elems(const WideKv& c) {
  return (size_t)c.kv_heads * c.page_size * (size_t)(c.key_dim + c.value_dim);
}
__device__ __forceinline__ size_t key_at(const WideKv& c, int page, int g, int row) {
  return (size_t)page * page_elems(c) + ((size_t)g * c.page_size + row) * c.key_dim;
}
__device__ __forceinline__ size_t value_at(const WideKv& c, int page, int g, int row) {
  return (size_t)page * page_elems(c) + (size_t)c.kv_heads * c.page_size * c.key_dim +
         ((size_t)g * c.page_size + row) * c.value_dim;
}

// The first position a token at `pos` sees: the start of its chunk of `chunk` positions (0: no chunks), or the start
// of its window of `window` positions (0: none), whichever is later.
__device__ __forceinline__ int first_visible(int pos, int chunk, int window) {
  int first = chunk > 0 ? (pos / chunk) * chunk : 0;
  if (window > 0 && pos + 1 - window > first) first = pos + 1 - window;
  return first;
}
