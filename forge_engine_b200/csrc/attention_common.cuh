// The page layout every attention kernel of this engine agrees on.
//
// One layer's keys live in k_cache[num_pages][num_kv_heads][page_size][head_dim]
// (values likewise): inside a page all tokens of one kv head are contiguous, so a
// (page, head) tile is one contiguous block of page_size * head_dim elements.
// block_table[entry][i] is the physical page of tokens [i*page_size, (i+1)*page_size)
// of that entry's sequence, or -1 where a page was never leased or has been given back.
#pragma once
#include "common.cuh"

struct PagedKV {
  const void* k;
  const void* v;
  const int* block_table;  // [entries, max_pages]
  int max_pages;
  int page_size;
  int num_pages;
  int num_kv_heads;
  int head_dim;
};

// Element offset of (page, head, slot, 0).
__device__ __forceinline__ size_t kv_offset(const PagedKV& c, int page, int head, int slot) {
  return (((size_t)page * c.num_kv_heads + head) * c.page_size + slot) * c.head_dim;
}
