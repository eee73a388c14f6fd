// Where a key or value element lies in the paged cache.
//
// One layer's keys (and, separately, its values) are an array
//   [n_pages][n_kv_heads][kPageTokens][head_dim]
// so that the 64 rows of one head in one page are contiguous and one bulk copy
// brings them on chip.  Inside such a [64][head_dim] tile the 16-byte groups of
// 8 elements of row r are stored XOR-permuted by (r & 7) when head_dim is a
// multiple of 64: a tile copied verbatim to shared memory is then read by
// ldmatrix without bank conflicts.  For other head sizes rows are stored as
// they are.  Every kernel that touches the cache goes through kv_elem_offset().
//
// A sequence finds its pages through its row of the page table.  A layer group
// that keeps all keys uses table entry (position / 64); a group that keeps a
// window uses a ring of `ring_pages` entries: entry (position / 64) % ring_pages.
#pragma once
#include <stdint.h>

namespace hos {

constexpr int kPageTokens = 64;

__host__ __device__ __forceinline__ bool kv_is_swizzled(int head_dim) { return (head_dim & 63) == 0; }

// Element offset of (row, d) inside one [64][head_dim] tile.
__host__ __device__ __forceinline__ int kv_elem_offset(int row, int d, int head_dim) {
    int chunk = d >> 3;
    if (kv_is_swizzled(head_dim)) chunk ^= (row & 7);
    return row * head_dim + (chunk << 3) + (d & 7);
}

struct PagedKV {
    void* k_pages;           // this layer's keys
    void* v_pages;           // this layer's values
    const int* page_table;   // [n_slots][table_stride] physical page of each table entry
    int table_stride;
    int ring_pages;          // 0: all keys are kept; > 0: ring of that many pages
    int n_kv_heads;
    int head_dim;
};

// Table entry that holds logical page `lp` of a sequence.
__host__ __device__ __forceinline__ int kv_table_entry(const PagedKV& c, int lp) {
    return c.ring_pages > 0 ? lp % c.ring_pages : lp;
}

// Element offset of the [64][head_dim] tile of (physical page, kv head).
__host__ __device__ __forceinline__ size_t kv_tile_offset(const PagedKV& c, int page, int kv_head) {
    return ((size_t)page * c.n_kv_heads + kv_head) * (size_t)kPageTokens * c.head_dim;
}

}  // namespace hos
