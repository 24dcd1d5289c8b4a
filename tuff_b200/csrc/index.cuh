// Where a request's keys and states lie: the index arithmetic that every kernel over the paged
// cache shares, as plain functions of integers.  They compile for the host too, so a unit test can
// run them without a GPU.
//
// Pages are [page][kv_head][offset][head_dim]; a request's block table row holds the page of its
// positions [b * page_size, (b + 1) * page_size) in entry b.  States are [slot][...], one slot a
// request.
//
// A build with -DTUFF_DEBUG_BOUNDS range-checks every table row, table entry, page id and slot
// that a kernel takes from its inputs: an index outside its range leaves a code in the status word
// and the access is skipped.  (No memory checker runs where these kernels are developed; this build
// stands in for one.)  The normal build compiles the checks away.
#pragma once
#include <stddef.h>

#if defined(__CUDACC__)
#define TUFF_HD __host__ __device__ __forceinline__
#else
#define TUFF_HD inline
#endif

#ifdef TUFF_DEBUG_BOUNDS
#define TUFF_CHECKED 1
#else
#define TUFF_CHECKED 0
#endif

// Codes a checked build leaves in the status word (the first one stays).
#define TUFF_BOUNDS_ENTRY 71      // a position beyond the block table's width (or negative)
#define TUFF_BOUNDS_PAGE 72       // a page id outside the pool
#define TUFF_BOUNDS_SLOT 73       // a state slot outside the slots
#define TUFF_BOUNDS_ROW 74        // a batch row outside the block table

TUFF_HD int page_entry(int pos, int page_size) { return pos / page_size; }
TUFF_HD int page_offset(int pos, int page_size) { return pos % page_size; }
TUFF_HD bool page_entry_ok(int pos, int page_size, int max_blocks) { return pos >= 0 && pos / page_size < max_blocks; }
TUFF_HD bool page_ok(long long page, long long n_pages) { return page >= 0 && page < n_pages; }
TUFF_HD bool slot_ok(long long slot, long long n_slots) { return slot >= 0 && slot < n_slots; }
TUFF_HD bool row_ok(long long row, long long n_rows) { return row >= 0 && row < n_rows; }
// First element of (page, kv_head, offset) in pages of kv_heads heads, page_size offsets and head_dim elements.
TUFF_HD size_t page_elem(long long page, int kv_head, int offset, int kv_heads, int page_size, int head_dim) {
    return (((size_t)page * kv_heads + kv_head) * page_size + offset) * head_dim;
}
// First element of a slot's state of `per_slot` elements.
TUFF_HD size_t slot_elem(long long slot, size_t per_slot) { return (size_t)slot * per_slot; }

// What a kernel needs for the checks: the sizes of the pool it indexes and where to leave a code.
// n_rows: rows of the block table (or of the slot table); n: pages in the pool, or state slots.
struct Bounds {
    long long n_rows, n;
    int* status;
};

#if defined(__CUDACC__)
__device__ __forceinline__ void bounds_fault(const Bounds& b, int code) {
    if (b.status) atomicCAS(b.status, 0, code);
}
// True if the access may go ahead.  In the normal build this is the constant true.
__device__ __forceinline__ bool check_row(const Bounds& b, long long row) {
    if (TUFF_CHECKED && !row_ok(row, b.n_rows)) { bounds_fault(b, TUFF_BOUNDS_ROW); return false; }
    return true;
}
__device__ __forceinline__ bool check_entry(const Bounds& b, int pos, int page_size, int max_blocks) {
    if (TUFF_CHECKED && !page_entry_ok(pos, page_size, max_blocks)) { bounds_fault(b, TUFF_BOUNDS_ENTRY); return false; }
    return true;
}
__device__ __forceinline__ bool check_page(const Bounds& b, long long page) {
    if (TUFF_CHECKED && !page_ok(page, b.n)) { bounds_fault(b, TUFF_BOUNDS_PAGE); return false; }
    return true;
}
__device__ __forceinline__ bool check_slot(const Bounds& b, long long slot) {
    if (TUFF_CHECKED && !slot_ok(slot, b.n)) { bounds_fault(b, TUFF_BOUNDS_SLOT); return false; }
    return true;
}
#endif
