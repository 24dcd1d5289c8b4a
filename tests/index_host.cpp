// The index helpers of tuff_b200/csrc/index.cuh compiled for the host, behind C names that
// tests/test_index_helpers.py calls through ctypes.
#include "index.cuh"

extern "C" {
int h_page_entry(int pos, int page_size) { return page_entry(pos, page_size); }
int h_page_offset(int pos, int page_size) { return page_offset(pos, page_size); }
int h_page_entry_ok(int pos, int page_size, int max_blocks) { return page_entry_ok(pos, page_size, max_blocks) ? 1 : 0; }
int h_page_ok(long long page, long long n_pages) { return page_ok(page, n_pages) ? 1 : 0; }
int h_slot_ok(long long slot, long long n_slots) { return slot_ok(slot, n_slots) ? 1 : 0; }
int h_row_ok(long long row, long long n_rows) { return row_ok(row, n_rows) ? 1 : 0; }
unsigned long long h_page_elem(long long page, int kv_head, int offset, int kv_heads, int page_size, int head_dim) {
    return page_elem(page, kv_head, offset, kv_heads, page_size, head_dim);
}
unsigned long long h_slot_elem(long long slot, unsigned long long per_slot) { return slot_elem(slot, per_slot); }
}
