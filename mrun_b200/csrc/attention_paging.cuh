// Where a key lives in the paged cache (cache[page, kv_head, offset, :]), shared by the attention
// kernels.  `page_shift` is log2(page_size) when the page size is a power of two (shift and mask
// instead of a division), else -1.
#pragma once

struct Paging {
    const int* table;       // the request's block table: page id per logical block, < 0 = not held
    int kv_heads, kvh, page_size, page_shift;
};

// Element offset of key `key` of kv head pg.kvh.  `valid` comes in as "the key is inside the
// visible range" and goes out false as well when the page is not held; the offset of an invalid
// key must not be dereferenced.
template <int HEAD_DIM>
__device__ __forceinline__ long cache_row(const Paging& pg, int key, bool& valid) {
    int block, off;
    if (pg.page_shift >= 0) {
        block = key >> pg.page_shift;
        off = key & (pg.page_size - 1);
    } else {
        block = key / pg.page_size;
        off = key - block * pg.page_size;
    }
    const int page = valid ? pg.table[block] : -1;
    valid = page >= 0;
    return ((long)(page * pg.kv_heads + pg.kvh) * pg.page_size + off) * HEAD_DIM;
}

inline int page_shift_of(int page_size) {
    for (int s = 0; s < 31; ++s)
        if ((1 << s) == page_size) return s;
    return -1;
}
