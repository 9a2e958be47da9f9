// Paged fp16 K/V cache: host-side object and the device-side view kernels use.
#pragma once
#include <vector>

#include "common.cuh"

// What a kernel needs to address a row of the cache.  Pool layout:
// [layer][K|V][page][token_in_page][kv_head][head_dim] f16.
struct KvView {
    __half* pool;
    const int32_t* page_table;  // [max_seqs][max_pages_per_seq], -1 = not reserved
    int layers, kv_heads, head_dim;
    int page_tokens, page_shift;
    int num_pages, max_seqs, max_pages_per_seq;
    int64_t kv_stride;     // elements between the K and V halves of a layer
    int64_t layer_stride;  // elements between layers
};

struct tsb_kv {
    tsb_ctx* ctx = nullptr;
    KvView view{};
    int32_t* page_table_dev = nullptr;
    std::vector<int32_t> page_table_host;
    std::vector<int32_t> free_pages;
    std::vector<int32_t> pages_of_seq;
    std::vector<int64_t> cursor;
};

#ifdef __CUDACC__
// Row of (layer, which = 0 K / 1 V) holding position `pos` of stream `seq`; nullptr when the
// position is outside the reserved pages (the caller records TSB_DEV_BAD_INDEX and skips).
__device__ __forceinline__ __half* kv_row(const KvView& kv, int layer, int which, int seq, int pos) {
    const int lp = pos >> kv.page_shift;
    if (pos < 0 || lp >= kv.max_pages_per_seq) return nullptr;
    const int page = kv.page_table[(size_t)seq * kv.max_pages_per_seq + lp];
    if (page < 0) return nullptr;
    const int64_t row = (int64_t)kv.kv_heads * kv.head_dim;
    return kv.pool + (int64_t)layer * kv.layer_stride + (int64_t)which * kv.kv_stride +
           ((int64_t)page * kv.page_tokens + (pos & (kv.page_tokens - 1))) * row;
}
#endif
