// Paged, head-major KV storage of one decoder layer: device-side view and the host object behind the C ABI.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kFastPageSize = 64;  // page size the TMA/tensor-core attention path is built for

// What kernels see.  Pools are [page][kv_head][page_size][head_dim]; page_table is [sequences][pages_per_seq].
struct KvView {
    void* pool[2];  // 0 = K, 1 = V
    const int32_t* page_table;
    int32_t* lengths;
    int32_t sequences, pages_per_seq, page_size, kv_heads, head_dim, dtype, num_pages;
};

__device__ __forceinline__ int64_t kv_offset(const KvView& kv, int sequence, int position, int head) {
    const int page = __ldg(kv.page_table + static_cast<int64_t>(sequence) * kv.pages_per_seq + position / kv.page_size);
    const int slot = position % kv.page_size;
    return ((static_cast<int64_t>(page) * kv.kv_heads + head) * kv.page_size + slot) * kv.head_dim;
}

// Stores features d (even) and d+1 of one cached token.
__device__ __forceinline__ void kv_store_pair(const KvView& kv, int which, int sequence, int position, int head, int d,
                                              float a, float b) {
    const int64_t at = kv_offset(kv, sequence, position, head) + d;
    if (kv.dtype == B200_BF16) {
        *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(kv.pool[which]) + at) = __floats2bfloat162_rn(a, b);
    } else {
        *reinterpret_cast<float2*>(static_cast<float*>(kv.pool[which]) + at) = make_float2(a, b);
    }
}

// The same with the physical page of the position already known.
__device__ __forceinline__ void kv_store_pair_at(const KvView& kv, int which, int page, int position, int head, int d, float a, float b) {
    const int64_t at = ((static_cast<int64_t>(page) * kv.kv_heads + head) * kv.page_size + position % kv.page_size) * kv.head_dim + d;
    if (kv.dtype == B200_BF16) {
        *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(kv.pool[which]) + at) = __floats2bfloat162_rn(a, b);
    } else {
        *reinterpret_cast<float2*>(static_cast<float*>(kv.pool[which]) + at) = make_float2(a, b);
    }
}

__device__ __forceinline__ float kv_load(const KvView& kv, int which, int64_t at) {
    return kv.dtype == B200_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(kv.pool[which])[at])
                                 : static_cast<const float*>(kv.pool[which])[at];
}

KvView kv_view(const b200_kv_cache* cache);
// Tensor maps (bf16 pools with head_dim % 64 == 0 and 64-token pages only); nullptr otherwise.
const CUtensorMap* kv_tensor_map(const b200_kv_cache* cache, int which);

}  // namespace b200

struct b200_kv_cache {
    int32_t device, dtype, sequences, kv_heads, head_dim, capacity, page_size, pages_per_seq, num_pages;
    size_t pool_bytes;
    void* pool[2];
    int32_t* page_table;
    int32_t* lengths;
    bool has_maps;
    bool even_lengths;   // host-side knowledge: every sequence has the same length (set_lengths with unequal entries clears it)
    alignas(64) CUtensorMap map[2];
};
