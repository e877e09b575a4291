// Helpers shared by the host sources; not part of the public surface.
#pragma once

#include "dl/dl.h"

#include <cstdint>
#include <cstring>
#include <stdexcept>

namespace dl {
namespace runtime {
void check(int status, const char* what);       // throws std::runtime_error with b200_last_error()
void check_cuda(int error, const char* what);   // throws "CUDA: ..." for a non-zero cudaError_t
void set_device(int device);
void copy_bytes(void* dst, Device dst_device, const void* src, Device src_device, std::size_t bytes);
// KV-head tensor parallelism: one NCCL communicator per device (runtime/collective.cpp).
void tp_unique_id(void* out128);
void tp_init(int device, int rank, int world, const void* id128);
void tp_finalize(int device);
int tp_world(int device);
int tp_rank(int device);
void tp_all_reduce(int device, float* data, std::size_t count);
void tp_symmetric_handle(int device, std::size_t slot_bytes, void* handle64);
void tp_symmetric_open(int device, const void* handles, int world);
void tp_set_push(int device, bool push);   // partial sums pushed by the projections (true) or pulled by the sums (false, default)
bool tp_push(int device);
bool tp_symmetric_ready(int device, std::size_t bytes);   // mapped on all ranks and a slot holds `bytes`
float* tp_partial_slot(int device, int slot, int owner = -1);   // this rank's partial rows of sum 0 or 1 in rank `owner`'s region (own by default)
void tp_argmax_finish(int device, std::int32_t first_index, const float* best_value, const std::int32_t* best_index, std::int32_t parts,
                      std::int64_t rows, std::int64_t* next, std::int64_t* ids, std::int64_t* history, std::int64_t history_rows,
                      std::int32_t* counter, b200_kv_cache* const* caches, std::int32_t cache_count);
void tp_reduce_shadow(int device, int slot, std::int64_t rows, std::int64_t width, const void* norm_weight, int norm_dtype, float* out,
                      void* out_hi, void* out_lo, float* sumsq_out);
}  // namespace runtime

namespace internal {

// f32 -> bf16 round-to-nearest-even, NaN kept quiet (the reference's include/dl/half.h:43-47 rule).
inline std::uint16_t to_bf16(float value) {
    std::uint32_t word;
    std::memcpy(&word, &value, sizeof word);
    if ((word & 0x7fffffffu) > 0x7f800000u) return static_cast<std::uint16_t>((word >> 16) | 0x0040u);
    word += 0x7fffu + ((word >> 16) & 1u);
    return static_cast<std::uint16_t>(word >> 16);
}
inline float from_bf16(std::uint16_t bits) {
    const std::uint32_t word = static_cast<std::uint32_t>(bits) << 16;
    float value;
    std::memcpy(&value, &word, sizeof value);
    return value;
}

// RAII owner of a kernel-level KV cache.
class KvHandle {
public:
    KvHandle(int device, int dtype, Index sequences, Index kv_heads, Index head_dim, Index capacity, Index page_size) {
        runtime::check(b200_kv_cache_create(device, dtype, static_cast<int32_t>(sequences), static_cast<int32_t>(kv_heads),
                                            static_cast<int32_t>(head_dim), static_cast<int32_t>(capacity),
                                            static_cast<int32_t>(page_size), &cache_), "KV cache allocation");
    }
    ~KvHandle() { b200_kv_cache_release(cache_); }
    KvHandle(const KvHandle&) = delete;
    KvHandle& operator=(const KvHandle&) = delete;
    b200_kv_cache* get() const { return cache_; }
private:
    b200_kv_cache* cache_ = nullptr;
};

}  // namespace internal
}  // namespace dl
