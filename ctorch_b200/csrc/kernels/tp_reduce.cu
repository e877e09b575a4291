// Tensor-parallel sum of the ranks' partial rows over NVLink peer memory, fused with what follows it in the decoder:
// the new residual stream, its per-row sum of squares and the activation shadow of the next RMSNorm.
//
// Every rank owns a "symmetric" region in its own device memory that all ranks of the group have mapped (CUDA IPC):
//     [0, 4096)   control: arrive[r] (written by rank r, read by the owner), the owner's call counter and exit ticket
//     2 x W slots partial rows [rows, width] f32, one slot per (sum, sender): rank s deposits the partial rows of its
//                 projection in slot (sum, s) of EVERY rank's region - the local one as the projection's result, the peers'
//                 as extra destinations of the same epilogue (plain peer stores), so the rows cross NVLink while the
//                 projection is still running (sum 0: output projection, sum 1: FFN down-projection; alternating sums
//                 make overwriting safe, see below)
// One call on every rank (same stream position on each):
//   1. CTA 0 publishes "my rows of call e are written everywhere" to every rank: __threadfence_system after the
//      projection kernel has completed, then a system-scope release store of e into arrive[my rank] of each peer's
//      region (plain peer stores, no multicast).
//   2. Thread 0 of every CTA waits until arrive[r] >= e for all r in its OWN region (local polling, acquire loads).
//      The wait is bounded (~2 s of %globaltimer); on expiry the device status word is set, the kernel still finishes
//      its bookkeeping and every later call skips the wait, so a lost rank surfaces as an error status, not a hang.
//   3. A CTA takes 1024 columns of one row, one 16-byte vector per thread: it reads them from the W sender slots of its OWN
//      region (local memory; ld.global.cv, because the peers wrote those lines and a stale L1 copy of the slot's previous
//      use must not be served), adds them in rank order 0..W-1 (every rank computes the same bits),
//      (`pull` mode: the projections wrote only their own region, and sender r's rows are read from rank r's region over
//      NVLink instead - one round trip per call; measured faster than pushing at two ranks, see the plan)
//      writes the f32 values, the shadow planes of value * norm_weight, and its partial of the row's sum of squares.
//   4. The last CTA to leave stores the call number (exit ticket), so the next call sees e + 1.
// Slot reuse: a rank overwrites its slots of sum s two calls later.  By then it has passed the wait of the call in
// between, which needs every peer's arrival for that call, and a peer arrives there only after its own kernel of the
// earlier call (the one that read sum s's slots) has completed in stream order.
// Reference arithmetic replaced: none - the reference has no tensor parallelism; the sums it would compute inside one
// matmul (src/kernels/cpu/matmul.h:10-22) are split over ranks here.
#include "linear_common.cuh"

#include "ctorch_b200_kernels.h"

namespace b200 {
namespace {

constexpr int kControlBytes = 4096;
constexpr int kMaxRanks = 16;
constexpr int kReduceThreads = 256;

struct Control {
    uint32_t arrive[kMaxRanks];   // arrive[r]: latest call whose partial rows rank r has published
    uint32_t pad[16];
    uint32_t calls;               // completed calls of the owner
    uint32_t ticket;              // CTAs of the running call that have finished
    uint32_t chosen[kMaxRanks];   // the same handshake for the exchange of argmax candidates (vocabulary split over the ranks)
    uint32_t choices;             // completed candidate exchanges of the owner
};
constexpr int kCandidateRows = 1024;   // rows of the candidate area: [sender][row] pairs (value, index) behind the slots

struct PeerTable { char* region[kMaxRanks]; };

__device__ __forceinline__ void store_release_system(uint32_t* address, uint32_t value) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t* address) {
    uint32_t value;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(kReduceThreads) tp_reduce_shadow_kernel(const PeerTable peers, int rank, int world, int slot,
                                                                         int64_t slot_bytes, int64_t rows, int64_t width,
                                                                         const void* norm_weight, int norm_dtype, float* out,
                                                                         __nv_bfloat16* out_hi, __nv_bfloat16* out_lo, float* sumsq_out,
                                                                         int32_t* status, int pull) {
    __shared__ float partial[32];
    __shared__ uint32_t proceed;
    grid_dependency_wait();   // the projection that wrote this rank's slot precedes this kernel in the stream
    grid_launch_dependents();
    auto* mine = reinterpret_cast<Control*>(peers.region[rank]);
    const uint32_t call = mine->calls + 1;   // stable during the kernel: only the last CTA to leave advances it
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0 && blockIdx.y == 0) {
            __threadfence_system();
            for (int r = 0; r < world; ++r) store_release_system(&reinterpret_cast<Control*>(peers.region[r])->arrive[rank], call);
        }
        uint32_t ok = 1;
        if (*reinterpret_cast<volatile int32_t*>(status) != 0) {
            ok = 0;   // an earlier wait gave up: do not wait again
        } else {
            const uint64_t start = global_timer_ns();
            for (int r = 0; r < world && ok; ++r) {
                while (static_cast<int32_t>(load_acquire_system(&mine->arrive[r]) - call) < 0) {
                    if (global_timer_ns() - start > 2000000000ull) {
                        atomicExch(status, B200_DEVICE_TIMEOUT);
                        ok = 0;
                        break;
                    }
                    __nanosleep(64);
                }
            }
        }
        proceed = ok;
    }
    __syncthreads();
    const int64_t row = blockIdx.y;
    float squares = 0.0f;
    // One 16-byte vector per thread: every peer load of the CTA is in flight at once (one NVLink round trip per call).
    const int64_t vectors = width >> 2;   // width % 4 == 0 (checked by the launcher)
    const int64_t v = static_cast<int64_t>(blockIdx.x) * kReduceThreads + threadIdx.x;
    if (proceed && row < rows && v < vectors) {
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float4 part[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < world) {
                const float4* source = reinterpret_cast<const float4*>(peers.region[pull ? r : rank] + kControlBytes
                                                                       + (static_cast<int64_t>(slot) * world + r) * slot_bytes)
                                       + row * vectors + v;
                part[r] = __ldcv(source);
            }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < world) {
                sum.x = __fadd_rn(sum.x, part[r].x); sum.y = __fadd_rn(sum.y, part[r].y);
                sum.z = __fadd_rn(sum.z, part[r].z); sum.w = __fadd_rn(sum.w, part[r].w);
            }
        }
        reinterpret_cast<float4*>(out + row * width)[v] = sum;
        squares = sum.x * sum.x + sum.y * sum.y + sum.z * sum.z + sum.w * sum.w;
        const int64_t c = v * 4;
        float w[4] = {1.0f, 1.0f, 1.0f, 1.0f};
        if (norm_weight) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                w[i] = norm_dtype == B200_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(norm_weight)[c + i])
                                               : static_cast<const float*>(norm_weight)[c + i];
        }
        const float e[4] = {__fmul_rn(sum.x, w[0]), __fmul_rn(sum.y, w[1]), __fmul_rn(sum.z, w[2]), __fmul_rn(sum.w, w[3])};
        const __nv_bfloat162 h0 = __floats2bfloat162_rn(e[0], e[1]), h1 = __floats2bfloat162_rn(e[2], e[3]);
        const __nv_bfloat162 l0 = __floats2bfloat162_rn(e[0] - __low2float(h0), e[1] - __high2float(h0));
        const __nv_bfloat162 l1 = __floats2bfloat162_rn(e[2] - __low2float(h1), e[3] - __high2float(h1));
        uint2 hi, lo;
        hi.x = *reinterpret_cast<const uint32_t*>(&h0); hi.y = *reinterpret_cast<const uint32_t*>(&h1);
        lo.x = *reinterpret_cast<const uint32_t*>(&l0); lo.y = *reinterpret_cast<const uint32_t*>(&l1);
        *reinterpret_cast<uint2*>(out_hi + row * width + c) = hi;
        *reinterpret_cast<uint2*>(out_lo + row * width + c) = lo;
    }
    for (int o = 16; o > 0; o >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, o);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = squares;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0f;
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0 && row < rows) sumsq_out[static_cast<int64_t>(blockIdx.x) * rows + row] = v;   // one partial per column chunk
    }
    // exit ticket: the last CTA of the call advances the owner's call counter
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t finished = atomicAdd(&mine->ticket, 1u);
        if (finished == gridDim.x * gridDim.y - 1) {
            mine->ticket = 0;
            __threadfence();
            mine->calls = call;
        }
    }
}

// Greedy choice with the vocabulary split over the ranks: every rank has reduced its slice of the logits to one candidate
// (value, index inside the slice) per row and feature tile.  One CTA: (1) warp w merges the tiles of rows w, w + warps, ...
// under the reference's rule (first maximum, first NaN wins; src/kernels/cpu/reduction.cpp:141-145), adds the slice's
// first index and deposits the row's candidate in slot [my rank][row] of EVERY rank's candidate area (8-byte peer stores);
// (2) "my candidates are written" goes to every rank (system-scope release), all ranks' signals are awaited in the own
// region (bounded, then the status word is set); (3) the W candidates of a row are merged under the same rule - the
// global index breaks ties, so every rank chooses the same token - and the token bookkeeping of the step follows.
struct LengthTable { int32_t* lengths[64]; int32_t counts[64]; int32_t caches; };
__global__ void __launch_bounds__(1024) tp_argmax_finish_kernel(const PeerTable peers, int rank, int world, int64_t area_offset, int32_t first_index,
                                                                const float* best_value, const int32_t* best_index, int parts, int64_t rows,
                                                                int64_t* next, int64_t* ids, int64_t* history, int64_t history_rows,
                                                                int32_t* counter, const LengthTable advance, int32_t* status) {
    __shared__ uint32_t proceed;
    grid_dependency_wait();
    grid_launch_dependents();
    auto* mine = reinterpret_cast<Control*>(peers.region[rank]);
    const uint32_t call = mine->choices + 1;
    const int32_t step = *counter;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int64_t row = warp; row < rows; row += warps) {
        Candidate best{-INFINITY, INT32_MAX};
        for (int t = lane; t < parts; t += 32) {
            const Candidate seen{__ldg(best_value + static_cast<int64_t>(t) * rows + row), __ldg(best_index + static_cast<int64_t>(t) * rows + row)};
            if (preferred(seen, best)) best = seen;
        }
        for (int o = 16; o > 0; o >>= 1) {
            const Candidate other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
            if (preferred(other, best)) best = other;
        }
        if (best.index != INT32_MAX) best.index += first_index;
        const unsigned long long packed = (static_cast<unsigned long long>(static_cast<uint32_t>(best.index)) << 32) | __float_as_uint(best.value);
        if (lane < world)
            *reinterpret_cast<unsigned long long*>(peers.region[lane] + area_offset + (static_cast<int64_t>(rank) * kCandidateRows + row) * 8) = packed;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int r = 0; r < world; ++r) store_release_system(&reinterpret_cast<Control*>(peers.region[r])->chosen[rank], call);
        uint32_t ok = 1;
        if (*reinterpret_cast<volatile int32_t*>(status) != 0) {
            ok = 0;
        } else {
            const uint64_t start = global_timer_ns();
            for (int r = 0; r < world && ok; ++r) {
                while (static_cast<int32_t>(load_acquire_system(&mine->chosen[r]) - call) < 0) {
                    if (global_timer_ns() - start > 2000000000ull) {
                        atomicExch(status, B200_DEVICE_TIMEOUT);
                        ok = 0;
                        break;
                    }
                    __nanosleep(64);
                }
            }
        }
        proceed = ok;
    }
    __syncthreads();
    for (int64_t row = warp; row < rows; row += warps) {
        Candidate best{-INFINITY, INT32_MAX};
        if (lane < world && proceed) {
            const unsigned long long packed = __ldcv(reinterpret_cast<const unsigned long long*>(
                peers.region[rank] + area_offset + (static_cast<int64_t>(lane) * kCandidateRows + row) * 8));
            best = Candidate{__uint_as_float(static_cast<uint32_t>(packed)), static_cast<int32_t>(packed >> 32)};
        }
        for (int o = 16; o > 0; o >>= 1) {
            const Candidate other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
            if (preferred(other, best)) best = other;
        }
        if (lane == 0) {
            const int64_t token = best.index == INT32_MAX ? 0 : best.index;
            next[row] = token;
            if (ids) ids[row] = token;
            if (history && step < history_rows) history[static_cast<int64_t>(step) * rows + row] = token;
        }
    }
    for (int c = 0; c < advance.caches; ++c)
        for (int i = threadIdx.x; i < advance.counts[c]; i += blockDim.x) advance.lengths[c][i] += 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        *counter = step + 1;
        mine->choices = call;
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int32_t b200_tp_reduce_parts(int64_t width) { return width > 0 ? static_cast<int32_t>((width + 4 * kReduceThreads - 1) / (4 * kReduceThreads)) : 0; }

size_t b200_tp_region_bytes(size_t slot_bytes, int32_t world) {
    const size_t ranks = static_cast<size_t>(world > 0 ? world : 1);
    return kControlBytes + 2 * ranks * slot_bytes + ranks * kCandidateRows * 8;   // control, slots per (sum, sender), candidate area
}

void* b200_tp_slot(void* region, size_t slot_bytes, int32_t world, int32_t slot, int32_t sender) {
    if (!region || world < 1 || slot < 0 || slot > 1 || sender < 0 || sender >= world) return nullptr;
    return static_cast<char*>(region) + kControlBytes + (static_cast<size_t>(slot) * world + sender) * slot_bytes;
}

int b200_tp_reduce_shadow(void* const* regions, int32_t rank, int32_t world, int32_t slot, size_t slot_bytes, int32_t pull, int64_t rows, int64_t width,
                          const void* norm_weight, int32_t norm_dtype, float* out, void* out_hi, void* out_lo, float* sumsq_out,
                          void* stream) {
    if (!regions || world < 1 || world > 8 || rank < 0 || rank >= world || slot < 0 || slot > 1 || rows <= 0 || width <= 0 || (width & 3)
        || !out || !out_hi || !out_lo || !sumsq_out || static_cast<size_t>(rows) * width * sizeof(float) > slot_bytes) {
        set_error("b200_tp_reduce_shadow: bad pointer, group or size");
        return B200_BAD_ARGUMENT;
    }
    PeerTable table{};
    for (int r = 0; r < world; ++r) {
        if (!regions[r]) { set_error("b200_tp_reduce_shadow: region of rank %d is not mapped", r); return B200_BAD_ARGUMENT; }
        table.region[r] = static_cast<char*>(regions[r]);
    }
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    int32_t* status = device_status_word(device);
    if (!status) { set_error("b200_tp_reduce_shadow: the device status word could not be allocated"); return B200_NO_DEVICE; }
    const dim3 grid(static_cast<unsigned>(b200_tp_reduce_parts(width)), static_cast<unsigned>(rows));
    return cuda_status(launch_dependent(tp_reduce_shadow_kernel, grid, dim3(kReduceThreads), 0, as_stream(stream), table,
                                        static_cast<int>(rank), static_cast<int>(world), static_cast<int>(slot), static_cast<int64_t>(slot_bytes),
                                        rows, width, norm_weight, static_cast<int>(norm_dtype), out, static_cast<__nv_bfloat16*>(out_hi),
                                        static_cast<__nv_bfloat16*>(out_lo), sumsq_out, status, static_cast<int>(pull != 0)),
                       "tp_reduce_shadow_kernel launch");
}

int b200_tp_argmax_finish(void* const* regions, int32_t rank, int32_t world, size_t slot_bytes, int32_t first_index, const float* best_value,
                          const int32_t* best_index, int32_t parts, int64_t rows, int64_t* next, int64_t* ids, int64_t* history,
                          int64_t history_rows, int32_t* counter, b200_kv_cache* const* caches, int32_t cache_count, void* stream) {
    if (!regions || world < 1 || world > 8 || rank < 0 || rank >= world || !best_value || !best_index || !next || !counter || parts <= 0
        || rows <= 0 || rows > kCandidateRows || first_index < 0 || cache_count < 0 || cache_count > 64 || (cache_count > 0 && !caches)) {
        set_error("b200_tp_argmax_finish: bad pointer, group or size (at most %d rows, 64 caches)", kCandidateRows);
        return B200_BAD_ARGUMENT;
    }
    PeerTable table{};
    for (int r = 0; r < world; ++r) {
        if (!regions[r]) { set_error("b200_tp_argmax_finish: region of rank %d is not mapped", r); return B200_BAD_ARGUMENT; }
        table.region[r] = static_cast<char*>(regions[r]);
    }
    LengthTable advance{};
    advance.caches = cache_count;
    for (int i = 0; i < cache_count; ++i) {
        if (!caches[i]) { set_error("b200_tp_argmax_finish: cache %d is NULL", i); return B200_BAD_ARGUMENT; }
        advance.lengths[i] = caches[i]->lengths;
        advance.counts[i] = caches[i]->sequences;
    }
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    int32_t* status = device_status_word(device);
    if (!status) { set_error("b200_tp_argmax_finish: the device status word could not be allocated"); return B200_NO_DEVICE; }
    const int64_t area = kControlBytes + 2 * static_cast<int64_t>(world) * static_cast<int64_t>(slot_bytes);
    const unsigned threads = rows >= 32 ? 1024 : static_cast<unsigned>(rows) * 32;
    return cuda_status(launch_dependent(tp_argmax_finish_kernel, dim3(1), dim3(threads), 0, as_stream(stream), table, static_cast<int>(rank),
                                        static_cast<int>(world), area, first_index, best_value, best_index, static_cast<int>(parts), rows, next,
                                        ids, history, history_rows, counter, advance, status),
                       "tp_argmax_finish_kernel launch");
}

}  // extern "C"
