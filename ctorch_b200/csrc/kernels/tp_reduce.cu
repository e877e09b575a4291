// Tensor-parallel sum of the ranks' partial rows over NVLink peer memory, fused with what follows it in the decoder:
// the new residual stream, its per-row sum of squares and the activation shadow of the next RMSNorm.
//
// Every rank owns a "symmetric" region in its own device memory that all ranks of the group have mapped (CUDA IPC):
//     [0, 4096)   control: arrive[r] (written by rank r, read by the owner), the owner's call counter and exit ticket
//     two slots   partial rows [rows, width] f32 written by the owner's projection kernel (slot 0: output projection,
//                 slot 1: FFN down-projection; alternating slots make overwriting safe, see below)
// One call on every rank (same stream position on each):
//   1. CTA 0 publishes "my slot holds call e" to every rank: __threadfence_system, then a system-scope release store of e
//      into arrive[my rank] of each peer's region (plain peer stores, no multicast).
//   2. Thread 0 of every CTA waits until arrive[r] >= e for all r in its OWN region (local polling, acquire loads).
//      The wait is bounded (~2 s of %globaltimer); on expiry the device status word is set, the kernel still finishes
//      its bookkeeping and every later call skips the wait, so a lost rank surfaces as an error status, not a hang.
//   3. A CTA takes 1024 columns of one row, one 16-byte vector per thread: it pulls them from every rank's slot with uncached loads (ld.global.cv: remote
//      lines must not be served from a stale L1), adds them in rank order 0..W-1 (every rank computes the same bits),
//      writes the f32 values, the shadow planes of value * norm_weight, and its partial of the row's sum of squares.
//   4. The last CTA to leave stores the call number (exit ticket), so the next call sees e + 1.
// Slot reuse: a rank overwrites slot s two calls later.  By then it has passed the wait of the call in between, which
// needs every peer's arrival for that call, and a peer arrives there only after its own kernel of the earlier call (the
// one that read slot s) has completed in stream order.
// Reference arithmetic replaced: none - the reference has no tensor parallelism; the sums it would compute inside one
// matmul (src/kernels/cpu/matmul.h:10-22) are split over ranks here.
#include "common.cuh"

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
};

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
                                                                         int32_t* status) {
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
                const float4* source = reinterpret_cast<const float4*>(peers.region[r] + kControlBytes + static_cast<int64_t>(slot) * slot_bytes)
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

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int32_t b200_tp_reduce_parts(int64_t width) { return width > 0 ? static_cast<int32_t>((width + 4 * kReduceThreads - 1) / (4 * kReduceThreads)) : 0; }

size_t b200_tp_region_bytes(size_t slot_bytes) { return kControlBytes + 2 * slot_bytes; }

void* b200_tp_slot(void* region, size_t slot_bytes, int32_t slot) {
    return region ? static_cast<char*>(region) + kControlBytes + static_cast<size_t>(slot) * slot_bytes : nullptr;
}

int b200_tp_reduce_shadow(void* const* regions, int32_t rank, int32_t world, int32_t slot, size_t slot_bytes, int64_t rows, int64_t width,
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
                                        static_cast<__nv_bfloat16*>(out_lo), sumsq_out, status),
                       "tp_reduce_shadow_kernel launch");
}

}  // extern "C"
