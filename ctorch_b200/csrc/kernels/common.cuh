// Shared device/host helpers of the sm_100a decoder kernels.
#pragma once

#include <mutex>
#include "ctorch_b200_kernels.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

namespace b200 {

// ---- host: error text ------------------------------------------------------------------------------------
void set_error(const char* format, ...);
int cuda_status(cudaError_t error, const char* what);

#define B200_CUDA(call)                                                 \
    do {                                                                \
        cudaError_t status_ = (call);                                   \
        if (status_ != cudaSuccess) return b200::cuda_status(status_, #call); \
    } while (0)

inline cudaStream_t as_stream(void* stream) { return static_cast<cudaStream_t>(stream); }

// Device-resident health word (one per device), set by kernels that abandon a bounded wait.
int32_t* device_status_word(int device);
// The same word if it already exists (it is created with the first KV cache of a device), else nullptr; never allocates.
int32_t* device_status_word_if_allocated(int device);

// ---- device helpers -------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

__device__ __forceinline__ float load_as_f32(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float load_as_f32(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ void store_from_f32(float* p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void store_from_f32(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// 16-byte read-only streaming load that does not allocate in L1 (weights and KV are read once per step).
__device__ __forceinline__ uint4 load_stream_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <class T> __device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// SiLU exactly as the reference states it: v * sigmoid(v), sigmoid through exp(-|v|) in two branches
// (src/kernels/cpu/pointwise.cpp:31-34,57 of the reference).
__device__ __forceinline__ float silu_reference(float v) {
    const float e = expf(-fabsf(v));
    const float s = v >= 0.0f ? __fdiv_rn(1.0f, __fadd_rn(1.0f, e)) : __fdiv_rn(e, __fadd_rn(1.0f, e));
    return __fmul_rn(v, s);
}

// The same function for the bf16 paths, whose results are rounded to 16 mantissa bits anyway: hardware exponential and
// approximate division (relative error around 1e-6) instead of the IEEE sequence above, a fifth of the instructions.  A row
// of a SwiGLU epilogue is a dependent chain per lane, so this is what bounds that epilogue's time.
__device__ __forceinline__ float silu_fast(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// Asks for the 128-byte line at `address` to be brought into L2; nothing waits for it.
__device__ __forceinline__ void prefetch_l2(const void* address) { asm volatile("prefetch.global.L2 [%0];" ::"l"(address)); }

// ---- mbarrier / TMA (cp.async.bulk.tensor, no multicast) --------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait: gives up after `limit` polls (each try_wait already blocks for a hardware-defined slice) and
// reports false so that the caller can set the device status word and leave instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = 4000000u) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// One lane of a fully active warp (the same lane on every call).  The warp-specialised loops below keep the whole warp in
// uniform control flow and put only the issuing instruction under this predicate: TMA and tcgen05 instructions take their
// operands from uniform registers, which the compiler can only fill cheaply while control flow is warp-uniform.  A loop
// run by one lane alone (`if (lane == 0) for (...)`) pays a chain of per-operand transfers for every instruction issued.
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(chosen));
    return chosen != 0;
}

// The same for waits that last a whole main loop (epilogue warps waiting for an accumulator): the warp sleeps between
// polls, so that its polling does not compete with the warps that issue the loads and the products.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, uint32_t limit = 4000000u) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(128);
    }
    return false;
}

// 2-D tiled TMA load global -> shared, completion on an mbarrier, this CTA only.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- programmatic dependent launch -----------------------------------------------------------------------------
// A kernel launched with launch_dependent() may begin while its predecessor in the stream is still running.  It must
// execute grid_dependency_wait() before it touches anything the predecessor writes (and before it writes anything
// the predecessor reads); everything before that point may only read constants such as weights.  A kernel calls
// grid_launch_dependents() to let its successor start early.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class... Params, class... Args>
cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// Same, for a grid made of thread-block clusters of `cluster` CTAs (distributed shared memory between them).
template <class... Params, class... Args>
cudaError_t launch_dependent_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, dim3 cluster,
                                     Args&&... args) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2]{};
    attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[0].val.programmaticStreamSerializationAllowed = 1;
    attributes[1].id = cudaLaunchAttributeClusterDimension;
    attributes[1].val.clusterDim.x = cluster.x;
    attributes[1].val.clusterDim.y = cluster.y;
    attributes[1].val.clusterDim.z = cluster.z;
    config.attrs = attributes;
    config.numAttrs = 2;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// ---- thread-block clusters: hardware barrier over all threads of the cluster, and loads from a peer CTA's shared memory ----
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_peer_shared(uint32_t local_address, uint32_t peer_rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_address), "r"(peer_rank));
    return remote;
}
// Not volatile: the cluster barrier orders these loads against the peers' stores, and independent loads should overlap.
__device__ __forceinline__ float2 load_cluster_float2(uint32_t cluster_address) {
    float2 value;
    asm("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(value.x), "=f"(value.y) : "r"(cluster_address));
    return value;
}

// Number of SMs of a device (cached; 148 when the device cannot be queried).
inline int sm_count(int device) {
    static std::mutex mutex;
    static int counts[64];
    std::lock_guard<std::mutex> lock(mutex);
    if (device < 0 || device >= 64) return 148;
    if (!counts[device] && cudaDeviceGetAttribute(&counts[device], cudaDevAttrMultiProcessorCount, device) != cudaSuccess) counts[device] = 148;
    return counts[device];
}

// Host: cuTensorMapEncodeTiled resolved through the runtime so that the library has no link-time dependency on
// the driver library (it must load on machines without a GPU).
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn tensor_map_encoder();

}  // namespace b200
