// NCCL behind a dlopen'ed function table: the library keeps no link-time dependency on NCCL (it must load on
// machines without it) and uses whichever libnccl.so.2 the process already has (the one PyTorch loaded, if any).
// Used only by the KV-head tensor-parallel plan: all-reduce(sum) of the [rows, D] partial sums after the output
// projection and after the FFN down-projection, enqueued on the library's compute stream (capturable in a graph).
#include "dl/internal.h"

#include "ctorch_b200_kernels.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <future>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>

namespace dl::runtime {

namespace {

struct UniqueId { char bytes[128]; };
using Comm = void*;

struct Nccl {
    int (*get_unique_id)(UniqueId*) = nullptr;
    int (*comm_init_rank)(Comm*, int, UniqueId, int) = nullptr;
    int (*all_reduce)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
    int (*comm_destroy)(Comm) = nullptr;
    const char* (*error_string)(int) = nullptr;
};

Nccl& nccl() {
    static Nccl table = [] {
        Nccl t;
        void* handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!handle) throw std::runtime_error(std::string("NCCL is not available: ") + dlerror());
        auto load = [&](const char* name) {
            void* symbol = dlsym(handle, name);
            if (!symbol) throw std::runtime_error(std::string("NCCL symbol missing: ") + name);
            return symbol;
        };
        t.get_unique_id = reinterpret_cast<decltype(t.get_unique_id)>(load("ncclGetUniqueId"));
        t.comm_init_rank = reinterpret_cast<decltype(t.comm_init_rank)>(load("ncclCommInitRank"));
        t.all_reduce = reinterpret_cast<decltype(t.all_reduce)>(load("ncclAllReduce"));
        t.comm_destroy = reinterpret_cast<decltype(t.comm_destroy)>(load("ncclCommDestroy"));
        t.error_string = reinterpret_cast<decltype(t.error_string)>(load("ncclGetErrorString"));
        return t;
    }();
    return table;
}

void check_nccl(int result, const char* what) {
    if (result != 0) throw std::runtime_error(std::string("NCCL: ") + what + ": " + nccl().error_string(result));
}

std::mutex group_mutex;
// `region`: this rank's symmetric memory (control words + two slots of partial rows) and every rank's mapping of it.
struct Group {
    Comm comm = nullptr;
    int rank = 0, world = 1;
    void* regions[16] = {};
    std::size_t slot_bytes = 0;
    bool mapped = false;
    bool push = false;   // projections push their partial rows into the peers' regions (else the sums pull them)
};
Group groups[64];

void check_runtime(cudaError_t status, const char* what) {
    if (status != cudaSuccess) throw std::runtime_error(std::string("CUDA: ") + what + ": " + cudaGetErrorString(status));
}

}  // namespace

void tp_unique_id(void* out128) {
    UniqueId id;
    check_nccl(nccl().get_unique_id(&id), "ncclGetUniqueId");
    std::memcpy(out128, id.bytes, sizeof id.bytes);
}

void tp_init(int device, int rank, int world, const void* id128) {
    if (device < 0 || device >= 64 || world < 1 || rank < 0 || rank >= world || !id128)
        throw std::invalid_argument("bad tensor-parallel group arguments");
    std::lock_guard<std::mutex> lock(group_mutex);
    if (groups[device].comm) throw std::logic_error("this device already belongs to a tensor-parallel group");
    set_device(device);
    stream(device);
    UniqueId id;
    std::memcpy(id.bytes, id128, sizeof id.bytes);
    // ncclCommInitRank returns only when every rank of the group has joined.  It runs on a helper thread while this one
    // waits with a deadline (CTORCH_B200_TP_INIT_TIMEOUT_S, 120 s by default): a rank that never joins then costs the
    // caller an error instead of a process that hangs for good.  The helper owns its state; after a timeout it is left
    // behind (it ends with the process) and the device stays outside any group.
    nccl();   // resolve the library on this thread, so that a missing NCCL is reported here
    struct Attempt {
        std::promise<int> done;
        Comm comm = nullptr;
    };
    auto attempt = std::make_shared<Attempt>();
    std::future<int> result = attempt->done.get_future();
    std::thread([attempt, device, world, rank, id] {
        int status = -1;
        try {
            set_device(device);
            status = nccl().comm_init_rank(&attempt->comm, world, id, rank);
        } catch (...) {
            status = -1;
        }
        attempt->done.set_value(status);
    }).detach();
    double seconds = 120.0;
    if (const char* text = std::getenv("CTORCH_B200_TP_INIT_TIMEOUT_S")) {
        const double wanted = std::atof(text);
        if (wanted > 0.0) seconds = wanted;
    }
    if (result.wait_for(std::chrono::duration<double>(seconds)) != std::future_status::ready)
        throw std::runtime_error("NCCL: ncclCommInitRank timed out after " + std::to_string(seconds) + " s: not every rank of the group of "
                                 + std::to_string(world) + " joined");
    const int status = result.get();
    if (status == -1) throw std::runtime_error("NCCL: ncclCommInitRank could not run on the helper thread");
    check_nccl(status, "ncclCommInitRank");
    Comm comm = attempt->comm;
    groups[device] = Group{};
    groups[device].comm = comm;
    groups[device].rank = rank;
    groups[device].world = world;
    if (const char* text = std::getenv("CTORCH_B200_TP_PUSH")) groups[device].push = std::atoi(text) != 0;
}

// How the partial sums travel: push = the projection's epilogue stores its rows into every peer's region and the sum reads
// local memory; pull (default) = the projection writes its own region and the sum loads the peers' rows over NVLink.
// Measured on the 8B shape at two ranks: pull 6.63 ms per step, push 6.86 ms.
void tp_set_push(int device, bool push) {
    std::lock_guard<std::mutex> lock(group_mutex);
    if (device < 0 || device >= 64 || !groups[device].comm) throw std::logic_error("tensor-parallel group is not initialised on this device");
    groups[device].push = push;
}
bool tp_push(int device) {
    std::lock_guard<std::mutex> lock(group_mutex);
    return device >= 0 && device < 64 && groups[device].comm && groups[device].push;
}

void tp_finalize(int device) {
    std::lock_guard<std::mutex> lock(group_mutex);
    if (device < 0 || device >= 64 || !groups[device].comm) return;
    set_device(device);
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream(device)));
    Group& group = groups[device];
    for (int r = 0; r < group.world && r < 16; ++r) {
        if (!group.regions[r]) continue;
        if (r == group.rank) cudaFree(group.regions[r]);
        else cudaIpcCloseMemHandle(group.regions[r]);
    }
    nccl().comm_destroy(group.comm);
    group = Group{};
}

// Symmetric memory for the one-shot sum over peer memory (kernels/tp_reduce.cu).  Each rank allocates its region, hands
// the 64-byte CUDA IPC handle to the application, which gathers the handles of all ranks (any transport) and gives the
// table back; only then is the peer path used.  Without the table the plan keeps the NCCL all-reduce.
void tp_symmetric_handle(int device, std::size_t slot_bytes, void* handle64) {
    std::lock_guard<std::mutex> lock(group_mutex);
    if (device < 0 || device >= 64 || !groups[device].comm) throw std::logic_error("tensor-parallel group is not initialised on this device");
    Group& group = groups[device];
    if (group.world > 8) throw std::invalid_argument("the peer-memory sum serves at most 8 ranks");
    if (group.regions[group.rank]) throw std::logic_error("symmetric memory was already allocated on this device");
    if (!handle64 || slot_bytes == 0 || (slot_bytes & 255)) throw std::invalid_argument("slot size must be a positive multiple of 256 bytes");
    set_device(device);
    void* region = nullptr;
    const std::size_t bytes = b200_tp_region_bytes(slot_bytes, group.world);
    check_runtime(cudaMalloc(&region, bytes), "cudaMalloc(symmetric region)");
    check_runtime(cudaMemset(region, 0, bytes), "cudaMemset(symmetric region)");
    check_runtime(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    cudaIpcMemHandle_t handle;
    const cudaError_t status = cudaIpcGetMemHandle(&handle, region);
    if (status != cudaSuccess) {
        cudaFree(region);
        check_runtime(status, "cudaIpcGetMemHandle");
    }
    static_assert(sizeof handle == 64, "CUDA IPC handles are 64 bytes");
    std::memcpy(handle64, &handle, sizeof handle);
    group.regions[group.rank] = region;
    group.slot_bytes = slot_bytes;
}

void tp_symmetric_open(int device, const void* handles, int world) {
    std::lock_guard<std::mutex> lock(group_mutex);
    if (device < 0 || device >= 64 || !groups[device].comm) throw std::logic_error("tensor-parallel group is not initialised on this device");
    Group& group = groups[device];
    if (!handles || world != group.world || !group.regions[group.rank]) throw std::invalid_argument("handle table does not match the group");
    set_device(device);
    for (int r = 0; r < world; ++r) {
        if (r == group.rank || group.regions[r]) continue;
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, static_cast<const char*>(handles) + 64 * static_cast<std::size_t>(r), sizeof handle);
        void* mapped = nullptr;
        check_runtime(cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
        group.regions[r] = mapped;
    }
    group.mapped = true;
}

bool tp_symmetric_ready(int device, std::size_t bytes) {
    std::lock_guard<std::mutex> lock(group_mutex);
    return device >= 0 && device < 64 && groups[device].mapped && bytes <= groups[device].slot_bytes;
}

// Where this rank's partial rows of sum `slot` go in the region of rank `owner` (its own region, or a peer's as mapped here).
float* tp_partial_slot(int device, int slot, int owner) {
    std::lock_guard<std::mutex> lock(group_mutex);
    const Group& group = groups[device];
    if (owner < 0) owner = group.rank;
    return static_cast<float*>(b200_tp_slot(group.regions[owner], group.slot_bytes, group.world, slot, group.rank));
}

void tp_reduce_shadow(int device, int slot, std::int64_t rows, std::int64_t width, const void* norm_weight, int norm_dtype, float* out,
                      void* out_hi, void* out_lo, float* sumsq_out) {
    Group group;
    {
        std::lock_guard<std::mutex> lock(group_mutex);
        group = groups[device];
    }
    check(b200_tp_reduce_shadow(group.regions, group.rank, group.world, slot, group.slot_bytes, group.push ? 0 : 1, rows, width, norm_weight, norm_dtype, out,
                                out_hi, out_lo, sumsq_out, stream(device)), "peer-memory sum");
}

void tp_argmax_finish(int device, std::int32_t first_index, const float* best_value, const std::int32_t* best_index, std::int32_t parts,
                      std::int64_t rows, std::int64_t* next, std::int64_t* ids, std::int64_t* history, std::int64_t history_rows,
                      std::int32_t* counter, b200_kv_cache* const* caches, std::int32_t cache_count) {
    Group group;
    {
        std::lock_guard<std::mutex> lock(group_mutex);
        group = groups[device];
    }
    check(b200_tp_argmax_finish(group.regions, group.rank, group.world, group.slot_bytes, first_index, best_value, best_index, parts, rows, next,
                                ids, history, history_rows, counter, caches, cache_count, stream(device)), "cross-rank greedy choice");
}

int tp_world(int device) {
    std::lock_guard<std::mutex> lock(group_mutex);
    return device >= 0 && device < 64 && groups[device].comm ? groups[device].world : 1;
}
int tp_rank(int device) {
    std::lock_guard<std::mutex> lock(group_mutex);
    return device >= 0 && device < 64 && groups[device].comm ? groups[device].rank : 0;
}

// In-place sum over the group's ranks of `count` floats, ordered on the device's compute stream.
void tp_all_reduce(int device, float* data, std::size_t count) {
    Comm comm;
    {
        std::lock_guard<std::mutex> lock(group_mutex);
        comm = device >= 0 && device < 64 ? groups[device].comm : nullptr;
    }
    if (!comm) throw std::logic_error("tensor-parallel group is not initialised on this device");
    check_nccl(nccl().all_reduce(data, data, count, /*ncclFloat32*/ 7, /*ncclSum*/ 0, comm, static_cast<cudaStream_t>(stream(device))),
               "ncclAllReduce");
}

}  // namespace dl::runtime
