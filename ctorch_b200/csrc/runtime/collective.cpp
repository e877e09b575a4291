// NCCL behind a dlopen'ed function table: the library keeps no link-time dependency on NCCL (it must load on
// machines without it) and uses whichever libnccl.so.2 the process already has (the one PyTorch loaded, if any).
// Used only by the KV-head tensor-parallel plan: all-reduce(sum) of the [rows, D] partial sums after the output
// projection and after the FFN down-projection, enqueued on the library's compute stream (capturable in a graph).
#include "dl/internal.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>

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
struct Group { Comm comm = nullptr; int rank = 0, world = 1; };
Group groups[64];

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
    Comm comm = nullptr;
    check_nccl(nccl().comm_init_rank(&comm, world, id, rank), "ncclCommInitRank");
    groups[device] = Group{comm, rank, world};
}

void tp_finalize(int device) {
    std::lock_guard<std::mutex> lock(group_mutex);
    if (device < 0 || device >= 64 || !groups[device].comm) return;
    set_device(device);
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream(device)));
    nccl().comm_destroy(groups[device].comm);
    groups[device] = Group{};
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
