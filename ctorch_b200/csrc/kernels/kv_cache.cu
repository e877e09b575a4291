// Host object and small kernels of the paged KV cache (see kv_cache.cuh for the layout).
#include "kv_cache.cuh"

#include <new>
#include <vector>

namespace b200 {

KvView kv_view(const b200_kv_cache* c) {
    return KvView{{c->pool[0], c->pool[1]}, c->page_table, c->lengths, c->sequences, c->pages_per_seq,
                  c->page_size, c->kv_heads, c->head_dim, c->dtype, c->num_pages};
}
const CUtensorMap* kv_tensor_map(const b200_kv_cache* c, int which) { return c->has_maps ? &c->map[which] : nullptr; }

namespace {

__global__ void fill_lengths_kernel(int32_t* lengths, int n, int32_t value) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) lengths[i] = value;
}

struct AdvanceList { int32_t* lengths[64]; int32_t counts[64]; };
__global__ void advance_kernel(AdvanceList list, int caches, int32_t delta) {
    grid_dependency_wait();   // earlier kernels of the step still read the old lengths
    grid_launch_dependents();
    const int c = blockIdx.x;
    if (c >= caches) return;
    for (int i = threadIdx.x; i < list.counts[c]; i += blockDim.x) list.lengths[c][i] += delta;
}

// out [sequences, kv_heads, length, head_dim] f32
__global__ void gather_kernel(KvView kv, int which, int length, float* out) {
    const int64_t total = static_cast<int64_t>(kv.sequences) * kv.kv_heads * length * kv.head_dim;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(i % kv.head_dim);
        const int64_t r = i / kv.head_dim;
        const int position = static_cast<int>(r % length);
        const int head = static_cast<int>((r / length) % kv.kv_heads);
        const int sequence = static_cast<int>(r / length / kv.kv_heads);
        out[i] = kv_load(kv, which, kv_offset(kv, sequence, position, head) + d);
    }
}

// key/value [sequences, kv_heads, count, head_dim] f32 -> positions lengths[s] + t
__global__ void append_kernel(KvView kv, const float* key, const float* value, int count) {
    const int64_t pairs = static_cast<int64_t>(kv.sequences) * kv.kv_heads * count * (kv.head_dim / 2);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < pairs;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int half = kv.head_dim / 2;
        const int d = static_cast<int>(i % half) * 2;
        const int64_t r = i / half;
        const int t = static_cast<int>(r % count);
        const int head = static_cast<int>((r / count) % kv.kv_heads);
        const int sequence = static_cast<int>(r / count / kv.kv_heads);
        const int position = kv.lengths[sequence] + t;
        if (position >= kv.pages_per_seq * kv.page_size) continue;
        const int64_t at = r * kv.head_dim + d;
        kv_store_pair(kv, 0, sequence, position, head, d, key[at], key[at + 1]);
        kv_store_pair(kv, 1, sequence, position, head, d, value[at], value[at + 1]);
    }
}

int make_maps(b200_kv_cache* c) {
    c->has_maps = false;
    if (c->dtype != B200_BF16 || c->page_size != kFastPageSize || c->head_dim % 64 != 0) return B200_OK;
    encode_tiled_fn encode = tensor_map_encoder();
    if (!encode) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return B200_NO_DEVICE; }
    // 2-D view [token rows][head_dim] of a pool; one box = 64 tokens x 64 features (128-byte rows, 128B swizzle).
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(c->head_dim),
                                static_cast<cuuint64_t>(c->num_pages) * c->kv_heads * c->page_size};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(c->head_dim) * 2};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(kFastPageSize)};
    const cuuint32_t element_strides[2] = {1, 1};
    for (int which = 0; which < 2; ++which) {
        const CUresult result = encode(&c->map[which], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c->pool[which], dims, strides,
                                       box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (result != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with %d", static_cast<int>(result)); return B200_BAD_ARGUMENT; }
    }
    c->has_maps = true;
    return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_kv_cache_create(int32_t device, int32_t dtype, int32_t sequences, int32_t kv_heads, int32_t head_dim,
                         int32_t capacity, int32_t page_size, b200_kv_cache** out) {
    if (!out) return B200_BAD_ARGUMENT;
    *out = nullptr;
    if ((dtype != B200_F32 && dtype != B200_BF16) || sequences <= 0 || kv_heads <= 0 || head_dim <= 0 || (head_dim & 1)
        || capacity <= 0 || page_size <= 0) {
        set_error("b200_kv_cache_create: bad shape or dtype");
        return B200_BAD_ARGUMENT;
    }
    B200_CUDA(cudaSetDevice(device));
    device_status_word(device);  // allocated here so that no kernel launch (possibly under stream capture) has to
    auto* c = new (std::nothrow) b200_kv_cache{};
    if (!c) return B200_BAD_ARGUMENT;
    c->device = device; c->dtype = dtype; c->sequences = sequences; c->kv_heads = kv_heads; c->head_dim = head_dim;
    c->capacity = capacity; c->page_size = page_size;
    c->pages_per_seq = (capacity + page_size - 1) / page_size;
    c->num_pages = c->pages_per_seq * sequences;
    c->pool_bytes = static_cast<size_t>(c->num_pages) * kv_heads * page_size * head_dim * (dtype == B200_BF16 ? 2 : 4);
    auto fail = [&](int status) { b200_kv_cache_release(c); return status; };
    for (int which = 0; which < 2; ++which) {
        cudaError_t e = cudaMalloc(&c->pool[which], c->pool_bytes);
        if (e != cudaSuccess) return fail(cuda_status(e, "cudaMalloc(KV pool)"));
        // Pages start as zeros so that masked positions of a partly filled page are finite.
        e = cudaMemset(c->pool[which], 0, c->pool_bytes);
        if (e != cudaSuccess) return fail(cuda_status(e, "cudaMemset(KV pool)"));
    }
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->page_table), sizeof(int32_t) * c->num_pages);
    if (e != cudaSuccess) return fail(cuda_status(e, "cudaMalloc(page table)"));
    e = cudaMalloc(reinterpret_cast<void**>(&c->lengths), sizeof(int32_t) * sequences);
    if (e != cudaSuccess) return fail(cuda_status(e, "cudaMalloc(lengths)"));
    // Default assignment: logical page p of sequence s lives in physical page p * sequences + s, so that the
    // pages the batch touches in one step are neighbours in memory.
    std::vector<int32_t> table(static_cast<size_t>(c->num_pages));
    for (int s = 0; s < sequences; ++s)
        for (int p = 0; p < c->pages_per_seq; ++p) table[static_cast<size_t>(s) * c->pages_per_seq + p] = p * sequences + s;
    e = cudaMemcpy(c->page_table, table.data(), sizeof(int32_t) * table.size(), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(cuda_status(e, "cudaMemcpy(page table)"));
    e = cudaMemset(c->lengths, 0, sizeof(int32_t) * sequences);
    if (e != cudaSuccess) return fail(cuda_status(e, "cudaMemset(lengths)"));
    c->even_lengths = true;
    const int status = make_maps(c);
    if (status != B200_OK) return fail(status);
    *out = c;
    return B200_OK;
}

void b200_kv_cache_release(b200_kv_cache* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaFree(c->pool[0]); cudaFree(c->pool[1]); cudaFree(c->page_table); cudaFree(c->lengths);
    delete c;
}

int b200_kv_cache_set_lengths(b200_kv_cache* c, const int32_t* host_lengths, void* stream) {
    if (!c || !host_lengths) return B200_BAD_ARGUMENT;
    for (int s = 0; s < c->sequences; ++s)
        if (host_lengths[s] < 0 || host_lengths[s] > c->capacity) { set_error("KV cache length outside [0, capacity]"); return B200_BAD_ARGUMENT; }
    B200_CUDA(cudaMemcpyAsync(c->lengths, host_lengths, sizeof(int32_t) * c->sequences, cudaMemcpyHostToDevice, as_stream(stream)));
    B200_CUDA(cudaStreamSynchronize(as_stream(stream)));  // host_lengths may be pageable and reused by the caller
    c->even_lengths = true;
    for (int s = 1; s < c->sequences; ++s) c->even_lengths = c->even_lengths && host_lengths[s] == host_lengths[0];
    return B200_OK;
}
int b200_kv_cache_fill_lengths(b200_kv_cache* c, int32_t length, void* stream) {
    if (!c || length < 0 || length > c->capacity) { set_error("KV cache length outside [0, capacity]"); return B200_BAD_ARGUMENT; }
    fill_lengths_kernel<<<(c->sequences + 127) / 128, 128, 0, as_stream(stream)>>>(c->lengths, c->sequences, length);
    c->even_lengths = true;
    return cuda_status(cudaGetLastError(), "fill_lengths_kernel launch");
}
int b200_kv_cache_set_page_table(b200_kv_cache* c, const int32_t* host_table, void* stream) {
    if (!c || !host_table) return B200_BAD_ARGUMENT;
    std::vector<char> seen(static_cast<size_t>(c->num_pages), 0);
    for (int i = 0; i < c->num_pages; ++i) {
        if (host_table[i] < 0 || host_table[i] >= c->num_pages || seen[static_cast<size_t>(host_table[i])]) {
            set_error("page table must be a permutation of [0, pages)");
            return B200_BAD_ARGUMENT;
        }
        seen[static_cast<size_t>(host_table[i])] = 1;
    }
    B200_CUDA(cudaMemcpyAsync(c->page_table, host_table, sizeof(int32_t) * c->num_pages, cudaMemcpyHostToDevice, as_stream(stream)));
    B200_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return B200_OK;
}
int32_t* b200_kv_cache_lengths(b200_kv_cache* c) { return c->lengths; }
int32_t* b200_kv_cache_page_table(b200_kv_cache* c) { return c->page_table; }
void* b200_kv_cache_pool(b200_kv_cache* c, int32_t which) { return c->pool[which ? 1 : 0]; }
int32_t b200_kv_cache_pages_per_sequence(const b200_kv_cache* c) { return c->pages_per_seq; }
int32_t b200_kv_cache_page_size(const b200_kv_cache* c) { return c->page_size; }
size_t b200_kv_cache_pool_bytes(const b200_kv_cache* c) { return c->pool_bytes; }

int b200_kv_cache_advance(b200_kv_cache* const* caches, int32_t count, int32_t delta, void* stream) {
    if (!caches || count < 0) return B200_BAD_ARGUMENT;
    for (int first = 0; first < count; first += 64) {
        AdvanceList list{};
        const int n = count - first < 64 ? count - first : 64;
        for (int i = 0; i < n; ++i) { list.lengths[i] = caches[first + i]->lengths; list.counts[i] = caches[first + i]->sequences; }
        const int status = cuda_status(launch_dependent(advance_kernel, dim3(n), dim3(128), 0, as_stream(stream), list, n, delta), "advance_kernel launch");
        if (status != B200_OK) return status;
    }
    return B200_OK;
}

int b200_kv_cache_gather(const b200_kv_cache* c, int32_t which, int32_t length, float* out, void* stream) {
    if (!c || !out || length < 0 || length > c->capacity) { set_error("b200_kv_cache_gather: bad length"); return B200_BAD_ARGUMENT; }
    if (length == 0) return B200_OK;
    const int64_t total = static_cast<int64_t>(c->sequences) * c->kv_heads * length * c->head_dim;
    const int blocks = static_cast<int>((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    gather_kernel<<<blocks, 256, 0, as_stream(stream)>>>(kv_view(c), which ? 1 : 0, length, out);
    return cuda_status(cudaGetLastError(), "gather_kernel launch");
}

int b200_kv_cache_append(b200_kv_cache* c, const float* key, const float* value, int32_t count, void* stream) {
    if (!c || !key || !value || count < 0) return B200_BAD_ARGUMENT;
    if (count == 0) return B200_OK;
    const int64_t pairs = static_cast<int64_t>(c->sequences) * c->kv_heads * count * (c->head_dim / 2);
    const int blocks = static_cast<int>((pairs + 255) / 256 < 4096 ? (pairs + 255) / 256 : 4096);
    append_kernel<<<blocks, 256, 0, as_stream(stream)>>>(kv_view(c), key, value, count);
    return cuda_status(cudaGetLastError(), "append_kernel launch");
}

}  // extern "C"
