// Small operators of the token loop (embedding gather, stand-alone RMSNorm, argmax, row select) and the host
// utilities shared by the kernel files (error text, driver entry point lookup, device status word).
#include "linear_common.cuh"
#include "kv_cache.cuh"

#include <cstring>
#include <mutex>


namespace b200 {

namespace {
thread_local char error_text[512];
std::mutex status_mutex;
int32_t* status_words[64];
}  // namespace

void set_error(const char* format, ...) {
    va_list args;
    va_start(args, format);
    std::vsnprintf(error_text, sizeof error_text, format, args);
    va_end(args);
}

int cuda_status(cudaError_t error, const char* what) {
    if (error == cudaSuccess) return B200_OK;
    set_error("CUDA: %s: %s", what, cudaGetErrorString(error));
    return static_cast<int>(error);
}

int32_t* device_status_word(int device) {
    std::lock_guard<std::mutex> lock(status_mutex);
    if (device < 0 || device >= 64) return nullptr;
    if (!status_words[device]) {
        int current = 0;
        cudaGetDevice(&current);
        cudaSetDevice(device);
        if (cudaMalloc(reinterpret_cast<void**>(&status_words[device]), sizeof(int32_t)) == cudaSuccess)
            cudaMemset(status_words[device], 0, sizeof(int32_t));
        else
            status_words[device] = nullptr;
        cudaSetDevice(current);
    }
    return status_words[device];
}

int32_t* device_status_word_if_allocated(int device) {
    std::lock_guard<std::mutex> lock(status_mutex);
    return device >= 0 && device < 64 ? status_words[device] : nullptr;
}

encode_tiled_fn tensor_map_encoder() {
    static encode_tiled_fn cached = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess
            || result != cudaDriverEntryPointSuccess)
            entry = nullptr;
        return reinterpret_cast<encode_tiled_fn>(entry);
    }();
    return cached;
}

namespace {

template <class T>
__global__ void embedding_kernel(const T* table, const int64_t* ids, int64_t rows, int64_t vocab, int64_t width, float* out,
                                 int32_t* status) {
    grid_dependency_wait();   // the ids may come from the previous step's token feedback
    grid_launch_dependents();
    const int64_t row = blockIdx.x;
    int64_t id = ids[row];
    if (id < 0 || id >= vocab) {  // the host API validates ids it can see; device-resident ids are clamped and flagged
        if (threadIdx.x == 0) atomicExch(status, B200_BAD_ARGUMENT);
        id = id < 0 ? 0 : vocab - 1;
    }
    for (int64_t c = threadIdx.x; c < width; c += blockDim.x) out[row * width + c] = load_as_f32(table, id * width + c);
}

// One CTA per row; f64 accumulation and f64 scale, one rounding (src/kernels/cpu/normalization.cpp:39-51).
template <class T>
__global__ void rms_norm_kernel(const float* x, const T* weight, int64_t width, double eps, float* out) {
    __shared__ double partial[32];
    __shared__ double inverse_std;
    const float* row = x + blockIdx.x * width;
    double squares = 0.0;
    for (int64_t c = threadIdx.x; c < width; c += blockDim.x) {
        const double v = static_cast<double>(row[c]);
        squares += v * v;
    }
    squares = warp_sum(squares);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = squares;
    __syncthreads();
    if (threadIdx.x < 32) {
        double v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0;
        v = warp_sum(v);
        if (threadIdx.x == 0) inverse_std = 1.0 / sqrt(v / static_cast<double>(width) + eps);
    }
    __syncthreads();
    for (int64_t c = threadIdx.x; c < width; c += blockDim.x) {
        double v = static_cast<double>(row[c]) * inverse_std;
        if (weight) v *= static_cast<double>(load_as_f32(weight, c));
        out[blockIdx.x * width + c] = static_cast<float>(v);
    }
}

// (value, index) ordering of the reference: a NaN beats everything and the first NaN / first maximum wins.
struct Best { float value; int64_t index; };
__device__ __forceinline__ bool better(const Best& a, const Best& b) {  // is a preferred over b?
    const bool an = a.value != a.value, bn = b.value != b.value;
    if (an || bn) return an && (!bn || a.index < b.index);
    return a.value > b.value || (a.value == b.value && a.index < b.index);
}
__global__ void argmax_kernel(const float* x, int64_t width, int64_t* index) {
    __shared__ Best partial[32];
    grid_dependency_wait();
    grid_launch_dependents();
    const float* row = x + blockIdx.x * width;
    Best best{row[0], 0};
    for (int64_t c = threadIdx.x; c < width; c += blockDim.x) {
        const Best candidate{row[c], c};
        if (better(candidate, best)) best = candidate;
    }
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
        if (better(other, best)) best = other;
    }
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : Best{row[0], 0};
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
            if (better(other, best)) best = other;
        }
        if (threadIdx.x == 0) index[blockIdx.x] = best.index;
    }
}

__global__ void select_rows_kernel(const float* x, int64_t first, int64_t stride, int64_t width, float* out) {
    const float* row = x + (first + blockIdx.x * stride) * width;
    for (int64_t c = threadIdx.x; c < width; c += blockDim.x) out[blockIdx.x * width + c] = row[c];
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

const char* b200_last_error(void) { return error_text; }

int b200_embedding(const void* table, int32_t table_dtype, const int64_t* ids, int64_t rows, int64_t vocab, int64_t width,
                   float* out, void* stream) {
    if (!table || !ids || !out || rows < 0 || vocab <= 0 || width <= 0) { set_error("b200_embedding: bad pointer or size"); return B200_BAD_ARGUMENT; }
    if (rows == 0) return B200_OK;
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    int32_t* status = device_status_word(device);
    if (!status) { set_error("b200_embedding: the device status word could not be allocated"); return B200_NO_DEVICE; }
    const int threads = width >= 256 ? 256 : 64;
    if (table_dtype == B200_BF16)
        return cuda_status(launch_dependent(embedding_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>(rows)), dim3(threads), 0, as_stream(stream),
                                            static_cast<const __nv_bfloat16*>(table), ids, rows, vocab, width, out, status), "embedding_kernel launch");
    if (table_dtype == B200_F32)
        return cuda_status(launch_dependent(embedding_kernel<float>, dim3(static_cast<unsigned>(rows)), dim3(threads), 0, as_stream(stream),
                                            static_cast<const float*>(table), ids, rows, vocab, width, out, status), "embedding_kernel launch");
    set_error("b200_embedding: table dtype %d is not f32 or bf16", table_dtype);
    return B200_UNSUPPORTED;
}

int b200_rms_norm(const float* x, const void* weight, int32_t weight_dtype, int64_t rows, int64_t width, double eps,
                  float* out, void* stream) {
    if (!x || !out || rows < 0 || width <= 0) { set_error("b200_rms_norm: bad pointer or size"); return B200_BAD_ARGUMENT; }
    if (rows == 0) return B200_OK;
    if (weight && weight_dtype == B200_BF16)
        rms_norm_kernel<<<static_cast<unsigned>(rows), 256, 0, as_stream(stream)>>>(x, static_cast<const __nv_bfloat16*>(weight), width, eps, out);
    else if (!weight || weight_dtype == B200_F32)
        rms_norm_kernel<<<static_cast<unsigned>(rows), 256, 0, as_stream(stream)>>>(x, static_cast<const float*>(weight), width, eps, out);
    else { set_error("b200_rms_norm: weight dtype %d is not f32 or bf16", weight_dtype); return B200_UNSUPPORTED; }
    return cuda_status(cudaGetLastError(), "rms_norm_kernel launch");
}

int b200_argmax(const float* x, int64_t rows, int64_t width, int64_t* index, void* stream) {
    if (!x || !index || rows < 0 || width <= 0) { set_error("b200_argmax: bad pointer or size"); return B200_BAD_ARGUMENT; }
    if (rows == 0) return B200_OK;
    return cuda_status(launch_dependent(argmax_kernel, dim3(static_cast<unsigned>(rows)), dim3(width >= 4096 ? 1024 : 256), 0, as_stream(stream),
                                        x, width, index), "argmax_kernel launch");
}

int b200_select_rows(const float* x, int64_t first, int64_t stride, int64_t rows_out, int64_t width, float* out, void* stream) {
    if (!x || !out || rows_out < 0 || width <= 0 || first < 0 || stride <= 0) { set_error("b200_select_rows: bad pointer or size"); return B200_BAD_ARGUMENT; }
    if (rows_out == 0) return B200_OK;
    select_rows_kernel<<<static_cast<unsigned>(rows_out), 256, 0, as_stream(stream)>>>(x, first, stride, width, out);
    return cuda_status(cudaGetLastError(), "select_rows_kernel launch");
}

int b200_take_device_status(int32_t device, void* stream, int32_t* status) {
    if (!status) return B200_BAD_ARGUMENT;
    int32_t* word = device_status_word(device);
    if (!word) { set_error("no status word for device %d", device); return B200_NO_DEVICE; }
    B200_CUDA(cudaMemcpyAsync(status, word, sizeof(int32_t), cudaMemcpyDeviceToHost, as_stream(stream)));
    B200_CUDA(cudaStreamSynchronize(as_stream(stream)));
    if (*status) B200_CUDA(cudaMemsetAsync(word, 0, sizeof(int32_t), as_stream(stream)));
    return B200_OK;
}

}  // extern "C"

namespace b200 {
namespace {

__global__ void rotary_kernel(const float* x, int64_t pairs, int64_t length, int64_t half, const float* cosine,
                              const float* sine, float* out) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < pairs;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t j = i % half, l = (i / half) % length;
        const float even = x[2 * i], odd = x[2 * i + 1];
        const float c = cosine[l * half + j], s = sine[l * half + j];
        out[2 * i] = __fsub_rn(__fmul_rn(even, c), __fmul_rn(odd, s));
        out[2 * i + 1] = __fadd_rn(__fmul_rn(even, s), __fmul_rn(odd, c));
    }
}

__global__ void permute_0213_kernel(const float* in, int64_t a, int64_t b, int64_t c, int64_t d, float* out) {
    const int64_t total = a * b * c * d;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t id = i % d, ib = (i / d) % b, ic = (i / d / b) % c, ia = i / d / b / c;  // i indexes out [a,c,b,d]
        out[i] = in[((ia * b + ib) * c + ic) * d + id];
    }
}

// Dense copy of a permuted view: out axis i is in axis order[i]; `size` and `stride` are those of the output axes, the
// strides measured in the input.
struct PermuteShape { int64_t size[8], stride[8]; int32_t rank; };
__global__ void permute_kernel(const float* in, const PermuteShape shape, int64_t total, float* out) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int64_t rest = i, source = 0;
        for (int axis = shape.rank - 1; axis >= 0; --axis) {
            source += (rest % shape.size[axis]) * shape.stride[axis];
            rest /= shape.size[axis];
        }
        out[i] = in[source];
    }
}

__global__ void token_feedback_kernel(const int64_t* next, int64_t batch, int64_t* ids, int64_t* history,
                                      int64_t history_rows, int32_t* counter) {
    grid_dependency_wait();
    grid_launch_dependents();
    const int32_t step = *counter;
    for (int64_t s = threadIdx.x; s < batch; s += blockDim.x) {
        const int64_t token = next[s];
        if (ids) ids[s] = token;
        if (history && step < history_rows) history[static_cast<int64_t>(step) * batch + s] = token;
    }
    __syncthreads();
    if (threadIdx.x == 0) *counter = step + 1;
}

// Merge of the per-tile candidates of the fused logits + argmax.  Every CTA takes eight rows, one per warp: the lanes walk the
// tiles, a butterfly leaves the row's choice, and lane 0 does the token bookkeeping of token_feedback_kernel for that row.
// The CTA that finishes last (a ticket in device memory; the library issues these launches on one stream per device, so
// one word serves) closes the step: cache lengths move on and the step counter is advanced - only then, because every
// CTA reads the counter when it starts.
struct LengthList { int32_t* lengths[64]; int32_t counts[64]; int32_t caches; };
__device__ unsigned int argmax_finish_ticket;
constexpr int kFinishWarps = 8;
__global__ void __launch_bounds__(kFinishWarps * 32) argmax_finish_kernel(const float* best_value, const int32_t* best_index, int parts, int64_t rows,
                                                                          int64_t* next, int64_t* ids, int64_t* history, int64_t history_rows,
                                                                          int32_t* counter, const LengthList advance) {
    __shared__ unsigned int last;
    grid_dependency_wait();
    grid_launch_dependents();
    const int32_t step = *counter;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kFinishWarps + warp;
    if (row < rows) {
        Candidate best{-INFINITY, INT32_MAX};
        for (int t0 = 0; t0 < parts; t0 += 32 * 8) {   // eight independent loads per lane in flight
            Candidate batch[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = t0 + u * 32 + lane;
                batch[u] = t < parts ? Candidate{__ldg(best_value + static_cast<int64_t>(t) * rows + row), __ldg(best_index + static_cast<int64_t>(t) * rows + row)}
                                     : Candidate{-INFINITY, INT32_MAX};
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (preferred(batch[u], best)) best = batch[u];
        }
        for (int o = 16; o > 0; o >>= 1) {
            const Candidate other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
            if (preferred(other, best)) best = other;
        }
        if (lane == 0) {
            const int64_t token = best.index;
            next[row] = token;
            if (ids) ids[row] = token;
            if (history && step < history_rows) history[static_cast<int64_t>(step) * rows + row] = token;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        last = atomicAdd(&argmax_finish_ticket, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!last) return;
    // end of a step: the caches (one per layer) move on by the token every earlier kernel of the step appended and read
    for (int c = 0; c < advance.caches; ++c)
        for (int i = threadIdx.x; i < advance.counts[c]; i += blockDim.x) advance.lengths[c][i] += 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        argmax_finish_ticket = 0;
        *counter = step + 1;
    }
}

// One CTA per row.  Thread t owns the contiguous slice [t * chunk, (t + 1) * chunk) of the row, so per-thread f64 sums
// followed by a scan over the threads give running sums in index order.
constexpr int kSampleThreads = 1024;
__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const float* x, int64_t width, float temperature, const double* uniform,
                                                                int64_t* index) {
    __shared__ float reduce_f[32];
    __shared__ double reduce_d[32];
    __shared__ double prefix[kSampleThreads];
    __shared__ long long chosen;
    grid_dependency_wait();
    grid_launch_dependents();
    const float* row = x + blockIdx.x * width;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t chunk = (width + kSampleThreads - 1) / kSampleThreads;
    const int64_t begin = min(width, threadIdx.x * chunk), end = min(width, begin + chunk);
    // max of x / T
    float m = -INFINITY;
    for (int64_t c = begin; c < end; ++c) m = fmaxf(m, __fdiv_rn(row[c], temperature));
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) reduce_f[warp] = m;
    __syncthreads();
    m = reduce_f[lane];
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // sum of exp(v - max): the softmax denominator (f32 terms, f64 sum)
    double mine = 0.0;
    for (int64_t c = begin; c < end; ++c) mine += static_cast<double>(expf(__fsub_rn(__fdiv_rn(row[c], temperature), m)));
    double total = mine;
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    __syncthreads();
    if (lane == 0) reduce_d[warp] = total;
    __syncthreads();
    total = 0.0;
    for (int w = 0; w < kSampleThreads / 32; ++w) total += reduce_d[w];
    const float denominator = static_cast<float>(total);
    // probabilities p = e / denominator (f32), their f64 running sums per thread, scan over threads
    double slice = 0.0;
    for (int64_t c = begin; c < end; ++c) slice += static_cast<double>(__fdiv_rn(expf(__fsub_rn(__fdiv_rn(row[c], temperature), m)), denominator));
    prefix[threadIdx.x] = slice;
    if (threadIdx.x == 0) chosen = -1;
    __syncthreads();
    if (warp == 0) {   // exclusive scan of 1024 slices: each lane scans 32 consecutive entries, then the lanes
        double run = 0.0;
        for (int i = 0; i < 32; ++i) {
            const double v = prefix[lane * 32 + i];
            prefix[lane * 32 + i] = run;
            run += v;
        }
        double before = run;
        for (int o = 1; o < 32; o <<= 1) {
            const double other = __shfl_up_sync(0xffffffffu, before, o);
            if (lane >= o) before += other;
        }
        before -= run;
        for (int i = 0; i < 32; ++i) prefix[lane * 32 + i] += before;
        if (lane == 31) reduce_d[0] = before + run;   // sum of all p
    }
    __syncthreads();
    const double target = uniform[blockIdx.x] * reduce_d[0];
    const double start = prefix[threadIdx.x];
    if (begin < end && start <= target && target < start + slice) {
        double run = start;
        long long found = end - 1;
        for (int64_t c = begin; c < end; ++c) {
            run += static_cast<double>(__fdiv_rn(expf(__fsub_rn(__fdiv_rn(row[c], temperature), m)), denominator));
            if (run > target) { found = c; break; }
        }
        chosen = found;   // the slices are disjoint: at most one thread gets here
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        long long result = chosen;
        if (result < 0) {   // u * total landed on or past the last boundary: the last index with a non-zero probability
            result = width - 1;
            while (result > 0 && expf(__fsub_rn(__fdiv_rn(row[result], temperature), m)) == 0.0f) --result;
        }
        index[blockIdx.x] = result;
    }
}

unsigned blocks_for(int64_t n) { return static_cast<unsigned>((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192); }

}  // namespace
}  // namespace b200

extern "C" {

int b200_rotary(const float* x, int64_t outer, int64_t length, int64_t head_dim, const float* cosine, const float* sine,
                float* out, void* stream) {
    if (!x || !cosine || !sine || !out || outer < 0 || length < 0 || head_dim <= 0 || (head_dim & 1)) { set_error("b200_rotary: bad pointer or size"); return B200_BAD_ARGUMENT; }
    const int64_t pairs = outer * length * (head_dim / 2);
    if (pairs == 0) return B200_OK;
    b200::rotary_kernel<<<b200::blocks_for(pairs), 256, 0, as_stream(stream)>>>(x, pairs, length, head_dim / 2, cosine, sine, out);
    return cuda_status(cudaGetLastError(), "rotary_kernel launch");
}

int b200_argmax_finish(const float* best_value, const int32_t* best_index, int32_t parts, int64_t rows, int64_t* next, int64_t* ids,
                       int64_t* history, int64_t history_rows, int32_t* counter, b200_kv_cache* const* caches, int32_t cache_count,
                       void* stream) {
    if (!best_value || !best_index || !next || !counter || parts <= 0 || rows <= 0 || cache_count < 0 || cache_count > 64
        || (cache_count > 0 && !caches)) {
        set_error("b200_argmax_finish: bad pointer or size");
        return B200_BAD_ARGUMENT;
    }
    b200::LengthList advance{};
    advance.caches = cache_count;
    for (int i = 0; i < cache_count; ++i) {
        if (!caches[i]) { set_error("b200_argmax_finish: cache %d is NULL", i); return B200_BAD_ARGUMENT; }
        advance.lengths[i] = caches[i]->lengths;
        advance.counts[i] = caches[i]->sequences;
    }
    const unsigned ctas = static_cast<unsigned>((rows + b200::kFinishWarps - 1) / b200::kFinishWarps);
    return cuda_status(launch_dependent(b200::argmax_finish_kernel, dim3(ctas), dim3(b200::kFinishWarps * 32), 0, as_stream(stream), best_value, best_index,
                                        static_cast<int>(parts), rows, next, ids, history, history_rows, counter, advance),
                       "argmax_finish_kernel launch");
}

int b200_sample(const float* x, int64_t rows, int64_t width, double temperature, const double* uniform, int64_t* index, void* stream) {
    if (!x || !uniform || !index || rows < 0 || width <= 0 || !(temperature > 0.0)) { set_error("b200_sample: bad pointer, size or temperature"); return B200_BAD_ARGUMENT; }
    if (rows == 0) return B200_OK;
    return cuda_status(launch_dependent(b200::sample_kernel, dim3(static_cast<unsigned>(rows)), dim3(b200::kSampleThreads), 0, as_stream(stream),
                                        x, width, static_cast<float>(temperature), uniform, index), "sample_kernel launch");
}

int b200_permute_0213(const float* in, int64_t a, int64_t b, int64_t c, int64_t d, float* out, void* stream) {
    if (!in || !out || a < 0 || b < 0 || c < 0 || d < 0) { set_error("b200_permute_0213: bad pointer or size"); return B200_BAD_ARGUMENT; }
    if (a * b * c * d == 0) return B200_OK;
    b200::permute_0213_kernel<<<b200::blocks_for(a * b * c * d), 256, 0, as_stream(stream)>>>(in, a, b, c, d, out);
    return cuda_status(cudaGetLastError(), "permute_0213_kernel launch");
}

int b200_permute(const float* in, const int64_t* sizes, const int64_t* order, int32_t rank, float* out, void* stream) {
    if (!in || !out || !sizes || !order || rank < 1 || rank > 8) { set_error("b200_permute: bad pointer or rank"); return B200_BAD_ARGUMENT; }
    b200::PermuteShape shape{};
    int64_t stride[8], count = 1;
    bool seen[8] = {false, false, false, false, false, false, false, false};
    for (int i = rank - 1; i >= 0; --i) {
        if (sizes[i] < 0) { set_error("b200_permute: negative size"); return B200_BAD_ARGUMENT; }
        stride[i] = count;
        count *= sizes[i];
    }
    for (int i = 0; i < rank; ++i) {
        if (order[i] < 0 || order[i] >= rank || seen[order[i]]) { set_error("b200_permute: order is not a permutation"); return B200_BAD_ARGUMENT; }
        seen[order[i]] = true;
        shape.size[i] = sizes[order[i]];
        shape.stride[i] = stride[order[i]];
    }
    shape.rank = rank;
    if (count == 0) return B200_OK;
    b200::permute_kernel<<<b200::blocks_for(count), 256, 0, as_stream(stream)>>>(in, shape, count, out);
    return cuda_status(cudaGetLastError(), "permute_kernel launch");
}

int b200_token_feedback(const int64_t* next, int64_t batch, int64_t* ids, int64_t* history, int64_t history_rows,
                        int32_t* counter, void* stream) {
    if (!next || !counter || batch <= 0) { set_error("b200_token_feedback: bad pointer or size"); return B200_BAD_ARGUMENT; }
    return cuda_status(launch_dependent(b200::token_feedback_kernel, dim3(1), dim3(256), 0, as_stream(stream), next, batch, ids, history,
                                        history_rows, counter), "token_feedback_kernel launch");
}

}  // extern "C"

namespace b200 {
namespace {
__global__ void scaled_add_kernel(float* y, const float* x, float scale, int64_t count) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        y[i] = __fadd_rn(y[i], __fmul_rn(x[i], scale));
}
}  // namespace
}  // namespace b200

extern "C" int b200_scaled_add(float* y, const float* x, float scale, int64_t count, void* stream) {
    if (!y || !x || count < 0) { set_error("b200_scaled_add: bad pointer or size"); return B200_BAD_ARGUMENT; }
    if (count == 0) return B200_OK;
    b200::scaled_add_kernel<<<b200::blocks_for(count), 256, 0, as_stream(stream)>>>(y, x, scale, count);
    return cuda_status(cudaGetLastError(), "scaled_add_kernel launch");
}

namespace b200 {
namespace {
// One CTA per row: gather, f32 copy, shadow of row * norm_weight, the row's sum of squares (parts = 1).
template <class T>
__global__ void embedding_shadow_kernel(const T* table, const int64_t* ids, int64_t vocab, int64_t width, const void* norm_weight,
                                        int norm_dtype, float* out, __nv_bfloat16* out_hi, __nv_bfloat16* out_lo,
                                        float* sumsq_out, int32_t* status) {
    __shared__ float partial[32];
    grid_dependency_wait();   // the ids may come from the previous step's token feedback
    grid_launch_dependents();
    const int64_t row = blockIdx.x;
    int64_t id = ids ? ids[row] : row;   // without ids the table is the activation matrix itself
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(status, B200_BAD_ARGUMENT);
        id = id < 0 ? 0 : vocab - 1;
    }
    float squares = 0.0f;
    for (int64_t c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = load_as_f32(table, id * width + c);
        if (out) out[row * width + c] = v;
        squares += v * v;
        float w = 1.0f;
        if (norm_weight)
            w = norm_dtype == B200_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(norm_weight)[c])
                                        : static_cast<const float*>(norm_weight)[c];
        const float scaled = __fmul_rn(v, w);
        const __nv_bfloat16 hi = __float2bfloat16_rn(scaled);
        out_hi[row * width + c] = hi;
        out_lo[row * width + c] = __float2bfloat16_rn(scaled - __bfloat162float(hi));
    }
    squares = warp_sum(squares);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = squares;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0f;
        v = warp_sum(v);
        if (threadIdx.x == 0) sumsq_out[row] = v;
    }
}
}  // namespace
}  // namespace b200

extern "C" int b200_embedding_shadow(const void* table, int32_t table_dtype, const int64_t* ids, int64_t rows, int64_t vocab,
                                     int64_t width, const void* norm_weight, int32_t norm_dtype, float* out, void* out_hi,
                                     void* out_lo, float* sumsq_out, void* stream) {
    if (!table || !ids || !out || !out_hi || !out_lo || !sumsq_out || rows < 0 || vocab <= 0 || width <= 0) {
        set_error("b200_embedding_shadow: bad pointer or size");
        return B200_BAD_ARGUMENT;
    }
    if (rows == 0) return B200_OK;
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    int32_t* status = device_status_word(device);
    if (!status) { set_error("b200_embedding_shadow: the device status word could not be allocated"); return B200_NO_DEVICE; }
    auto* hi = static_cast<__nv_bfloat16*>(out_hi);
    auto* lo = static_cast<__nv_bfloat16*>(out_lo);
    if (table_dtype == B200_BF16)
        return cuda_status(launch_dependent(b200::embedding_shadow_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>(rows)), dim3(256), 0,
                                            as_stream(stream), static_cast<const __nv_bfloat16*>(table), ids, vocab, width, norm_weight,
                                            static_cast<int>(norm_dtype), out, hi, lo, sumsq_out, status), "embedding_shadow_kernel launch");
    if (table_dtype == B200_F32)
        return cuda_status(launch_dependent(b200::embedding_shadow_kernel<float>, dim3(static_cast<unsigned>(rows)), dim3(256), 0,
                                            as_stream(stream), static_cast<const float*>(table), ids, vocab, width, norm_weight,
                                            static_cast<int>(norm_dtype), out, hi, lo, sumsq_out, status), "embedding_shadow_kernel launch");
    set_error("b200_embedding_shadow: table dtype %d is not f32 or bf16", table_dtype);
    return B200_UNSUPPORTED;
}

extern "C" int b200_shadow_from_rows(const float* x, int64_t rows, int64_t width, const void* norm_weight, int32_t norm_dtype,
                                     void* out_hi, void* out_lo, float* sumsq_out, void* stream) {
    if (!x || !out_hi || !out_lo || !sumsq_out || rows < 0 || width <= 0) { set_error("b200_shadow_from_rows: bad pointer or size"); return B200_BAD_ARGUMENT; }
    if (rows == 0) return B200_OK;
    int device = 0;
    B200_CUDA(cudaGetDevice(&device));
    int32_t* status = device_status_word(device);
    if (!status) { set_error("b200_shadow_from_rows: the device status word could not be allocated"); return B200_NO_DEVICE; }
    return cuda_status(launch_dependent(b200::embedding_shadow_kernel<float>, dim3(static_cast<unsigned>(rows)), dim3(256), 0, as_stream(stream),
                                        x, static_cast<const int64_t*>(nullptr), rows, width, norm_weight, static_cast<int>(norm_dtype),
                                        static_cast<float*>(nullptr), static_cast<__nv_bfloat16*>(out_hi), static_cast<__nv_bfloat16*>(out_lo),
                                        sumsq_out, status), "shadow_from_rows launch");
}
