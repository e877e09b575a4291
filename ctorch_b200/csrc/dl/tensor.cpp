// Device context, storage, dense tensors and the functional operators of the decoder path.
#include "dl/dl.h"

#include <algorithm>
#include "dl/internal.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <limits>
#include <mutex>
#include <stdexcept>

namespace dl {

namespace runtime {

namespace {
std::mutex stream_mutex;
cudaStream_t streams[64];
}  // namespace

void check(int status, const char* what) {
    if (status == B200_OK) return;
    throw std::runtime_error(std::string(what) + ": " + b200_last_error());
}
void check_cuda(int error, const char* what) {
    if (error == 0) return;
    throw std::runtime_error(std::string("CUDA: ") + what + ": " + cudaGetErrorString(static_cast<cudaError_t>(error)));
}

void* stream(int device) {
    std::lock_guard<std::mutex> lock(stream_mutex);
    if (device < 0 || device >= 64) throw std::invalid_argument("CUDA device index out of range");
    if (!streams[device]) {
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || device >= count)
            throw std::runtime_error("CUDA: no such device; this library has no CPU compute path");
        check_cuda(cudaSetDevice(device), "cudaSetDevice");
        check_cuda(cudaStreamCreateWithFlags(&streams[device], cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
    }
    return streams[device];
}

void set_device(int device) { check_cuda(cudaSetDevice(device), "cudaSetDevice"); }

Storage::Storage(std::size_t size, Device where, bool pin) : bytes(size), device(where), pinned(pin) {
    const std::size_t request = size ? size : 1;
    if (device.type == DeviceType::cuda) {
        stream(device.index);
        set_device(device.index);
        check_cuda(cudaMalloc(&data, request), "cudaMalloc");
    } else if (pinned) {
        check_cuda(cudaMallocHost(&data, request), "cudaMallocHost");
    } else {
        data = std::malloc(request);
        if (!data) throw std::bad_alloc();
    }
}
Storage::~Storage() {
    if (!data) return;
    if (device.type == DeviceType::cuda) {
        cudaSetDevice(device.index);
        cudaFree(data);
    } else if (pinned) {
        cudaFreeHost(data);
    } else {
        std::free(data);
    }
}

// Copies `bytes` between any two places; device copies are ordered on the device's stream and completed
// before returning when the host is involved.
void copy_bytes(void* dst, Device dst_device, const void* src, Device src_device, std::size_t bytes) {
    if (bytes == 0) return;
    if (dst_device.type == DeviceType::cpu && src_device.type == DeviceType::cpu) {
        std::memcpy(dst, src, bytes);
        return;
    }
    const int device = dst_device.type == DeviceType::cuda ? dst_device.index : src_device.index;
    auto s = static_cast<cudaStream_t>(stream(device));
    set_device(device);
    if (dst_device.type == DeviceType::cuda && src_device.type == DeviceType::cuda && dst_device.index != src_device.index) {
        check_cuda(cudaMemcpyPeerAsync(dst, dst_device.index, src, src_device.index, bytes, s), "cudaMemcpyPeerAsync");
        check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        return;
    }
    check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, s), "cudaMemcpyAsync");
    if (dst_device.type == DeviceType::cpu || src_device.type == DeviceType::cpu)
        check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize");
}

}  // namespace runtime

void synchronize(Device device) {
    if (device.type != DeviceType::cuda) return;
    runtime::set_device(device.index);
    runtime::check_cuda(cudaStreamSynchronize(static_cast<cudaStream_t>(runtime::stream(device.index))), "cudaStreamSynchronize");
}

// ---- Tensor ---------------------------------------------------------------------------------------------
namespace {
Shape dense_strides(const Shape& shape) {
    Shape strides(shape.size(), 1);
    for (std::size_t i = shape.size(); i-- > 1;) strides[i - 1] = strides[i] * (shape[i] > 0 ? shape[i] : 1);
    return strides;
}
Index count(const Shape& shape) {
    Index n = 1;
    for (auto d : shape) {
        if (d < 0) throw std::invalid_argument("negative dimension");
        n *= d;
    }
    return n;
}
Index wrap_axis(Index axis, Index rank) {
    if (axis < -rank || axis >= rank) throw std::out_of_range("axis out of range");
    return axis < 0 ? axis + rank : axis;
}
}  // namespace

Tensor::Tensor(std::shared_ptr<runtime::Storage> storage, Shape shape, DType dtype, std::size_t offset_bytes)
    : storage_(std::move(storage)), shape_(std::move(shape)), strides_(dense_strides(shape_)), dtype_(dtype), offset_(offset_bytes) {}

Index Tensor::size(Index axis) const { return shape_[static_cast<std::size_t>(wrap_axis(axis, ndim()))]; }
Index Tensor::numel() const { return count(shape_); }

Tensor empty(Shape shape, TensorOptions options) {
    const auto bytes = static_cast<std::size_t>(count(shape)) * element_size(options.dtype);
    return Tensor(std::make_shared<runtime::Storage>(bytes, options.device), std::move(shape), options.dtype);
}

namespace {
void fill_host(void* data, DType dtype, Index n, double value) {
    switch (dtype) {
    case DType::f32: { auto* p = static_cast<float*>(data); for (Index i = 0; i < n; ++i) p[i] = static_cast<float>(value); break; }
    case DType::f64: { auto* p = static_cast<double*>(data); for (Index i = 0; i < n; ++i) p[i] = value; break; }
    case DType::i64: { auto* p = static_cast<Index*>(data); for (Index i = 0; i < n; ++i) p[i] = static_cast<Index>(value); break; }
    case DType::boolean: { auto* p = static_cast<bool*>(data); for (Index i = 0; i < n; ++i) p[i] = value != 0; break; }
    case DType::bf16: { auto* p = static_cast<std::uint16_t*>(data); const auto b = internal::to_bf16(static_cast<float>(value)); for (Index i = 0; i < n; ++i) p[i] = b; break; }
    case DType::f16: throw std::invalid_argument("f16 tensors are outside the decoder path");
    }
}
}  // namespace

Tensor full(Shape shape, double value, TensorOptions options) {
    Tensor host = empty(shape, {options.dtype, Device::cpu()});
    fill_host(host.mutable_data(), options.dtype, host.numel(), value);
    return host.to(options.device);
}
Tensor zeros(Shape shape, TensorOptions options) { return full(std::move(shape), 0.0, options); }
Tensor ones(Shape shape, TensorOptions options) { return full(std::move(shape), 1.0, options); }

Tensor detail::from_host(const void* data, Shape shape, DType dtype, bool, Device device) {
    Tensor result = empty(std::move(shape), {dtype, device});
    runtime::copy_bytes(result.mutable_data(), device, data, Device::cpu(), result.nbytes());
    return result;
}

Tensor Tensor::to(Device target) const {
    if (target == device()) return *this;
    Tensor result = empty(shape_, {dtype_, target});
    runtime::copy_bytes(result.mutable_data(), target, raw_data(), device(), nbytes());
    return result;
}

Tensor Tensor::clone() const {
    Tensor result = empty(shape_, {dtype_, device()});
    runtime::copy_bytes(result.mutable_data(), device(), raw_data(), device(), nbytes());
    return result;
}

void Tensor::copy_to_host(void* destination) const {
    runtime::copy_bytes(destination, Device::cpu(), raw_data(), device(), nbytes());
}

template <class T> std::vector<T> Tensor::to_vector() const {
    constexpr DType want = std::is_same_v<T, float> ? DType::f32 : std::is_same_v<T, double> ? DType::f64 : DType::i64;
    Tensor host = to(Device::cpu()).astype(want);
    const T* p = host.data<T>();
    return std::vector<T>(p, p + host.numel());
}
template std::vector<float> Tensor::to_vector<float>() const;
template std::vector<double> Tensor::to_vector<double>() const;
template std::vector<Index> Tensor::to_vector<Index>() const;

Tensor Tensor::astype(DType target) const {
    if (target == dtype_) return *this;
    if (device().type == DeviceType::cuda) return to(Device::cpu()).astype(target).to(device());
    Tensor result = empty(shape_, {target, Device::cpu()});
    const Index n = numel();
    auto read = [&](Index i) -> double {
        switch (dtype_) {
        case DType::f32: return data<float>()[i];
        case DType::f64: return data<double>()[i];
        case DType::i64: return static_cast<double>(data<Index>()[i]);
        case DType::boolean: return data<bool>()[i] ? 1.0 : 0.0;
        case DType::bf16: return internal::from_bf16(data<std::uint16_t>()[i]);
        case DType::f16: break;
        }
        throw std::invalid_argument("f16 tensors are outside the decoder path");
    };
    for (Index i = 0; i < n; ++i) {
        const double v = read(i);
        switch (target) {
        case DType::f32: static_cast<float*>(result.mutable_data())[i] = static_cast<float>(v); break;
        case DType::f64: static_cast<double*>(result.mutable_data())[i] = v; break;
        case DType::i64: static_cast<Index*>(result.mutable_data())[i] = static_cast<Index>(v); break;
        case DType::boolean: static_cast<bool*>(result.mutable_data())[i] = v != 0; break;
        case DType::bf16: static_cast<std::uint16_t*>(result.mutable_data())[i] = internal::to_bf16(static_cast<float>(v)); break;
        case DType::f16: throw std::invalid_argument("f16 tensors are outside the decoder path");
        }
    }
    return result;
}

Tensor Tensor::reshape(Shape shape) const {
    Index known = 1, unknown = -1;
    for (std::size_t i = 0; i < shape.size(); ++i) {
        if (shape[i] == -1) {
            if (unknown >= 0) throw std::invalid_argument("reshape allows one inferred dimension");
            unknown = static_cast<Index>(i);
        } else known *= shape[i];
    }
    if (unknown >= 0) {
        if (known == 0 || numel() % known) throw std::invalid_argument("reshape cannot infer the dimension");
        shape[static_cast<std::size_t>(unknown)] = numel() / known;
    }
    if (count(shape) != numel()) throw std::invalid_argument("reshape changes the number of elements");
    return Tensor(storage_, std::move(shape), dtype_, offset_);
}

Tensor Tensor::narrow(Index axis, Index start, Index length) const {
    axis = wrap_axis(axis, ndim());
    const Index extent = shape_[static_cast<std::size_t>(axis)];
    if (start < 0) start += extent;
    if (start < 0 || length < 0 || start + length > extent) throw std::out_of_range("narrow range outside the axis");
    Index outer = 1, inner = 1;
    for (Index i = 0; i < axis; ++i) outer *= shape_[static_cast<std::size_t>(i)];
    for (Index i = axis + 1; i < ndim(); ++i) inner *= shape_[static_cast<std::size_t>(i)];
    Shape shape = shape_;
    shape[static_cast<std::size_t>(axis)] = length;
    const std::size_t row = static_cast<std::size_t>(inner) * element_size(dtype_);
    if (outer == 1) return Tensor(storage_, std::move(shape), dtype_, offset_ + static_cast<std::size_t>(start) * row);
    Tensor result = empty(shape, {dtype_, device()});
    if (result.numel() == 0) return result;
    const char* source = static_cast<const char*>(raw_data()) + static_cast<std::size_t>(start) * row;
    if (device().type == DeviceType::cpu) {
        for (Index o = 0; o < outer; ++o)
            std::memcpy(static_cast<char*>(result.mutable_data()) + static_cast<std::size_t>(o * length) * row,
                        source + static_cast<std::size_t>(o * extent) * row, static_cast<std::size_t>(length) * row);
    } else {
        runtime::set_device(device().index);
        runtime::check_cuda(cudaMemcpy2DAsync(result.mutable_data(), static_cast<std::size_t>(length) * row, source,
                                              static_cast<std::size_t>(extent) * row, static_cast<std::size_t>(length) * row,
                                              static_cast<std::size_t>(outer), cudaMemcpyDeviceToDevice,
                                              static_cast<cudaStream_t>(runtime::stream(device().index))),
                            "cudaMemcpy2DAsync");
    }
    return result;
}

Tensor Tensor::select(Index axis, Index index) const {
    axis = wrap_axis(axis, ndim());
    Tensor part = narrow(axis, index, 1);
    Shape shape = part.shape();
    shape.erase(shape.begin() + axis);
    return part.reshape(std::move(shape));
}

// ---- functional operators -------------------------------------------------------------------------------
namespace {
int cuda_index(const Tensor& t, const char* op) {
    if (t.device().type != DeviceType::cuda)
        throw std::invalid_argument(std::string(op) + ": tensors must live on a CUDA device (this library has no CPU compute path)");
    return t.device().index;
}
int weight_code(DType dtype, const char* op) {
    if (dtype == DType::f32) return B200_F32;
    if (dtype == DType::bf16) return B200_BF16;
    throw std::invalid_argument(std::string(op) + ": weights must be f32 or bf16");
}
Tensor as_f32(const Tensor& t) { return t.dtype() == DType::f32 ? t : t.astype(DType::f32); }
}  // namespace

Tensor linear(const Tensor& input, const Tensor& weight, std::optional<Tensor> bias) {
    const int device = cuda_index(input, "linear");
    if (weight.device() != input.device()) throw std::invalid_argument("linear inputs must share a device");
    if (bias) throw std::invalid_argument("linear: bias is not part of the decoder path");
    if (weight.ndim() != 2 || input.ndim() < 1 || input.size(-1) != weight.size(1))
        throw std::invalid_argument("linear: input features do not match the weight");
    const Tensor x = as_f32(input);
    Shape shape = x.shape();
    shape.back() = weight.size(0);
    Tensor result = empty(shape, {DType::f32, input.device()});
    const Index rows = x.numel() / x.size(-1);
    runtime::set_device(device);
    runtime::check(b200_linear(x.data<float>(), rows, x.size(-1), weight.raw_data(), weight_code(weight.dtype(), "linear"),
                               weight.size(0), nullptr, 0, 0.0, B200_EPI_STORE, nullptr, nullptr,
                               static_cast<float*>(result.mutable_data()), runtime::stream(device)), "linear");
    return result;
}

Tensor embedding(const Tensor& indices, const Tensor& weight) {
    const int device = cuda_index(indices, "embedding");
    if (weight.device() != indices.device()) throw std::invalid_argument("embedding inputs must share a device");
    if (indices.dtype() != DType::i64 || weight.ndim() != 2) throw std::invalid_argument("embedding expects int64 indices and a matrix");
    Shape shape = indices.shape();
    shape.push_back(weight.size(1));
    Tensor result = empty(shape, {DType::f32, indices.device()});
    runtime::set_device(device);
    runtime::check(b200_embedding(weight.raw_data(), weight_code(weight.dtype(), "embedding"), indices.data<Index>(), indices.numel(),
                                  weight.size(0), weight.size(1), static_cast<float*>(result.mutable_data()), runtime::stream(device)),
                   "embedding");
    return result;
}

Tensor rms_norm(const Tensor& input, const Shape& normalized_shape, std::optional<Tensor> weight, std::optional<double> epsilon) {
    const int device = cuda_index(input, "rms_norm");
    const Index width = count(normalized_shape);
    if (width <= 0 || input.numel() % width || normalized_shape.size() != 1 || input.size(-1) != width)
        throw std::invalid_argument("rms_norm normalises the last axis");
    if (weight && (weight->numel() != width || weight->device() != input.device()))
        throw std::invalid_argument("rms_norm weight does not match");
    const Tensor x = as_f32(input);
    Tensor result = empty(x.shape(), {DType::f32, input.device()});
    const double eps = epsilon.value_or(std::numeric_limits<float>::epsilon());
    runtime::set_device(device);
    runtime::check(b200_rms_norm(x.data<float>(), weight ? weight->raw_data() : nullptr,
                                 weight ? weight_code(weight->dtype(), "rms_norm") : B200_F32, x.numel() / width, width, eps,
                                 static_cast<float*>(result.mutable_data()), runtime::stream(device)), "rms_norm");
    return result;
}

Tensor argmax(const Tensor& input, Index axis, KeepDim keep) {
    const int device = cuda_index(input, "argmax");
    if (wrap_axis(axis, input.ndim()) != input.ndim() - 1) throw std::invalid_argument("argmax: only the last axis is on the decoder path");
    const Tensor x = as_f32(input);
    Shape shape = x.shape();
    if (keep == KeepDim::yes) shape.back() = 1; else shape.pop_back();
    Tensor result = empty(shape, {DType::i64, input.device()});
    runtime::set_device(device);
    runtime::check(b200_argmax(x.data<float>(), x.numel() / x.size(-1), x.size(-1), static_cast<Index*>(result.mutable_data()),
                               runtime::stream(device)), "argmax");
    return result;
}

// dl::tensordot (src/ops/contraction.cpp:9-42): the contracted axes of `a` go last, those of `b` last as well (so that
// the product is the linear kernel's x @ W^T), the result has a's remaining axes followed by b's.
Tensor tensordot(const Tensor& a, const Tensor& b, Shape axes_a, Shape axes_b) {
    const int device = cuda_index(a, "tensordot");
    if (b.device() != a.device()) throw std::invalid_argument("tensordot inputs must share a device");
    auto axes = [](Shape values, Index rank) {
        Shape seen;
        for (auto& axis : values) {
            axis = wrap_axis(axis, rank);
            if (std::find(seen.begin(), seen.end(), axis) != seen.end()) throw std::invalid_argument("tensordot axes must be distinct");
            seen.push_back(axis);
        }
        return values;
    };
    axes_a = axes(std::move(axes_a), a.ndim());
    axes_b = axes(std::move(axes_b), b.ndim());
    if (axes_a.size() != axes_b.size()) throw std::invalid_argument("tensordot axis counts differ");
    if (a.ndim() > 8 || b.ndim() > 8) throw std::invalid_argument("tensordot: at most 8 axes per operand");
    Index inner = 1;
    for (std::size_t i = 0; i < axes_a.size(); ++i) {
        if (a.size(axes_a[i]) != b.size(axes_b[i])) throw std::invalid_argument("tensordot contracted dimensions differ");
        inner *= a.size(axes_a[i]);
    }
    auto remaining = [](Index rank, const Shape& contracted) {
        Shape result;
        for (Index i = 0; i < rank; ++i)
            if (std::find(contracted.begin(), contracted.end(), i) == contracted.end()) result.push_back(i);
        return result;
    };
    Shape left = remaining(a.ndim(), axes_a), right = remaining(b.ndim(), axes_b), output;
    Index rows = 1, columns = 1;
    for (auto axis : left) { output.push_back(a.size(axis)); rows *= a.size(axis); }
    for (auto axis : right) { output.push_back(b.size(axis)); columns *= b.size(axis); }
    left.insert(left.end(), axes_a.begin(), axes_a.end());      // a: [remaining..., contracted...] = [rows, inner]
    right.insert(right.end(), axes_b.begin(), axes_b.end());    // b: [remaining..., contracted...] = [columns, inner]
    Tensor result = empty(output, {DType::f32, a.device()});
    if (rows == 0 || columns == 0) return result;
    runtime::set_device(device);
    void* stream = runtime::stream(device);
    if (inner == 0) {
        runtime::check_cuda(cudaMemsetAsync(result.mutable_data(), 0, result.nbytes(), static_cast<cudaStream_t>(stream)), "cudaMemsetAsync");
        synchronize(a.device());
        return result;
    }
    auto dense = [&](const Tensor& source, const Shape& order, Index first, Index second) {
        const Tensor x = as_f32(source);
        Tensor out = empty({first, second}, {DType::f32, source.device()});
        if (order.empty()) return x.reshape({first, second});
        runtime::check(b200_permute(x.data<float>(), x.shape().data(), order.data(), static_cast<std::int32_t>(order.size()),
                                    static_cast<float*>(out.mutable_data()), stream), "permute");
        return out;
    };
    const Tensor x = dense(a, left, rows, inner), w = dense(b, right, columns, inner);
    runtime::check(b200_linear(x.data<float>(), rows, inner, w.raw_data(), B200_F32, columns, nullptr, 0, 0.0, B200_EPI_STORE, nullptr, nullptr,
                               static_cast<float*>(result.mutable_data()), stream), "tensordot");
    synchronize(a.device());   // the dense copies die with this scope
    return result;
}

Tensor rotary_embedding(const Tensor& input, const Tensor& cosine, const Tensor& sine) {
    const int device = cuda_index(input, "rotary_embedding");
    const Index hd = input.size(-1);
    if (hd == 0 || hd % 2) throw std::invalid_argument("rotary embedding requires a positive even dimension");
    if (input.ndim() < 2 || cosine.ndim() != 2 || cosine.size(0) != input.size(-2) || cosine.size(1) != hd / 2
        || sine.shape() != cosine.shape() || cosine.device() != input.device() || sine.device() != input.device())
        throw std::invalid_argument("rotary tables must be [length, dimensions/2] on the input's device");
    const Tensor x = as_f32(input), c = as_f32(cosine), s = as_f32(sine);
    Tensor result = empty(x.shape(), {DType::f32, input.device()});
    runtime::set_device(device);
    runtime::check(b200_rotary(x.data<float>(), x.numel() / (x.size(-2) * hd), x.size(-2), hd, c.data<float>(), s.data<float>(),
                               static_cast<float*>(result.mutable_data()), runtime::stream(device)), "rotary_embedding");
    return result;
}

Tensor grouped_query_attention(const Tensor& query, const Tensor& key, const Tensor& value, std::optional<Tensor> keep_mask) {
    const int device = cuda_index(query, "grouped_query_attention");
    if (keep_mask) throw std::invalid_argument("grouped_query_attention: explicit masks are outside the decoder path");
    if (query.ndim() != 4 || key.ndim() != 4 || value.ndim() != 4)
        throw std::invalid_argument("grouped-query attention expects [batch,heads,length,features]");
    const Index batch = query.size(0), heads = query.size(1), kv_heads = key.size(1), length = query.size(2);
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || value.size(1) != kv_heads)
        throw std::invalid_argument("query heads must be divisible by matching key/value heads");
    if (key.size(0) != batch || value.size(0) != batch || query.size(3) != key.size(3) || key.size(2) != value.size(2)
        || value.size(3) != key.size(3))
        throw std::invalid_argument("attention batch, key dimension and key/value lengths must match");
    const Index source = key.size(2), hd = query.size(3);
    const Tensor q = as_f32(query), k = as_f32(key), v = as_f32(value);
    runtime::set_device(device);
    void* stream = runtime::stream(device);
    internal::KvHandle cache(device, B200_F32, batch, kv_heads, hd, source, 64);
    runtime::check(b200_kv_cache_append(cache.get(), k.data<float>(), v.data<float>(), static_cast<int32_t>(source), stream), "KV append");
    runtime::check(b200_kv_cache_fill_lengths(cache.get(), static_cast<int32_t>(source), stream), "KV lengths");
    // [B,H,L,hd] -> [B,L,H,hd] rows for the kernel, and back
    Tensor rows = empty({batch, length, heads, hd}, {DType::f32, query.device()});
    runtime::check(b200_permute_0213(q.data<float>(), batch, heads, length, hd, static_cast<float*>(rows.mutable_data()), stream), "permute");
    const std::size_t scratch_bytes = b200_attention_scratch_bytes(batch * length, static_cast<int32_t>(heads), static_cast<int32_t>(kv_heads),
                                                                   static_cast<int32_t>(hd), static_cast<int32_t>(source), 64);
    Tensor scratch = empty({static_cast<Index>(scratch_bytes / 4 + 1)}, {DType::f32, query.device()});
    Tensor attended = empty({batch, length, heads, hd}, {DType::f32, query.device()});
    runtime::check(b200_attention_decode(rows.data<float>(), batch * length, static_cast<int32_t>(length), static_cast<int32_t>(heads),
                                         cache.get(), static_cast<int32_t>(source), 0, scratch.mutable_data(), scratch_bytes,
                                         static_cast<float*>(attended.mutable_data()), stream), "attention");
    Tensor result = empty({batch, heads, length, hd}, {DType::f32, query.device()});
    runtime::check(b200_permute_0213(attended.data<float>(), batch, length, heads, hd, static_cast<float*>(result.mutable_data()), stream), "permute");
    synchronize(query.device());  // the temporary cache dies with this scope
    return result;
}

}  // namespace dl
