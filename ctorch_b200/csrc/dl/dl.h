// C++20 host surface of the B200 decoder path.  It mirrors the part of the reference's dl:: interface that the
// decoder token loop touches (reference headers named per declaration), so that code written against
// dl::nn::TransformerDecoder / KVCache / Linear / Embedding / RMSNorm keeps its shape.  All compute runs in the
// sm_100a kernels behind ctorch_b200_kernels.h; there is no CPU compute path: an operator given CPU tensors throws.
#pragma once

#include "ctorch_b200_kernels.h"

#include <filesystem>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <span>
#include <string>
#include <string_view>
#include <utility>
#include <vector>

namespace dl {

// ---- include/dl/types.h:11-43 of the reference -------------------------------------------------------------
using Index = std::int64_t;
using Shape = std::vector<Index>;

enum class DType : std::uint8_t { f32, f64, i64, boolean, f16, bf16 };
enum class DeviceType : std::uint8_t { cpu, cuda };
enum class KeepDim { no, yes };

struct Device {
    DeviceType type = DeviceType::cpu;
    int index = 0;
    static constexpr Device cpu() { return {}; }
    static constexpr Device cuda(int index = 0) { return {DeviceType::cuda, index}; }
    bool operator==(const Device&) const = default;
};

struct TensorOptions {
    DType dtype = DType::f32;
    Device device = Device::cpu();
    bool requires_grad = false;  // accepted for signature compatibility; the decode path never records gradients
};

constexpr std::size_t element_size(DType dtype) {
    constexpr std::size_t sizes[] = {4, 8, 8, 1, 2, 2};
    return sizes[static_cast<std::size_t>(dtype)];
}

void synchronize(Device device);

// ---- runtime --------------------------------------------------------------------------------------------
namespace runtime {
// One non-blocking compute stream per CUDA device; every kernel and copy of the library is ordered on it.
void* stream(int device);
struct Storage {
    void* data = nullptr;
    std::size_t bytes = 0;
    Device device;
    bool pinned = false;
    Storage(std::size_t bytes, Device device, bool pinned = false);
    ~Storage();
    Storage(const Storage&) = delete;
    Storage& operator=(const Storage&) = delete;
};
}  // namespace runtime

// ---- include/dl/tensor.h:16-113 of the reference (the subset the token loop needs) ----------------------------
// Handles share storage; every tensor is dense row-major.  select/narrow/reshape of a dense tensor along the
// leading axis share storage, otherwise they copy (the reference returns strided views; values are identical).
class Tensor {
public:
    Tensor() = default;
    Tensor(std::shared_ptr<runtime::Storage> storage, Shape shape, DType dtype, std::size_t offset_bytes = 0);
    bool defined() const { return static_cast<bool>(storage_); }
    const Shape& shape() const { return shape_; }
    const Shape& strides() const { return strides_; }
    Index size(Index axis) const;
    Index ndim() const { return static_cast<Index>(shape_.size()); }
    Index numel() const;
    DType dtype() const { return dtype_; }
    Device device() const { return storage_->device; }
    std::size_t nbytes() const { return static_cast<std::size_t>(numel()) * element_size(dtype_); }
    template <class T> const T* data() const { return static_cast<const T*>(raw_data()); }
    void* mutable_data() const { return const_cast<void*>(raw_data()); }
    const void* raw_data() const { return static_cast<const char*>(storage_->data) + offset_; }

    Tensor to(Device device) const;
    Tensor astype(DType dtype) const;  // f32 <-> bf16 <-> f64 and i64 on host tensors; device tensors go through the host
    Tensor clone() const;
    Tensor reshape(Shape shape) const;
    Tensor select(Index axis, Index index) const;
    Tensor narrow(Index axis, Index start, Index length) const;
    void copy_to_host(void* destination) const;  // synchronises
    template <class T> std::vector<T> to_vector() const;
    template <class T> T item() const { return to_vector<T>().at(0); }

private:
    std::shared_ptr<runtime::Storage> storage_;
    Shape shape_, strides_;
    DType dtype_ = DType::f32;
    std::size_t offset_ = 0;
};

Tensor empty(Shape shape, TensorOptions options = {});
Tensor full(Shape shape, double value, TensorOptions options = {});
Tensor zeros(Shape shape, TensorOptions options = {});
Tensor ones(Shape shape, TensorOptions options = {});
namespace detail {
Tensor from_host(const void* data, Shape shape, DType dtype, bool requires_grad, Device device);
}

// ---- include/dl/ops.h:57,100-101,149-158,191,341-342 of the reference ---------------------------------------
Tensor linear(const Tensor& input, const Tensor& weight, std::optional<Tensor> bias = std::nullopt);
Tensor embedding(const Tensor& indices, const Tensor& weight);
Tensor rms_norm(const Tensor& input, const Shape& normalized_shape, std::optional<Tensor> weight = std::nullopt,
                std::optional<double> epsilon = std::nullopt);
Tensor argmax(const Tensor& input, Index axis, KeepDim keep = KeepDim::no);
Tensor tensordot(const Tensor& a, const Tensor& b, Shape axes_a, Shape axes_b);
Tensor rotary_embedding(const Tensor& input, const Tensor& cosine, const Tensor& sine);
Tensor grouped_query_attention(const Tensor& query, const Tensor& key, const Tensor& value,
                               std::optional<Tensor> keep_mask = std::nullopt);

using NamedTensor = std::pair<std::string, Tensor>;
using StateDict = std::vector<NamedTensor>;

namespace nn {

// ---- include/dl/nn.h:29-110 of the reference ---------------------------------------------------------------
class Module {
public:
    virtual ~Module() = default;
    StateDict state_dict() const;                                  // parameters then buffers, dotted names
    void load_state_dict(std::span<const NamedTensor> state);      // same name, shape and dtype required for every entry
    void to(Device device);
    void train(bool enabled = true);
    void eval() { train(false); }
    bool is_training() const { return training_; }
    // Bumped whenever parameter storage changes (to / load_state_dict); execution plans re-pack when it moves.
    std::uint64_t version() const;

protected:
    Tensor& register_parameter(std::string name, Tensor value);
    Tensor& register_buffer(std::string name, Tensor value);
    void register_module(std::string name, std::shared_ptr<Module> child);
    template <class Child, class... Args> std::shared_ptr<Child> add_module(std::string name, Args&&... args) {
        auto child = std::make_shared<Child>(std::forward<Args>(args)...);
        register_module(std::move(name), child);
        return child;
    }

private:
    void collect(const std::string& prefix, bool buffers, std::vector<std::pair<std::string, Tensor*>>& out);
    std::vector<std::pair<std::string, std::unique_ptr<Tensor>>> parameters_, buffers_;
    std::vector<std::pair<std::string, std::shared_ptr<Module>>> children_;
    bool training_ = true;
    std::uint64_t version_ = 0;
};

class UnaryModule : public Module {
public:
    virtual Tensor forward(const Tensor& input) = 0;
    Tensor operator()(const Tensor& input) { return forward(input); }
};

// include/dl/nn.h:113-124
class Linear : public UnaryModule {
public:
    Linear(Index input_features, Index output_features, bool bias = true, TensorOptions options = {});
    explicit Linear(Tensor weight, std::optional<Tensor> bias = std::nullopt);
    Tensor forward(const Tensor& input) override;
    const Tensor& weight() const { return *weight_; }
    const std::optional<Tensor>& bias() const { return bias_; }
private:
    Tensor* weight_;
    std::optional<Tensor> bias_;
};

// include/dl/nn.h:210-219
class Embedding : public UnaryModule {
public:
    Embedding(Index vocabulary, Index dimensions, TensorOptions options = {});
    explicit Embedding(Tensor weight);
    Tensor forward(const Tensor& indices) override;
    const Tensor& weight() const { return *weight_; }
private:
    Tensor* weight_;
};

// include/dl/nn.h:381-390
class RMSNorm : public UnaryModule {
public:
    explicit RMSNorm(Shape normalized_shape, std::optional<double> epsilon = std::nullopt, bool affine = true,
                     TensorOptions options = {});
    Tensor forward(const Tensor& input) override;
    const Tensor* weight() const { return weight_; }
    double epsilon() const { return epsilon_; }
private:
    Shape normalized_shape_;
    double epsilon_;
    Tensor* weight_ = nullptr;
};

// ---- include/dl/decoder.h:8-107 of the reference -------------------------------------------------------------
class SwiGLU : public UnaryModule {
public:
    SwiGLU(Index dimensions, Index hidden, bool bias = false, TensorOptions options = {});
    Tensor forward(const Tensor& input) override;
    const Linear& gate() const { return *gate_; }
    const Linear& up() const { return *up_; }
    const Linear& down() const { return *down_; }
private:
    std::shared_ptr<Linear> gate_, up_, down_;
    Tensor packed_;  // gate/up rows interleaved for the fused epilogue
    std::uint64_t packed_version_ = ~0ull;
};

class LoRALinear : public UnaryModule {
public:
    LoRALinear(const Linear& base, Index rank, double alpha = 1.0);
    Tensor forward(const Tensor& input) override;
    std::shared_ptr<Linear> merged() const;
    const Tensor& weight() const { return *weight_; }
    const Linear& down() const { return *down_; }
    const Linear& up() const { return *up_; }
    double scale() const { return scale_; }
    Index rank() const { return rank_; }
private:
    Tensor* weight_;
    double scale_;
    Index rank_;
    std::shared_ptr<Linear> down_, up_;
};

class RotaryEmbedding : public UnaryModule {
public:
    RotaryEmbedding(Index dimensions, Index capacity, double base = 10000.0, TensorOptions options = {});
    Tensor forward(const Tensor& input) override { return forward(input, 0); }
    Tensor forward(const Tensor& input, Index offset);
    const Tensor& cosine() const { return *cosine_; }
    const Tensor& sine() const { return *sine_; }
private:
    Tensor *cosine_, *sine_;
};

// Storage of one layer's keys and values for one request.  Unlike the reference's dense buffer the storage is
// paged and head-major on the device (b200_kv_cache); the observable behaviour (capacity, one length for the batch,
// lazy allocation at the first append, clear/truncate reuse, move-only) is the reference's
// (include/dl/decoder.h:45-62, src/nn/kv_cache.cpp:9-43).
class KVCache {
public:
    explicit KVCache(Index capacity);
    ~KVCache();
    KVCache(const KVCache&) = delete;
    KVCache& operator=(const KVCache&) = delete;
    KVCache(KVCache&& other) noexcept;
    KVCache& operator=(KVCache&& other) noexcept;
    void append(const Tensor& key, const Tensor& value);  // [batch, kv_heads, count, head_dim] f32 CUDA tensors
    Tensor key() const;
    Tensor value() const;
    Index length() const { return length_; }
    Index capacity() const { return capacity_; }
    void clear();
    void truncate(Index length);

    // B200 extensions used by the execution plan.
    void set_storage_dtype(DType dtype) { storage_dtype_ = dtype; }  // before the first append; default f32
    DType storage_dtype() const { return storage_dtype_; }
    b200_kv_cache* ensure(int device, Index batch, Index kv_heads, Index head_dim);  // allocate or validate
    b200_kv_cache* handle() const { return cache_; }
    void commit(Index count) { length_ += count; }  // host mirror after the device lengths were advanced
    std::uint64_t id() const { return id_; }

private:
    Tensor gather(int which) const;
    Index capacity_, length_ = 0;
    DType storage_dtype_ = DType::f32;
    b200_kv_cache* cache_ = nullptr;
    int device_ = 0;
    Index batch_ = 0, kv_heads_ = 0, head_dim_ = 0;
    std::uint64_t id_ = 0;
};

class GroupedQueryAttention : public UnaryModule {
public:
    GroupedQueryAttention(Index dimensions, Index heads, Index kv_heads, Index context, TensorOptions options = {});
    Tensor forward(const Tensor& input) override;
    Tensor decode(const Tensor& input, KVCache& cache);
    // Installs adapters on the query and value projections (the reference can only host merged weights here,
    // include/dl/decoder.h:75); nullptr removes them.
    void set_adapters(std::shared_ptr<LoRALinear> query, std::shared_ptr<LoRALinear> value);
    Index dimensions() const { return dimensions_; }
    Index heads() const { return heads_; }
    Index kv_heads() const { return kv_heads_; }
    const Linear& query() const { return *query_; }
    const Linear& key() const { return *key_; }
    const Linear& value() const { return *value_; }
    const Linear& output() const { return *output_; }
    const RotaryEmbedding& rotary() const { return *rotary_; }
    const LoRALinear* query_adapter() const { return query_adapter_.get(); }
    const LoRALinear* value_adapter() const { return value_adapter_.get(); }
private:
    Index dimensions_, heads_, kv_heads_, context_;
    std::shared_ptr<Linear> query_, key_, value_, output_;
    std::shared_ptr<RotaryEmbedding> rotary_;
    std::shared_ptr<LoRALinear> query_adapter_, value_adapter_;
};

class TransformerDecoderLayer : public UnaryModule {
public:
    static constexpr double norm_epsilon = 1e-5;
    TransformerDecoderLayer(Index dimensions, Index heads, Index kv_heads, Index hidden, Index context,
                            TensorOptions options = {});
    Tensor forward(const Tensor& input) override;
    Tensor decode(const Tensor& input, KVCache& cache);
    GroupedQueryAttention& attention() const { return *attention_; }
    SwiGLU& feedforward() const { return *feedforward_; }
    const RMSNorm& attention_norm() const { return *attention_norm_; }
    const RMSNorm& feedforward_norm() const { return *feedforward_norm_; }
private:
    std::shared_ptr<GroupedQueryAttention> attention_;
    std::shared_ptr<SwiGLU> feedforward_;
    std::shared_ptr<RMSNorm> attention_norm_, feedforward_norm_;
};

class DecodePlan;  // fixed execution plan, plan.h

class TransformerDecoder : public UnaryModule {
public:
    TransformerDecoder(Index layers, Index dimensions, Index heads, Index kv_heads, Index hidden, Index context,
                       TensorOptions options = {});
    ~TransformerDecoder() override;
    Tensor forward(const Tensor& input) override;
    std::vector<KVCache> make_cache() const;
    Index layer_count() const { return static_cast<Index>(layers_.size()); }
    Tensor decode(const Tensor& input, std::span<KVCache> cache);

    // B200 extensions.
    Index dimensions() const { return dimensions_; }
    Index heads() const { return heads_; }
    Index kv_heads() const { return kv_heads_; }
    Index hidden() const { return hidden_; }
    Index context() const { return context_; }
    DType dtype() const { return dtype_; }
    TransformerDecoderLayer& layer(Index i) const { return *layers_[static_cast<std::size_t>(i)]; }
    const RMSNorm& normalization() const { return *normalization_; }
    // f32 (default): activations between the kernels keep ~16 mantissa bits (bf16 hi + lo planes).  bf16: passes over more
    // than 16 rows (prefill, large decode batches) feed the tensor cores the hi plane only.
    void set_activation_dtype(DType dtype);
    DType activation_dtype() const { return activation_dtype_; }
    void set_cache_dtype(DType dtype) { cache_dtype_ = dtype; }  // storage dtype of caches made by make_cache()
    // KV-head tensor parallelism: this object computes the slice `rank` of `world` (query heads, KV heads and SwiGLU
    // features are split evenly; norms, residual stream, embedding and logits stay replicated) and sums the partial
    // results of the output and down projections over the device's tensor-parallel group.
    void set_tensor_parallel(int rank, int world);
    int tp_rank() const { return tp_rank_; }
    int tp_world() const { return tp_world_; }
    DType cache_dtype() const { return cache_dtype_; }
    DecodePlan& plan();

private:
    Index dimensions_, heads_, kv_heads_, hidden_, context_;
    DType dtype_, cache_dtype_, activation_dtype_ = DType::f32;
    int tp_rank_ = 0, tp_world_ = 1;
    std::vector<std::shared_ptr<TransformerDecoderLayer>> layers_;
    std::shared_ptr<RMSNorm> normalization_;
    std::unique_ptr<DecodePlan> plan_;
};

}  // namespace nn

// ---- include/dl/io.h of the reference: weight archives (".ct"), see checkpoint.cpp for the layout --------------
namespace io {
void save(const std::filesystem::path& path, std::span<const NamedTensor> state);
StateDict load(const std::filesystem::path& path);   // tensors in host memory
}  // namespace io

// ---- extensions/onnx/include/dl/onnx.h:30-35 of the reference: the decoder with its KV cache as graph ports ----
namespace onnx {
void save_decoder(const std::string& path, const nn::TransformerDecoder& decoder);
void save_decoder(const std::string& path, const nn::Embedding& embedding, const nn::TransformerDecoder& decoder, const nn::Linear& output);
}  // namespace onnx

}  // namespace dl
