// Module registry and the decoder's layers.  Structure and names follow the reference modules
// (src/nn/module.cpp, src/nn/layers.cpp, src/nn/decoder.cpp, src/nn/kv_cache.cpp) so that state_dict keys match:
//   layer{i}.attention.{query,key,value,output}.weight, layer{i}.attention.rotary.{cosine,sine},
//   layer{i}.feedforward.{gate,up,down}.weight, layer{i}.{attention_norm,feedforward_norm}.weight, normalization.weight
#include "dl/dl.h"
#include "dl/internal.h"
#include "dl/plan.h"

#include <atomic>
#include <cmath>
#include <random>
#include <stdexcept>
#include <unordered_map>

namespace dl::nn {

// ---- Module ---------------------------------------------------------------------------------------------
Tensor& Module::register_parameter(std::string name, Tensor value) {
    parameters_.emplace_back(std::move(name), std::make_unique<Tensor>(std::move(value)));
    return *parameters_.back().second;
}
Tensor& Module::register_buffer(std::string name, Tensor value) {
    buffers_.emplace_back(std::move(name), std::make_unique<Tensor>(std::move(value)));
    return *buffers_.back().second;
}
void Module::register_module(std::string name, std::shared_ptr<Module> child) {
    children_.emplace_back(std::move(name), std::move(child));
}

void Module::collect(const std::string& prefix, bool buffers, std::vector<std::pair<std::string, Tensor*>>& out) {
    for (auto& [name, tensor] : buffers ? buffers_ : parameters_) out.emplace_back(prefix + name, tensor.get());
    for (auto& [name, child] : children_) child->collect(prefix + name + ".", buffers, out);
}

StateDict Module::state_dict() const {
    std::vector<std::pair<std::string, Tensor*>> slots;
    auto* self = const_cast<Module*>(this);
    self->collect("", false, slots);
    self->collect("", true, slots);
    StateDict result;
    for (auto& [name, tensor] : slots) result.emplace_back(name, *tensor);
    return result;
}

void Module::load_state_dict(std::span<const NamedTensor> state) {
    std::unordered_map<std::string_view, const Tensor*> source;
    for (const auto& [name, tensor] : state) source.emplace(name, &tensor);
    std::vector<std::pair<std::string, Tensor*>> slots;
    collect("", false, slots);
    collect("", true, slots);
    // Validate everything before the first write so that a bad entry leaves the module untouched.
    for (auto& [name, tensor] : slots) {
        auto found = source.find(name);
        if (found == source.end()) throw std::out_of_range("state entry missing: " + name);
        if (found->second->shape() != tensor->shape() || found->second->dtype() != tensor->dtype())
            throw std::invalid_argument("state tensor shape, dtype or write access differs: " + name);
    }
    for (auto& [name, tensor] : slots) {
        const Tensor& value = *source.at(name);
        runtime::copy_bytes(tensor->mutable_data(), tensor->device(), value.raw_data(), value.device(), value.nbytes());
    }
    for (auto& [name, tensor] : slots)
        if (tensor->device().type == DeviceType::cuda) { synchronize(tensor->device()); break; }
    ++version_;
}

void Module::to(Device device) {
    for (auto& [name, tensor] : parameters_) *tensor = tensor->to(device);
    for (auto& [name, tensor] : buffers_) *tensor = tensor->to(device);
    for (auto& [name, child] : children_) child->to(device);
    ++version_;
}
void Module::train(bool enabled) {
    training_ = enabled;
    for (auto& [name, child] : children_) child->train(enabled);
}
std::uint64_t Module::version() const {
    std::uint64_t total = version_;
    for (const auto& [name, child] : children_) total += child->version();
    return total;
}

// ---- initialisation -------------------------------------------------------------------------------------
namespace {
std::atomic<std::uint64_t> init_counter{0x9e3779b97f4a7c15ull};

// uniform(-1/sqrt(fan_in), 1/sqrt(fan_in)) like the reference's nn/initialization.h:15-18 (values differ: the
// reference draws from its global Philox generator; models that need specific weights load a state_dict).
Tensor uniform_parameter(Shape shape, Index fan_in, TensorOptions options) {
    Tensor host = empty(shape, {DType::f32, Device::cpu()});
    std::mt19937_64 engine(init_counter.fetch_add(0x632be59bd9b4e019ull));
    const float bound = 1.0f / std::sqrt(static_cast<float>(fan_in > 0 ? fan_in : 1));
    std::uniform_real_distribution<float> draw(-bound, bound);
    auto* p = static_cast<float*>(host.mutable_data());
    for (Index i = 0; i < host.numel(); ++i) p[i] = draw(engine);
    return host.astype(options.dtype).to(options.device);
}
void require_float(DType dtype) {
    if (dtype != DType::f32 && dtype != DType::bf16)
        throw std::invalid_argument("the B200 decoder path stores weights in f32 or bf16");
}
}  // namespace

// ---- generic layers ---------------------------------------------------------------------------------------
Linear::Linear(Index input_features, Index output_features, bool bias, TensorOptions options)
    : weight_(&register_parameter("weight", uniform_parameter({output_features, input_features}, input_features, options))) {
    require_float(options.dtype);
    if (bias) throw std::invalid_argument("Linear: bias is not part of the decoder path");
}
Linear::Linear(Tensor weight, std::optional<Tensor> bias) : weight_(&register_parameter("weight", std::move(weight))) {
    if (bias) throw std::invalid_argument("Linear: bias is not part of the decoder path");
    if (weight_->ndim() != 2) throw std::invalid_argument("Linear weight must be a matrix");
}
Tensor Linear::forward(const Tensor& input) { return linear(input, *weight_); }

Embedding::Embedding(Index vocabulary, Index dimensions, TensorOptions options)
    : Embedding(uniform_parameter({vocabulary, dimensions}, 1, options)) {}
Embedding::Embedding(Tensor weight) : weight_(&register_parameter("weight", std::move(weight))) {
    if (weight_->ndim() != 2) throw std::invalid_argument("Embedding weight must be a matrix");
}
Tensor Embedding::forward(const Tensor& indices) { return embedding(indices, *weight_); }

RMSNorm::RMSNorm(Shape normalized_shape, std::optional<double> epsilon, bool affine, TensorOptions options)
    : normalized_shape_(std::move(normalized_shape)),
      epsilon_(epsilon.value_or(std::numeric_limits<float>::epsilon())) {
    if (affine) weight_ = &register_parameter("weight", ones(normalized_shape_, {options.dtype, options.device}));
}
Tensor RMSNorm::forward(const Tensor& input) {
    return rms_norm(input, normalized_shape_, weight_ ? std::optional{*weight_} : std::nullopt, epsilon_);
}

// ---- SwiGLU (src/nn/decoder.cpp:11-16) ------------------------------------------------------------------------
SwiGLU::SwiGLU(Index dimensions, Index hidden, bool bias, TensorOptions options) {
    gate_ = add_module<Linear>("gate", dimensions, hidden, bias, options);
    up_ = add_module<Linear>("up", dimensions, hidden, bias, options);
    down_ = add_module<Linear>("down", hidden, dimensions, bias, options);
}
Tensor SwiGLU::forward(const Tensor& input) {
    if (input.device().type != DeviceType::cuda) throw std::invalid_argument("SwiGLU: tensors must live on a CUDA device");
    const int device = input.device().index;
    if (packed_version_ != version() || !packed_.defined()) {
        packed_ = interleave_rows(gate_->weight(), up_->weight());
        packed_version_ = version();
    }
    const Tensor x = input.dtype() == DType::f32 ? input : input.astype(DType::f32);
    const Index rows = x.numel() / x.size(-1), hidden = gate_->weight().size(0);
    Tensor activated = empty({rows, hidden}, {DType::f32, input.device()});
    const int code = gate_->weight().dtype() == DType::bf16 ? B200_BF16 : B200_F32;
    runtime::set_device(device);
    runtime::check(b200_linear(x.data<float>(), rows, x.size(-1), packed_.raw_data(), code, 2 * hidden, nullptr, 0, 0.0,
                               B200_EPI_SWIGLU, nullptr, nullptr, static_cast<float*>(activated.mutable_data()),
                               runtime::stream(device)), "SwiGLU gate/up");
    Shape shape = x.shape();
    return linear(activated, down_->weight()).reshape(shape);
}

// ---- LoRALinear (src/nn/decoder.cpp:18-35) ------------------------------------------------------------------------
LoRALinear::LoRALinear(const Linear& base, Index rank, double alpha)
    : weight_(&register_parameter("weight", base.weight().clone())), scale_(alpha / static_cast<double>(rank)), rank_(rank) {
    if (rank <= 0) throw std::invalid_argument("LoRA rank must be positive");
    const TensorOptions options{weight_->dtype(), weight_->device()};
    down_ = add_module<Linear>("down", weight_->size(1), rank, false, options);
    up_ = add_module<Linear>("up", zeros({weight_->size(0), rank}, options));
}
Tensor LoRALinear::forward(const Tensor& input) {
    if (input.device().type != DeviceType::cuda) throw std::invalid_argument("LoRALinear: tensors must live on a CUDA device");
    // base(x) + up(down(x)) * f32(alpha/rank): three skinny linears and a scaled add on the device
    Tensor base = linear(input, *weight_);
    Tensor delta = linear(linear(input, down_->weight()), up_->weight());
    const int device = input.device().index;
    runtime::set_device(device);
    runtime::check(b200_scaled_add(static_cast<float*>(base.mutable_data()), delta.data<float>(), static_cast<float>(scale_),
                                   base.numel(), runtime::stream(device)), "LoRA add");
    return base;
}
std::shared_ptr<Linear> LoRALinear::merged() const {
    // W + (up @ down) * scale in f32, rounded to W's dtype.  One-off host arithmetic at load time (weights are
    // parameters, not activations); the token loop never runs it.
    const Tensor w = weight_->to(Device::cpu()).astype(DType::f32);
    const Tensor d = down_->weight().to(Device::cpu()).astype(DType::f32);
    const Tensor u = up_->weight().to(Device::cpu()).astype(DType::f32);
    const Index out = w.size(0), in = w.size(1);
    Tensor merged = empty({out, in}, {DType::f32, Device::cpu()});
    const float scale = static_cast<float>(scale_);
    auto* m = static_cast<float*>(merged.mutable_data());
    for (Index o = 0; o < out; ++o)
        for (Index i = 0; i < in; ++i) {
            float sum = 0.0f;
            for (Index r = 0; r < rank_; ++r) sum = sum + u.data<float>()[o * rank_ + r] * d.data<float>()[r * in + i];
            m[o * in + i] = w.data<float>()[o * in + i] + sum * scale;
        }
    return std::make_shared<Linear>(merged.astype(weight_->dtype()).to(weight_->device()));
}

// ---- RotaryEmbedding (src/nn/decoder.cpp:38-59) ---------------------------------------------------------------
namespace {
// angle[p,i] = f32(p) * expf(f32(i) * f32(-2 ln(base)/dimensions)); cos/sin of the f32 angle, all on the host with
// the C library's single-precision functions, exactly as the reference builds its buffers.
std::pair<Tensor, Tensor> rotary_tables(Index dimensions, Index capacity, double base) {
    if (dimensions <= 0 || dimensions % 2 != 0 || capacity <= 0 || base <= 0)
        throw std::invalid_argument("RoPE needs an even positive dimension, positive capacity and base");
    const Index half = dimensions / 2;
    Tensor cosine = empty({capacity, half}, {DType::f32, Device::cpu()}), sine = empty({capacity, half}, {DType::f32, Device::cpu()});
    const float factor = static_cast<float>(-2.0 * std::log(base) / static_cast<double>(dimensions));
    auto* c = static_cast<float*>(cosine.mutable_data());
    auto* s = static_cast<float*>(sine.mutable_data());
    for (Index p = 0; p < capacity; ++p)
        for (Index i = 0; i < half; ++i) {
            const float frequency = expf(static_cast<float>(i) * factor);
            const float angle = static_cast<float>(p) * frequency;
            c[p * half + i] = cosf(angle);
            s[p * half + i] = sinf(angle);
        }
    return {cosine, sine};
}
}  // namespace

RotaryEmbedding::RotaryEmbedding(Index dimensions, Index capacity, double base, TensorOptions options) {
    auto [cosine, sine] = rotary_tables(dimensions, capacity, base);
    cosine_ = &register_buffer("cosine", cosine.to(options.device));
    sine_ = &register_buffer("sine", sine.to(options.device));
}
Tensor RotaryEmbedding::forward(const Tensor& input, Index offset) {
    if (offset < 0 || input.size(-2) > cosine_->size(0) - offset) throw std::out_of_range("RoPE positions exceed the table capacity");
    return rotary_embedding(input, cosine_->narrow(0, offset, input.size(-2)), sine_->narrow(0, offset, input.size(-2)));
}

// ---- KVCache (src/nn/kv_cache.cpp:9-43) -----------------------------------------------------------------------
namespace {
std::atomic<std::uint64_t> cache_ids{1};
}
KVCache::KVCache(Index capacity) : capacity_(capacity), id_(cache_ids.fetch_add(1)) {
    if (capacity <= 0) throw std::invalid_argument("KV cache capacity must be positive");
}
KVCache::~KVCache() {
    if (cache_) {
        try { synchronize(Device::cuda(device_)); } catch (...) {}
        b200_kv_cache_release(cache_);
    }
}
KVCache::KVCache(KVCache&& other) noexcept
    : capacity_(other.capacity_), length_(other.length_), storage_dtype_(other.storage_dtype_), cache_(other.cache_),
      device_(other.device_), batch_(other.batch_), kv_heads_(other.kv_heads_), head_dim_(other.head_dim_), id_(other.id_) {
    other.cache_ = nullptr;
}
KVCache& KVCache::operator=(KVCache&& other) noexcept {
    if (this != &other) {
        if (cache_) {
            try { synchronize(Device::cuda(device_)); } catch (...) {}
            b200_kv_cache_release(cache_);
        }
        capacity_ = other.capacity_; length_ = other.length_; storage_dtype_ = other.storage_dtype_; cache_ = other.cache_;
        device_ = other.device_; batch_ = other.batch_; kv_heads_ = other.kv_heads_; head_dim_ = other.head_dim_; id_ = other.id_;
        other.cache_ = nullptr;
    }
    return *this;
}
b200_kv_cache* KVCache::ensure(int device, Index batch, Index kv_heads, Index head_dim) {
    if (!cache_) {
        const int code = storage_dtype_ == DType::bf16 ? B200_BF16 : B200_F32;
        runtime::check(b200_kv_cache_create(device, code, static_cast<int32_t>(batch), static_cast<int32_t>(kv_heads),
                                            static_cast<int32_t>(head_dim), static_cast<int32_t>(capacity_), 64, &cache_),
                       "KV cache allocation");
        device_ = device; batch_ = batch; kv_heads_ = kv_heads; head_dim_ = head_dim;
        if (length_) runtime::check(b200_kv_cache_fill_lengths(cache_, static_cast<int32_t>(length_), runtime::stream(device)), "KV lengths");
    } else if (device != device_ || batch != batch_ || kv_heads != kv_heads_ || head_dim != head_dim_) {
        throw std::invalid_argument("KV cache shape, dtype or device changed");
    }
    return cache_;
}
void KVCache::append(const Tensor& key, const Tensor& value) {
    if (key.ndim() != 4 || value.shape() != key.shape()) throw std::invalid_argument("KV cache append expects matching [batch,kv_heads,count,head_dim]");
    const Index count = key.size(-2);
    if (count != value.size(-2) || count > capacity_ - length_)
        throw std::invalid_argument("KV cache append exceeds capacity or has unequal key/value lengths");
    if (key.device().type != DeviceType::cuda || value.device() != key.device())
        throw std::invalid_argument("KV cache append: tensors must live on one CUDA device");
    const int device = key.device().index;
    ensure(device, key.size(0), key.size(1), key.size(3));
    const Tensor k = key.dtype() == DType::f32 ? key : key.astype(DType::f32), v = value.dtype() == DType::f32 ? value : value.astype(DType::f32);
    runtime::set_device(device);
    runtime::check(b200_kv_cache_append(cache_, k.data<float>(), v.data<float>(), static_cast<int32_t>(count), runtime::stream(device)), "KV append");
    runtime::check(b200_kv_cache_advance(&cache_, 1, static_cast<int32_t>(count), runtime::stream(device)), "KV advance");
    length_ += count;
}
Tensor KVCache::gather(int which) const {
    if (!cache_) throw std::logic_error(which ? "KV cache has no value tensor before its first append"
                                              : "KV cache has no key tensor before its first append");
    Tensor result = empty({batch_, kv_heads_, length_, head_dim_}, {DType::f32, Device::cuda(device_)});
    runtime::set_device(device_);
    runtime::check(b200_kv_cache_gather(cache_, which, static_cast<int32_t>(length_), static_cast<float*>(result.mutable_data()),
                                        runtime::stream(device_)), "KV gather");
    return result;
}
Tensor KVCache::key() const { return gather(0); }
Tensor KVCache::value() const { return gather(1); }
void KVCache::clear() {
    length_ = 0;
    if (cache_) runtime::check(b200_kv_cache_fill_lengths(cache_, 0, runtime::stream(device_)), "KV lengths");
}
void KVCache::truncate(Index length) {
    if (length < 0 || length > length_) throw std::out_of_range("KV cache truncation must keep an existing prefix");
    length_ = length;
    if (cache_) runtime::check(b200_kv_cache_fill_lengths(cache_, static_cast<int32_t>(length), runtime::stream(device_)), "KV lengths");
}

// ---- GroupedQueryAttention (src/nn/decoder.cpp:61-89) ----------------------------------------------------------
GroupedQueryAttention::GroupedQueryAttention(Index dimensions, Index heads, Index kv_heads, Index context, TensorOptions options)
    : dimensions_(dimensions), heads_(heads), kv_heads_(kv_heads), context_(context) {
    if (heads <= 0 || kv_heads <= 0 || dimensions <= 0 || dimensions % heads || heads % kv_heads)
        throw std::invalid_argument("attention dimensions and query/key head counts must divide evenly");
    query_ = add_module<Linear>("query", dimensions, dimensions, false, options);
    key_ = add_module<Linear>("key", dimensions, kv_heads * (dimensions / heads), false, options);
    value_ = add_module<Linear>("value", dimensions, kv_heads * (dimensions / heads), false, options);
    output_ = add_module<Linear>("output", dimensions, dimensions, false, options);
    rotary_ = add_module<RotaryEmbedding>("rotary", dimensions / heads, context, 10000.0, options);
}
void GroupedQueryAttention::set_adapters(std::shared_ptr<LoRALinear> query, std::shared_ptr<LoRALinear> value) {
    if (static_cast<bool>(query) != static_cast<bool>(value)) throw std::invalid_argument("adapters are installed on query and value together");
    if (query && (query->weight().shape() != query_->weight().shape() || value->weight().shape() != value_->weight().shape()
                  || query->rank() != value->rank()))
        throw std::invalid_argument("adapter shapes do not match the projections");
    query_adapter_ = std::move(query);
    value_adapter_ = std::move(value);
    to(query_->weight().device());  // bumps the version so that plans re-pack
}
// A stand-alone attention block runs the same plan as a one-layer stack without the feed-forward half; the decoder
// never calls these two (it drives whole layers), they exist for interface parity.
Tensor GroupedQueryAttention::forward(const Tensor& input) {
    KVCache scratch(context_);
    return decode(input, scratch);
}
Tensor GroupedQueryAttention::decode(const Tensor& input, KVCache& cache) { return attention_block(*this, input, cache); }

// ---- TransformerDecoderLayer / TransformerDecoder (src/nn/decoder.cpp:91-142) ------------------------------------
TransformerDecoderLayer::TransformerDecoderLayer(Index dimensions, Index heads, Index kv_heads, Index hidden, Index context,
                                                 TensorOptions options) {
    attention_ = add_module<GroupedQueryAttention>("attention", dimensions, heads, kv_heads, context, options);
    feedforward_ = add_module<SwiGLU>("feedforward", dimensions, hidden, false, options);
    attention_norm_ = add_module<RMSNorm>("attention_norm", Shape{dimensions}, norm_epsilon, true, options);
    feedforward_norm_ = add_module<RMSNorm>("feedforward_norm", Shape{dimensions}, norm_epsilon, true, options);
}
Tensor TransformerDecoderLayer::forward(const Tensor& input) {
    KVCache scratch(attention_->rotary().cosine().size(0));
    return decode(input, scratch);
}
Tensor TransformerDecoderLayer::decode(const Tensor& input, KVCache& cache) {
    // x + attention(norm(x)), then r + feedforward(norm(r)) (src/nn/decoder.cpp:102-106), op by op
    Tensor residual = add(input, attention_->decode((*attention_norm_)(input), cache));
    return add(residual, (*feedforward_)((*feedforward_norm_)(residual)));
}

TransformerDecoder::TransformerDecoder(Index layers, Index dimensions, Index heads, Index kv_heads, Index hidden, Index context,
                                       TensorOptions options)
    : dimensions_(dimensions), heads_(heads), kv_heads_(kv_heads), hidden_(hidden), context_(context), dtype_(options.dtype),
      cache_dtype_(options.dtype == DType::bf16 ? DType::bf16 : DType::f32) {
    if (layers <= 0) throw std::invalid_argument("decoder requires at least one layer");
    require_float(options.dtype);
    for (Index i = 0; i < layers; ++i)
        layers_.push_back(add_module<TransformerDecoderLayer>("layer" + std::to_string(i), dimensions, heads, kv_heads, hidden,
                                                              context, options));
    normalization_ = add_module<RMSNorm>("normalization", Shape{dimensions}, TransformerDecoderLayer::norm_epsilon, true, options);
}
TransformerDecoder::~TransformerDecoder() = default;

void TransformerDecoder::set_activation_dtype(DType dtype) {
    if (dtype != DType::f32 && dtype != DType::bf16) throw std::invalid_argument("activation dtype must be f32 or bf16");
    if (dtype == DType::bf16 && dtype_ != DType::bf16) throw std::invalid_argument("bf16 activations need a bf16 decoder");
    activation_dtype_ = dtype;
}

void TransformerDecoder::set_tensor_parallel(int rank, int world) {
    if (world < 1 || rank < 0 || rank >= world) throw std::invalid_argument("tensor-parallel rank must lie in [0, world)");
    const Index hd = dimensions_ / heads_;
    if (heads_ % world || kv_heads_ % world || hidden_ % world || ((hidden_ / world) % 8) || ((heads_ / world * hd) % 8))
        throw std::invalid_argument("query heads, KV heads and SwiGLU features must split evenly (in multiples of 8 features) over the ranks");
    tp_rank_ = rank;
    tp_world_ = world;
    to(normalization_->weight()->device());  // bumps the version: plans re-pack their slices
}

Tensor TransformerDecoder::forward(const Tensor& input) {
    // A full causal pass equals decoding the whole sequence into an empty cache (the property the reference's
    // tests/state.cpp:54-63 pins); the cache is dropped afterwards.
    auto cache = make_cache();
    return decode(input, cache);
}
std::vector<KVCache> TransformerDecoder::make_cache() const {
    std::vector<KVCache> result;
    result.reserve(layers_.size());
    for (std::size_t i = 0; i < layers_.size(); ++i) {
        result.emplace_back(context_);
        result.back().set_storage_dtype(cache_dtype_);
    }
    return result;
}
DecodePlan& TransformerDecoder::plan() {
    if (!plan_) plan_ = std::make_unique<DecodePlan>(*this);
    return *plan_;
}
Tensor TransformerDecoder::decode(const Tensor& input, std::span<KVCache> cache) { return plan().decode(input, cache); }

}  // namespace dl::nn
