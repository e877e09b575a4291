// C17 boundary: opaque handles over the dl:: objects, exceptions turned into DL_ERROR plus a thread-local message
// (the contract of the reference's src/api/common.h:53-69 and src/api/decoder.cpp:10-70).
#include "ctorch_b200_c_api.h"
#include "dl/dl.h"
#include "dl/internal.h"
#include "dl/plan.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <exception>
#include <mutex>

struct dl_tensor { dl::Tensor value; };
struct dl_module { std::shared_ptr<dl::nn::UnaryModule> value; };
struct dl_state { dl::StateDict value; };
struct dl_decoder_cache { std::vector<dl::nn::KVCache> value; };
struct dl_generation { std::unique_ptr<dl::nn::Generation> value; };

namespace {

thread_local char last_error[2048];

void set_error(const char* message) noexcept { std::snprintf(last_error, sizeof last_error, "%s", message); }

template <class Function> dl_status invoke(Function&& function) noexcept {
    try {
        function();
        set_error("");
        return DL_OK;
    } catch (const std::exception& error) {
        set_error(error.what());
    } catch (...) {
        set_error("unknown C++ exception");
    }
    return DL_ERROR;
}

template <class Handle, class Function> dl_status make_handle(Handle** output, Function&& function) noexcept {
    if (!output) { set_error("output slot is NULL"); return DL_ERROR; }
    *output = nullptr;
    return invoke([&] { *output = new Handle{function()}; });
}

template <class T> const T& need(const T* handle, const char* what) {
    if (!handle) throw std::invalid_argument(std::string(what) + " handle is NULL");
    return *handle;
}
template <class T> T& need(T* handle, const char* what) {
    if (!handle) throw std::invalid_argument(std::string(what) + " handle is NULL");
    return *handle;
}

dl::Device convert(dl_device value) { return {static_cast<dl::DeviceType>(value.type), value.index}; }
dl_device convert(dl::Device value) { return {static_cast<dl_device_type>(value.type), value.index}; }
dl::Shape convert(dl_shape value) { return value.size == 0 ? dl::Shape{} : dl::Shape(value.data, value.data + value.size); }
dl::TensorOptions convert(dl_tensor_options value) {
    return {static_cast<dl::DType>(value.dtype), convert(value.device), value.requires_grad != 0};
}

template <class Module> Module& as(dl_module* module, const char* what) {
    auto* typed = dynamic_cast<Module*>(need(module, "module").value.get());
    if (!typed) throw std::invalid_argument(std::string("module is not a ") + what);
    return *typed;
}
template <class Module> std::shared_ptr<Module> shared_as(const dl_module* module, const char* what) {
    auto typed = std::dynamic_pointer_cast<Module>(need(module, "module").value);
    if (!typed) throw std::invalid_argument(std::string("module is not a ") + what);
    return typed;
}

std::mutex timer_mutex;
cudaEvent_t timer_events[64][2];

}  // namespace

extern "C" {

const char* dl_version(void) { return DL_VERSION; }
const char* dl_last_error(void) { return last_error; }
dl_tensor_options dl_default_tensor_options(void) { return {DL_F32, {DL_CPU, 0}, 0}; }

// ---- tensors ------------------------------------------------------------------------------------------------
void dl_tensor_release(dl_tensor* tensor) { delete tensor; }
dl_status dl_tensor_retain(const dl_tensor* tensor, dl_tensor** output) {
    return make_handle(output, [&] { return need(tensor, "tensor").value; });
}
dl_tensor_info dl_tensor_get_info(const dl_tensor* tensor) {
    const auto& t = tensor->value;
    return {static_cast<dl_dtype>(t.dtype()), convert(t.device()), t.numel(), 1, 0, 1};
}
dl_shape dl_tensor_shape(const dl_tensor* tensor) { return {tensor->value.shape().data(), tensor->value.shape().size()}; }
dl_shape dl_tensor_strides(const dl_tensor* tensor) { return {tensor->value.strides().data(), tensor->value.strides().size()}; }
const void* dl_tensor_data(const dl_tensor* tensor) { return tensor->value.raw_data(); }
size_t dl_tensor_nbytes(const dl_tensor* tensor) { return tensor->value.nbytes(); }
dl_status dl_tensor_copy_to_host(const dl_tensor* tensor, void* destination) {
    return invoke([&] {
        if (!destination) throw std::invalid_argument("destination is NULL");
        need(tensor, "tensor").value.copy_to_host(destination);
    });
}
dl_status dl_from_host(const void* data, dl_shape shape, dl_tensor_options options, dl_tensor** output) {
    return make_handle(output, [&] {
        if (!data) throw std::invalid_argument("data is NULL");
        return dl::detail::from_host(data, convert(shape), static_cast<dl::DType>(options.dtype), false, convert(options.device));
    });
}
dl_status dl_full(dl_shape shape, double value, dl_tensor_options options, dl_tensor** output) {
    return make_handle(output, [&] { return dl::full(convert(shape), value, convert(options)); });
}
dl_status dl_zeros(dl_shape shape, dl_tensor_options options, dl_tensor** output) {
    return make_handle(output, [&] { return dl::zeros(convert(shape), convert(options)); });
}
dl_status dl_ones(dl_shape shape, dl_tensor_options options, dl_tensor** output) {
    return make_handle(output, [&] { return dl::ones(convert(shape), convert(options)); });
}
dl_status dl_clone(const dl_tensor* input, dl_tensor** output) {
    return make_handle(output, [&] { return need(input, "tensor").value.clone(); });
}
dl_status dl_astype(const dl_tensor* input, dl_dtype dtype, dl_tensor** output) {
    return make_handle(output, [&] { return need(input, "tensor").value.astype(static_cast<dl::DType>(dtype)); });
}
dl_status dl_to(const dl_tensor* input, dl_device device, dl_tensor** output) {
    return make_handle(output, [&] { return need(input, "tensor").value.to(convert(device)); });
}
dl_status dl_reshape(const dl_tensor* input, dl_shape shape, dl_tensor** output) {
    return make_handle(output, [&] { return need(input, "tensor").value.reshape(convert(shape)); });
}
dl_status dl_select(const dl_tensor* input, int64_t axis, int64_t index, dl_tensor** output) {
    return make_handle(output, [&] {
        const auto& t = need(input, "tensor").value;
        const auto a = axis < 0 ? axis + t.ndim() : axis;
        if (a < 0 || a >= t.ndim()) throw std::out_of_range("axis out of range");
        const auto extent = t.shape()[static_cast<std::size_t>(a)];
        return t.select(a, index < 0 ? index + extent : index);
    });
}
dl_status dl_narrow(const dl_tensor* input, int64_t axis, int64_t start, int64_t length, dl_tensor** output) {
    return make_handle(output, [&] { return need(input, "tensor").value.narrow(axis, start, length); });
}

// ---- operators ------------------------------------------------------------------------------------------
dl_status dl_argmax(const dl_tensor* input, int64_t axis, int32_t keepdim, dl_tensor** output) {
    return make_handle(output, [&] { return dl::argmax(need(input, "tensor").value, axis, keepdim ? dl::KeepDim::yes : dl::KeepDim::no); });
}
dl_status dl_linear(const dl_tensor* input, const dl_tensor* weight, const dl_tensor* bias, dl_tensor** output) {
    return make_handle(output, [&] {
        return dl::linear(need(input, "tensor").value, need(weight, "tensor").value, bias ? std::optional{bias->value} : std::nullopt);
    });
}
dl_status dl_embedding(const dl_tensor* indices, const dl_tensor* weight, dl_tensor** output) {
    return make_handle(output, [&] { return dl::embedding(need(indices, "tensor").value, need(weight, "tensor").value); });
}
dl_status dl_rms_norm(const dl_tensor* input, dl_shape normalized_shape, const dl_tensor* weight, const double* epsilon,
                      dl_tensor** output) {
    return make_handle(output, [&] {
        return dl::rms_norm(need(input, "tensor").value, convert(normalized_shape), weight ? std::optional{weight->value} : std::nullopt,
                            epsilon ? std::optional{*epsilon} : std::nullopt);
    });
}
dl_status dl_synchronize(dl_device device) { return invoke([&] { dl::synchronize(convert(device)); }); }
dl_status dl_rotary_embedding(const dl_tensor* input, const dl_tensor* cosine, const dl_tensor* sine, dl_tensor** output) {
    return make_handle(output, [&] {
        return dl::rotary_embedding(need(input, "tensor").value, need(cosine, "tensor").value, need(sine, "tensor").value);
    });
}
dl_status dl_tensordot(const dl_tensor* a, const dl_tensor* b, dl_shape axes_a, dl_shape axes_b, dl_tensor** output) {
    return make_handle(output, [&] { return dl::tensordot(need(a, "tensor").value, need(b, "tensor").value, convert(axes_a), convert(axes_b)); });
}
dl_status dl_grouped_query_attention(const dl_tensor* query, const dl_tensor* key, const dl_tensor* value,
                                     const dl_tensor* keep_mask, dl_tensor** output) {
    return make_handle(output, [&] {
        return dl::grouped_query_attention(need(query, "tensor").value, need(key, "tensor").value, need(value, "tensor").value,
                                           keep_mask ? std::optional{keep_mask->value} : std::nullopt);
    });
}

// ---- modules ------------------------------------------------------------------------------------------------
void dl_module_release(dl_module* module) { delete module; }
dl_status dl_module_retain(const dl_module* module, dl_module** output) {
    return make_handle(output, [&] { return need(module, "module").value; });
}
dl_status dl_linear_create(int64_t input_features, int64_t output_features, int32_t bias, dl_tensor_options options,
                           dl_module** output) {
    return make_handle(output, [&] { return std::make_shared<dl::nn::Linear>(input_features, output_features, bias != 0, convert(options)); });
}
dl_status dl_linear_from_tensors(const dl_tensor* weight, const dl_tensor* bias, dl_module** output) {
    return make_handle(output, [&] {
        return std::make_shared<dl::nn::Linear>(need(weight, "tensor").value, bias ? std::optional{bias->value} : std::nullopt);
    });
}
dl_status dl_embedding_create(int64_t vocabulary, int64_t dimensions, dl_tensor_options options, dl_module** output) {
    return make_handle(output, [&] { return std::make_shared<dl::nn::Embedding>(vocabulary, dimensions, convert(options)); });
}
dl_status dl_embedding_from_tensor(const dl_tensor* weight, dl_module** output) {
    return make_handle(output, [&] { return std::make_shared<dl::nn::Embedding>(need(weight, "tensor").value); });
}
dl_status dl_rms_norm_create(dl_shape normalized_shape, const double* epsilon, int32_t affine, dl_tensor_options options,
                             dl_module** output) {
    return make_handle(output, [&] {
        return std::make_shared<dl::nn::RMSNorm>(convert(normalized_shape), epsilon ? std::optional{*epsilon} : std::nullopt,
                                                 affine != 0, convert(options));
    });
}
dl_status dl_module_forward(dl_module* module, const dl_tensor* input, dl_tensor** output) {
    return make_handle(output, [&] { return need(module, "module").value->forward(need(input, "tensor").value); });
}
dl_status dl_module_train(dl_module* module, int32_t training) {
    return invoke([&] { need(module, "module").value->train(training != 0); });
}
int32_t dl_module_is_training(const dl_module* module) { return module && module->value->is_training(); }
dl_status dl_module_to(dl_module* module, dl_device device) {
    return invoke([&] { need(module, "module").value->to(convert(device)); });
}
dl_status dl_module_state(const dl_module* module, dl_state** output) {
    return make_handle(output, [&] { return need(module, "module").value->state_dict(); });
}
dl_status dl_module_load_state(dl_module* module, const dl_state* state) {
    return invoke([&] { need(module, "module").value->load_state_dict(need(state, "state").value); });
}
void dl_state_release(dl_state* state) { delete state; }
size_t dl_state_size(const dl_state* state) { return state ? state->value.size() : 0; }
const char* dl_state_name(const dl_state* state, size_t index) {
    return state && index < state->value.size() ? state->value[index].first.c_str() : nullptr;
}
dl_status dl_state_tensor(const dl_state* state, size_t index, dl_tensor** output) {
    return make_handle(output, [&] { return need(state, "state").value.at(index).second; });
}
dl_status dl_state_create(const char* const* names, const dl_tensor* const* tensors, size_t count, dl_state** output) {
    return make_handle(output, [&] {
        dl::StateDict result;
        for (size_t i = 0; i < count; ++i) result.emplace_back(names[i], need(tensors[i], "tensor").value);
        return result;
    });
}

dl_status dl_state_save(const char* path, const dl_state* state) {
    return invoke([&] {
        if (!path) throw std::invalid_argument("path is NULL");
        dl::io::save(path, need(state, "state").value);
    });
}
dl_status dl_state_load(const char* path, dl_state** output) {
    return make_handle(output, [&] {
        if (!path) throw std::invalid_argument("path is NULL");
        return dl::io::load(path);
    });
}

// ---- decoder ------------------------------------------------------------------------------------------------
dl_status dl_swiglu_create(int64_t dimensions, int64_t hidden, int32_t bias, dl_tensor_options options, dl_module** output) {
    return make_handle(output, [&] { return std::make_shared<dl::nn::SwiGLU>(dimensions, hidden, bias != 0, convert(options)); });
}
dl_status dl_lora_linear_create(const dl_module* base, int64_t rank, double alpha, dl_module** output) {
    return make_handle(output, [&] { return std::make_shared<dl::nn::LoRALinear>(*shared_as<dl::nn::Linear>(base, "Linear"), rank, alpha); });
}
dl_status dl_lora_linear_merge(const dl_module* adapter, dl_module** output) {
    return make_handle(output, [&] { return shared_as<dl::nn::LoRALinear>(adapter, "LoRALinear")->merged(); });
}
dl_status dl_rotary_embedding_create(int64_t dimensions, int64_t capacity, double base, dl_tensor_options options,
                                     dl_module** output) {
    return make_handle(output, [&] { return std::make_shared<dl::nn::RotaryEmbedding>(dimensions, capacity, base, convert(options)); });
}
dl_status dl_rotary_embedding_forward(dl_module* rotary, const dl_tensor* input, int64_t offset, dl_tensor** output) {
    return make_handle(output, [&] { return as<dl::nn::RotaryEmbedding>(rotary, "RotaryEmbedding").forward(need(input, "tensor").value, offset); });
}
dl_status dl_grouped_query_attention_create(int64_t dimensions, int64_t heads, int64_t kv_heads, int64_t context,
                                            dl_tensor_options options, dl_module** output) {
    return make_handle(output, [&] {
        return std::make_shared<dl::nn::GroupedQueryAttention>(dimensions, heads, kv_heads, context, convert(options));
    });
}
dl_status dl_transformer_decoder_create(int64_t layers, int64_t dimensions, int64_t heads, int64_t kv_heads, int64_t hidden,
                                        int64_t context, dl_tensor_options options, dl_module** output) {
    return make_handle(output, [&] {
        return std::make_shared<dl::nn::TransformerDecoder>(layers, dimensions, heads, kv_heads, hidden, context, convert(options));
    });
}
dl_status dl_decoder_cache_create(const dl_module* decoder, dl_decoder_cache** output) {
    return make_handle(output, [&] { return shared_as<dl::nn::TransformerDecoder>(decoder, "TransformerDecoder")->make_cache(); });
}
void dl_decoder_cache_release(dl_decoder_cache* cache) { delete cache; }
dl_status dl_decoder_cache_clear(dl_decoder_cache* cache) {
    return invoke([&] { for (auto& layer : need(cache, "cache").value) layer.clear(); });
}
dl_status dl_decoder_cache_truncate(dl_decoder_cache* cache, int64_t length) {
    return invoke([&] {
        auto& layers = need(cache, "cache").value;
        for (const auto& layer : layers)
            if (length < 0 || length > layer.length()) throw std::out_of_range("KV cache truncation must keep an existing prefix");
        for (auto& layer : layers) layer.truncate(length);
    });
}
dl_status dl_decoder_cache_length(const dl_decoder_cache* cache, int64_t* length) {
    return invoke([&] {
        if (!length) throw std::invalid_argument("length slot is NULL");
        const auto& layers = need(cache, "cache").value;
        *length = layers.empty() ? 0 : layers.front().length();
    });
}
dl_status dl_transformer_decoder_decode(dl_module* decoder, const dl_tensor* input, dl_decoder_cache* cache, dl_tensor** output) {
    return make_handle(output, [&] {
        return as<dl::nn::TransformerDecoder>(decoder, "TransformerDecoder").decode(need(input, "tensor").value, need(cache, "cache").value);
    });
}

// ---- new entry points ---------------------------------------------------------------------------------------
dl_status dl_transformer_decoder_set_activation_dtype(dl_module* decoder, dl_dtype dtype) {
    return invoke([&] { as<dl::nn::TransformerDecoder>(decoder, "TransformerDecoder").set_activation_dtype(static_cast<dl::DType>(dtype)); });
}
dl_status dl_transformer_decoder_set_cache_dtype(dl_module* decoder, dl_dtype dtype) {
    return invoke([&] {
        if (dtype != DL_F32 && dtype != DL_BF16) throw std::invalid_argument("cache dtype must be f32 or bf16");
        as<dl::nn::TransformerDecoder>(decoder, "TransformerDecoder").set_cache_dtype(static_cast<dl::DType>(dtype));
    });
}
dl_status dl_transformer_decoder_set_adapters(dl_module* decoder, int64_t layer, const dl_module* query, const dl_module* value) {
    return invoke([&] {
        auto& model = as<dl::nn::TransformerDecoder>(decoder, "TransformerDecoder");
        if (layer < 0 || layer >= model.layer_count()) throw std::out_of_range("layer index out of range");
        model.layer(layer).attention().set_adapters(query ? shared_as<dl::nn::LoRALinear>(query, "LoRALinear") : nullptr,
                                                    value ? shared_as<dl::nn::LoRALinear>(value, "LoRALinear") : nullptr);
    });
}
dl_status dl_generation_create(dl_module* decoder, dl_module* embedding, dl_module* output, dl_decoder_cache* cache,
                               int64_t batch, int64_t max_steps, dl_generation** result) {
    return make_handle(result, [&] {
        return std::make_unique<dl::nn::Generation>(shared_as<dl::nn::TransformerDecoder>(decoder, "TransformerDecoder"),
                                                    shared_as<dl::nn::Embedding>(embedding, "Embedding"),
                                                    shared_as<dl::nn::Linear>(output, "Linear"), &need(cache, "cache").value, batch, max_steps);
    });
}
void dl_generation_release(dl_generation* generation) { delete generation; }
dl_status dl_generation_prefill(dl_generation* generation, const dl_tensor* prompt) {
    return invoke([&] { need(generation, "generation").value->prefill(need(prompt, "tensor").value); });
}
dl_status dl_generation_step(dl_generation* generation, int64_t steps) {
    return invoke([&] { need(generation, "generation").value->step(steps); });
}
dl_status dl_generation_step_host(dl_generation* generation, const int64_t* ids_in, int64_t* ids_out) {
    return invoke([&] { need(generation, "generation").value->step_host(ids_in, ids_out); });
}
dl_status dl_onnx_save_decoder(const char* path, const dl_module* decoder, const dl_module* embedding, const dl_module* output) {
    return invoke([&] {
        if (!path) throw std::invalid_argument("path is NULL");
        const auto model = std::dynamic_pointer_cast<dl::nn::TransformerDecoder>(need(decoder, "module").value);
        if (!model) throw std::invalid_argument("module is not a TransformerDecoder");
        if (!embedding && !output) return dl::onnx::save_decoder(path, *model);
        if (!embedding || !output) throw std::invalid_argument("decoder export needs both embedding and output layers");
        const auto table = std::dynamic_pointer_cast<dl::nn::Embedding>(embedding->value);
        const auto head = std::dynamic_pointer_cast<dl::nn::Linear>(output->value);
        if (!table || !head) throw std::invalid_argument("decoder export needs an Embedding and a Linear");
        dl::onnx::save_decoder(path, *table, *model, *head);
    });
}
int64_t dl_b200_shadow_partial_rows(int64_t dimensions, int64_t hidden) {
    return dimensions > 0 && hidden > 0 ? dl::nn::shadow_partial_rows(dimensions, hidden) : 0;
}
dl_status dl_generation_run_host(dl_generation* generation, const int64_t* ids_in, int64_t steps, int64_t* ids_out) {
    return invoke([&] {
        auto& run = *need(generation, "generation").value;
        if (steps < 0 || (steps > 0 && !ids_out)) throw std::invalid_argument("run_host needs a non-negative step count and a result buffer");
        const int64_t batch = run.batch();
        for (int64_t i = 0; i < steps; ++i) run.step_host(i == 0 ? ids_in : ids_out + (i - 1) * batch, ids_out + i * batch);
    });
}
dl_status dl_generation_step_sampled(dl_generation* generation, double temperature, const double* uniforms, int64_t* ids_out) {
    return invoke([&] { need(generation, "generation").value->step_sampled(temperature, uniforms, ids_out); });
}
dl_status dl_generation_tokens(dl_generation* generation, dl_tensor** output) {
    return make_handle(output, [&] { return need(generation, "generation").value->tokens(); });
}
dl_status dl_generation_logits(dl_generation* generation, dl_tensor** output) {
    return make_handle(output, [&] { return need(generation, "generation").value->last_logits(); });
}
int64_t dl_generation_launches_per_step(const dl_generation* generation) {
    return generation ? generation->value->launches_per_step() : 0;
}
dl_status dl_generation_profile_step(dl_generation* generation, double milliseconds[4]) {
    return invoke([&] {
        if (!milliseconds) throw std::invalid_argument("result slot is NULL");
        const auto profile = need(generation, "generation").value->profile_step();
        milliseconds[0] = profile.linear_ms; milliseconds[1] = profile.attention_ms; milliseconds[2] = profile.other_ms;
        milliseconds[3] = static_cast<double>(profile.launches);
    });
}
dl_status dl_decoder_generate(dl_module* decoder, dl_module* embedding, dl_module* output, const dl_tensor* prompt,
                              int64_t steps, dl_decoder_cache* cache, dl_tensor** tokens) {
    return make_handle(tokens, [&] {
        const auto& ids = need(prompt, "tensor").value;
        if (steps <= 0) throw std::invalid_argument("generation needs at least one step");
        if (ids.ndim() != 2) throw std::invalid_argument("prompt must be int64 [batch, length]");
        dl::nn::Generation generation(shared_as<dl::nn::TransformerDecoder>(decoder, "TransformerDecoder"),
                                      shared_as<dl::nn::Embedding>(embedding, "Embedding"), shared_as<dl::nn::Linear>(output, "Linear"),
                                      &need(cache, "cache").value, ids.size(0), steps);
        generation.prefill(ids);
        generation.step(steps - 1);
        return generation.tokens().to(ids.device());
    });
}

dl_status dl_b200_tp_unique_id(void* id128) {
    return invoke([&] {
        if (!id128) throw std::invalid_argument("id slot is NULL");
        dl::runtime::tp_unique_id(id128);
    });
}
dl_status dl_b200_tp_init(dl_device device, int32_t rank, int32_t world, const void* id128) {
    return invoke([&] {
        if (device.type != DL_CUDA) throw std::invalid_argument("tensor parallelism needs a CUDA device");
        dl::runtime::tp_init(device.index, rank, world, id128);
    });
}
dl_status dl_b200_tp_symmetric_handle(dl_device device, size_t slot_bytes, void* handle64) {
    return invoke([&] { dl::runtime::tp_symmetric_handle(device.index, slot_bytes, handle64); });
}
dl_status dl_b200_tp_symmetric_open(dl_device device, const void* handles, int32_t world) {
    return invoke([&] { dl::runtime::tp_symmetric_open(device.index, handles, world); });
}
dl_status dl_b200_tp_set_push(dl_device device, int32_t push) {
    return invoke([&] { dl::runtime::tp_set_push(device.index, push != 0); });
}
dl_status dl_b200_tp_finalize(dl_device device) { return invoke([&] { dl::runtime::tp_finalize(device.index); }); }
dl_status dl_transformer_decoder_set_tensor_parallel(dl_module* decoder, int32_t rank, int32_t world) {
    return invoke([&] { as<dl::nn::TransformerDecoder>(decoder, "TransformerDecoder").set_tensor_parallel(rank, world); });
}

dl_status dl_b200_timer_start(dl_device device) {
    return invoke([&] {
        if (device.type != DL_CUDA || device.index < 0 || device.index >= 64) throw std::invalid_argument("timer needs a CUDA device");
        std::lock_guard<std::mutex> lock(timer_mutex);
        dl::runtime::set_device(device.index);
        auto stream = static_cast<cudaStream_t>(dl::runtime::stream(device.index));
        for (auto& event : timer_events[device.index])
            if (!event) dl::runtime::check_cuda(cudaEventCreate(&event), "cudaEventCreate");
        dl::runtime::check_cuda(cudaEventRecord(timer_events[device.index][0], stream), "cudaEventRecord");
    });
}
dl_status dl_b200_timer_stop(dl_device device, double* milliseconds) {
    return invoke([&] {
        if (device.type != DL_CUDA || device.index < 0 || device.index >= 64 || !milliseconds) throw std::invalid_argument("timer needs a CUDA device and a result slot");
        std::lock_guard<std::mutex> lock(timer_mutex);
        if (!timer_events[device.index][0]) throw std::logic_error("timer was not started");
        dl::runtime::set_device(device.index);
        auto stream = static_cast<cudaStream_t>(dl::runtime::stream(device.index));
        dl::runtime::check_cuda(cudaEventRecord(timer_events[device.index][1], stream), "cudaEventRecord");
        dl::runtime::check_cuda(cudaEventSynchronize(timer_events[device.index][1]), "cudaEventSynchronize");
        float ms = 0.0f;
        dl::runtime::check_cuda(cudaEventElapsedTime(&ms, timer_events[device.index][0], timer_events[device.index][1]), "cudaEventElapsedTime");
        *milliseconds = ms;
    });
}
void* dl_b200_stream(dl_device device) {
    void* stream = nullptr;
    invoke([&] { stream = dl::runtime::stream(device.index); });
    return stream;
}

}  // extern "C"
