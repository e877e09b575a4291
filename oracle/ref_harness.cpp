// ref_harness.cpp -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// A C-ABI window onto the UNMODIFIED Ctorch reference CPU library (compiled by oracle/Makefile from the
// reference's own sources into oracle/_ref/libctorch_ref.a).  It drives the reference strictly through its
// public C++ API (dl::nn::TransformerDecoder, Embedding, Linear, KVCache, dl::grouped_query_attention, ...)
// the way examples/decoder_model.h:10-39 and examples/decoder_generate.cpp:16-31 do, so that
//   * oracle/decoder_oracle.c can be validated bit-for-bit against the real thing,
//   * golden vectors under tests/golden/ can be generated, and
//   * the reference's CPU decoder can be timed as the CPU baseline on the benchmark host.
// Function names and argument meaning mirror decoder_oracle.c with the prefix ref_.
#include "dl/dl.h"
#include "dl/onnx.h"

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cmath>
#include <memory>
#include <random>
#include <string>
#include <barrier>
#include <chrono>
#include <thread>
#include <vector>

namespace {

struct Config {  // must match oracle_config in decoder_oracle.c
    int64_t vocab, d_model, layers, heads, kv_heads, hidden, context;
    int32_t weight_dtype, tied;
    double eps, rope_base;
    int64_t lora_rank;
    double lora_alpha;
};

thread_local char last_error[512];

template <class Function> int guarded(Function&& function) noexcept {
    try {
        function();
        return 0;
    } catch (const std::exception& error) {
        std::snprintf(last_error, sizeof last_error, "%s", error.what());
    } catch (...) {
        std::snprintf(last_error, sizeof last_error, "unknown exception");
    }
    return 1;
}

dl::DType dtype_of_code(int32_t code) { return code == 5 ? dl::DType::bf16 : dl::DType::f32; }

dl::Tensor host_tensor(const void* data, dl::Shape shape, dl::DType dtype) {
    return dl::detail::from_host(data, std::move(shape), dtype, false, dl::Device::cpu());
}

// A "generator" whose every draw makes std::generate_canonical<double, 53> return a chosen u = k / 2^53: with a 64-bit
// range libstdc++ takes one draw v and returns double(v) / 2^64.
struct FixedBits {
    using result_type = std::uint64_t;
    double u;
    static constexpr result_type min() { return 0; }
    static constexpr result_type max() { return ~static_cast<result_type>(0); }
    result_type operator()() const { return static_cast<result_type>(std::ldexp(u, 53)) << 11; }
};

struct Model {
    Config cfg;
    std::shared_ptr<dl::nn::Embedding> tokens;
    std::shared_ptr<dl::nn::TransformerDecoder> decoder;
    std::shared_ptr<dl::nn::Linear> output;
};

struct Cache {
    std::vector<dl::nn::KVCache> layers;
};

void copy_out(const dl::Tensor& tensor, float* destination) {
    auto dense = tensor.astype(dl::DType::f32).contiguous();
    std::memcpy(destination, dense.data<float>(), sizeof(float) * static_cast<std::size_t>(dense.numel()));
}

dl::Tensor model_decode(Model& model, Cache& cache, const int64_t* ids, int64_t batch, int64_t length) {
    dl::NoGradGuard inference;
    auto input = host_tensor(ids, {batch, length}, dl::DType::i64);
    return (*model.output)(model.decoder->decode((*model.tokens)(input), cache.layers));
}

}  // namespace

extern "C" {

const char* ref_last_error(void) { return last_error; }

// Same tensor order as oracle_decoder_create.  Adapters cannot be hosted inside the reference's
// GroupedQueryAttention (typed Linear members, include/dl/decoder.h:75), so lora must be NULL here; use
// ref_lora_linear / ref_lora_merge for the adapter arithmetic.
void* ref_decoder_create(const Config* cfg, const void* const* tensors, const void* const* lora) {
    Model* model = nullptr;
    if (guarded([&] {
            if (lora || cfg->lora_rank) throw std::invalid_argument("reference decoder cannot host unmerged adapters");
            const auto dtype = dtype_of_code(cfg->weight_dtype);
            const dl::TensorOptions options{.dtype = dtype};
            const int64_t D = cfg->d_model, F = cfg->hidden, hd = D / cfg->heads, KV = cfg->kv_heads * hd, V = cfg->vocab;
            auto fresh = std::make_unique<Model>();
            fresh->cfg = *cfg;
            int64_t next = 0;
            fresh->tokens = std::make_shared<dl::nn::Embedding>(host_tensor(tensors[next++], {V, D}, dtype));
            fresh->decoder = std::make_shared<dl::nn::TransformerDecoder>(cfg->layers, D, cfg->heads, cfg->kv_heads, F,
                                                                         cfg->context, options);
            dl::StateDict state = fresh->decoder->state_dict();
            auto replace = [&](const std::string& name, dl::Shape shape) {
                for (auto& entry : state)
                    if (entry.first == name) {
                        entry.second = host_tensor(tensors[next++], std::move(shape), dtype);
                        return;
                    }
                throw std::invalid_argument("missing state entry " + name);
            };
            for (int64_t i = 0; i < cfg->layers; ++i) {
                const auto p = "layer" + std::to_string(i) + ".";
                replace(p + "attention.query.weight", {D, D});
                replace(p + "attention.key.weight", {KV, D});
                replace(p + "attention.value.weight", {KV, D});
                replace(p + "attention.output.weight", {D, D});
                replace(p + "feedforward.gate.weight", {F, D});
                replace(p + "feedforward.up.weight", {F, D});
                replace(p + "feedforward.down.weight", {D, F});
                replace(p + "attention_norm.weight", {D});
                replace(p + "feedforward_norm.weight", {D});
            }
            replace("normalization.weight", {D});
            fresh->decoder->load_state_dict(state);
            fresh->decoder->eval();
            fresh->output = cfg->tied ? std::make_shared<dl::nn::Linear>(fresh->tokens->weight())
                                      : std::make_shared<dl::nn::Linear>(host_tensor(tensors[next++], {V, D}, dtype));
            model = fresh.release();
        }))
        return nullptr;
    return model;
}
void ref_decoder_release(void* model) { delete static_cast<Model*>(model); }

// The cosine / sine buffers of layer0's rotary module, [context, hd/2] f32.
int ref_decoder_rope_tables(void* handle, float* cosine, float* sine) {
    return guarded([&] {
        for (const auto& [name, tensor] : static_cast<Model*>(handle)->decoder->state_dict()) {
            if (name == "layer0.attention.rotary.cosine") copy_out(tensor, cosine);
            if (name == "layer0.attention.rotary.sine") copy_out(tensor, sine);
        }
    });
}

// Writes the state_dict names, newline separated, into text (truncated to capacity).
int ref_decoder_state_names(void* handle, char* text, int64_t capacity) {
    return guarded([&] {
        std::string all;
        for (const auto& [name, tensor] : static_cast<Model*>(handle)->decoder->state_dict()) {
            all += name + " " + std::to_string(static_cast<int>(tensor.dtype())) + "\n";
        }
        std::snprintf(text, static_cast<std::size_t>(capacity), "%s", all.c_str());
    });
}

void* ref_cache_create(void* model) {
    Cache* cache = nullptr;
    if (guarded([&] { cache = new Cache{static_cast<Model*>(model)->decoder->make_cache()}; })) return nullptr;
    return cache;
}
void ref_cache_release(void* cache) { delete static_cast<Cache*>(cache); }
int64_t ref_cache_length(void* cache) {
    auto& layers = static_cast<Cache*>(cache)->layers;
    return layers.empty() ? 0 : layers.front().length();
}
void ref_cache_clear(void* cache) {
    for (auto& layer : static_cast<Cache*>(cache)->layers) layer.clear();
}
int ref_cache_truncate(void* cache, int64_t length) {
    return guarded([&] {
        for (auto& layer : static_cast<Cache*>(cache)->layers) layer.truncate(length);
    });
}
// dtype code of the cached keys of a layer (-1 before the first append); documents that the reference keeps
// an f32 cache even for bf16 weights.
int ref_cache_dtype(void* cache, int64_t layer) {
    int code = -1;
    guarded([&] { code = static_cast<int>(static_cast<Cache*>(cache)->layers[static_cast<std::size_t>(layer)].key().dtype()); });
    return code;
}
int ref_cache_copy(void* cache, int64_t layer, int32_t which, float* destination) {
    return guarded([&] {
        auto& entry = static_cast<Cache*>(cache)->layers[static_cast<std::size_t>(layer)];
        copy_out(which ? entry.value() : entry.key(), destination);  // [batch, kv_heads, length, hd]
    });
}

int ref_decoder_decode(void* handle, void* cache, const float* x, int64_t batch, int64_t length, float* out) {
    return guarded([&] {
        auto& model = *static_cast<Model*>(handle);
        auto input = host_tensor(x, {batch, length, model.cfg.d_model}, dl::DType::f32);
        copy_out(model.decoder->decode(input, static_cast<Cache*>(cache)->layers), out);
    });
}

int ref_model_decode(void* handle, void* cache, const int64_t* ids, int64_t batch, int64_t length, float* logits) {
    return guarded([&] {
        copy_out(model_decode(*static_cast<Model*>(handle), *static_cast<Cache*>(cache), ids, batch, length), logits);
    });
}

// examples/decoder_generate.cpp:20-31 for a batch.
int ref_generate(void* handle, void* cache_handle, const int64_t* prompt, int64_t batch, int64_t prompt_length,
                 int64_t steps, int64_t* tokens, float* logits) {
    return guarded([&] {
        auto& model = *static_cast<Model*>(handle);
        auto& cache = *static_cast<Cache*>(cache_handle);
        const int64_t V = model.cfg.vocab;
        std::vector<int64_t> next(prompt, prompt + batch * prompt_length);
        int64_t length = prompt_length;
        for (int64_t step = 0; step < steps; ++step) {
            auto last = model_decode(model, cache, next.data(), batch, length).select(1, length - 1);
            auto chosen = dl::argmax(last, -1).to_vector<int64_t>();
            if (logits) copy_out(last, logits + step * batch * V);
            for (int64_t b = 0; b < batch; ++b) tokens[b * steps + step] = chosen[static_cast<std::size_t>(b)];
            next = chosen;
            length = 1;
        }
    });
}

// CPU baseline: `threads` workers share one read-only model; each owns a cache and runs the greedy loop on its
// own slice of the batch (one or more sequences per worker).  The reference's mutable globals are thread_local.
int ref_generate_threads(void* handle, const int64_t* prompt, int64_t batch, int64_t prompt_length, int64_t steps,
                         int64_t threads, int64_t* tokens) {
    std::vector<int> status(static_cast<std::size_t>(threads), 0);
    std::vector<std::thread> workers;
    const int64_t share = (batch + threads - 1) / threads;
    for (int64_t t = 0; t < threads; ++t) {
        workers.emplace_back([&, t] {
            const int64_t first = t * share, count = std::min(share, batch - first);
            if (count <= 0) return;
            void* cache = ref_cache_create(handle);
            status[static_cast<std::size_t>(t)] = !cache || ref_generate(handle, cache, prompt + first * prompt_length, count,
                                                                           prompt_length, steps, tokens + first * steps, nullptr);
            ref_cache_release(cache);
        });
    }
    for (auto& worker : workers) worker.join();
    for (int value : status)
        if (value) return 1;
    return 0;
}

// CPU-baseline timing: every worker prefills its slice of the batch and runs `warmup` single-token steps, all
// workers meet at a barrier, then each runs `steps` timed single-token steps (greedy feedback) and they meet again.
// seconds = wall time between the two barriers.
// `cached` > 0: before the prompt is decoded every layer cache receives `cached` positions of seeded pseudo-random K and V
// through the public KVCache::append, so that the timed steps attend over `cached + prompt_length + ...` positions without
// paying a CPU prefill of that length (step time depends on the context length, not on the cached values).
int ref_timed_decode(void* handle, const int64_t* prompt, int64_t batch, int64_t prompt_length, int64_t warmup,
                     int64_t steps, int64_t threads, int64_t cached, double* seconds) {
    if (threads > batch) threads = batch;
    std::vector<int> status(static_cast<std::size_t>(threads), 0);
    std::chrono::steady_clock::time_point begin, end;
    std::barrier start(static_cast<std::ptrdiff_t>(threads), [&]() noexcept { begin = std::chrono::steady_clock::now(); });
    std::barrier finish(static_cast<std::ptrdiff_t>(threads), [&]() noexcept { end = std::chrono::steady_clock::now(); });
    const int64_t share = (batch + threads - 1) / threads;
    std::vector<std::thread> workers;
    for (int64_t t = 0; t < threads; ++t) {
        workers.emplace_back([&, t] {
            const int64_t first = t * share, count = std::max<int64_t>(0, std::min(share, batch - first));
            std::vector<int64_t> next;
            Cache cache;
            int failed = guarded([&] {
                if (!count) return;
                auto& model = *static_cast<Model*>(handle);
                cache.layers = model.decoder->make_cache();
                if (cached > 0) {
                    const int64_t hd = model.cfg.d_model / model.cfg.heads;
                    std::vector<float> filler(static_cast<std::size_t>(count * model.cfg.kv_heads * cached * hd));
                    std::uint32_t state = 0x9e3779b9u + static_cast<std::uint32_t>(t);
                    for (auto& value : filler) {   // uniform in [-1, 1): a linear congruential sequence is enough here
                        state = state * 1664525u + 1013904223u;
                        value = static_cast<float>(static_cast<std::int32_t>(state)) * (1.0f / 2147483648.0f);
                    }
                    const auto block = host_tensor(filler.data(), {count, model.cfg.kv_heads, cached, hd}, dl::DType::f32);
                    for (auto& layer : cache.layers) layer.append(block, block);
                }
                auto last = model_decode(model, cache, prompt + first * prompt_length, count, prompt_length).select(1, prompt_length - 1);
                next = dl::argmax(last, -1).to_vector<int64_t>();
                for (int64_t i = 0; i < warmup; ++i)
                    next = dl::argmax(model_decode(model, cache, next.data(), count, 1).select(1, 0), -1).to_vector<int64_t>();
            });
            start.arrive_and_wait();
            if (!failed)
                failed = guarded([&] {
                    auto& model = *static_cast<Model*>(handle);
                    for (int64_t i = 0; i < steps && count; ++i)
                        next = dl::argmax(model_decode(model, cache, next.data(), count, 1).select(1, 0), -1).to_vector<int64_t>();
                });
            finish.arrive_and_wait();
            status[static_cast<std::size_t>(t)] = failed;
        });
    }
    for (auto& worker : workers) worker.join();
    *seconds = std::chrono::duration<double>(end - begin).count();
    for (int value : status)
        if (value) return 1;
    return 0;
}

// The model written by the reference's ONNX exporter (extensions/onnx/src/decoder.cpp): with_head != 0 exports
// input_ids -> logits with the (tied) table, otherwise features -> hidden states.
int ref_save_onnx(void* handle, const char* path, int with_head) {
    return guarded([&] {
        auto& model = *static_cast<Model*>(handle);
        if (with_head) dl::onnx::save_decoder(path, *model.tokens, *model.decoder, *model.output);
        else dl::onnx::save_decoder(path, *model.decoder);
    });
}

int ref_gqa_attention(const float* query, const float* key, const float* value, int64_t batch, int64_t heads,
                      int64_t kv_heads, int64_t length, int64_t source, int64_t head_dim, int64_t causal_offset,
                      float* out) {
    return guarded([&] {
        dl::NoGradGuard inference;
        auto q = host_tensor(query, {batch, heads, length, head_dim}, dl::DType::f32);
        auto k = host_tensor(key, {batch, kv_heads, source, head_dim}, dl::DType::f32);
        auto v = host_tensor(value, {batch, kv_heads, source, head_dim}, dl::DType::f32);
        if (causal_offset >= 0) {
            // The public op has no offset argument; an explicit keep mask states the same rule
            // (key position <= query position, src/ops/attention.cpp:52-57).
            std::vector<uint8_t> keep(static_cast<std::size_t>(length * source));
            for (int64_t l = 0; l < length; ++l)
                for (int64_t s = 0; s < source; ++s) keep[static_cast<std::size_t>(l * source + s)] = s <= causal_offset + l;
            auto mask = host_tensor(keep.data(), {length, source}, dl::DType::boolean);
            copy_out(dl::grouped_query_attention(q, k, v, mask), out);
        } else {
            copy_out(dl::grouped_query_attention(q, k, v), out);
        }
    });
}

int ref_rms_norm(const float* x, const float* weight, int64_t rows, int64_t width, double eps, float* y) {
    return guarded([&] {
        dl::NoGradGuard inference;
        auto input = host_tensor(x, {rows, width}, dl::DType::f32);
        auto w = host_tensor(weight, {width}, dl::DType::f32);
        copy_out(dl::rms_norm(input, {width}, w, eps), y);
    });
}

// weight given as f32 values or bf16 bit patterns according to weight_dtype.
int ref_linear(const float* x, const void* w, int32_t weight_dtype, int64_t rows, int64_t in, int64_t out, float* y) {
    return guarded([&] {
        dl::NoGradGuard inference;
        auto input = host_tensor(x, {rows, in}, dl::DType::f32);
        auto weight = host_tensor(w, {out, in}, dtype_of_code(weight_dtype));
        copy_out(dl::linear(input, weight), y);
    });
}

int ref_silu_mul(const float* gate, const float* up, int64_t count, float* y) {
    return guarded([&] {
        dl::NoGradGuard inference;
        copy_out(dl::silu(host_tensor(gate, {count}, dl::DType::f32)) * host_tensor(up, {count}, dl::DType::f32), y);
    });
}

int ref_rotary(const float* x, int64_t batch, int64_t heads, int64_t length, int64_t head_dim, double base,
               int64_t capacity, int64_t offset, float* y) {
    return guarded([&] {
        dl::NoGradGuard inference;
        dl::nn::RotaryEmbedding rotary(head_dim, capacity, base);
        copy_out(rotary.forward(host_tensor(x, {batch, heads, length, head_dim}, dl::DType::f32), offset), y);
    });
}

int ref_argmax(const float* x, int64_t rows, int64_t width, int64_t* index) {
    return guarded([&] {
        auto chosen = dl::argmax(host_tensor(x, {rows, width}, dl::DType::f32), -1).to_vector<int64_t>();
        std::memcpy(index, chosen.data(), sizeof(int64_t) * chosen.size());
    });
}

// LoRALinear::forward and ::merged through the reference classes; weights in weight_dtype.
int ref_lora_linear(const float* x, const void* w, const void* down, const void* up, int32_t weight_dtype,
                    int64_t rows, int64_t in, int64_t out, int64_t rank, double alpha, float* y, void* merged) {
    return guarded([&] {
        dl::NoGradGuard inference;
        const auto dtype = dtype_of_code(weight_dtype);
        dl::nn::Linear base(host_tensor(w, {out, in}, dtype));
        dl::nn::LoRALinear adapter(base, rank, alpha);
        dl::StateDict state = adapter.state_dict();
        for (auto& [name, tensor] : state) {
            if (name == "down.weight") tensor = host_tensor(down, {rank, in}, dtype);
            if (name == "up.weight") tensor = host_tensor(up, {out, rank}, dtype);
        }
        adapter.load_state_dict(state);
        if (y) copy_out(adapter.forward(host_tensor(x, {rows, in}, dl::DType::f32)), y);
        if (merged) {
            auto weight = adapter.merged()->weight().contiguous();
            std::memcpy(merged, weight.data<char>(), dl::element_size(dtype) * static_cast<std::size_t>(weight.numel()));
        }
    });
}

// Weight archive written by the reference's own dl::io::save (src/io/checkpoint.cpp:97-104): "tokens.weight" and the
// decoder's state under "decoder.", the names of examples/decoder_model.h.  ref_archive_entry reads one back through
// dl::io::load: shape (up to 8 extents), dtype code, and the first `capacity` bytes of the elements.
int ref_save_state(void* handle, const char* path) {
    return guarded([&] {
        auto& model = *static_cast<Model*>(handle);
        dl::StateDict state;
        for (auto& [name, tensor] : model.tokens->state_dict()) state.emplace_back("tokens." + name, tensor);
        for (auto& [name, tensor] : model.decoder->state_dict()) state.emplace_back("decoder." + name, tensor);
        dl::io::save(path, state);
    });
}

int64_t ref_archive_size(const char* path) {
    int64_t count = -1;
    guarded([&] { count = static_cast<int64_t>(dl::io::load(path).size()); });
    return count;
}

int ref_archive_entry(const char* path, int64_t index, char* name, int64_t name_capacity, int64_t* shape8, int64_t* rank,
                      int32_t* dtype, void* bytes, int64_t capacity) {
    return guarded([&] {
        const auto state = dl::io::load(path);
        const auto& [entry_name, tensor] = state.at(static_cast<std::size_t>(index));
        std::snprintf(name, static_cast<std::size_t>(name_capacity), "%s", entry_name.c_str());
        *rank = tensor.ndim();
        for (int64_t i = 0; i < tensor.ndim() && i < 8; ++i) shape8[i] = tensor.shape()[static_cast<std::size_t>(i)];
        *dtype = static_cast<int32_t>(tensor.dtype());
        const auto dense = tensor.contiguous();
        const auto total = static_cast<int64_t>(dense.numel()) * static_cast<int64_t>(dl::element_size(dense.dtype()));
        std::memcpy(bytes, dense.data<char>(), static_cast<std::size_t>(std::min(total, capacity)));
    });
}

// The sampling lines of examples/text_generate.cpp:38-39 on the reference library: softmax(logits / temperature), then
// std::discrete_distribution driven by a generator that yields the caller's uniform variate (a multiple of 2^-53).
int ref_sample(const float* x, int64_t rows, int64_t width, double temperature, const double* uniform, int64_t* index) {
    return guarded([&] {
        dl::NoGradGuard inference;
        for (int64_t r = 0; r < rows; ++r) {
            auto logits = host_tensor(x + r * width, {width}, dl::DType::f32);
            auto probabilities = dl::softmax(logits / temperature, 0).to_vector<float>();
            FixedBits bits{uniform[r]};
            index[r] = std::discrete_distribution<int>(probabilities.begin(), probabilities.end())(bits);
        }
    });
}

}  // extern "C"
