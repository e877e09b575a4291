// Fixed execution plan of the decoder token loop and the device-resident greedy generation built on it.
//
// The reference walks Module::forward op by op (src/nn/decoder.cpp:77-142: ~35 launches per layer and token, every
// intermediate freshly allocated).  The plan instead owns packed weights (q|k|v rows concatenated, gate/up rows
// interleaved), persistent workspaces and a fixed kernel sequence per layer:
//     [adapter down-projection]  ->  RMSNorm + QKV + RoPE + KV append  ->  split-K attention (+ combine)
//     ->  o-projection + residual  ->  RMSNorm + gate/up + SiLU*up  ->  down-projection + residual
// For single-token steps the whole token loop body (embedding ... argmax, token feedback, cache length advance)
// is captured once into a CUDA graph and replayed.
#pragma once

#include "dl/dl.h"

#include <cuda_runtime.h>

#include <utility>

namespace dl::nn {

Tensor interleave_rows(const Tensor& even_rows, const Tensor& odd_rows);  // [n,k],[n,k] -> [2n,k]
Tensor concat_rows(std::span<const Tensor> parts);                          // [n_i,k] -> [sum n_i,k]
Tensor add(const Tensor& a, const Tensor& b);                               // f32 CUDA tensors of one shape
Tensor attention_block(GroupedQueryAttention& attention, const Tensor& input, KVCache& cache);
// Rows of the plan's partial-sum-of-squares buffers for a residual stream of width D and a (per-rank) SwiGLU width F.
Index shadow_partial_rows(Index D, Index F);

class DecodePlan {
public:
    explicit DecodePlan(TransformerDecoder& owner);
    ~DecodePlan();

    // TransformerDecoder::decode: features [batch, length, D] -> normalised features, caches advanced by `length`.
    Tensor decode(const Tensor& input, std::span<KVCache> cache);

    // Pieces used by Generation.  `x` holds rows = batch*length feature rows; the residual stream ends in hidden().
    void validate(Index batch, Index length, std::span<KVCache> cache, int device);
    // `shadow_ready`: the caller already produced the input shadow and its sums of squares (token path, see embed()).
    void run_layers(const float* x, Index batch, Index length, std::span<KVCache> cache, Index max_length, void* stream,
                    bool shadow_ready = false);
    // Token ids -> first hidden rows `x` (plus the input shadow when the shadow protocol is active).
    void embed(const Embedding& tokens, const Index* ids, Index rows, float* x, void* stream);
    // Logits of the last run_layers' rows (decode step: final norm folded into the projection).
    void logits(const Linear& output, Index rows, float* out, void* stream);
    // Fused logits + greedy choice (no logits in memory): prepare_choice() sizes the per-tile candidate buffers and says
    // whether the fused path serves this projection and row count; choose() enqueues the projection with the argmax
    // epilogue and the merge, which also feeds the chosen ids back (ids, history, counter as b200_token_feedback).
    bool prepare_choice(const Linear& output, Index rows, int device);
    // This rank's rows of the output table under tensor parallelism with mapped peer memory (first row, count); the whole
    // table otherwise.  The ranks then exchange one (value, index) candidate per row instead of each reading the table.
    std::pair<Index, Index> vocabulary_slice(const Linear& output, Index rows, int device) const;
    // `advance`: caches (at most 64) whose lengths the merge kernel moves on by one token, sparing the step a launch.
    void choose(const Linear& output, Index rows, Index* next, Index* ids, Index* history, Index history_rows, std::int32_t* counter,
                std::span<b200_kv_cache* const> advance, void* stream);
    // Who ran the plan last: the final hidden state in the workspaces belongs to that user (nullptr: Module::decode).
    void set_user(const void* user) { user_ = user; }
    const void* user() const { return user_; }
    // Whether a pass over `rows` activation rows runs on the shadow protocol (bf16 model and every projection inside
    // the limits of the kernel that serves that row count).
    bool shadows_for(Index rows) const;
    void reserve(Index rows, Index max_length, int device);
    float* hidden() const { return static_cast<float*>(h_.mutable_data()); }
    void refresh();  // re-pack weights when the owner's parameters moved
    std::uint64_t buffer_epoch() const { return buffer_epoch_; }  // moves when a workspace was reallocated

private:
    struct Layer {
        Tensor wqkv, wgu, lora_down, wo_slice, wd_slice;  // slices: tensor-parallel column cuts of o-proj / down
        const void *wo, *wd, *norm1, *norm2, *q_up, *v_up;
        int rank;
        float scale;
    };
    TransformerDecoder& owner_;
    std::vector<Layer> layers_;
    std::uint64_t packed_version_ = ~0ull;
    Index reserved_rows_ = 0;
    std::size_t scratch_bytes_ = 0;
    std::uint64_t buffer_epoch_ = 0;
    Tensor h_, q_, attended_, activated_, low_, scratch_;
    // shadow protocol (bf16 models whose widths fit the streaming kernel): activations travel as bf16 hi + lo planes
    bool shadow_ = false;
    int last_parts_ = 0;
    Tensor hs_hi_, hs_lo_, att_hi_, att_lo_, act_hi_, act_lo_, sq_attn_, sq_ffn_;
    Tensor best_value_, best_index_;   // [tiles][rows] candidates of the fused logits + argmax
    const void* user_ = nullptr;
};

// Greedy generation with the token loop resident on the device (the loop of examples/decoder_generate.cpp:20-31).
class Generation {
public:
    Generation(std::shared_ptr<TransformerDecoder> decoder, std::shared_ptr<Embedding> tokens, std::shared_ptr<Linear> output,
               std::vector<KVCache>* cache, Index batch, Index max_steps);
    ~Generation();
    // Prefill the prompt [batch, P] (int64, host or device) in chunks and choose the first token.
    void prefill(const Tensor& prompt);
    // Enqueue `steps` single-token steps (graph replays); no host synchronisation.
    void step(Index steps);
    // One step driven from the host: ids_in [batch] host -> H2D, step, D2H -> ids_out [batch] host (the reference's
    // per-token host round trip, examples/decoder_generate.cpp:28-30).  ids_in may be NULL to continue from the device ids.
    void step_host(const Index* ids_in, Index* ids_out);
    // One token drawn from softmax(logits / temperature) instead of the argmax, host in the loop: uniforms [batch] in
    // [0, 1) come from the caller's generator (the reference example owns a std::mt19937, examples/text_generate.cpp:29),
    // the chosen ids go to ids_out [batch] (may be NULL) and feed the next step.
    void step_sampled(double temperature, const double* uniforms, Index* ids_out);
    Index generated() const { return generated_; }
    Index batch() const { return batch_; }
    Tensor tokens() const;         // [batch, generated] int64 on the host (synchronises)
    // [batch, vocab] f32 on the device: logits the latest token was chosen from.  Steps choose their token without
    // writing logits; they are computed here, on demand, from the final hidden state of the last step, which is only
    // possible while nothing else has used the decoder since (logic_error otherwise).
    Tensor last_logits();
    Index launches_per_step() const { return launches_per_step_; }
    // One real step run eagerly with a CUDA event after every launch: milliseconds spent in the skinny-linear
    // launches, in the attention launches and in everything else, and the number of launches.
    struct StepProfile { double linear_ms, attention_ms, other_ms; Index launches; };
    StepProfile profile_step();

private:
    void enqueue_step(void* stream, Index max_length);
    void prepare();   // workspaces of a single-token step, before anything is enqueued or captured
    void capture();
    std::shared_ptr<TransformerDecoder> decoder_;
    std::shared_ptr<Embedding> tokens_;
    std::shared_ptr<Linear> output_;
    std::vector<KVCache>* cache_;
    Index batch_, max_steps_, generated_ = 0, launches_per_step_ = 0;
    bool fused_choice_ = false, logits_current_ = false;
    int device_ = 0;
    Tensor ids_, next_, logits_, history_, counter_, x_, uniform_;
    std::shared_ptr<runtime::Storage> pinned_;
    cudaGraphExec_t graph_ = nullptr;
    std::uint64_t graph_version_ = ~0ull, graph_epoch_ = ~0ull;
};

}  // namespace dl::nn
