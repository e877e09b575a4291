// Fixed execution plan and device-resident greedy generation (see plan.h).
#include "dl/plan.h"
#include "dl/internal.h"

#include <algorithm>
#include <stdexcept>

namespace dl::nn {

namespace {

constexpr Index kShadowDenseRows = 17;   // from this row count on the dense tensor-core kernels serve a shadow linear

// Optional per-launch event trail (Generation::profile_step); kinds: 0 linear, 1 attention, 2 other.
struct StepProbe {
    cudaStream_t stream;
    std::vector<cudaEvent_t> events;
    std::vector<int> kinds;
    void mark(int kind) {
        cudaEvent_t event;
        runtime::check_cuda(cudaEventCreate(&event), "cudaEventCreate");
        runtime::check_cuda(cudaEventRecord(event, stream), "cudaEventRecord");
        events.push_back(event);
        kinds.push_back(kind);
    }
};
thread_local StepProbe* step_probe = nullptr;
void probe(int kind) { if (step_probe) step_probe->mark(kind); }

int code_of(DType dtype) { return dtype == DType::bf16 ? B200_BF16 : B200_F32; }

cudaStream_t cuda_stream(int device) { return static_cast<cudaStream_t>(runtime::stream(device)); }

void require_cuda(const Tensor& t, const char* what) {
    if (t.device().type != DeviceType::cuda)
        throw std::invalid_argument(std::string(what) + ": tensors must live on a CUDA device (this library has no CPU compute path)");
}

// Device-side row copy: dst rows [first, first+n) of a [*, width] matrix with `pitch` bytes per destination row.
void copy_rows(void* dst, std::size_t dst_pitch, const Tensor& src, int device) {
    const std::size_t row = static_cast<std::size_t>(src.size(1)) * element_size(src.dtype());
    runtime::check_cuda(cudaMemcpy2DAsync(dst, dst_pitch, src.raw_data(), row, row, static_cast<std::size_t>(src.size(0)),
                                          cudaMemcpyDeviceToDevice, cuda_stream(device)), "cudaMemcpy2DAsync");
}

}  // namespace

Tensor interleave_rows(const Tensor& even_rows, const Tensor& odd_rows) {
    require_cuda(even_rows, "interleave_rows");
    if (even_rows.shape() != odd_rows.shape() || even_rows.dtype() != odd_rows.dtype() || even_rows.ndim() != 2)
        throw std::invalid_argument("interleave_rows: matrices must match");
    const int device = even_rows.device().index;
    runtime::set_device(device);
    Tensor result = empty({2 * even_rows.size(0), even_rows.size(1)}, {even_rows.dtype(), even_rows.device()});
    const std::size_t row = static_cast<std::size_t>(even_rows.size(1)) * element_size(even_rows.dtype());
    copy_rows(result.mutable_data(), 2 * row, even_rows, device);
    copy_rows(static_cast<char*>(result.mutable_data()) + row, 2 * row, odd_rows, device);
    return result;
}

Tensor concat_rows(std::span<const Tensor> parts) {
    Index rows = 0;
    for (const auto& part : parts) {
        require_cuda(part, "concat_rows");
        if (part.ndim() != 2 || part.size(1) != parts.front().size(1) || part.dtype() != parts.front().dtype())
            throw std::invalid_argument("concat_rows: matrices must share width and dtype");
        rows += part.size(0);
    }
    const int device = parts.front().device().index;
    runtime::set_device(device);
    Tensor result = empty({rows, parts.front().size(1)}, {parts.front().dtype(), parts.front().device()});
    std::size_t offset = 0;
    for (const auto& part : parts) {
        runtime::check_cuda(cudaMemcpyAsync(static_cast<char*>(result.mutable_data()) + offset, part.raw_data(), part.nbytes(),
                                            cudaMemcpyDeviceToDevice, cuda_stream(device)), "cudaMemcpyAsync");
        offset += part.nbytes();
    }
    return result;
}

Tensor add(const Tensor& a, const Tensor& b) {
    require_cuda(a, "add");
    if (a.shape() != b.shape() || a.device() != b.device()) throw std::invalid_argument("add: shapes and devices must match");
    Tensor result = (a.dtype() == DType::f32 ? a : a.astype(DType::f32)).clone();
    const Tensor other = b.dtype() == DType::f32 ? b : b.astype(DType::f32);
    runtime::check(b200_scaled_add(static_cast<float*>(result.mutable_data()), other.data<float>(), 1.0f, result.numel(),
                                   runtime::stream(a.device().index)), "add");
    return result;
}

namespace {

struct AttentionWeights {
    Tensor wqkv, lora_down;
    const void *q_up = nullptr, *v_up = nullptr;
    int rank = 0;
    float scale = 0.0f;
};

AttentionWeights pack_attention(const GroupedQueryAttention& a, int rank = 0, int world = 1) {
    AttentionWeights w;
    const auto* qa = a.query_adapter();
    const auto* va = a.value_adapter();
    // rows of this rank's query heads and KV heads (all rows when world == 1)
    const Index q_rows = a.dimensions() / world, kv_rows = a.kv_heads() * (a.dimensions() / a.heads()) / world;
    const Tensor parts[3] = {(qa ? qa->weight() : a.query().weight()).narrow(0, rank * q_rows, q_rows),
                             a.key().weight().narrow(0, rank * kv_rows, kv_rows),
                             (va ? va->weight() : a.value().weight()).narrow(0, rank * kv_rows, kv_rows)};
    w.wqkv = concat_rows(parts);
    if (qa) {
        const Tensor downs[2] = {qa->down().weight(), va->down().weight()};
        w.lora_down = concat_rows(downs);
        w.q_up = qa->up().weight().narrow(0, rank * q_rows, q_rows).raw_data();
        w.v_up = va->up().weight().narrow(0, rank * kv_rows, kv_rows).raw_data();
        w.rank = static_cast<int>(qa->rank());
        w.scale = static_cast<float>(qa->scale());
        if (static_cast<float>(va->scale()) != w.scale) throw std::invalid_argument("query and value adapters must share alpha/rank");
    }
    return w;
}

// RMSNorm? + QKV + RoPE + append, attention, output projection.  `norm` may be null.  y = residual + o-proj when
// residual != nullptr, else y = o-proj.
void enqueue_attention(const GroupedQueryAttention& a, const AttentionWeights& w, const float* x, const Tensor* norm, double eps,
                       Index batch, Index length, KVCache& cache, Index max_length, float* q, float* attended, float* low,
                       void* scratch, std::size_t scratch_bytes, const float* residual, float* y, int device, void* stream) {
    const Index D = a.dimensions(), H = a.heads(), HK = a.kv_heads(), hd = D / H, rows = batch * length;
    const int wcode = code_of(a.key().weight().dtype());
    b200_kv_cache* kv = cache.ensure(device, batch, HK, hd);
    b200_qkv_args args{};
    args.heads = static_cast<int32_t>(H); args.kv_heads = static_cast<int32_t>(HK); args.head_dim = static_cast<int32_t>(hd);
    args.tokens_per_sequence = static_cast<int32_t>(length);
    args.cosine = a.rotary().cosine().data<float>(); args.sine = a.rotary().sine().data<float>();
    args.context = static_cast<int32_t>(a.rotary().cosine().size(0));
    args.cache = kv; args.q_out = q;
    const void* norm_w = norm ? norm->raw_data() : nullptr;
    const int norm_code = norm ? code_of(norm->dtype()) : B200_F32;
    if (w.rank > 0) {
        runtime::check(b200_linear(x, rows, D, w.lora_down.raw_data(), wcode, 2 * w.rank, norm_w, norm_code, eps, B200_EPI_STORE,
                                   nullptr, nullptr, low, stream), "adapter down-projection");
        probe(0);
        args.lora_rank = w.rank; args.lora_scale = w.scale; args.low = low; args.q_up = w.q_up; args.v_up = w.v_up;
    }
    runtime::check(b200_linear(x, rows, D, w.wqkv.raw_data(), wcode, D + 2 * HK * hd, norm_w, norm_code, eps, B200_EPI_QKV, nullptr,
                               &args, q, stream), "q/k/v projection");
    probe(0);
    runtime::check(b200_attention_decode(q, rows, static_cast<int32_t>(length), static_cast<int32_t>(H), kv,
                                         static_cast<int32_t>(max_length), 1, scratch, scratch_bytes, attended, stream), "attention");
    probe(1);
    runtime::check(b200_linear(attended, rows, D, a.output().weight().raw_data(), code_of(a.output().weight().dtype()), D, nullptr, 0,
                               0.0, residual ? B200_EPI_RESIDUAL : B200_EPI_STORE, residual, nullptr, y, stream), "output projection");
    probe(0);
}

}  // namespace

Tensor attention_block(GroupedQueryAttention& a, const Tensor& input, KVCache& cache) {
    require_cuda(input, "GroupedQueryAttention");
    if (input.ndim() != 3 || input.size(2) != a.dimensions()) throw std::invalid_argument("attention expects [batch,length,dimensions]");
    const Index batch = input.size(0), length = input.size(1), D = a.dimensions(), rows = batch * length;
    if (length > cache.capacity() - cache.length())
        throw std::invalid_argument("KV cache append exceeds capacity or has unequal key/value lengths");
    if (length > a.rotary().cosine().size(0) - cache.length()) throw std::out_of_range("RoPE positions exceed the table capacity");
    const int device = input.device().index;
    runtime::set_device(device);
    void* stream = runtime::stream(device);
    const Tensor x = input.dtype() == DType::f32 ? input : input.astype(DType::f32);
    const AttentionWeights w = pack_attention(a);
    const TensorOptions f32{DType::f32, input.device()};
    Tensor q = empty({rows, D}, f32), attended = empty({rows, D}, f32), y = empty({batch, length, D}, f32);
    Tensor low = empty({rows, std::max<Index>(1, 2 * w.rank)}, f32);
    const Index max_length = cache.length() + length;
    const std::size_t scratch_bytes = b200_attention_scratch_bytes(rows, static_cast<int32_t>(a.heads()), static_cast<int32_t>(a.kv_heads()),
                                                                   static_cast<int32_t>(D / a.heads()), static_cast<int32_t>(max_length), 64);
    Tensor scratch = empty({static_cast<Index>(scratch_bytes / 4 + 1)}, f32);
    enqueue_attention(a, w, x.data<float>(), nullptr, 0.0, batch, length, cache, max_length, static_cast<float*>(q.mutable_data()),
                      static_cast<float*>(attended.mutable_data()), static_cast<float*>(low.mutable_data()), scratch.mutable_data(),
                      scratch_bytes, nullptr, static_cast<float*>(y.mutable_data()), device, stream);
    b200_kv_cache* handle = cache.handle();
    runtime::check(b200_kv_cache_advance(&handle, 1, static_cast<int32_t>(length), stream), "KV advance");
    cache.commit(length);
    synchronize(input.device());  // temporaries above are released on return
    return y;
}

// ---- DecodePlan -----------------------------------------------------------------------------------------
DecodePlan::DecodePlan(TransformerDecoder& owner) : owner_(owner) {}
DecodePlan::~DecodePlan() = default;

void DecodePlan::refresh() {
    const auto version = owner_.version();
    if (version == packed_version_ && !layers_.empty()) return;
    const Tensor& probe = owner_.normalization().weight() ? *owner_.normalization().weight() : owner_.layer(0).attention().key().weight();
    require_cuda(probe, "TransformerDecoder");
    runtime::set_device(probe.device().index);
    layers_.clear();
    for (Index i = 0; i < owner_.layer_count(); ++i) {
        auto& layer = owner_.layer(i);
        const int rank = owner_.tp_rank(), world = owner_.tp_world();
        const AttentionWeights a = pack_attention(layer.attention(), rank, world);
        Layer packed{};
        packed.wqkv = a.wqkv; packed.lora_down = a.lora_down; packed.q_up = a.q_up; packed.v_up = a.v_up;
        packed.rank = a.rank; packed.scale = a.scale;
        const Index f_rows = owner_.hidden() / world, d_cols = owner_.dimensions() / world;
        packed.wgu = interleave_rows(layer.feedforward().gate().weight().narrow(0, rank * f_rows, f_rows),
                                     layer.feedforward().up().weight().narrow(0, rank * f_rows, f_rows));
        packed.wo = layer.attention().output().weight().raw_data();
        packed.wd = layer.feedforward().down().weight().raw_data();
        if (world > 1) {  // column cuts: this rank's input features of the two row-parallel projections
            packed.wo_slice = layer.attention().output().weight().narrow(1, rank * d_cols, d_cols);
            packed.wd_slice = layer.feedforward().down().weight().narrow(1, rank * f_rows, f_rows);
            packed.wo = packed.wo_slice.raw_data();
            packed.wd = packed.wd_slice.raw_data();
        }
        packed.norm1 = layer.attention_norm().weight()->raw_data();
        packed.norm2 = layer.feedforward_norm().weight()->raw_data();
        layers_.push_back(std::move(packed));
    }
    synchronize(probe.device());
    packed_version_ = version;
    // Shadow protocol: bf16 weights and bf16 norm weights; whether a given row count can use it is decided per pass.
    shadow_ = owner_.dtype() == DType::bf16;
    for (Index i = 0; shadow_ && i < owner_.layer_count(); ++i) {
        auto& layer = owner_.layer(i);
        shadow_ = layer.attention_norm().weight()->dtype() == DType::bf16 && layer.feedforward_norm().weight()->dtype() == DType::bf16;
    }
}

// Rows of the [parts, rows] buffers that carry the per-row partial sums of squares between two kernels: the largest count
// any producer of a residual stream of width D may write - one partial per feature tile of the streaming kernel (whose
// tiles shrink to 8 features when the inner size is large, so up to D / 8), of the dense kernels (D / 128) or of the
// cross-GPU sum - whatever the row count of the pass (the producers choose their tiling from the inner sizes D and F).
Index shadow_partial_rows(Index D, Index F) {
    Index parts = 1;
    for (const Index rows : {Index{1}, Index{kShadowDenseRows}})
        for (const Index inner : {D, F})
            parts = std::max<Index>(parts, b200_linear_shadow_parts(rows, inner, D));
    return std::max<Index>(parts, b200_tp_reduce_parts(D));
}

bool DecodePlan::shadows_for(Index rows) const {
    if (!shadow_ || rows <= 0) return false;
    const Index world = owner_.tp_world();
    const Index D = owner_.dimensions(), F = owner_.hidden() / world, KV = owner_.kv_heads() * (D / owner_.heads()) / world;
    return b200_linear_shadow_parts(rows, D, D / world + 2 * KV) > 0 && b200_linear_shadow_parts(rows, D / world, D) > 0
        && b200_linear_shadow_parts(rows, D, 2 * F) > 0 && b200_linear_shadow_parts(rows, F, D) > 0;
}

void DecodePlan::reserve(Index rows, Index max_length, int device) {
    const Index D = owner_.dimensions(), F = owner_.hidden();
    const std::size_t need = b200_attention_scratch_bytes(rows, static_cast<int32_t>(owner_.heads()), static_cast<int32_t>(owner_.kv_heads()),
                                                          static_cast<int32_t>(D / owner_.heads()), static_cast<int32_t>(max_length), 64);
    const TensorOptions f32{DType::f32, Device::cuda(device)};
    if (rows > reserved_rows_ || !h_.defined() || h_.device().index != device || (shadow_ && !hs_hi_.defined())) {
        synchronize(Device::cuda(device));
        int max_rank = 0;
        for (const auto& layer : layers_) max_rank = std::max(max_rank, layer.rank);
        h_ = empty({rows, D}, f32); q_ = empty({rows, D}, f32); attended_ = empty({rows, D}, f32);
        activated_ = empty({rows, F}, f32); low_ = empty({rows, std::max(1, 2 * max_rank)}, f32);
        if (shadow_) {
            const TensorOptions half{DType::bf16, Device::cuda(device)};
            hs_hi_ = empty({rows, D}, half); hs_lo_ = empty({rows, D}, half);
            att_hi_ = empty({rows, D}, half); att_lo_ = empty({rows, D}, half);
            act_hi_ = empty({rows, F}, half); act_lo_ = empty({rows, F}, half);
            const Index parts = shadow_partial_rows(D, F / owner_.tp_world());
            sq_attn_ = empty({parts, rows}, f32); sq_ffn_ = empty({parts, rows}, f32);
        }
        reserved_rows_ = rows;
        ++buffer_epoch_;
    }
    if (need > scratch_bytes_ || !scratch_.defined() || scratch_.device().index != device) {
        synchronize(Device::cuda(device));
        scratch_ = empty({static_cast<Index>(need / 4 + 1)}, f32);
        scratch_bytes_ = need;
        ++buffer_epoch_;
    }
}

void DecodePlan::validate(Index batch, Index length, std::span<KVCache> cache, int device) {
    if (static_cast<Index>(cache.size()) != owner_.layer_count()) throw std::invalid_argument("decoder requires one cache per layer");
    const Index prefix = cache.front().length();
    for (const auto& layer : cache)
        if (layer.length() != prefix) throw std::invalid_argument("decoder cache positions differ");
    // Everything that can fail is checked before the first kernel is enqueued, so a rejected chunk leaves every
    // layer at the prefix it had (the reference reaches the same state by truncating after the throw,
    // src/nn/decoder.cpp:137-141).
    for (const auto& layer : cache)
        if (length > layer.capacity() - layer.length())
            throw std::invalid_argument("KV cache append exceeds capacity or has unequal key/value lengths");
    if (length > owner_.context() - prefix) throw std::out_of_range("RoPE positions exceed the table capacity");
    const Index hd = owner_.dimensions() / owner_.heads();
    for (auto& layer : cache) layer.ensure(device, batch, owner_.kv_heads() / owner_.tp_world(), hd);
}

namespace {
void shadow_linear(const b200_shadow_linear_args& args, void* stream, const char* what) {
    runtime::check(b200_linear_shadow(&args, stream), what);
    probe(0);
}
}  // namespace

void DecodePlan::embed(const Embedding& tokens, const Index* ids, Index rows, float* x, void* stream) {
    const Tensor& table = tokens.weight();
    if (!shadows_for(rows)) {
        runtime::check(b200_embedding(table.raw_data(), code_of(table.dtype()), ids, rows, table.size(0), table.size(1), x, stream), "embedding");
        probe(2);
        return;
    }
    const Tensor* norm = owner_.layer(0).attention_norm().weight();
    runtime::check(b200_embedding_shadow(table.raw_data(), code_of(table.dtype()), ids, rows, table.size(0), table.size(1), norm->raw_data(),
                                         code_of(norm->dtype()), x, hs_hi_.mutable_data(), hs_lo_.mutable_data(),
                                         static_cast<float*>(sq_attn_.mutable_data()), stream), "embedding");
    probe(2);
}

void DecodePlan::logits(const Linear& output, Index rows, float* out, void* stream) {
    const Tensor* norm = owner_.normalization().weight();
    const Index V = output.weight().size(0), D = owner_.dimensions();
    if (shadows_for(rows) && output.weight().dtype() == DType::bf16 && b200_linear_shadow_parts(rows, D, V) > 0) {
        b200_shadow_linear_args args{};
        args.x_hi = hs_hi_.raw_data(); args.rows = rows; args.in = D;
        args.x_lo = owner_.activation_dtype() == DType::bf16 && rows >= 17 ? nullptr : hs_lo_.raw_data();
        args.weight = output.weight().raw_data(); args.out = V;
        args.sumsq_in = sq_attn_.data<float>(); args.parts_in = last_parts_; args.eps = owner_.normalization().epsilon();
        args.epilogue = B200_EPI_STORE; args.y = out;
        shadow_linear(args, stream, "logits");
        return;
    }
    runtime::check(b200_linear(hidden(), rows, D, output.weight().raw_data(), code_of(output.weight().dtype()), V, norm->raw_data(),
                               code_of(norm->dtype()), owner_.normalization().epsilon(), B200_EPI_STORE, nullptr, nullptr, out, stream),
                   "logits");
    probe(0);
}

// With tensor parallelism over mapped peer memory the vocabulary is split over the ranks in whole 128-row tiles: this rank's
// slice of the output table, as (first row, rows).  {0, V} otherwise.
std::pair<Index, Index> DecodePlan::vocabulary_slice(const Linear& output, Index rows, int device) const {
    const Index V = output.weight().size(0);
    const int world = owner_.tp_world(), rank = owner_.tp_rank();
    if (world <= 1 || rows > 1024 || !runtime::tp_symmetric_ready(device, 1)) return {0, V};
    const Index tiles = (V + 127) / 128, each = (tiles + world - 1) / world * 128;
    if (each * (world - 1) >= V) return {0, V};   // a vocabulary too small to give every rank a slice: replicated logits
    const Index first = each * rank;
    return {first, std::min(each, V - first)};
}

bool DecodePlan::prepare_choice(const Linear& output, Index rows, int device) {
    const Index D = owner_.dimensions();
    if (!shadows_for(rows) || output.weight().dtype() != DType::bf16 || output.weight().size(1) != D) return false;
    const Index slice = vocabulary_slice(output, rows, device).second;
    const Index parts = b200_linear_argmax_parts(rows, D, slice);
    if (parts <= 0) return false;
    if (!best_value_.defined() || best_value_.numel() < parts * rows || best_value_.device().index != device) {
        synchronize(Device::cuda(device));
        const TensorOptions f32{DType::f32, Device::cuda(device)};
        best_value_ = empty({parts * rows}, f32);
        best_index_ = empty({parts * rows}, f32);   // int32 payload
        ++buffer_epoch_;
    }
    return true;
}

void DecodePlan::choose(const Linear& output, Index rows, Index* next, Index* ids, Index* history, Index history_rows, std::int32_t* counter,
                        std::span<b200_kv_cache* const> advance, void* stream) {
    const Index V = output.weight().size(0), D = owner_.dimensions();
    const int device = h_.device().index;
    const auto [first, slice] = vocabulary_slice(output, rows, device);
    const bool split = slice != V;
    const Index parts = b200_linear_argmax_parts(rows, D, slice);
    if (parts <= 0 || !best_value_.defined() || best_value_.numel() < parts * rows)
        throw std::logic_error("fused logits + argmax was not prepared for this row count");
    b200_shadow_linear_args args{};
    args.x_hi = hs_hi_.raw_data(); args.rows = rows; args.in = D;
    args.x_lo = owner_.activation_dtype() == DType::bf16 && rows >= 17 ? nullptr : hs_lo_.raw_data();
    args.weight = static_cast<const char*>(output.weight().raw_data()) + static_cast<std::size_t>(first) * static_cast<std::size_t>(D) * 2;
    args.out = slice;
    args.sumsq_in = sq_attn_.data<float>(); args.parts_in = last_parts_; args.eps = owner_.normalization().epsilon();
    args.epilogue = B200_EPI_ARGMAX;
    args.best_value = static_cast<float*>(best_value_.mutable_data());
    args.best_index = static_cast<std::int32_t*>(best_index_.mutable_data());
    shadow_linear(args, stream, "logits + argmax");
    if (split) {
        // every rank holds the best of its slice; the candidates meet over peer memory and every rank picks the same token
        runtime::tp_argmax_finish(device, static_cast<std::int32_t>(first), args.best_value, args.best_index, static_cast<std::int32_t>(parts), rows,
                                  next, ids, history, history_rows, counter, advance.data(), static_cast<std::int32_t>(advance.size()));
    } else {
        runtime::check(b200_argmax_finish(args.best_value, args.best_index, static_cast<std::int32_t>(parts), rows, next, ids, history, history_rows,
                                          counter, advance.data(), static_cast<std::int32_t>(advance.size()), stream), "argmax merge");
    }
    probe(2);
}

void DecodePlan::run_layers(const float* x, Index batch, Index length, std::span<KVCache> cache, Index max_length, void* stream,
                            bool shadow_ready) {
    const Index D = owner_.dimensions(), F = owner_.hidden(), rows = batch * length;
    const int device = h_.device().index;
    const double eps = TransformerDecoderLayer::norm_epsilon;
    float* h = hidden();
    if (owner_.tp_world() > 1 && !shadows_for(rows))
        throw std::invalid_argument("tensor parallelism needs a bf16 decoder whose slices fit the shadow kernels");
    if (shadows_for(rows)) {
        // Tensor parallel (world > 1): this rank owns H/world query heads, HK/world KV heads and F/world SwiGLU features;
        // the output and down projections produce partial sums over their input slices, rank 0 adds the residual, an
        // all-reduce makes every rank's residual stream identical, and the next shadow is rebuilt from it.
        const int world = owner_.tp_world(), rank = owner_.tp_rank();
        const bool parallel = world > 1;
        const Index hd = D / owner_.heads();
        const Index H = owner_.heads() / world, HK = owner_.kv_heads() / world, Dl = H * hd, Fl = F / world;
        // With symmetric memory mapped (and the rows fitting a slot) the projections write their partial rows into this
        // rank's slot and one kernel sums the ranks' slots over NVLink and rebuilds the shadow; otherwise NCCL.
        const bool peer_sum = parallel && runtime::tp_symmetric_ready(device, static_cast<std::size_t>(rows * D) * sizeof(float));
        const bool push_sums = peer_sum && runtime::tp_push(device);
        const int parts_summed = peer_sum ? b200_tp_reduce_parts(D) : 1;   // partial sums of squares the rebuilt shadow comes with
        const int parts_o = parallel ? parts_summed : b200_linear_shadow_parts(rows, D, D);
        const int parts_down = parallel ? parts_summed : b200_linear_shadow_parts(rows, F, D);
        auto* sq_attn = static_cast<float*>(sq_attn_.mutable_data());
        auto* sq_ffn = static_cast<float*>(sq_ffn_.mutable_data());
        // bf16 activations: the dense kernel (more than 16 rows) is given the hi plane only
        const bool single_plane = owner_.activation_dtype() == DType::bf16 && rows >= 17;
        auto lo_plane = [&](const Tensor& plane) -> const void* { return single_plane ? nullptr : plane.raw_data(); };
        auto rebuild_shadow = [&](const Tensor* norm, float* sums, int slot) {
            if (peer_sum) {
                runtime::tp_reduce_shadow(device, slot, rows, D, norm->raw_data(), code_of(norm->dtype()), h, hs_hi_.mutable_data(),
                                          hs_lo_.mutable_data(), sums);
                probe(2);
                return;
            }
            runtime::tp_all_reduce(device, h, static_cast<std::size_t>(rows * D));
            probe(2);
            runtime::check(b200_shadow_from_rows(h, rows, D, norm->raw_data(), code_of(norm->dtype()), hs_hi_.mutable_data(),
                                                 hs_lo_.mutable_data(), sums, stream), "shadow after all-reduce");
            probe(2);
        };
        if (!shadow_ready) {
            const Tensor* norm = owner_.layer(0).attention_norm().weight();
            runtime::check(b200_shadow_from_rows(x, rows, D, norm->raw_data(), code_of(norm->dtype()), hs_hi_.mutable_data(),
                                                 hs_lo_.mutable_data(), sq_attn, stream), "input shadow");
            probe(2);
        }
        int parts_attn = 1;
        for (Index i = 0; i < owner_.layer_count(); ++i) {
            auto& layer = owner_.layer(i);
            const auto& a = layer.attention();
            const Layer& packed = layers_[static_cast<std::size_t>(i)];
            const float* in = i == 0 ? x : h;
            b200_kv_cache* kv = cache[static_cast<std::size_t>(i)].ensure(device, batch, HK, hd);
            b200_qkv_args qkv{};
            qkv.heads = static_cast<int32_t>(H); qkv.kv_heads = static_cast<int32_t>(HK); qkv.head_dim = static_cast<int32_t>(hd);
            qkv.tokens_per_sequence = static_cast<int32_t>(length);
            qkv.cosine = a.rotary().cosine().data<float>(); qkv.sine = a.rotary().sine().data<float>();
            qkv.context = static_cast<int32_t>(a.rotary().cosine().size(0));
            qkv.cache = kv; qkv.q_out = static_cast<float*>(q_.mutable_data());
            b200_shadow_linear_args base{};
            base.x_hi = hs_hi_.raw_data(); base.x_lo = lo_plane(hs_lo_); base.rows = rows; base.in = D;
            base.sumsq_in = sq_attn; base.parts_in = parts_attn; base.eps = eps;
            if (packed.rank > 0) {
                b200_shadow_linear_args low = base;
                low.weight = packed.lora_down.raw_data(); low.out = 2 * packed.rank; low.epilogue = B200_EPI_STORE;
                low.y = static_cast<float*>(low_.mutable_data());
                shadow_linear(low, stream, "adapter down-projection");
                qkv.lora_rank = packed.rank; qkv.lora_scale = packed.scale; qkv.low = low.y; qkv.q_up = packed.q_up; qkv.v_up = packed.v_up;
            }
            b200_shadow_linear_args project = base;
            project.weight = packed.wqkv.raw_data(); project.out = Dl + 2 * HK * hd; project.epilogue = B200_EPI_QKV; project.qkv = &qkv;
            shadow_linear(project, stream, "q/k/v projection");
            runtime::check(b200_attention_decode_shadow(qkv.q_out, rows, static_cast<int32_t>(length), static_cast<int32_t>(H), kv,
                                                        static_cast<int32_t>(max_length), 1, scratch_.mutable_data(), scratch_bytes_,
                                                        att_hi_.mutable_data(), att_lo_.mutable_data(), stream), "attention");
            probe(1);
            const Tensor* ffn_norm = layer.feedforward_norm().weight();
            const bool adds_residual = !parallel || rank == 0;
            b200_shadow_linear_args out_proj{};
            out_proj.x_hi = att_hi_.raw_data(); out_proj.x_lo = lo_plane(att_lo_); out_proj.rows = rows; out_proj.in = Dl;
            out_proj.weight = packed.wo; out_proj.out = D; out_proj.y = peer_sum ? runtime::tp_partial_slot(device, 0) : h;
            float* o_copies[7];
            if (peer_sum && push_sums) {   // the partial rows go to this rank's slot in every peer's memory from the projection's own epilogue
                for (int r = 0, c = 0; r < world; ++r)
                    if (r != rank) o_copies[c++] = runtime::tp_partial_slot(device, 0, r);
                out_proj.y_copies = o_copies; out_proj.copies = world - 1;
            }
            out_proj.epilogue = adds_residual ? B200_EPI_RESIDUAL : B200_EPI_STORE; out_proj.residual = adds_residual ? in : nullptr;
            if (!parallel) {
                out_proj.out_hi = hs_hi_.mutable_data(); out_proj.out_lo = hs_lo_.mutable_data();
                out_proj.out_norm_weight = ffn_norm->raw_data(); out_proj.out_norm_dtype = code_of(ffn_norm->dtype()); out_proj.sumsq_out = sq_ffn;
            }
            shadow_linear(out_proj, stream, "output projection");
            if (parallel) rebuild_shadow(ffn_norm, sq_ffn, 0);
            b200_shadow_linear_args gate_up{};
            gate_up.x_hi = hs_hi_.raw_data(); gate_up.x_lo = lo_plane(hs_lo_); gate_up.rows = rows; gate_up.in = D;
            gate_up.weight = packed.wgu.raw_data(); gate_up.out = 2 * Fl; gate_up.sumsq_in = sq_ffn; gate_up.parts_in = parts_o; gate_up.eps = eps;
            gate_up.epilogue = B200_EPI_SWIGLU; gate_up.out_hi = act_hi_.mutable_data(); gate_up.out_lo = act_lo_.mutable_data();
            shadow_linear(gate_up, stream, "gate/up projection");
            const Tensor* next_norm = i + 1 < owner_.layer_count() ? owner_.layer(i + 1).attention_norm().weight() : owner_.normalization().weight();
            b200_shadow_linear_args down{};
            down.x_hi = act_hi_.raw_data(); down.x_lo = lo_plane(act_lo_); down.rows = rows; down.in = Fl;
            down.weight = packed.wd; down.out = D; down.y = peer_sum ? runtime::tp_partial_slot(device, 1) : h;
            float* down_copies[7];
            if (peer_sum && push_sums) {
                for (int r = 0, c = 0; r < world; ++r)
                    if (r != rank) down_copies[c++] = runtime::tp_partial_slot(device, 1, r);
                down.y_copies = down_copies; down.copies = world - 1;
            }
            down.epilogue = adds_residual ? B200_EPI_RESIDUAL : B200_EPI_STORE; down.residual = adds_residual ? h : nullptr;
            if (!parallel) {
                down.out_hi = hs_hi_.mutable_data(); down.out_lo = hs_lo_.mutable_data();
                down.out_norm_weight = next_norm->raw_data(); down.out_norm_dtype = code_of(next_norm->dtype()); down.sumsq_out = sq_attn;
            }
            shadow_linear(down, stream, "down projection");
            if (parallel) rebuild_shadow(next_norm, sq_attn, 1);
            parts_attn = parts_down;
        }
        last_parts_ = parts_attn;
        return;
    }
    auto* act = static_cast<float*>(activated_.mutable_data());
    for (Index i = 0; i < owner_.layer_count(); ++i) {
        auto& layer = owner_.layer(i);
        const Layer& packed = layers_[static_cast<std::size_t>(i)];
        const float* in = i == 0 ? x : h;
        AttentionWeights w;
        w.wqkv = packed.wqkv; w.lora_down = packed.lora_down; w.q_up = packed.q_up; w.v_up = packed.v_up; w.rank = packed.rank; w.scale = packed.scale;
        enqueue_attention(layer.attention(), w, in, layer.attention_norm().weight(), eps, batch, length, cache[static_cast<std::size_t>(i)],
                          max_length, static_cast<float*>(q_.mutable_data()), static_cast<float*>(attended_.mutable_data()),
                          static_cast<float*>(low_.mutable_data()), scratch_.mutable_data(), scratch_bytes_, in, h, device, stream);
        const int wcode = code_of(layer.feedforward().gate().weight().dtype());
        runtime::check(b200_linear(h, rows, D, packed.wgu.raw_data(), wcode, 2 * F, packed.norm2, code_of(layer.feedforward_norm().weight()->dtype()),
                                   eps, B200_EPI_SWIGLU, nullptr, nullptr, act, stream), "gate/up projection");
        probe(0);
        runtime::check(b200_linear(act, rows, F, packed.wd, wcode, D, nullptr, 0, 0.0, B200_EPI_RESIDUAL, h, nullptr, h, stream),
                       "down projection");
        probe(0);
    }
}

Tensor DecodePlan::decode(const Tensor& input, std::span<KVCache> cache) {
    require_cuda(input, "TransformerDecoder::decode");
    if (input.ndim() != 3 || input.size(2) != owner_.dimensions())
        throw std::invalid_argument("decoder expects [batch,length,dimensions]");
    const Index batch = input.size(0), length = input.size(1), rows = batch * length;
    const int device = input.device().index;
    runtime::set_device(device);
    refresh();
    user_ = nullptr;
    validate(batch, length, cache, device);
    Tensor result = empty(input.shape(), {DType::f32, input.device()});
    if (rows == 0) return result;
    const Tensor x = input.dtype() == DType::f32 ? input : input.astype(DType::f32);
    const Index max_length = cache.front().length() + length;
    reserve(rows, max_length, device);
    void* stream = runtime::stream(device);
    run_layers(x.data<float>(), batch, length, cache, max_length, stream);
    const Tensor* norm = owner_.normalization().weight();
    runtime::check(b200_rms_norm(hidden(), norm->raw_data(), code_of(norm->dtype()), rows, owner_.dimensions(),
                                 owner_.normalization().epsilon(), static_cast<float*>(result.mutable_data()), stream), "final norm");
    std::vector<b200_kv_cache*> handles;
    for (auto& layer : cache) handles.push_back(layer.handle());
    runtime::check(b200_kv_cache_advance(handles.data(), static_cast<int32_t>(handles.size()), static_cast<int32_t>(length), stream), "KV advance");
    for (auto& layer : cache) layer.commit(length);
    synchronize(input.device());  // `x` may be a temporary; results are complete when the call returns
    return result;
}

// ---- Generation -----------------------------------------------------------------------------------------
Generation::Generation(std::shared_ptr<TransformerDecoder> decoder, std::shared_ptr<Embedding> tokens, std::shared_ptr<Linear> output,
                       std::vector<KVCache>* cache, Index batch, Index max_steps)
    : decoder_(std::move(decoder)), tokens_(std::move(tokens)), output_(std::move(output)), cache_(cache), batch_(batch),
      max_steps_(max_steps) {
    if (!decoder_ || !tokens_ || !output_ || !cache_) throw std::invalid_argument("generation needs a decoder, an embedding, an output layer and a cache");
    if (batch <= 0 || max_steps <= 0) throw std::invalid_argument("generation needs a positive batch and step budget");
    require_cuda(tokens_->weight(), "generation");
    if (tokens_->weight().size(1) != decoder_->dimensions() || output_->weight().size(1) != decoder_->dimensions())
        throw std::invalid_argument("embedding and output widths must equal the decoder's dimensions");
    device_ = tokens_->weight().device().index;
    runtime::set_device(device_);
    const Device where = Device::cuda(device_);
    ids_ = zeros({batch}, {DType::i64, where});
    next_ = zeros({batch}, {DType::i64, where});
    logits_ = empty({batch, output_->weight().size(0)}, {DType::f32, where});
    history_ = zeros({max_steps, batch}, {DType::i64, where});
    counter_ = zeros({1}, {DType::i64, where});  // the kernel uses the first 32 bits
    x_ = empty({batch, decoder_->dimensions()}, {DType::f32, where});
    uniform_ = zeros({batch}, {DType::f64, where});
    // pinned staging: ids in, ids out, uniform variates
    pinned_ = std::make_shared<runtime::Storage>(sizeof(Index) * static_cast<std::size_t>(batch) * 3, Device::cpu(), true);
}
Generation::~Generation() {
    try { synchronize(Device::cuda(device_)); } catch (...) {}
    if (graph_) cudaGraphExecDestroy(graph_);
}

// logits of `rows` hidden rows (final RMSNorm fused into the projection), argmax, token feedback
static void enqueue_head(TransformerDecoder& decoder, const Linear& output, const float* hidden, Index batch, float* logits,
                         Index* next, Index* ids, Index* history, Index history_rows, int32_t* counter, void* stream) {
    const Tensor* norm = decoder.normalization().weight();
    const Index V = output.weight().size(0), D = decoder.dimensions();
    runtime::check(b200_linear(hidden, batch, D, output.weight().raw_data(), code_of(output.weight().dtype()), V, norm->raw_data(),
                               code_of(norm->dtype()), decoder.normalization().epsilon(), B200_EPI_STORE, nullptr, nullptr, logits, stream),
                   "logits");
    probe(0);
    runtime::check(b200_argmax(logits, batch, V, next, stream), "argmax");
    runtime::check(b200_token_feedback(next, batch, ids, history, history_rows, counter, stream), "token feedback");
    probe(2);
}

void Generation::prefill(const Tensor& prompt) {
    if (prompt.ndim() != 2 || prompt.size(0) != batch_ || prompt.dtype() != DType::i64 || prompt.size(1) <= 0)
        throw std::invalid_argument("prompt must be int64 [batch, length] with a positive length");
    const Index P = prompt.size(1), D = decoder_->dimensions();
    runtime::set_device(device_);
    void* stream = runtime::stream(device_);
    if (prompt.device().type == DeviceType::cpu) {
        const Index V = tokens_->weight().size(0);
        for (Index i = 0; i < prompt.numel(); ++i)
            if (prompt.data<Index>()[i] < 0 || prompt.data<Index>()[i] >= V) throw std::out_of_range("embedding index out of range");
    }
    const Tensor device_prompt = prompt.to(Device::cuda(device_));
    auto& plan = decoder_->plan();
    plan.refresh();
    plan.validate(batch_, P, *cache_, device_);
    if (generated_ >= max_steps_) throw std::out_of_range("generation step budget exhausted");
    // Chunked prefill: at most ~8192 rows per pass; chunked decode equals one pass (tests/state.cpp:54-63 of the reference).
    const Index chunk = std::max<Index>(1, std::min<Index>(P, 8192 / batch_ > 0 ? 8192 / batch_ : 1));
    Tensor features = empty({batch_ * chunk, D}, {DType::f32, Device::cuda(device_)});
    Index done = 0;
    while (done < P) {
        const Index count = std::min(chunk, P - done);
        const Tensor part = count == P ? device_prompt : device_prompt.narrow(1, done, count);
        runtime::check(b200_embedding(tokens_->weight().raw_data(), code_of(tokens_->weight().dtype()), part.data<Index>(), batch_ * count,
                                      tokens_->weight().size(0), D, static_cast<float*>(features.mutable_data()), stream), "embedding");
        const Index max_length = cache_->front().length() + count;
        plan.reserve(batch_ * count, max_length, device_);
        plan.run_layers(features.data<float>(), batch_, count, *cache_, max_length, stream);
        std::vector<b200_kv_cache*> handles;
        for (auto& layer : *cache_) handles.push_back(layer.handle());
        runtime::check(b200_kv_cache_advance(handles.data(), static_cast<int32_t>(handles.size()), static_cast<int32_t>(count), stream), "KV advance");
        for (auto& layer : *cache_) layer.commit(count);
        done += count;
        if (done == P) {
            // last position of every sequence -> first generated token
            runtime::check(b200_select_rows(plan.hidden(), count - 1, count, batch_, D, static_cast<float*>(x_.mutable_data()), stream), "select");
            enqueue_head(*decoder_, *output_, x_.data<float>(), batch_, static_cast<float*>(logits_.mutable_data()),
                         static_cast<Index*>(next_.mutable_data()), static_cast<Index*>(ids_.mutable_data()),
                         static_cast<Index*>(history_.mutable_data()), max_steps_, static_cast<int32_t*>(counter_.mutable_data()), stream);
        }
        synchronize(Device::cuda(device_));  // `part` and the chunk buffers are reused
    }
    plan.set_user(this);
    logits_current_ = true;   // the prompt's last position went through the materialised head
    ++generated_;
}

void Generation::enqueue_step(void* stream, Index max_length) {
    auto& plan = decoder_->plan();
    const Index D = decoder_->dimensions();
    plan.embed(*tokens_, ids_.data<Index>(), batch_, static_cast<float*>(x_.mutable_data()), stream);
    plan.run_layers(x_.data<float>(), batch_, 1, *cache_, max_length, stream, plan.shadows_for(batch_));
    std::vector<b200_kv_cache*> handles;
    for (auto& layer : *cache_) handles.push_back(layer.handle());
    if (fused_choice_ && handles.size() <= 64) {   // the merge kernel of the fused choice also advances the caches
        plan.choose(*output_, batch_, static_cast<Index*>(next_.mutable_data()), static_cast<Index*>(ids_.mutable_data()),
                    static_cast<Index*>(history_.mutable_data()), max_steps_, static_cast<int32_t*>(counter_.mutable_data()), handles, stream);
        return;
    }
    runtime::check(b200_kv_cache_advance(handles.data(), static_cast<int32_t>(handles.size()), 1, stream), "KV advance");
    probe(2);
    if (fused_choice_) {
        plan.choose(*output_, batch_, static_cast<Index*>(next_.mutable_data()), static_cast<Index*>(ids_.mutable_data()),
                    static_cast<Index*>(history_.mutable_data()), max_steps_, static_cast<int32_t*>(counter_.mutable_data()), {}, stream);
        return;
    }
    plan.logits(*output_, batch_, static_cast<float*>(logits_.mutable_data()), stream);
    runtime::check(b200_argmax(logits_.data<float>(), batch_, output_->weight().size(0), static_cast<Index*>(next_.mutable_data()), stream), "argmax");
    runtime::check(b200_token_feedback(next_.data<Index>(), batch_, static_cast<Index*>(ids_.mutable_data()),
                                       static_cast<Index*>(history_.mutable_data()), max_steps_,
                                       static_cast<int32_t*>(counter_.mutable_data()), stream), "token feedback");
    probe(2);
}

void Generation::prepare() {
    auto& plan = decoder_->plan();
    plan.reserve(batch_, cache_->front().capacity(), device_);
    fused_choice_ = plan.prepare_choice(*output_, batch_, device_);
}

void Generation::capture() {
    auto& plan = decoder_->plan();
    plan.refresh();
    const std::uint64_t version = decoder_->version() + tokens_->version() + output_->version();
    runtime::set_device(device_);
    const Index capacity = cache_->front().capacity();
    prepare();
    if (graph_ && graph_version_ == version && graph_epoch_ == plan.buffer_epoch()) return;
    if (graph_) { cudaGraphExecDestroy(graph_); graph_ = nullptr; }
    cudaStream_t stream = cuda_stream(device_);
    runtime::check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    runtime::check_cuda(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    cudaGraph_t graph = nullptr;
    try {
        enqueue_step(stream, capacity);
    } catch (...) {
        cudaStreamEndCapture(stream, &graph);
        if (graph) cudaGraphDestroy(graph);
        throw;
    }
    runtime::check_cuda(cudaStreamEndCapture(stream, &graph), "cudaStreamEndCapture");
    std::size_t nodes = 0;
    cudaGraphGetNodes(graph, nullptr, &nodes);
    launches_per_step_ = static_cast<Index>(nodes);
    const auto status = cudaGraphInstantiate(&graph_, graph, 0);
    cudaGraphDestroy(graph);
    runtime::check_cuda(status, "cudaGraphInstantiate");
    graph_version_ = version;
    graph_epoch_ = plan.buffer_epoch();
}

void Generation::step(Index steps) {
    if (steps < 0) throw std::invalid_argument("negative step count");
    if (generated_ == 0) throw std::logic_error("prefill a prompt before stepping");
    if (generated_ + steps > max_steps_) throw std::out_of_range("generation step budget exhausted");
    runtime::set_device(device_);
    decoder_->plan().refresh();
    decoder_->plan().validate(batch_, steps, *cache_, device_);  // capacity for all `steps` single-token appends
    capture();
    if (steps > 0) {
        decoder_->plan().set_user(this);
        logits_current_ = !fused_choice_;
    }
    cudaStream_t stream = cuda_stream(device_);
    for (Index i = 0; i < steps; ++i) runtime::check_cuda(cudaGraphLaunch(graph_, stream), "cudaGraphLaunch");
    for (auto& layer : *cache_) layer.commit(steps);
    generated_ += steps;
}

void Generation::step_host(const Index* ids_in, Index* ids_out) {
    runtime::set_device(device_);
    cudaStream_t stream = cuda_stream(device_);
    auto* staging = static_cast<Index*>(pinned_->data);
    if (ids_in) {
        const Index V = tokens_->weight().size(0);
        for (Index b = 0; b < batch_; ++b) {
            if (ids_in[b] < 0 || ids_in[b] >= V) throw std::out_of_range("embedding index out of range");
            staging[b] = ids_in[b];
        }
        runtime::check_cuda(cudaMemcpyAsync(ids_.mutable_data(), staging, sizeof(Index) * static_cast<std::size_t>(batch_),
                                            cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync");
        if (generated_ == 0) generated_ = 1;  // the caller supplied the first token itself
    }
    step(1);
    runtime::check_cuda(cudaMemcpyAsync(staging + batch_, next_.raw_data(), sizeof(Index) * static_cast<std::size_t>(batch_),
                                        cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync");
    runtime::check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    if (ids_out) std::copy(staging + batch_, staging + 2 * batch_, ids_out);
}

void Generation::step_sampled(double temperature, const double* uniforms, Index* ids_out) {
    if (!(temperature > 0.0)) throw std::invalid_argument("temperature must be positive");
    if (!uniforms) throw std::invalid_argument("uniform variates are NULL");
    if (generated_ == 0) throw std::logic_error("prefill a prompt before stepping");
    if (generated_ + 1 > max_steps_) throw std::out_of_range("generation step budget exhausted");
    for (Index b = 0; b < batch_; ++b)
        if (!(uniforms[b] >= 0.0 && uniforms[b] < 1.0)) throw std::invalid_argument("uniform variates must lie in [0, 1)");
    runtime::set_device(device_);
    auto& plan = decoder_->plan();
    plan.refresh();
    plan.validate(batch_, 1, *cache_, device_);
    const Index capacity = cache_->front().capacity();
    plan.reserve(batch_, capacity, device_);
    plan.set_user(this);
    cudaStream_t stream = cuda_stream(device_);
    auto* staging = static_cast<Index*>(pinned_->data);
    auto* variates = reinterpret_cast<double*>(staging + 2 * batch_);
    std::copy(uniforms, uniforms + batch_, variates);
    runtime::check_cuda(cudaMemcpyAsync(uniform_.mutable_data(), variates, sizeof(double) * static_cast<std::size_t>(batch_),
                                        cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync");
    plan.embed(*tokens_, ids_.data<Index>(), batch_, static_cast<float*>(x_.mutable_data()), stream);
    plan.run_layers(x_.data<float>(), batch_, 1, *cache_, capacity, stream, plan.shadows_for(batch_));
    std::vector<b200_kv_cache*> handles;
    for (auto& layer : *cache_) handles.push_back(layer.handle());
    runtime::check(b200_kv_cache_advance(handles.data(), static_cast<int32_t>(handles.size()), 1, stream), "KV advance");
    plan.logits(*output_, batch_, static_cast<float*>(logits_.mutable_data()), stream);
    runtime::check(b200_sample(logits_.data<float>(), batch_, output_->weight().size(0), temperature, uniform_.data<double>(),
                               static_cast<Index*>(next_.mutable_data()), stream), "sampling");
    runtime::check(b200_token_feedback(next_.data<Index>(), batch_, static_cast<Index*>(ids_.mutable_data()),
                                       static_cast<Index*>(history_.mutable_data()), max_steps_,
                                       static_cast<int32_t*>(counter_.mutable_data()), stream), "token feedback");
    for (auto& layer : *cache_) layer.commit(1);
    ++generated_;
    logits_current_ = true;
    runtime::check_cuda(cudaMemcpyAsync(staging + batch_, next_.raw_data(), sizeof(Index) * static_cast<std::size_t>(batch_),
                                        cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync");
    runtime::check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    if (ids_out) std::copy(staging + batch_, staging + 2 * batch_, ids_out);
}

Generation::StepProfile Generation::profile_step() {
    if (generated_ == 0) throw std::logic_error("prefill a prompt before stepping");
    if (generated_ + 1 > max_steps_) throw std::out_of_range("generation step budget exhausted");
    runtime::set_device(device_);
    auto& plan = decoder_->plan();
    plan.refresh();
    plan.validate(batch_, 1, *cache_, device_);
    prepare();
    plan.set_user(this);
    logits_current_ = !fused_choice_;
    cudaStream_t stream = cuda_stream(device_);
    runtime::check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    StepProbe trail{stream, {}, {}};
    trail.mark(2);
    step_probe = &trail;
    try {
        enqueue_step(stream, cache_->front().capacity());
    } catch (...) {
        step_probe = nullptr;
        throw;
    }
    step_probe = nullptr;
    runtime::check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    for (auto& layer : *cache_) layer.commit(1);
    ++generated_;
    StepProfile result{0.0, 0.0, 0.0, static_cast<Index>(trail.events.size()) - 1};
    for (std::size_t i = 1; i < trail.events.size(); ++i) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, trail.events[i - 1], trail.events[i]);
        (trail.kinds[i] == 0 ? result.linear_ms : trail.kinds[i] == 1 ? result.attention_ms : result.other_ms) += ms;
    }
    for (auto event : trail.events) cudaEventDestroy(event);
    return result;
}

Tensor Generation::tokens() const {
    synchronize(Device::cuda(device_));
    // history is [step, batch]; the caller-facing layout is [batch, step]
    const Tensor host = history_.narrow(0, 0, generated_).to(Device::cpu());
    Tensor result = empty({batch_, generated_}, {DType::i64, Device::cpu()});
    for (Index s = 0; s < generated_; ++s)
        for (Index b = 0; b < batch_; ++b)
            static_cast<Index*>(result.mutable_data())[b * generated_ + s] = host.data<Index>()[s * batch_ + b];
    return result;
}
Tensor Generation::last_logits() {
    if (logits_current_) return logits_;
    if (generated_ == 0) throw std::logic_error("nothing has been generated yet");
    auto& plan = decoder_->plan();
    if (plan.user() != this) throw std::logic_error("the decoder has run something else since this generation's last step");
    runtime::set_device(device_);
    plan.logits(*output_, batch_, static_cast<float*>(logits_.mutable_data()), runtime::stream(device_));
    logits_current_ = true;
    return logits_;
}

}  // namespace dl::nn
