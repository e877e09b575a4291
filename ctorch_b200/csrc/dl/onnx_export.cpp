// ONNX export of the decoder with its KV cache as graph ports (dl::onnx::save_decoder, extensions/onnx/include/dl/onnx.h:30-35
// of the reference; graph layout extensions/onnx/src/decoder.cpp:53-118).  The file is a protobuf ModelProto (ir 12, opset
// 24, producer "Ctorch") whose graph "CtorchDecoder" takes `features` [batch, tokens, width] (or int64 `input_ids` when an
// embedding and an output layer are given) plus, per layer i, `past_key_i` / `past_value_i` [batch, kv_heads, past, head],
// and returns `hidden_states` (or `logits`) plus `present_key_i` / `present_value_i` [batch, kv_heads, total, head].  Per
// layer: RMSNormalization, MatMul projections, RotaryEmbedding (interleaved = adjacent pairs, positions past .. past +
// tokens), causal Attention fed with the past ports, SwiGLU as Mul(gate * Sigmoid(gate), up).  Weights become f32
// initializers; a tensor used twice (tied embedding / output table) is written once.
//
// Everything is read from the module objects of this library (state_dict names of src/nn/decoder.cpp:111-114), on the host:
// no kernel runs.  The writer emits fields in the order in which the reference's exporter does, so that the two files
// are equal byte for byte for equal weights.
#include "dl/dl.h"

#include <bit>
#include <cstdint>
#include <fstream>
#include <stdexcept>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

namespace dl::onnx {
namespace {

// Append-only protobuf encoder: varints, length-delimited fields, 32-bit floats.
class Proto {
public:
    void number(unsigned field, std::uint64_t value) { varint(static_cast<std::uint64_t>(field) << 3); varint(value); }
    void text(unsigned field, std::string_view value) {
        varint((static_cast<std::uint64_t>(field) << 3) | 2u);
        varint(value.size());
        buffer_.append(value);
    }
    void nested(unsigned field, const Proto& child) { text(field, child.buffer_); }
    void real(unsigned field, float value) {
        varint((static_cast<std::uint64_t>(field) << 3) | 5u);
        std::uint32_t bits = std::bit_cast<std::uint32_t>(value);
        for (int byte = 0; byte < 4; ++byte, bits >>= 8) buffer_.push_back(static_cast<char>(bits & 0xffu));
    }
    const std::string& bytes() const { return buffer_; }

private:
    void varint(std::uint64_t value) {
        for (; value >= 0x80u; value >>= 7) buffer_.push_back(static_cast<char>((value & 0x7fu) | 0x80u));
        buffer_.push_back(static_cast<char>(value));
    }
    std::string buffer_;
};

// onnx.proto field numbers used below
namespace field {
constexpr unsigned model_ir = 1, model_producer = 2, model_graph = 7, model_opset = 8, opset_version = 2;
constexpr unsigned graph_node = 1, graph_name = 2, graph_initializer = 5, graph_input = 11, graph_output = 12;
constexpr unsigned node_input = 1, node_output = 2, node_type = 4, node_attribute = 5;
constexpr unsigned tensor_dim = 1, tensor_type = 2, tensor_name = 8, tensor_raw = 9;
constexpr unsigned attr_name = 1, attr_float = 2, attr_int = 3, attr_ints = 8, attr_kind = 20;
constexpr unsigned info_name = 1, info_type = 2, type_tensor = 1, tensor_elem = 1, tensor_shape = 2, shape_dim = 1, dim_value = 1, dim_name = 2;
}  // namespace field

int element_code(DType dtype) {   // TensorProto.DataType
    switch (dtype) {
    case DType::f32: return 1;
    case DType::f64: return 11;
    case DType::i64: return 7;
    case DType::boolean: return 9;
    case DType::f16: return 10;
    case DType::bf16: return 16;
    }
    return 0;
}

struct Attribute {
    enum class Kind { integer, real, integers } kind;
    std::string name;
    Index integer = 0;
    double real = 0.0;
    Shape integers;
    static Attribute of(std::string name, Index value) { return {Kind::integer, std::move(name), value, 0.0, {}}; }
    static Attribute of(std::string name, double value) { return {Kind::real, std::move(name), 0, value, {}}; }
    static Attribute of(std::string name, Shape values) { return {Kind::integers, std::move(name), 0, 0.0, std::move(values)}; }
};

struct Extent {   // a fixed size or a named (run-time) one
    Index size = -1;
    std::string_view name;
    Extent(Index fixed) : size(fixed) {}
    Extent(const char* symbol) : name(symbol) {}
};

class DecoderGraph {
public:
    explicit DecoderGraph(const nn::TransformerDecoder& decoder) {
        graph_.text(field::graph_name, "CtorchDecoder");
        for (auto& entry : decoder.state_dict()) state_.emplace(entry.first, entry.second);
    }

    const Tensor& parameter(const std::string& name) const {
        const auto found = state_.find(name);
        if (found == state_.end()) throw std::invalid_argument("decoder state has no entry " + name);
        return found->second;
    }

    void port(bool output, const std::string& name, DType dtype, std::initializer_list<Extent> extents) {
        Proto shape;
        for (const Extent& extent : extents) {
            Proto dimension;
            if (extent.size >= 0) dimension.number(field::dim_value, static_cast<std::uint64_t>(extent.size));
            else dimension.text(field::dim_name, extent.name);
            shape.nested(field::shape_dim, dimension);
        }
        Proto tensor, type, info;
        tensor.number(field::tensor_elem, static_cast<std::uint64_t>(element_code(dtype)));
        tensor.nested(field::tensor_shape, shape);
        type.nested(field::type_tensor, tensor);
        info.text(field::info_name, name);
        info.nested(field::info_type, type);
        graph_.nested(output ? field::graph_output : field::graph_input, info);
    }

    std::string next_name() { return "value_" + std::to_string(counter_++); }

    // An initializer holding a host tensor as it is.
    std::string constant(const Tensor& value) {
        const Tensor host = value.device().type == DeviceType::cpu ? value : value.to(Device::cpu());
        const std::string name = next_name();
        Proto tensor;
        for (const Index extent : host.shape()) tensor.number(field::tensor_dim, static_cast<std::uint64_t>(extent));
        tensor.number(field::tensor_type, static_cast<std::uint64_t>(element_code(host.dtype())));
        tensor.text(field::tensor_name, name);
        static_assert(std::endian::native == std::endian::little, "raw tensor data is little-endian");
        tensor.text(field::tensor_raw, std::string_view(static_cast<const char*>(host.raw_data()), host.nbytes()));
        graph_.nested(field::graph_initializer, tensor);
        return name;
    }
    std::string integers(const Shape& values) {
        return constant(dl::detail::from_host(values.data(), {static_cast<Index>(values.size())}, DType::i64, false, Device::cpu()));
    }
    std::string scalar(Index value) { return constant(dl::detail::from_host(&value, {}, DType::i64, false, Device::cpu())); }

    // A weight as an f32 initializer; the same storage is written once (tied embedding and output tables).
    std::string weight(const Tensor& tensor) {
        const auto found = written_.find(tensor.raw_data());
        if (found != written_.end()) return found->second;
        const Tensor host = tensor.device().type == DeviceType::cpu ? tensor : tensor.to(Device::cpu());
        const std::string name = constant(host.astype(DType::f32));
        written_.emplace(tensor.raw_data(), name);
        return name;
    }

    void node(std::string_view type, const std::vector<std::string>& inputs, const std::vector<std::string>& outputs,
              const std::vector<Attribute>& attributes = {}) {
        Proto op;
        for (const auto& name : inputs) op.text(field::node_input, name);
        for (const auto& name : outputs) op.text(field::node_output, name);
        op.text(field::node_type, type);
        for (const Attribute& attribute : attributes) {
            Proto encoded;
            encoded.text(field::attr_name, attribute.name);
            switch (attribute.kind) {
            case Attribute::Kind::integer:
                encoded.number(field::attr_kind, 2);
                encoded.number(field::attr_int, static_cast<std::uint64_t>(attribute.integer));
                break;
            case Attribute::Kind::real:
                encoded.number(field::attr_kind, 1);
                encoded.real(field::attr_float, static_cast<float>(attribute.real));
                break;
            case Attribute::Kind::integers:
                encoded.number(field::attr_kind, 7);
                for (const Index item : attribute.integers) encoded.number(field::attr_ints, static_cast<std::uint64_t>(item));
                break;
            }
            op.nested(field::node_attribute, encoded);
        }
        graph_.nested(field::graph_node, op);
    }
    // One-output node with a generated name.
    std::string apply(std::string_view type, const std::vector<std::string>& inputs, const std::vector<Attribute>& attributes = {}) {
        const std::string name = next_name();
        node(type, inputs, {name}, attributes);
        return name;
    }

    std::string project(const std::string& x, const Tensor& matrix) {   // x @ W^T with W stored [out, in]
        const std::string stored = weight(matrix);
        const std::string transposed = apply("Transpose", {stored}, {Attribute::of("perm", Shape{1, 0})});
        return apply("MatMul", {x, transposed});
    }
    std::string normalise(const std::string& x, const std::string& weight_name) {
        const std::string scale = weight(parameter(weight_name));
        return apply("RMSNormalization", {x, scale}, {Attribute::of("epsilon", nn::TransformerDecoderLayer::norm_epsilon)});
    }

    // positions of the new tokens: past .. past + tokens, one row per sequence
    std::string positions(const std::string& input) {
        const std::string one = scalar(1), two = scalar(2);
        const std::string batch_tokens = apply("Shape", {input}, {Attribute::of("end", Index{2})});
        const std::string tokens = apply("Gather", {batch_tokens, one});
        const std::string cache_shape = apply("Shape", {"past_key_0"});
        const std::string past = apply("Gather", {cache_shape, two});
        const std::string end = apply("Add", {past, tokens});
        const std::string range = apply("Range", {past, end, one});
        return apply("Expand", {range, batch_tokens});
    }

    std::string layer(Index index, const std::string& x, const std::string& position_ids) {
        const std::string number = std::to_string(index), prefix = "layer" + number + ".";
        const std::string attention = prefix + "attention.", feedforward = prefix + "feedforward.";
        const Tensor& cosine = parameter(attention + "rotary.cosine");
        const Tensor& sine = parameter(attention + "rotary.sine");
        const Index width = parameter(attention + "query.weight").size(0);
        const Index head = 2 * cosine.size(1);
        const Index kv_heads = parameter(attention + "key.weight").size(0) / head;
        const std::string past_key = "past_key_" + number, past_value = "past_value_" + number;
        const std::string present_key = "present_key_" + number, present_value = "present_value_" + number;
        port(false, past_key, DType::f32, {"batch", kv_heads, "past", head});
        port(false, past_value, DType::f32, {"batch", kv_heads, "past", head});
        port(true, present_key, DType::f32, {"batch", kv_heads, "total", head});
        port(true, present_value, DType::f32, {"batch", kv_heads, "total", head});

        const std::string normalized = normalise(x, prefix + "attention_norm.weight");
        const std::vector<Attribute> heads_outward{Attribute::of("perm", Shape{0, 2, 1, 3})};
        auto heads_of = [&](const char* which, Index count) {   // [batch, tokens, count * head] -> [batch, count, tokens, head]
            const std::string projected = project(normalized, parameter(attention + which + ".weight"));
            const std::string shape = integers({0, 0, count, head});
            const std::string split = apply("Reshape", {projected, shape});
            return apply("Transpose", {split}, heads_outward);
        };
        auto rotated = [&](const std::string& input) {
            const std::string cosine_table = weight(cosine), sine_table = weight(sine);
            return apply("RotaryEmbedding", {input, cosine_table, sine_table, position_ids}, {Attribute::of("interleaved", Index{1})});
        };
        const std::string q = rotated(heads_of("query", width / head));
        const std::string k = rotated(heads_of("key", kv_heads));
        const std::string v = heads_of("value", kv_heads);
        const std::string attended = next_name();
        node("Attention", {q, k, v, "", past_key, past_value}, {attended, present_key, present_value}, {Attribute::of("is_causal", Index{1})});
        const std::string heads_inward = apply("Transpose", {attended}, heads_outward);
        const std::string merged_shape = integers({0, 0, width});
        const std::string merged = apply("Reshape", {heads_inward, merged_shape});
        const std::string attention_out = project(merged, parameter(attention + "output.weight"));
        const std::string residual = apply("Add", {x, attention_out});
        const std::string features = normalise(residual, prefix + "feedforward_norm.weight");
        const std::string gate = project(features, parameter(feedforward + "gate.weight"));
        const std::string sigmoid = apply("Sigmoid", {gate});
        const std::string silu = apply("Mul", {gate, sigmoid});
        const std::string up = project(features, parameter(feedforward + "up.weight"));
        const std::string hidden = apply("Mul", {silu, up});
        const std::string down = project(hidden, parameter(feedforward + "down.weight"));
        return apply("Add", {residual, down});
    }

    void write(const std::string& path) const {
        Proto model, opset;
        model.number(field::model_ir, 12);
        model.text(field::model_producer, "Ctorch");
        model.nested(field::model_graph, graph_);
        opset.number(field::opset_version, 24);
        model.nested(field::model_opset, opset);
        std::ofstream file;
        file.exceptions(std::ios::failbit | std::ios::badbit);
        try {
            file.open(path, std::ios::binary | std::ios::trunc);
            file.write(model.bytes().data(), static_cast<std::streamsize>(model.bytes().size()));
            file.close();
        } catch (const std::ios_base::failure&) {
            throw std::runtime_error("cannot write ONNX file " + path);
        }
    }

private:
    Proto graph_;
    std::unordered_map<std::string, Tensor> state_;
    std::unordered_map<const void*, std::string> written_;
    std::size_t counter_ = 0;
};

void export_decoder(const std::string& path, const nn::TransformerDecoder& decoder, const nn::Embedding* embedding, const nn::Linear* output) {
    DecoderGraph graph(decoder);
    const Index width = graph.parameter("normalization.weight").size(0);
    const std::string input = embedding ? "input_ids" : "features", result = output ? "logits" : "hidden_states";
    if (embedding) {
        if (embedding->weight().size(1) != width || output->weight().size(1) != width)
            throw std::invalid_argument("decoder input and output projections must match its hidden width");
        graph.port(false, input, DType::i64, {"batch", "tokens"});
    } else {
        graph.port(false, input, DType::f32, {"batch", "tokens", width});
    }
    graph.port(true, result, DType::f32, {"batch", "tokens", output ? output->weight().size(0) : width});
    const std::string position_ids = graph.positions(input);
    std::string x = input;
    if (embedding) {
        const std::string table = graph.weight(embedding->weight());
        x = graph.apply("Gather", {table, input});
    }
    for (Index i = 0; i < decoder.layer_count(); ++i) x = graph.layer(i, x, position_ids);
    x = graph.normalise(x, "normalization.weight");
    if (output) {
        x = graph.project(x, output->weight());
        if (output->bias()) {
            const std::string bias = graph.weight(*output->bias());
            x = graph.apply("Add", {x, bias});
        }
    }
    graph.node("Identity", {x}, {result});
    graph.write(path);
}

}  // namespace

void save_decoder(const std::string& path, const nn::TransformerDecoder& decoder) { export_decoder(path, decoder, nullptr, nullptr); }

void save_decoder(const std::string& path, const nn::Embedding& embedding, const nn::TransformerDecoder& decoder, const nn::Linear& output) {
    export_decoder(path, decoder, &embedding, &output);
}

}  // namespace dl::onnx
