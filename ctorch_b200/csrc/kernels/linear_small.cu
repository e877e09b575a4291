// Skinny linear for the decode step: y = epilogue(rmsnorm?(x) @ W^T), x f32 [rows, in] with few rows, W [out, in]
// row-major in f32 or bf16.  The work is weight streaming (HBM-bound): every warp owns two adjacent output
// features, its lanes stride over K with 128-bit non-allocating loads, the activation tile lives in shared
// memory, accumulation is f32 and the cross-lane reduction uses warp shuffles.  Rows beyond the register tile
// are covered by blockIdx.x so that CTAs that share a weight block run back to back and hit L2.
//
// Fused around the contraction (reference: src/nn/decoder.cpp:77-106 runs these as separate ops):
//   prologue  RMSNorm of x in f64 (src/kernels/cpu/normalization.cpp:39-51)
//   epilogue  store | residual add | SiLU(gate)*up on interleaved rows | RoPE + KV-cache append (+ LoRA delta)
#include "linear_common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kNF = 2;           // output features per warp (RoPE and SwiGLU consume adjacent pairs)
constexpr int kChunk = 2048;     // activation columns staged per pass


template <class W> struct Vec;
template <> struct Vec<__nv_bfloat16> { static constexpr int n = 8; };
template <> struct Vec<float> { static constexpr int n = 4; };

// Position of activation column k inside a staged row.  For bf16 weights a lane consumes 8 consecutive
// columns with two 16-byte shared loads; splitting the two halves into separate planes keeps consecutive lanes
// 16 bytes apart (no bank conflicts).
template <int V> __device__ __forceinline__ int staged_index(int k, int plane) {
    if constexpr (V == 8) return ((k >> 3) << 2) + (k & 3) + ((k >> 2) & 1) * plane;
    else return k;
}

template <class W, int R, int EPI, bool VECTOR>
__global__ void __launch_bounds__(kThreads) linear_small_kernel(const LinearParams p) {
    constexpr int V = VECTOR ? Vec<W>::n : 1;
    extern __shared__ __align__(16) float xs[];  // [R][stride]
    __shared__ double inverse_std[R];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * R;
    const int feature0 = (blockIdx.y * kWarps + warp) * kNF;
    const bool active = feature0 < p.out;
    const W* weight = static_cast<const W*>(p.weight);

    const int chunk_max = p.in < kChunk ? p.in : kChunk;
    const int stride = ((chunk_max + 7) >> 3) << 3;  // staged row length, multiple of 8
    const int plane = stride >> 1;

    if (p.norm_weight) {
        // One warp per row: sum of squares in f64, as the reference's CPU kernel does.
        for (int r = warp; r < R; r += kWarps) {
            double squares = 0.0;
            if (row0 + r < p.rows) {
                const float* row = p.x + static_cast<int64_t>(row0 + r) * p.in;
                for (int k = lane; k < p.in; k += 32) {
                    const double v = static_cast<double>(row[k]);
                    squares += v * v;
                }
            }
            squares = warp_sum(squares);
            if (lane == 0) inverse_std[r] = 1.0 / sqrt(squares / static_cast<double>(p.in) + p.eps);
        }
        __syncthreads();
    }

    float acc[kNF][R];
#pragma unroll
    for (int f = 0; f < kNF; ++f)
#pragma unroll
        for (int r = 0; r < R; ++r) acc[f][r] = 0.0f;

    for (int base = 0; base < p.in; base += kChunk) {
        const int width = (p.in - base) < kChunk ? (p.in - base) : kChunk;
        if (base) __syncthreads();
        // Stage (and normalise) the activation chunk.
        for (int i = threadIdx.x; i < R * stride; i += kThreads) {
            const int r = i / stride, k = i - r * stride;
            float value = 0.0f;
            if (k < width && row0 + r < p.rows) {
                value = p.x[static_cast<int64_t>(row0 + r) * p.in + base + k];
                if (p.norm_weight) {
                    double scaled = static_cast<double>(value) * inverse_std[r];
                    const double w = p.norm_dtype == B200_BF16
                        ? static_cast<double>(__bfloat162float(static_cast<const __nv_bfloat16*>(p.norm_weight)[base + k]))
                        : static_cast<double>(static_cast<const float*>(p.norm_weight)[base + k]);
                    scaled *= w;
                    value = static_cast<float>(scaled);
                }
            }
            xs[r * stride + staged_index<V>(k, plane)] = value;
        }
        __syncthreads();
        if (!active) continue;

        const W* w0 = weight + static_cast<int64_t>(feature0) * p.in + base;
        const bool second = feature0 + 1 < p.out;
        const W* w1 = second ? w0 + p.in : w0;
        if constexpr (V == 8) {
#pragma unroll 2
            for (int k = lane * 8; k < width; k += 256) {
                const uint4 a = load_stream_16(w0 + k);
                const uint4 b = load_stream_16(w1 + k);
                const float wa[8] = {bf16_lo(a.x), bf16_hi(a.x), bf16_lo(a.y), bf16_hi(a.y),
                                     bf16_lo(a.z), bf16_hi(a.z), bf16_lo(a.w), bf16_hi(a.w)};
                const float wb[8] = {bf16_lo(b.x), bf16_hi(b.x), bf16_lo(b.y), bf16_hi(b.y),
                                     bf16_lo(b.z), bf16_hi(b.z), bf16_lo(b.w), bf16_hi(b.w)};
                const int at = (k >> 3) << 2;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float4 lo = *reinterpret_cast<const float4*>(xs + r * stride + at);
                    const float4 hi = *reinterpret_cast<const float4*>(xs + r * stride + plane + at);
                    const float xv[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        acc[0][r] = fmaf(wa[j], xv[j], acc[0][r]);
                        acc[1][r] = fmaf(wb[j], xv[j], acc[1][r]);
                    }
                }
            }
        } else if constexpr (V == 4) {
#pragma unroll 2
            for (int k = lane * 4; k < width; k += 128) {
                const uint4 a = load_stream_16(w0 + k);
                const uint4 b = load_stream_16(w1 + k);
                const float wa[4] = {__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w)};
                const float wb[4] = {__uint_as_float(b.x), __uint_as_float(b.y), __uint_as_float(b.z), __uint_as_float(b.w)};
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float4 v = *reinterpret_cast<const float4*>(xs + r * stride + k);
                    const float xv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[0][r] = fmaf(wa[j], xv[j], acc[0][r]);
                        acc[1][r] = fmaf(wb[j], xv[j], acc[1][r]);
                    }
                }
            }
        } else {
            for (int k = lane; k < width; k += 32) {
                const float a = load_as_f32(w0, k), b = load_as_f32(w1, k);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float v = xs[r * stride + k];
                    acc[0][r] = fmaf(a, v, acc[0][r]);
                    acc[1][r] = fmaf(b, v, acc[1][r]);
                }
            }
        }
    }
    if (!active) return;

#pragma unroll
    for (int f = 0; f < kNF; ++f)
#pragma unroll
        for (int r = 0; r < R; ++r) acc[f][r] = warp_sum(acc[f][r]);

    // Lane r finishes row r of this warp's feature pair.
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (lane != r) continue;
        const int row = row0 + r;
        if (row >= p.rows) continue;
        float a = acc[0][r], b = acc[1][r];
        linear_epilogue<EPI>(p, row, feature0, a, b);
    }
}

template <class W, int R, int EPI, bool VECTOR> int launch(const LinearParams& p, cudaStream_t stream) {
    const int row_tiles = (p.rows + R - 1) / R;
    const int feature_blocks = (p.out + kWarps * kNF - 1) / (kWarps * kNF);
    const int chunk = p.in < kChunk ? p.in : kChunk;
    const size_t smem = sizeof(float) * R * (((chunk + 7) >> 3) << 3);
    auto kernel = linear_small_kernel<W, R, EPI, VECTOR>;
    if (smem > 48 * 1024) B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kernel<<<dim3(row_tiles, feature_blocks), kThreads, smem, stream>>>(p);
    return cuda_status(cudaGetLastError(), "linear_small_kernel launch");
}

template <class W, int EPI> int pick_rows(const LinearParams& p, bool vector, cudaStream_t stream) {
    if (!vector) return launch<W, 8, EPI, false>(p, stream);
    if (p.rows == 1) return launch<W, 1, EPI, true>(p, stream);
    if (p.rows == 2) return launch<W, 2, EPI, true>(p, stream);
    if (p.rows <= 4) return launch<W, 4, EPI, true>(p, stream);
    return launch<W, 8, EPI, true>(p, stream);
}

template <class W> int pick_epilogue(const LinearParams& p, int epilogue, bool vector, cudaStream_t stream) {
    switch (epilogue) {
    case B200_EPI_STORE: return pick_rows<W, B200_EPI_STORE>(p, vector, stream);
    case B200_EPI_RESIDUAL: return pick_rows<W, B200_EPI_RESIDUAL>(p, vector, stream);
    case B200_EPI_SWIGLU: return pick_rows<W, B200_EPI_SWIGLU>(p, vector, stream);
    case B200_EPI_QKV: return pick_rows<W, B200_EPI_QKV>(p, vector, stream);
    }
    set_error("b200_linear: unknown epilogue %d", epilogue);
    return B200_BAD_ARGUMENT;
}

}  // namespace
}  // namespace b200

namespace b200 {
namespace {
// Copies and checks the operands of the q|k|v epilogue.
int fill_qkv(LinearParams& p, int epilogue, const b200_qkv_args* qkv, int64_t rows, int64_t out) {
    if (epilogue != B200_EPI_QKV) return B200_OK;
        if (!qkv || !qkv->cache || !qkv->q_out || !qkv->cosine || !qkv->sine || qkv->tokens_per_sequence <= 0 || (qkv->head_dim & 1)
            || out != static_cast<int64_t>(qkv->heads + 2 * qkv->kv_heads) * qkv->head_dim) {
            set_error("b200_linear: inconsistent QKV epilogue arguments");
            return B200_BAD_ARGUMENT;
        }
        p.heads = qkv->heads; p.kv_heads = qkv->kv_heads; p.head_dim = qkv->head_dim;
        p.tokens_per_sequence = qkv->tokens_per_sequence; p.context = qkv->context;
        p.cosine = qkv->cosine; p.sine = qkv->sine; p.kv = kv_view(qkv->cache); p.q_out = qkv->q_out;
        if (p.kv.kv_heads != qkv->kv_heads || p.kv.head_dim != qkv->head_dim
            || rows != static_cast<int64_t>(p.kv.sequences) * qkv->tokens_per_sequence) {
            set_error("b200_linear: KV cache shape does not match the projection");
            return B200_BAD_ARGUMENT;
        }
        p.lora_rank = qkv->lora_rank; p.lora_scale = qkv->lora_scale; p.low = qkv->low; p.q_up = qkv->q_up; p.v_up = qkv->v_up;
        if (p.lora_rank > 0 && (!p.low || !p.q_up || !p.v_up)) { set_error("b200_linear: adapter pointers missing"); return B200_BAD_ARGUMENT; }
        return B200_OK;
}
}  // namespace
}  // namespace b200

extern "C" int b200_linear(const float* x, int64_t rows, int64_t in, const void* weight, int32_t weight_dtype,
                           int64_t out, const void* norm_weight, int32_t norm_dtype, double eps,
                           b200_epilogue epilogue, const float* residual, const b200_qkv_args* qkv, float* y,
                           void* stream) {
    using namespace b200;
    if (!x || !weight || !y || rows < 0 || in <= 0 || out <= 0 || rows > INT32_MAX || in > INT32_MAX || out > INT32_MAX) {
        set_error("b200_linear: bad pointer or size");
        return B200_BAD_ARGUMENT;
    }
    if (weight_dtype != B200_F32 && weight_dtype != B200_BF16) {
        set_error("b200_linear: weight dtype %d is not f32 or bf16", weight_dtype);
        return B200_UNSUPPORTED;
    }
    if (epilogue < B200_EPI_STORE || epilogue > B200_EPI_QKV) {
        set_error("b200_linear: epilogue %d is not available for f32 activation rows", static_cast<int>(epilogue));
        return B200_UNSUPPORTED;
    }
    if (rows == 0) return B200_OK;
    LinearParams p{};
    p.x = x; p.rows = static_cast<int>(rows); p.in = static_cast<int>(in); p.out = static_cast<int>(out);
    p.weight = weight; p.norm_weight = norm_weight; p.norm_dtype = norm_dtype; p.weight_dtype = weight_dtype; p.eps = eps;
    p.residual = residual; p.y = y;
    if (epilogue == B200_EPI_RESIDUAL && !residual) { set_error("b200_linear: residual epilogue without residual"); return B200_BAD_ARGUMENT; }
    if (epilogue == B200_EPI_SWIGLU && (out & 1)) { set_error("b200_linear: SwiGLU epilogue needs interleaved gate/up rows"); return B200_BAD_ARGUMENT; }
    {
        const int status = fill_qkv(p, epilogue, qkv, rows, out);
        if (status != B200_OK) return status;
    }
    cudaStream_t s = as_stream(stream);
    {
        // bf16 weights with a moderate inner size go to the tensor-core streaming kernel
        const int status = launch_linear_stream(p, epilogue, s);
        if (status != B200_UNSUPPORTED) return status;
    }
    const size_t element = weight_dtype == B200_BF16 ? 2 : 4;
    const bool vector = (in * element) % 16 == 0 && reinterpret_cast<uintptr_t>(weight) % 16 == 0;
    return weight_dtype == B200_BF16 ? pick_epilogue<__nv_bfloat16>(p, epilogue, vector, s)
                                     : pick_epilogue<float>(p, epilogue, vector, s);
}

extern "C" int b200_linear_shadow(const b200_shadow_linear_args* args, void* stream) {
    using namespace b200;
    if (!args || !args->x_hi || !args->weight || args->rows < 0 || args->in <= 0 || args->out <= 0
        || args->rows > INT32_MAX || args->in > INT32_MAX || args->out > INT32_MAX) {
        set_error("b200_linear_shadow: bad pointer or size");
        return B200_BAD_ARGUMENT;
    }
    if (args->rows == 0) return B200_OK;
    const int epilogue = args->epilogue;
    if (epilogue < B200_EPI_STORE || epilogue > B200_EPI_ARGMAX) { set_error("b200_linear_shadow: unknown epilogue"); return B200_BAD_ARGUMENT; }
    if ((epilogue != B200_EPI_SWIGLU && !args->y && epilogue != B200_EPI_QKV && epilogue != B200_EPI_ARGMAX)
        || (epilogue == B200_EPI_ARGMAX && (!args->best_value || !args->best_index)) || (epilogue == B200_EPI_RESIDUAL && !args->residual)
        || (epilogue == B200_EPI_SWIGLU && (args->out & 1)) || (epilogue == B200_EPI_SWIGLU && !args->y && !args->out_hi)
        || (args->out_hi && !args->out_lo) || (args->sumsq_in && args->parts_in <= 0)) {
        set_error("b200_linear_shadow: inconsistent epilogue operands");
        return B200_BAD_ARGUMENT;
    }
    LinearParams p{};
    p.rows = static_cast<int>(args->rows); p.in = static_cast<int>(args->in); p.out = static_cast<int>(args->out);
    p.weight = args->weight; p.weight_dtype = B200_BF16; p.eps = args->eps;
    p.residual = args->residual; p.y = args->y;
    p.x_hi = static_cast<const __nv_bfloat16*>(args->x_hi); p.x_lo = static_cast<const __nv_bfloat16*>(args->x_lo);
    p.sumsq_in = args->sumsq_in; p.parts_in = args->parts_in;
    p.out_hi = static_cast<__nv_bfloat16*>(args->out_hi); p.out_lo = static_cast<__nv_bfloat16*>(args->out_lo);
    p.out_norm_weight = args->out_norm_weight; p.out_norm_dtype = args->out_norm_dtype; p.sumsq_out = args->sumsq_out;
    p.best_value = args->best_value; p.best_index = args->best_index;
    if (args->copies < 0 || args->copies > 7 || (args->copies > 0 && (!args->y_copies || (epilogue != B200_EPI_STORE && epilogue != B200_EPI_RESIDUAL)))) {
        set_error("b200_linear_shadow: at most 7 result copies, for store and residual epilogues only");
        return B200_BAD_ARGUMENT;
    }
    p.copies = args->copies;
    for (int c = 0; c < p.copies; ++c) {
        if (!args->y_copies[c]) { set_error("b200_linear_shadow: result copy %d is NULL", c); return B200_BAD_ARGUMENT; }
        p.y_copy[c] = args->y_copies[c];
    }
    const int status = fill_qkv(p, epilogue, args->qkv, args->rows, args->out);
    if (status != B200_OK) return status;
    const int launched = launch_linear_stream(p, epilogue, as_stream(stream));
    if (launched == B200_UNSUPPORTED) set_error("b200_linear_shadow: shape [%d, %d] is outside the streaming kernel", p.out, p.in);
    return launched;
}

extern "C" int32_t b200_linear_shadow_parts(int64_t rows, int64_t in, int64_t out) {
    if (rows <= 0 || in <= 0 || out <= 0 || rows > INT32_MAX || in > INT32_MAX || out > INT32_MAX) return 0;
    return b200::linear_stream_parts(static_cast<int>(rows), static_cast<int>(in), static_cast<int>(out));
}

extern "C" const char* b200_linear_shadow_kernel(int64_t rows, int64_t in, int64_t out) {
    // mirrors the dispatch of launch_linear_stream / launch_linear_gemm for a shadow call with bf16 weights
    if (rows <= 0 || in <= 0 || out <= 0 || rows > INT32_MAX) return "";
    if (rows >= b200::kGemmRows || in > 2048) {
        if (rows >= b200::kGemmRows && out <= 64 && rows <= 512) return "linear_thin_kernel";
        return b200::linear_decode_takes(static_cast<int>(rows)) ? "linear_decode_kernel" : "linear_gemm_kernel";
    }
    return "linear_stream_kernel";
}

extern "C" int32_t b200_linear_decode_launch_shape(int64_t rows, int64_t in, int64_t out, int32_t two_planes, int32_t* shape) {
    if (!shape || rows <= 0 || in <= 0 || out <= 0 || rows > INT32_MAX || in > INT32_MAX || out > INT32_MAX) return 0;
    if (!b200::linear_decode_takes(static_cast<int>(rows))) return 0;
    int device = 0;
    const int sms = cudaGetDevice(&device) == cudaSuccess ? b200::sm_count(device) : 148;
    cudaGetLastError();
    const b200::DecodeShape s = b200::linear_decode_shape(static_cast<int>(rows), static_cast<int>(in), static_cast<int>(out), two_planes != 0, sms);
    if (s.tiles == 0) return 0;
    const int32_t values[10] = {s.tiles, s.split, s.ctas, s.stages, s.stage_bytes, s.n_pad, s.tmem_columns, s.smem_bytes, s.token_tile, s.token_tiles};
    for (int i = 0; i < 10; ++i) shape[i] = values[i];
    return 1;
}

extern "C" int32_t b200_linear_argmax_parts(int64_t rows, int64_t in, int64_t out) {
    if (rows <= 0 || in <= 0 || out <= 0 || rows > INT32_MAX || in > INT32_MAX || out > INT32_MAX) return 0;
    return b200::linear_argmax_parts(static_cast<int>(rows), static_cast<int>(in), static_cast<int>(out));
}
