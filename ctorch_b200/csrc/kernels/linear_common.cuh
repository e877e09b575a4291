// Operands and epilogues shared by the skinny-linear kernels.
#pragma once

#include "common.cuh"

#include "kv_cache.cuh"

namespace b200 {

struct LinearParams {
    const float* x;
    int rows, in, out;
    const void* weight;
    const void* norm_weight;
    int norm_dtype, weight_dtype;
    double eps;
    const float* residual;
    float* y;
    // B200_EPI_QKV
    int heads, kv_heads, head_dim, tokens_per_sequence, context;
    const float *cosine, *sine;
    KvView kv;
    float* q_out;
    int lora_rank;
    float lora_scale;
    const float* low;
    const void *q_up, *v_up;
    // Activation shadows (streaming kernel only, all optional).  A shadow is an f32 matrix stored as two bf16
    // planes hi + lo (hi = bf16(v), lo = bf16(v - hi)), the form the tensor cores consume.
    const __nv_bfloat16 *x_hi, *x_lo;  // input shadow [rows, in]; replaces x
    const float* sumsq_in;             // [parts_in][rows] partial sums of squares of the input rows before their
    int parts_in;                      //   norm weight was folded in: the result is scaled by 1/sqrt(mean + eps)
    __nv_bfloat16 *out_hi, *out_lo;    // output shadow (residual: [rows, out]; SwiGLU: [rows, out/2])
    const void* out_norm_weight;       // weight of the RMSNorm that follows, folded into the output shadow
    int out_norm_dtype;
    float* sumsq_out;                  // [tiles][rows] per-tile sums of squares of the (un-weighted) result rows
    // B200_EPI_ARGMAX: per feature tile and row, the preferred value and its feature index
    float* best_value;                 // [tiles][rows]
    int32_t* best_index;               // [tiles][rows]
    // Store and residual epilogues: further [rows, out] f32 matrices that receive the same result rows as y.  Tensor
    // parallelism points them at this rank's slot in every peer's memory, so the partial sums travel over NVLink from
    // the projection's own epilogue (plain peer stores) and the sum that follows reads local memory only.
    float* y_copy[7];
    int copies;
};

// The result pair of (row, feature0) to every extra destination (see LinearParams::y_copy).  The destinations are named
// one by one: a loop over the array would index the kernel's parameters with a register, which costs a copy of the whole
// parameter block in local memory.
__device__ __forceinline__ void store_copy_pair(float* target, float a, float b, bool second) {
    if (second && (reinterpret_cast<uintptr_t>(target) & 7) == 0) {
        *reinterpret_cast<float2*>(target) = make_float2(a, b);
    } else {
        target[0] = a;
        if (second) target[1] = b;
    }
}
__device__ __forceinline__ void store_copies(const LinearParams& p, int64_t at, float a, float b, bool second) {
    if (p.copies > 0) store_copy_pair(p.y_copy[0] + at, a, b, second);
    if (p.copies > 1) store_copy_pair(p.y_copy[1] + at, a, b, second);
    if (p.copies > 2) store_copy_pair(p.y_copy[2] + at, a, b, second);
    if (p.copies > 3) store_copy_pair(p.y_copy[3] + at, a, b, second);
    if (p.copies > 4) store_copy_pair(p.y_copy[4] + at, a, b, second);
    if (p.copies > 5) store_copy_pair(p.y_copy[5] + at, a, b, second);
    if (p.copies > 6) store_copy_pair(p.y_copy[6] + at, a, b, second);
}
// The same for four adjacent features on a 16-byte boundary.
__device__ __forceinline__ void store_copies(const LinearParams& p, int64_t at, const float4& v) {
    if (p.copies > 0) *reinterpret_cast<float4*>(p.y_copy[0] + at) = v;
    if (p.copies > 1) *reinterpret_cast<float4*>(p.y_copy[1] + at) = v;
    if (p.copies > 2) *reinterpret_cast<float4*>(p.y_copy[2] + at) = v;
    if (p.copies > 3) *reinterpret_cast<float4*>(p.y_copy[3] + at) = v;
    if (p.copies > 4) *reinterpret_cast<float4*>(p.y_copy[4] + at) = v;
    if (p.copies > 5) *reinterpret_cast<float4*>(p.y_copy[5] + at) = v;
    if (p.copies > 6) *reinterpret_cast<float4*>(p.y_copy[6] + at) = v;
}

// (value, index) ordering of the reference's argmax (src/kernels/cpu/reduction.cpp:128-151): a NaN beats every number,
// and among equals (or among NaNs) the lower index wins.
struct Candidate { float value; int32_t index; };
__device__ __forceinline__ bool preferred(const Candidate& a, const Candidate& b) {
    const bool an = a.value != a.value, bn = b.value != b.value;
    if (an || bn) return an && (!bn || a.index < b.index);
    return a.value > b.value || (a.value == b.value && a.index < b.index);
}
// The better of the two adjacent features (feature0, feature0 + 1) of one row; feature0 + 1 may lie past `out`.
__device__ __forceinline__ Candidate pair_candidate(int feature0, float a, float b, int out) {
    Candidate first{a, feature0};
    const Candidate second{b, feature0 + 1};
    if (feature0 + 1 < out && preferred(second, first)) first = second;
    return first;
}

// Adapter delta of the feature pair (local, local + 1) of region q (0) or v (2) for activation row `row`, before the
// alpha / rank scale: up(down(x)), the products added in index order (src/nn/decoder.cpp:26-28).
__device__ __forceinline__ void lora_pair_delta(const LinearParams& p, int row, int region, int local, float& da, float& db) {
    // LoRALinear::forward: base + up(down(x)) * f32(alpha/rank)
    const float* low = p.low + static_cast<int64_t>(row) * 2 * p.lora_rank + (region == 2 ? p.lora_rank : 0);
    const void* up = region == 0 ? p.q_up : p.v_up;
    da = 0.0f; db = 0.0f;
    if (p.weight_dtype == B200_BF16 && (p.lora_rank & 7) == 0) {
        // 16-byte loads: eight up-projection weights of each feature and eight low-rank activations per step; the
        // products are added in the same order as the scalar loop below (j ascending)
        const uint4* ua = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(up) + static_cast<int64_t>(local) * p.lora_rank);
        const uint4* ub = ua + (p.lora_rank >> 3);
        const float4* lv = reinterpret_cast<const float4*>(low);
        for (int j = 0; j < (p.lora_rank >> 3); ++j) {
            const uint4 wa = __ldg(ua + j), wb = __ldg(ub + j);
            const float4 l0 = __ldg(lv + 2 * j), l1 = __ldg(lv + 2 * j + 1);
            const float l[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
            const uint32_t pa[4] = {wa.x, wa.y, wa.z, wa.w}, pb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                da = __fadd_rn(da, __fmul_rn(l[2 * i], __uint_as_float(pa[i] << 16)));
                db = __fadd_rn(db, __fmul_rn(l[2 * i], __uint_as_float(pb[i] << 16)));
                da = __fadd_rn(da, __fmul_rn(l[2 * i + 1], __uint_as_float(pa[i] & 0xffff0000u)));
                db = __fadd_rn(db, __fmul_rn(l[2 * i + 1], __uint_as_float(pb[i] & 0xffff0000u)));
            }
        }
    } else
    for (int j = 0; j < p.lora_rank; ++j) {
        const int64_t at = static_cast<int64_t>(local) * p.lora_rank + j;
        const float ua = p.weight_dtype == B200_BF16 ? load_as_f32(static_cast<const __nv_bfloat16*>(up), at)
                                                   : load_as_f32(static_cast<const float*>(up), at);
        const float ub = p.weight_dtype == B200_BF16 ? load_as_f32(static_cast<const __nv_bfloat16*>(up), at + p.lora_rank)
                                                   : load_as_f32(static_cast<const float*>(up), at + p.lora_rank);
        const float lj = __ldg(low + j);
        da = __fadd_rn(da, __fmul_rn(lj, ua));
        db = __fadd_rn(db, __fmul_rn(lj, ub));
    }
}

// Finishes one pair of adjacent output features (feature0 even) of activation row `row`.
//   store | residual add (src/nn/decoder.cpp:104-105) | SiLU(gate)*up on interleaved rows (src/nn/decoder.cpp:16) |
//   q|k|v: adapter delta (src/nn/decoder.cpp:26-28), adjacent-pair RoPE (src/ops/contraction.cpp:44-49), q store,
//   k/v append to the paged cache (src/nn/kv_cache.cpp:24-28)
//   `place` (optional, q|k|v only): the row's position and physical cache page, looked up once per row by the caller
//   (x = position, y = page) instead of once per feature pair here.
template <int EPI>
__device__ __forceinline__ void linear_epilogue(const LinearParams& p, int row, int feature0, float& a, float& b, const int2* place = nullptr,
                                                bool store = true) {
    const bool second = feature0 + 1 < p.out;
    if constexpr (EPI == B200_EPI_STORE) {
        p.y[static_cast<int64_t>(row) * p.out + feature0] = a;
        if (second) p.y[static_cast<int64_t>(row) * p.out + feature0 + 1] = b;
        store_copies(p, static_cast<int64_t>(row) * p.out + feature0, a, b, second);
    } else if constexpr (EPI == B200_EPI_RESIDUAL) {
        const int64_t at = static_cast<int64_t>(row) * p.out + feature0;
        a = __fadd_rn(p.residual[at], a);
        b = second ? __fadd_rn(p.residual[at + 1], b) : 0.0f;
        p.y[at] = a;
        if (second) p.y[at + 1] = b;
        store_copies(p, at, a, b, second);
    } else if constexpr (EPI == B200_EPI_SWIGLU) {
        // rows 2j (gate_j) and 2j+1 (up_j) of the interleaved weight
        a = __fmul_rn(p.x_hi ? silu_fast(a) : silu_reference(a), b);   // shadow input = bf16 model: see silu_fast
        if (p.y) p.y[static_cast<int64_t>(row) * (p.out >> 1) + (feature0 >> 1)] = a;
    } else if constexpr (EPI == B200_EPI_ARGMAX) {
        // nothing is stored: the kernels reduce the pairs of a tile to one candidate per row themselves
    } else {
        const int D = p.heads * p.head_dim, KV = p.kv_heads * p.head_dim;
        const int sequence = row / p.tokens_per_sequence;
        const int position = place ? place->x : __ldg(p.kv.lengths + sequence) + row % p.tokens_per_sequence;
        int region = 0, local = feature0;  // 0 = q, 1 = k, 2 = v
        if (local >= D) { region = 1; local -= D; }
        if (region == 1 && local >= KV) { region = 2; local -= KV; }
        if (p.lora_rank > 0 && region != 1) {
            float da, db;
            lora_pair_delta(p, row, region, local, da, db);
            a = __fadd_rn(a, __fmul_rn(da, p.lora_scale));
            b = __fadd_rn(b, __fmul_rn(db, p.lora_scale));
        }
        const int head = local / p.head_dim, d = local % p.head_dim;
        // (unsigned comparison: a warm-up pass may hand in a position that nobody has written yet)
        if (region != 2 && static_cast<unsigned>(position) < static_cast<unsigned>(p.context)) {
            // adjacent-pair rotation, each product rounded before the add (src/ops/contraction.cpp:44-49)
            const float c = __ldg(p.cosine + static_cast<int64_t>(position) * (p.head_dim >> 1) + (d >> 1));
            const float s = __ldg(p.sine + static_cast<int64_t>(position) * (p.head_dim >> 1) + (d >> 1));
            const float even = a, odd = b;
            a = __fsub_rn(__fmul_rn(even, c), __fmul_rn(odd, s));
            b = __fadd_rn(__fmul_rn(even, s), __fmul_rn(odd, c));
        }
        if (!store) {
            // warm-up pass of the caller: everything above has run, nothing is written
        } else if (region == 0) {
            float* q = p.q_out + static_cast<int64_t>(row) * D + local;
            q[0] = a;
            q[1] = b;
        } else if (place) {
            kv_store_pair_at(p.kv, region - 1, place->y, position, head, d, a, b);
        } else {
            kv_store_pair(p.kv, region - 1, sequence, position, head, d, a, b);
        }
    }
}

// Tensor-core streaming kernel for bf16 weights (linear_stream.cu); returns B200_UNSUPPORTED when the shape is
// outside what it handles, in which case the caller uses the CUDA-core kernel.
int launch_linear_stream(const LinearParams& p, int epilogue, cudaStream_t stream);
// Number of per-row sum-of-squares partials a residual-epilogue shadow call with these sizes writes (0: unsupported).
int linear_stream_parts(int rows, int in, int out);
// Number of per-row candidate slices the argmax epilogue of a shadow call with these sizes writes (0: unsupported).
int linear_argmax_parts(int rows, int in, int out);
// tcgen05 GEMM for many rows (linear_gemm.cu): shadow input only; B200_UNSUPPORTED otherwise.
int launch_linear_gemm(const LinearParams& p, int epilogue, cudaStream_t stream);
int linear_gemm_parts(int rows, int in, int out);
// Row count from which the dense tensor-core kernel replaces the streaming one.
constexpr int kGemmRows = 17;
// Decode batches on the tensor cores with the weights as the streamed operand (linear_decode.cu): up to 256 rows.
struct DecodeShape {
    int tiles, split, ctas, stages, stage_bytes, n_pad, n_alloc, tmem_columns, body_bytes, smem_bytes, token_tile, token_tiles;
};
DecodeShape linear_decode_shape(int rows, int in, int out, bool two_planes, int sms);
bool linear_decode_takes(int rows);
int linear_decode_parts(int rows, int in, int out);
int launch_linear_decode(const LinearParams& p, int epilogue, cudaStream_t stream);

}  // namespace b200
