/*
 * decoder_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C, single-threaded restatement of the arithmetic that the Ctorch reference performs on its CPU
 * path for the GQA decoder token loop.  Parity tests compare the CUDA kernels with this file; nothing in the
 * shipped library links, loads or calls it.  Every function names the reference source it follows
 * (paths are relative to the reference project root).
 *
 * Pinning: the reference ships no golden vectors for this path (its tests pin cached == uncached
 * self-consistency only), so this restatement is pinned against the reference itself: the unmodified
 * reference CPU sources are compiled by oracle/Makefile into oracle/_ref/ and
 * tests/test_oracle_vs_reference.py requires BIT-EXACT agreement of logits, features and token streams;
 * tests/golden/ holds committed vectors produced by that reference build for machines without the reference.
 *
 * Arithmetic rules restated (the order of roundings is part of the contract):
 *   - Linear: y[r,o] = sum_k x[r,k] * W[o,k], f32, strictly sequential in k, separate multiply and add
 *     (src/kernels/cpu/matmul.h:10-22; 16-bit weights are widened to f32 first, src/kernels/cpu/matmul.cpp:28-31).
 *   - RMSNorm: sum of squares, 1/sqrt(mean+eps) and the weight product in f64, one rounding to f32
 *     (src/kernels/cpu/normalization.cpp:39-51, src/kernels/cpu/moments.h:11-24).
 *   - RoPE: table angle[p,i] = f32(p) * expf(f32(i) * f32(-2 ln(base)/hd)), cosf/sinf of the f32 angle
 *     (src/nn/decoder.cpp:38-52); adjacent pairs, each product rounded before the sub/add
 *     (src/ops/contraction.cpp:44-49).
 *   - Attention: scores by sequential-k dot, one multiply by f32(1/sqrt(hd)), causal -inf mask only when the
 *     chunk's first query cannot see every key, softmax = max, expf(x-max), running f32 sum, divide
 *     (src/ops/attention.cpp:65-95, src/kernels/cpu/reduction.cpp:155-203), P.V sequential over keys.
 *   - SiLU: v * sigmoid(v), sigmoid through expf(-|v|) in two branches (src/kernels/cpu/pointwise.cpp:31-34,57).
 *   - Argmax: strict '>' keeps the first maximum, the first NaN wins (src/kernels/cpu/reduction.cpp:128-151).
 *
 * Build: gcc -std=c17 -O2 -ffp-contract=off (see oracle/Makefile).  Contraction must stay off.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_F32 0
#define ORACLE_BF16 5

typedef struct oracle_config {
    int64_t vocab, d_model, layers, heads, kv_heads, hidden, context;
    int32_t weight_dtype; /* ORACLE_F32 or ORACLE_BF16 (same codes as dl_dtype) */
    int32_t tied;         /* 1: logits use the embedding table (examples/decoder_model.h:13-18) */
    double eps, rope_base;
    int64_t lora_rank;    /* 0: no adapter; else rank of the q and v adapters */
    double lora_alpha;
} oracle_config;

typedef struct oracle_layer {
    float *wq, *wk, *wv, *wo, *wg, *wu, *wd, *norm1, *norm2;
    float *q_down, *q_up, *v_down, *v_up; /* LoRA, NULL when rank == 0 */
} oracle_layer;

typedef struct oracle_decoder {
    oracle_config cfg;
    float *embedding, *final_norm, *output; /* output == embedding when tied */
    oracle_layer* layer;
    float *cosine, *sine; /* [context, hd/2] */
} oracle_decoder;

typedef struct oracle_cache {
    int64_t layers, batch, kv_heads, capacity, head_dim, length;
    float **key, **value; /* per layer [batch, kv_heads, capacity, head_dim], allocated at first append */
} oracle_cache;

static _Thread_local char oracle_error[256];
const char* oracle_last_error(void) { return oracle_error; }
static int fail(const char* text) { snprintf(oracle_error, sizeof oracle_error, "%s", text); return 1; }

/* bf16 -> f32 widening is exact (include/dl/half.h). */
static float widen_bf16(uint16_t bits) {
    uint32_t word = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &word, sizeof value);
    return value;
}
/* f32 -> bf16 round-to-nearest-even (include/dl/half.h:43-47); NaN keeps a quiet payload. */
uint16_t oracle_round_bf16(float value) {
    uint32_t word;
    memcpy(&word, &value, sizeof word);
    if ((word & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((word >> 16) | 0x0040u);
    word += 0x7fffu + ((word >> 16) & 1u);
    return (uint16_t)(word >> 16);
}

static float* widen(const void* source, int64_t count, int32_t dtype) {
    float* result = (float*)malloc(sizeof(float) * (size_t)(count > 0 ? count : 1));
    if (!result) return NULL;
    if (dtype == ORACLE_BF16) {
        const uint16_t* bits = (const uint16_t*)source;
        for (int64_t i = 0; i < count; ++i) result[i] = widen_bf16(bits[i]);
    } else {
        memcpy(result, source, sizeof(float) * (size_t)count);
    }
    return result;
}

/* ---- stand-alone operators (also exported for kernel-level parity tests) ------------------------------- */

/* src/nn/decoder.cpp:38-52 (rotary_angles + cos/sin buffers), f32 throughout for f32 and bf16 models. */
void oracle_rope_tables(int64_t head_dim, int64_t capacity, double base, float* cosine, float* sine) {
    const int64_t half = head_dim / 2;
    const float factor = (float)(-2.0 * log(base) / (double)head_dim);
    for (int64_t p = 0; p < capacity; ++p) {
        for (int64_t i = 0; i < half; ++i) {
            const float frequency = expf((float)i * factor);
            const float angle = (float)p * frequency;
            cosine[p * half + i] = cosf(angle);
            sine[p * half + i] = sinf(angle);
        }
    }
}

/* src/kernels/cpu/normalization.cpp:21-56 with kind == rms (mean fixed at zero), f32 in, f32 out. */
void oracle_rms_norm(const float* x, const float* weight, int64_t rows, int64_t width, double eps, float* y) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* row = x + r * width;
        double squares = 0;
        for (int64_t c = 0; c < width; ++c) {
            const double value = (double)row[c];
            squares += value * value;
        }
        const double inverse_std = 1.0 / sqrt(squares / (double)width + eps);
        for (int64_t c = 0; c < width; ++c) {
            double value = (double)row[c] * inverse_std;
            if (weight) value *= weight[c];
            y[r * width + c] = (float)value;
        }
    }
}

/* src/kernels/cpu/matmul.h:10-22 as driven by numeric::linear (src/ops/numeric.cpp:199-209):
 * y[r,o] = sum over k in order of x[r,k] * w[o,k]; the accumulator starts at +0 and every step is a separate
 * f32 multiply followed by an f32 add. */
void oracle_linear(const float* x, const float* w, int64_t rows, int64_t in, int64_t out, float* y) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* a = x + r * in;
        for (int64_t o = 0; o < out; ++o) {
            const float* b = w + o * in;
            float sum = 0.0f;
            for (int64_t k = 0; k < in; ++k) {
                const float product = a[k] * b[k];
                sum = sum + product;
            }
            y[r * out + o] = sum;
        }
    }
}

/* src/kernels/cpu/pointwise.cpp:31-34,57 */
static float silu_value(float v) {
    const float e = expf(-fabsf(v));
    const float sigmoid = v >= 0.0f ? 1.0f / (1.0f + e) : e / (1.0f + e);
    return v * sigmoid;
}
void oracle_silu_mul(const float* gate, const float* up, int64_t count, float* y) {
    for (int64_t i = 0; i < count; ++i) {
        const float activated = silu_value(gate[i]);
        y[i] = activated * up[i];
    }
}

/* src/ops/contraction.cpp:44-49 on a [rows, heads, head_dim] block whose row r sits at position pos[r].
 * In place. */
static void rope_rows(float* x, int64_t rows, int64_t heads, int64_t head_dim, const int64_t* position,
                      const float* cosine, const float* sine) {
    const int64_t half = head_dim / 2;
    for (int64_t r = 0; r < rows; ++r) {
        const float* c = cosine + position[r] * half;
        const float* s = sine + position[r] * half;
        for (int64_t h = 0; h < heads; ++h) {
            float* v = x + (r * heads + h) * head_dim;
            for (int64_t i = 0; i < half; ++i) {
                const float even = v[2 * i], odd = v[2 * i + 1];
                const float ec = even * c[i], os = odd * s[i], es = even * s[i], oc = odd * c[i];
                v[2 * i] = ec - os;
                v[2 * i + 1] = es + oc;
            }
        }
    }
}
/* dl::rotary_embedding on [batch, heads, length, head_dim] with tables narrowed to [offset, offset+length). */
void oracle_rotary(const float* x, int64_t batch, int64_t heads, int64_t length, int64_t head_dim,
                   const float* cosine, const float* sine, int64_t offset, float* y) {
    const int64_t half = head_dim / 2;
    for (int64_t b = 0; b < batch * heads; ++b)
        for (int64_t l = 0; l < length; ++l) {
            const float* v = x + (b * length + l) * head_dim;
            float* o = y + (b * length + l) * head_dim;
            const float* c = cosine + (offset + l) * half;
            const float* s = sine + (offset + l) * half;
            for (int64_t i = 0; i < half; ++i) {
                const float even = v[2 * i], odd = v[2 * i + 1];
                const float ec = even * c[i], os = odd * s[i], es = even * s[i], oc = odd * c[i];
                o[2 * i] = ec - os;
                o[2 * i + 1] = es + oc;
            }
        }
}

/* One query row against `source` keys: src/ops/attention.cpp:65-95 + softmax src/kernels/cpu/reduction.cpp:155-203.
 * key/value rows are `stride` floats apart.  visible < 0: no mask.  Otherwise keys at index > visible are set
 * to -inf before the softmax, which then writes exact zeros for the trailing masked part. */
static void attend_row(const float* q, const float* key, const float* value, int64_t stride, int64_t source,
                       int64_t head_dim, float scale, int64_t visible, float* scores, float* out) {
    for (int64_t s = 0; s < source; ++s) {
        const float* k = key + s * stride;
        float sum = 0.0f;
        for (int64_t d = 0; d < head_dim; ++d) {
            const float product = q[d] * k[d];
            sum = sum + product;
        }
        scores[s] = sum * scale;
        if (visible >= 0 && s > visible) scores[s] = -INFINITY;
    }
    float maximum = -INFINITY;
    for (int64_t s = 0; s < source; ++s) {
        const float v = scores[s];
        maximum = isnan(v) ? v : (maximum < v ? v : maximum);
    }
    int64_t active = source;
    if (isfinite(maximum))
        while (active > 0 && scores[active - 1] == -INFINITY) --active;
    float total = 0.0f;
    for (int64_t s = 0; s < active; ++s) {
        const float e = expf(scores[s] - maximum);
        scores[s] = e;
        total += e;
    }
    for (int64_t s = 0; s < active; ++s) scores[s] /= total;
    for (int64_t s = active; s < source; ++s) scores[s] = 0.0f;
    for (int64_t d = 0; d < head_dim; ++d) out[d] = 0.0f;
    for (int64_t s = 0; s < source; ++s) {
        const float w = scores[s];
        const float* v = value + s * stride;
        for (int64_t d = 0; d < head_dim; ++d) {
            const float product = w * v[d];
            out[d] = out[d] + product;
        }
    }
}

/* dl::grouped_query_attention / detail::grouped_attention (src/ops/attention.cpp:155-188).
 * query [batch, heads, length, hd], key/value [batch, kv_heads, source, hd], out like query.
 * causal_offset < 0: unmasked.  Otherwise query row l sits at position causal_offset + l and the mask is
 * applied only when causal_offset < source - 1 (src/ops/attention.cpp:81). */
int oracle_gqa_attention(const float* query, const float* key, const float* value, int64_t batch, int64_t heads,
                         int64_t kv_heads, int64_t length, int64_t source, int64_t head_dim,
                         int64_t causal_offset, float* out) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return fail("query heads must be divisible by matching key/value heads");
    float* scores = (float*)malloc(sizeof(float) * (size_t)(source > 0 ? source : 1));
    if (!scores) return fail("out of memory");
    const float scale = (float)(1.0 / sqrt((double)head_dim));
    const int64_t group = heads / kv_heads;
    const int masked = causal_offset >= 0 && causal_offset < source - 1;
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t h = 0; h < heads; ++h)
            for (int64_t l = 0; l < length; ++l) {
                const int64_t kv = h / group;
                attend_row(query + ((b * heads + h) * length + l) * head_dim,
                           key + (b * kv_heads + kv) * source * head_dim,
                           value + (b * kv_heads + kv) * source * head_dim, head_dim, source, head_dim, scale,
                           masked ? causal_offset + l : -1, scores,
                           out + ((b * heads + h) * length + l) * head_dim);
            }
    free(scores);
    return 0;
}

/* src/kernels/cpu/reduction.cpp:128-151 along the last axis. */
void oracle_argmax(const float* x, int64_t rows, int64_t width, int64_t* index) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* row = x + r * width;
        float best = row[0];
        int64_t selected = 0;
        for (int64_t i = 1; i < width; ++i) {
            const float v = row[i];
            if (best == best && (v != v || v > best)) { best = v; selected = i; }
        }
        index[r] = selected;
    }
}

/* Temperature sampling of the sibling example (examples/text_generate.cpp:38-39): softmax(logits / temperature) with the
 * f32 softmax of src/kernels/cpu/reduction.cpp:155-203 (max, expf(v - max), running f32 sum in index order, divide), then
 * the categorical draw of std::discrete_distribution as libstdc++ documents it: probabilities normalised by their sum in
 * double, running sums with the last forced to one, and the first running sum greater than the uniform variate u
 * (std::upper_bound).  The caller supplies u in [0, 1), one per row. */
void oracle_sample(const float* x, int64_t rows, int64_t width, double temperature, const double* uniform, int64_t* index) {
    float* p = (float*)malloc(sizeof(float) * (size_t)width);
    const float t = (float)temperature;
    for (int64_t r = 0; r < rows; ++r) {
        const float* row = x + r * width;
        float maximum = -INFINITY;
        for (int64_t i = 0; i < width; ++i) {
            const float v = row[i] / t;
            p[i] = v;
            maximum = isnan(v) ? v : (maximum < v ? v : maximum);
        }
        float total = 0.0f;
        for (int64_t i = 0; i < width; ++i) {
            p[i] = expf(p[i] - maximum);
            total += p[i];
        }
        double sum = 0.0;
        for (int64_t i = 0; i < width; ++i) {
            p[i] /= total;
            sum += (double)p[i];
        }
        double running = 0.0;
        int64_t chosen = width - 1;
        for (int64_t i = 0; i < width; ++i) {
            running += (double)p[i] / sum;
            const double boundary = i == width - 1 ? 1.0 : running;
            if (boundary > uniform[r]) { chosen = i; break; }
        }
        index[r] = chosen;
    }
    free(p);
}

/* LoRALinear::forward (src/nn/decoder.cpp:26-28): base(x) + up(down(x)) * f32(alpha/rank). */
void oracle_lora_linear(const float* x, const float* w, const float* down, const float* up, int64_t rows,
                        int64_t in, int64_t out, int64_t rank, double alpha, float* y) {
    float* low = (float*)malloc(sizeof(float) * (size_t)(rows * rank));
    float* delta = (float*)malloc(sizeof(float) * (size_t)(rows * out));
    const float scale = (float)(alpha / (double)rank);
    oracle_linear(x, w, rows, in, out, y);
    oracle_linear(x, down, rows, in, rank, low);
    oracle_linear(low, up, rows, rank, out, delta);
    for (int64_t i = 0; i < rows * out; ++i) {
        const float scaled = delta[i] * scale;
        y[i] = y[i] + scaled;
    }
    free(low);
    free(delta);
}

/* LoRALinear::merged (src/nn/decoder.cpp:29-35): W + (up @ down) * scale in f32, rounded to W's dtype.
 * Weights here are already widened to f32; `round_to_bf16` re-applies the 16-bit rounding. */
void oracle_lora_merge(const float* w, const float* down, const float* up, int64_t in, int64_t out, int64_t rank,
                       double alpha, int32_t round_to_bf16, float* merged) {
    const float scale = (float)(alpha / (double)rank);
    for (int64_t o = 0; o < out; ++o)
        for (int64_t i = 0; i < in; ++i) {
            float sum = 0.0f;
            for (int64_t r = 0; r < rank; ++r) {
                const float product = up[o * rank + r] * down[r * in + i];
                sum = sum + product;
            }
            const float scaled = sum * scale;
            float value = w[o * in + i] + scaled;
            if (round_to_bf16) value = widen_bf16(oracle_round_bf16(value));
            merged[o * in + i] = value;
        }
}

/* ---- decoder object -------------------------------------------------------------------------------------- */

void oracle_decoder_release(oracle_decoder* model) {
    if (!model) return;
    if (model->layer) {
        for (int64_t i = 0; i < model->cfg.layers; ++i) {
            oracle_layer* l = &model->layer[i];
            free(l->wq); free(l->wk); free(l->wv); free(l->wo); free(l->wg); free(l->wu); free(l->wd);
            free(l->norm1); free(l->norm2); free(l->q_down); free(l->q_up); free(l->v_down); free(l->v_up);
        }
        free(model->layer);
    }
    if (model->output != model->embedding) free(model->output);
    free(model->embedding); free(model->final_norm); free(model->cosine); free(model->sine);
    free(model);
}

/* tensors, all in cfg.weight_dtype, in this order:
 *   [0] tokens.weight [V,D]
 *   per layer i (9 entries): query [D,D], key [Hkv*hd,D], value [Hkv*hd,D], output [D,D], gate [F,D], up [F,D],
 *                            down [D,F], attention_norm [D], feedforward_norm [D]
 *   then normalization [D], then (only when !tied) output.weight [V,D].
 * lora (NULL when lora_rank == 0), per layer 4 entries: q.down [r,D], q.up [D,r], v.down [r,D], v.up [Hkv*hd,r].
 * Names follow the reference state_dict (src/nn/decoder.cpp:66-70,92-96,110-114). */
oracle_decoder* oracle_decoder_create(const oracle_config* cfg, const void* const* tensors, const void* const* lora) {
    if (cfg->layers <= 0) { fail("decoder requires at least one layer"); return NULL; }
    if (cfg->heads <= 0 || cfg->kv_heads <= 0 || cfg->d_model <= 0 || cfg->d_model % cfg->heads || cfg->heads % cfg->kv_heads) {
        fail("attention dimensions and query/key head counts must divide evenly");
        return NULL;
    }
    const int64_t hd = cfg->d_model / cfg->heads;
    if (hd % 2 || cfg->context <= 0 || cfg->rope_base <= 0) {
        fail("RoPE needs an even positive dimension, positive capacity and base");
        return NULL;
    }
    oracle_decoder* model = (oracle_decoder*)calloc(1, sizeof *model);
    model->cfg = *cfg;
    const int32_t t = cfg->weight_dtype;
    const int64_t D = cfg->d_model, F = cfg->hidden, KV = cfg->kv_heads * hd, V = cfg->vocab;
    int64_t next = 0;
    model->embedding = widen(tensors[next++], V * D, t);
    model->layer = (oracle_layer*)calloc((size_t)cfg->layers, sizeof(oracle_layer));
    for (int64_t i = 0; i < cfg->layers; ++i) {
        oracle_layer* l = &model->layer[i];
        l->wq = widen(tensors[next++], D * D, t);
        l->wk = widen(tensors[next++], KV * D, t);
        l->wv = widen(tensors[next++], KV * D, t);
        l->wo = widen(tensors[next++], D * D, t);
        l->wg = widen(tensors[next++], F * D, t);
        l->wu = widen(tensors[next++], F * D, t);
        l->wd = widen(tensors[next++], D * F, t);
        l->norm1 = widen(tensors[next++], D, t);
        l->norm2 = widen(tensors[next++], D, t);
        if (cfg->lora_rank > 0 && lora) {
            const int64_t r = cfg->lora_rank;
            l->q_down = widen(lora[i * 4 + 0], r * D, t);
            l->q_up = widen(lora[i * 4 + 1], D * r, t);
            l->v_down = widen(lora[i * 4 + 2], r * D, t);
            l->v_up = widen(lora[i * 4 + 3], KV * r, t);
        }
    }
    model->final_norm = widen(tensors[next++], D, t);
    model->output = cfg->tied ? model->embedding : widen(tensors[next++], V * D, t);
    model->cosine = (float*)malloc(sizeof(float) * (size_t)(cfg->context * (hd / 2)));
    model->sine = (float*)malloc(sizeof(float) * (size_t)(cfg->context * (hd / 2)));
    oracle_rope_tables(hd, cfg->context, cfg->rope_base, model->cosine, model->sine);
    return model;
}

const float* oracle_decoder_cosine(const oracle_decoder* model) { return model->cosine; }
const float* oracle_decoder_sine(const oracle_decoder* model) { return model->sine; }

/* TransformerDecoder::make_cache (src/nn/decoder.cpp:121-126): one empty cache of `context` capacity per layer. */
oracle_cache* oracle_cache_create(const oracle_decoder* model) {
    oracle_cache* cache = (oracle_cache*)calloc(1, sizeof *cache);
    cache->layers = model->cfg.layers;
    cache->kv_heads = model->cfg.kv_heads;
    cache->capacity = model->cfg.context;
    cache->head_dim = model->cfg.d_model / model->cfg.heads;
    cache->key = (float**)calloc((size_t)cache->layers, sizeof(float*));
    cache->value = (float**)calloc((size_t)cache->layers, sizeof(float*));
    return cache;
}
void oracle_cache_release(oracle_cache* cache) {
    if (!cache) return;
    for (int64_t i = 0; i < cache->layers; ++i) { free(cache->key[i]); free(cache->value[i]); }
    free(cache->key); free(cache->value); free(cache);
}
int64_t oracle_cache_length(const oracle_cache* cache) { return cache->length; }
void oracle_cache_clear(oracle_cache* cache) { cache->length = 0; }
/* KVCache::truncate (src/nn/kv_cache.cpp:39-42) */
int oracle_cache_truncate(oracle_cache* cache, int64_t length) {
    if (length < 0 || length > cache->length) return fail("KV cache truncation must keep an existing prefix");
    cache->length = length;
    return 0;
}
/* Read-only view for tests: layer's K or V storage [batch, kv_heads, capacity, head_dim]. */
const float* oracle_cache_data(const oracle_cache* cache, int64_t layer, int32_t which) {
    return which ? cache->value[layer] : cache->key[layer];
}

/* Projection with optional adapter (src/nn/decoder.cpp:26-28, 80-85). */
static void project(const float* x, const float* w, const float* down, const float* up, int64_t rows, int64_t in,
                    int64_t out, const oracle_config* cfg, float* y) {
    if (down) oracle_lora_linear(x, w, down, up, rows, in, out, cfg->lora_rank, cfg->lora_alpha, y);
    else oracle_linear(x, w, rows, in, out, y);
}

/* TransformerDecoder::decode (src/nn/decoder.cpp:127-142) on features: x [batch, length, D] -> out [batch, length, D].
 * Transactional: on failure the cache keeps its previous length. */
int oracle_decoder_decode(const oracle_decoder* model, oracle_cache* cache, const float* x, int64_t batch,
                          int64_t length, float* out) {
    const oracle_config* cfg = &model->cfg;
    const int64_t D = cfg->d_model, F = cfg->hidden, H = cfg->heads, HK = cfg->kv_heads, hd = D / H, KV = HK * hd;
    const int64_t offset = cache->length, rows = batch * length, source = offset + length, cap = cache->capacity;
    if (cache->layers != cfg->layers) return fail("decoder requires one cache per layer");
    if (length > cap - offset) return fail("KV cache append exceeds capacity or has unequal key/value lengths");
    if (cache->key[0] && cache->batch != batch) return fail("KV cache shape, dtype or device changed");
    if (!cache->key[0]) {
        cache->batch = batch;
        for (int64_t i = 0; i < cfg->layers; ++i) {
            cache->key[i] = (float*)calloc((size_t)(batch * HK * cap * hd), sizeof(float));
            cache->value[i] = (float*)calloc((size_t)(batch * HK * cap * hd), sizeof(float));
        }
    }
    float* h = (float*)malloc(sizeof(float) * (size_t)(rows * D));
    float* n = (float*)malloc(sizeof(float) * (size_t)(rows * D));
    float* q = (float*)malloc(sizeof(float) * (size_t)(rows * D));
    float* k = (float*)malloc(sizeof(float) * (size_t)(rows * KV));
    float* v = (float*)malloc(sizeof(float) * (size_t)(rows * KV));
    float* a = (float*)malloc(sizeof(float) * (size_t)(rows * D));
    float* o = (float*)malloc(sizeof(float) * (size_t)(rows * D));
    float* g = (float*)malloc(sizeof(float) * (size_t)(rows * F));
    float* u = (float*)malloc(sizeof(float) * (size_t)(rows * F));
    float* scores = (float*)malloc(sizeof(float) * (size_t)source);
    int64_t* position = (int64_t*)malloc(sizeof(int64_t) * (size_t)rows);
    for (int64_t r = 0; r < rows; ++r) position[r] = offset + r % length;
    const float scale = (float)(1.0 / sqrt((double)hd));
    const int64_t group = H / HK;
    const int masked = offset < source - 1; /* src/ops/attention.cpp:81 */
    memcpy(h, x, sizeof(float) * (size_t)(rows * D));
    for (int64_t i = 0; i < cfg->layers; ++i) {
        const oracle_layer* l = &model->layer[i];
        /* TransformerDecoderLayer::decode, src/nn/decoder.cpp:102-106 */
        oracle_rms_norm(h, l->norm1, rows, D, cfg->eps, n);
        /* GroupedQueryAttention::run, src/nn/decoder.cpp:77-89 */
        project(n, l->wq, l->q_down, l->q_up, rows, D, D, cfg, q);
        project(n, l->wk, NULL, NULL, rows, D, KV, cfg, k);
        project(n, l->wv, l->v_down, l->v_up, rows, D, KV, cfg, v);
        rope_rows(q, rows, H, hd, position, model->cosine, model->sine);
        rope_rows(k, rows, HK, hd, position, model->cosine, model->sine);
        /* KVCache::append, src/nn/kv_cache.cpp:12-33 */
        for (int64_t b = 0; b < batch; ++b)
            for (int64_t t = 0; t < length; ++t)
                for (int64_t kh = 0; kh < HK; ++kh) {
                    const int64_t target = ((b * HK + kh) * cap + offset + t) * hd;
                    memcpy(cache->key[i] + target, k + ((b * length + t) * HK + kh) * hd, sizeof(float) * (size_t)hd);
                    memcpy(cache->value[i] + target, v + ((b * length + t) * HK + kh) * hd, sizeof(float) * (size_t)hd);
                }
        for (int64_t b = 0; b < batch; ++b)
            for (int64_t t = 0; t < length; ++t)
                for (int64_t qh = 0; qh < H; ++qh) {
                    const int64_t kh = qh / group, row = b * length + t;
                    attend_row(q + (row * H + qh) * hd, cache->key[i] + (b * HK + kh) * cap * hd,
                               cache->value[i] + (b * HK + kh) * cap * hd, hd, source, hd, scale,
                               masked ? offset + t : -1, scores, a + (row * H + qh) * hd);
                }
        oracle_linear(a, l->wo, rows, D, D, o);
        for (int64_t j = 0; j < rows * D; ++j) h[j] = h[j] + o[j];
        oracle_rms_norm(h, l->norm2, rows, D, cfg->eps, n);
        /* SwiGLU::forward, src/nn/decoder.cpp:11-16 */
        oracle_linear(n, l->wg, rows, D, F, g);
        oracle_linear(n, l->wu, rows, D, F, u);
        oracle_silu_mul(g, u, rows * F, g);
        oracle_linear(g, l->wd, rows, F, D, o);
        for (int64_t j = 0; j < rows * D; ++j) h[j] = h[j] + o[j];
    }
    oracle_rms_norm(h, model->final_norm, rows, D, cfg->eps, out);
    cache->length = source;
    free(h); free(n); free(q); free(k); free(v); free(a); free(o); free(g); free(u); free(scores); free(position);
    return 0;
}

/* ByteDecoder::decode (examples/decoder_model.h:31-34): embedding -> decoder -> tied/untied output Linear.
 * ids [batch, length] -> logits [batch, length, vocab]. */
int oracle_model_decode(const oracle_decoder* model, oracle_cache* cache, const int64_t* ids, int64_t batch,
                        int64_t length, float* logits) {
    const int64_t D = model->cfg.d_model, V = model->cfg.vocab, rows = batch * length;
    float* x = (float*)malloc(sizeof(float) * (size_t)(rows * D));
    float* y = (float*)malloc(sizeof(float) * (size_t)(rows * D));
    for (int64_t r = 0; r < rows; ++r) {
        if (ids[r] < 0 || ids[r] >= V) { free(x); free(y); return fail("embedding index out of range"); }
        memcpy(x + r * D, model->embedding + ids[r] * D, sizeof(float) * (size_t)D);
    }
    const int status = oracle_decoder_decode(model, cache, x, batch, length, y);
    if (!status) oracle_linear(y, model->output, rows, D, V, logits);
    free(x); free(y);
    return status;
}

/* The greedy loop of examples/decoder_generate.cpp:20-31 for a batch: prefill the whole prompt, take the last
 * position, argmax (first maximum), feed the token back.  tokens [batch, steps]; logits (optional)
 * [steps, batch, vocab] receives the logits each token was chosen from. */
int oracle_generate(const oracle_decoder* model, oracle_cache* cache, const int64_t* prompt, int64_t batch,
                    int64_t prompt_length, int64_t steps, int64_t* tokens, float* logits) {
    const int64_t V = model->cfg.vocab;
    if (prompt_length <= 0 || steps < 0 || cache->length + prompt_length + (steps > 0 ? steps - 1 : 0) > cache->capacity)
        return fail("prompt and generated tokens must fit the context");
    float* full = (float*)malloc(sizeof(float) * (size_t)(batch * prompt_length * V));
    float* last = (float*)malloc(sizeof(float) * (size_t)(batch * V));
    int64_t* next = (int64_t*)malloc(sizeof(int64_t) * (size_t)batch);
    int status = 0;
    for (int64_t step = 0; step < steps && !status; ++step) {
        if (step == 0) {
            status = oracle_model_decode(model, cache, prompt, batch, prompt_length, full);
            for (int64_t b = 0; b < batch && !status; ++b)
                memcpy(last + b * V, full + ((b + 1) * prompt_length - 1) * V, sizeof(float) * (size_t)V);
        } else {
            status = oracle_model_decode(model, cache, next, batch, 1, last);
        }
        if (status) break;
        oracle_argmax(last, batch, V, next);
        for (int64_t b = 0; b < batch; ++b) tokens[b * steps + step] = next[b];
        if (logits) memcpy(logits + step * batch * V, last, sizeof(float) * (size_t)(batch * V));
    }
    free(full); free(last); free(next);
    return status;
}
