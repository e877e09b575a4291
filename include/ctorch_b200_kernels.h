/*
 * ctorch_b200_kernels.h -- kernel-level C ABI of the B200 (sm_100a) decoder token loop.
 *
 * Plain pointers and sizes only.  This is the layer a Ctorch maintainer binds from src/nn (decoder.cpp,
 * kv_cache.cpp) in place of the per-op numeric:: dispatch (src/ops/numeric.cpp, src/backends/backend.h:21-108):
 * every entry point states which reference functions it replaces.  All pointers are DEVICE pointers unless a
 * comment says "host".  `stream` is a cudaStream_t passed as void*.  Every call only enqueues work; it returns
 * B200_OK or a negative B200_* code / positive cudaError_t, and never falls back to a CPU path.
 *
 * dtype codes are the reference's dl_dtype values (include/dl/c_api.h:34): 0 = f32, 5 = bf16.
 */
#ifndef CTORCH_B200_KERNELS_H
#define CTORCH_B200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

enum { B200_OK = 0, B200_BAD_ARGUMENT = -1, B200_UNSUPPORTED = -2, B200_NO_DEVICE = -3, B200_DEVICE_TIMEOUT = -4 };
enum { B200_F32 = 0, B200_BF16 = 5 };

/* Largest number of activation rows one skinny-linear launch keeps in registers; callers with more rows
 * (prefill chunks) are tiled over rows inside b200_linear. */
#define B200_LINEAR_ROW_TILE 8

/* Last error text of the calling thread (argument checks, CUDA errors). */
B200_API const char* b200_last_error(void);

/* ---- paged, head-major KV storage -------------------------------------------------------------------------
 * Replaces the dense [batch, kv_heads, capacity, head_dim] buffers of dl::nn::KVCache
 * (include/dl/decoder.h:45-62, src/nn/kv_cache.cpp:9-43).  One object holds the K pool and the V pool of ONE
 * layer, each laid out [page][kv_head][page_size][head_dim] (a (page, head) tile is contiguous, which is what
 * the TMA box of the attention kernel fetches), a page table [sequences][pages_per_sequence] (int32 page ids)
 * and the per-sequence cached length [sequences] (int32), all in device memory.  The object also owns the two
 * TMA tensor maps.  Lengths are per sequence; the reference behaviour (one length for the batch) is the case
 * where all entries are equal. */
typedef struct b200_kv_cache b200_kv_cache;

B200_API int b200_kv_cache_create(int32_t device, int32_t dtype, int32_t sequences, int32_t kv_heads,
                                  int32_t head_dim, int32_t capacity, int32_t page_size, b200_kv_cache** out);
B200_API void b200_kv_cache_release(b200_kv_cache* cache);
/* Host-side setters/getters: enqueue small copies on `stream`. */
B200_API int b200_kv_cache_set_lengths(b200_kv_cache* cache, const int32_t* host_lengths, void* stream);
B200_API int b200_kv_cache_fill_lengths(b200_kv_cache* cache, int32_t length, void* stream);
B200_API int b200_kv_cache_set_page_table(b200_kv_cache* cache, const int32_t* host_table, void* stream);
B200_API int32_t* b200_kv_cache_lengths(b200_kv_cache* cache);        /* device [sequences] */
B200_API int32_t* b200_kv_cache_page_table(b200_kv_cache* cache);     /* device [sequences][pages_per_sequence] */
B200_API void* b200_kv_cache_pool(b200_kv_cache* cache, int32_t which); /* 0 = K, 1 = V */
B200_API int32_t b200_kv_cache_pages_per_sequence(const b200_kv_cache* cache);
B200_API int32_t b200_kv_cache_page_size(const b200_kv_cache* cache);
B200_API size_t b200_kv_cache_pool_bytes(const b200_kv_cache* cache);
/* lengths[s] += delta for every sequence of every listed cache (the commit of KVCache::append's length_ += count,
 * src/nn/kv_cache.cpp:32). `caches` is a host array. */
B200_API int b200_kv_cache_advance(b200_kv_cache* const* caches, int32_t count, int32_t delta, void* stream);
/* Writes rows [0, length) of every sequence as dense f32 [sequences, kv_heads, length, head_dim]
 * (KVCache::key()/value(), src/nn/kv_cache.cpp:34-38). */
B200_API int b200_kv_cache_gather(const b200_kv_cache* cache, int32_t which, int32_t length, float* out, void* stream);
/* KVCache::append (src/nn/kv_cache.cpp:12-33) for stand-alone use: key/value f32 [sequences, kv_heads, count, head_dim]
 * written at positions lengths[s] .. lengths[s]+count-1 (lengths are NOT advanced). */
B200_API int b200_kv_cache_append(b200_kv_cache* cache, const float* key, const float* value, int32_t count, void* stream);

/* ---- operators ------------------------------------------------------------------------------------------ */

/* dl::embedding (src/ops/indexing.cpp:38-42): out[r,:] = f32(table[ids[r],:]).  ids are int64. */
B200_API int b200_embedding(const void* table, int32_t table_dtype, const int64_t* ids, int64_t rows, int64_t vocab,
                            int64_t width, float* out, void* stream);

/* dl::rms_norm (src/ops/normalization.cpp:136-142; CPU arithmetic src/kernels/cpu/normalization.cpp:39-51):
 * sum of squares, 1/sqrt(mean+eps) and the weight product in f64, one rounding to f32. weight may be NULL. */
B200_API int b200_rms_norm(const float* x, const void* weight, int32_t weight_dtype, int64_t rows, int64_t width,
                           double eps, float* out, void* stream);

/* What a skinny linear does with each finished output value. */
typedef enum b200_epilogue {
    B200_EPI_STORE = 0,     /* y[r,o] = acc                                   (dl::linear, src/ops/matmul.cpp:35-67) */
    B200_EPI_RESIDUAL = 1,  /* y[r,o] = residual[r,o] + acc                   (src/nn/decoder.cpp:104-105) */
    B200_EPI_SWIGLU = 2,    /* weight rows interleaved gate_j, up_j: y[r,j] = silu(gate) * up   (src/nn/decoder.cpp:16) */
    B200_EPI_QKV = 3,       /* fused q|k|v rows: RoPE on q and k, q stored, k and v appended to the KV cache
                               (src/nn/decoder.cpp:80-86) */
    B200_EPI_ARGMAX = 4     /* shadow linears only: nothing is stored; every feature tile leaves, per row, its best value
                               and the index of it under the reference's rule (first maximum, first NaN wins:
                               src/kernels/cpu/reduction.cpp:128-151).  b200_argmax_finish merges the tiles.  This is
                               logits + greedy choice without materialising the logits
                               (examples/decoder_generate.cpp:27-30). */
} b200_epilogue;

/* Extra operands of B200_EPI_QKV. */
typedef struct b200_qkv_args {
    int32_t heads, kv_heads, head_dim;
    int32_t tokens_per_sequence;  /* L: row r belongs to sequence r / L at position lengths[r / L] + r % L */
    const float* cosine;          /* [context, head_dim/2] f32 tables (src/nn/decoder.cpp:49-52) */
    const float* sine;
    int32_t context;
    b200_kv_cache* cache;
    float* q_out;                 /* [rows, heads, head_dim] f32 */
    /* optional adapters on q and v (LoRALinear::forward, src/nn/decoder.cpp:26-28); rank 0 = none.
     * low = [rows, 2*rank] f32 holds down_q(x) | down_v(x) computed by a previous b200_linear call. */
    int32_t lora_rank;
    float lora_scale;
    const float* low;
    const void* q_up;             /* [heads*head_dim, rank] weight dtype */
    const void* v_up;             /* [kv_heads*head_dim, rank] */
} b200_qkv_args;

/* y = epilogue(norm(x) @ W^T) for a skinny activation matrix: x f32 [rows, in], W [out, in] row-major
 * (f32 or bf16, widened to f32 exactly as src/kernels/cpu/matmul.cpp:28-31), f32 accumulation.
 * When norm_weight != NULL the RMSNorm of x (weights norm_weight, eps) is applied while x is staged
 * (TransformerDecoderLayer::decode applies the norm right before these projections, src/nn/decoder.cpp:104-105).
 * Replaces nn::Linear::forward -> numeric::linear -> matmul_into (src/nn/layers.cpp:21-23, src/ops/numeric.cpp:199-209).
 * `y` may alias `residual`.  For B200_EPI_SWIGLU y is [rows, out/2]. */
B200_API int b200_linear(const float* x, int64_t rows, int64_t in, const void* weight, int32_t weight_dtype,
                         int64_t out, const void* norm_weight, int32_t norm_dtype, double eps,
                         b200_epilogue epilogue, const float* residual, const b200_qkv_args* qkv, float* y, void* stream);

/* ---- activation shadows (no counterpart in the reference) -------------------------------------------------------
 * Between the kernels of a decode step an f32 activation matrix can travel as a "shadow": two bf16 planes hi + lo
 * (hi = bf16(v), lo = bf16(v - hi), about 16 mantissa bits together), the operand form of the tensor cores.  The
 * consumer fetches its rows with bulk copies straight into shared memory instead of converting f32 in every CTA.
 * An RMSNorm between producer and consumer is split: the producer folds the norm weight into the shadow and leaves
 * per-row partial sums of squares of the un-weighted values; the consumer multiplies its results by
 * 1/sqrt(sum/width + eps).  The f32 arithmetic differs from the reference's f64 norm by rounding only. */
typedef struct b200_shadow_linear_args {
    const void* x_hi;              /* bf16 [rows, in] */
    const void* x_lo;              /* may be NULL for calls the dense kernel serves (more than 16 rows or in > 2048): the
                                      activations then count as bf16 - half the operand traffic and tensor-core work */
    int64_t rows, in;
    const void* weight;            /* bf16 [out, in] */
    int64_t out;
    const float* sumsq_in;         /* [parts_in][rows] or NULL (no row scale) */
    int32_t parts_in;
    double eps;
    b200_epilogue epilogue;
    const float* residual;         /* B200_EPI_RESIDUAL */
    const b200_qkv_args* qkv;      /* B200_EPI_QKV */
    float* y;                      /* f32 result; may be NULL for B200_EPI_SWIGLU when only the shadow is wanted */
    void* out_hi;                  /* optional output shadow: residual epilogue [rows, out], SwiGLU epilogue [rows, out/2] */
    void* out_lo;
    const void* out_norm_weight;   /* residual epilogue: weight [out] of the norm that follows, folded into the shadow */
    int32_t out_norm_dtype;
    float* sumsq_out;              /* residual epilogue: [b200_linear_shadow_parts(rows, in, out)][rows] */
    float* best_value;             /* B200_EPI_ARGMAX: [b200_linear_argmax_parts(rows, in, out)][rows] */
    int32_t* best_index;           /* B200_EPI_ARGMAX: same shape, feature index of best_value */
    float* const* y_copies;        /* store / residual epilogues: `copies` (0..7) further [rows, out] f32 matrices that receive the */
    int32_t copies;                /*   same rows as y - a tensor-parallel rank's slot in each peer's memory (plain peer stores) */
} b200_shadow_linear_args;
/* Up to 16 rows with in <= 2048: streaming kernel (bulk-TMA weight ring, mma.sync).  More rows or a wider input:
 * dense tcgen05 kernel (TMA operand tiles, accumulator in tensor memory; K split over a thread-block cluster when the
 * tiles are few, a persistent variant for prefill-sized passes), except store-epilogue calls with at most 64 output
 * features (adapter down-projections), which a CUDA-core kernel serves.  B200_UNSUPPORTED when in % 8 != 0. */
B200_API int b200_linear_shadow(const b200_shadow_linear_args* args, void* stream);
/* Number of row-sum partials a residual-epilogue call with these sizes writes (its feature tiles), 0 if unsupported. */
B200_API int32_t b200_linear_shadow_parts(int64_t rows, int64_t in, int64_t out);
/* Number of candidate slices a B200_EPI_ARGMAX call with these sizes writes (one per CTA of the streaming kernel, one per
 * feature tile of the dense kernel), 0 if unsupported. */
B200_API int32_t b200_linear_argmax_parts(int64_t rows, int64_t in, int64_t out);
/* Name of the kernel family a b200_linear_shadow call with these sizes runs on ("linear_stream_kernel": up to 16 rows;
 * "linear_decode_kernel": decode batches on tcgen05 with the weights as the streamed operand; "linear_gemm_kernel": more
 * rows; "linear_thin_kernel": at most 64 output features).  For logs and benchmarks. */
B200_API const char* b200_linear_shadow_kernel(int64_t rows, int64_t in, int64_t out);
/* Launch shape the decode-batch kernel would take for these sizes (host-side; needs no GPU - without one the figures of a
 * 148-SM B200 are used): shape[0..9] = weight tiles per CTA, K split (cluster size), tile groups (grid y), ring stages,
 * bytes per stage, N of the products (rows of a token tile padded to 16), tensor-memory columns, dynamic shared memory,
 * rows per token tile, token tiles (grid x).  Returns 1, or 0 when that kernel does not take the row count.  Diagnostic. */
B200_API int32_t b200_linear_decode_launch_shape(int64_t rows, int64_t in, int64_t out, int32_t two_planes, int32_t* shape);
/* Second half of the fused logits + greedy choice: merges the `parts` per-tile candidates of every row (same rule), writes
 * the chosen feature index to next[rows], and does what b200_token_feedback does with it (ids, history, counter; any of
 * ids / history may be NULL).  With caches (at most 64, one per layer) it also does b200_kv_cache_advance(caches, count, 1): the
 * step's token becomes part of every cache.  One launch of one CTA. */
B200_API int b200_argmax_finish(const float* best_value, const int32_t* best_index, int32_t parts, int64_t rows, int64_t* next,
                                int64_t* ids, int64_t* history, int64_t history_rows, int32_t* counter,
                                b200_kv_cache* const* caches, int32_t cache_count, void* stream);
/* b200_embedding that also writes the shadow of out * norm_weight and one partial sum of squares per row ([1][rows]). */
B200_API int b200_embedding_shadow(const void* table, int32_t table_dtype, const int64_t* ids, int64_t rows, int64_t vocab,
                                   int64_t width, const void* norm_weight, int32_t norm_dtype, float* out, void* out_hi,
                                   void* out_lo, float* sumsq_out, void* stream);

/* Shadow of x * norm_weight (norm_weight may be NULL) and one partial sum of squares per row ([1][rows]) for f32 rows
 * that did not come out of one of the kernels above. */
B200_API int b200_shadow_from_rows(const float* x, int64_t rows, int64_t width, const void* norm_weight, int32_t norm_dtype,
                                   void* out_hi, void* out_lo, float* sumsq_out, void* stream);

/* Split-K flash-decode grouped-query attention over the paged cache.
 * Replaces detail::grouped_attention / grouped_block / attention_weights (src/ops/attention.cpp:65-95,161-188)
 * and the softmax of src/kernels/cpu/reduction.cpp:155-203 for queries whose keys are the cache:
 * q f32 [rows, heads, head_dim]; with causal != 0 row r belongs to sequence r / L and sees keys
 * 0 .. lengths[r/L] + r % L (the causal rule key_pos <= query_pos of src/ops/attention.cpp:52-57; for L == 1
 * that is every cached key, the new one included, which the cache must already hold); with causal == 0 every
 * row of sequence s sees keys 0 .. lengths[s]-1 (dl::grouped_query_attention without a mask).
 * out f32 [rows, heads*head_dim].
 * scratch: device workspace of at least b200_attention_scratch_bytes(...) bytes holding the per-split partial
 * (max, sum, accumulator) triples; no allocation happens inside the call.
 * max_length: upper bound of lengths[s] + L (sizes the split grid; may be the cache capacity). */
B200_API size_t b200_attention_scratch_bytes(int64_t rows, int32_t heads, int32_t kv_heads, int32_t head_dim,
                                             int32_t max_length, int32_t page_size);
B200_API int b200_attention_decode(const float* q, int64_t rows, int32_t tokens_per_sequence, int32_t heads,
                                   const b200_kv_cache* cache, int32_t max_length, int32_t causal, void* scratch,
                                   size_t scratch_bytes, float* out, void* stream);

/* b200_attention_decode writing its result as a shadow (bf16 planes [rows, heads*head_dim]) for a following
 * b200_linear_shadow instead of f32. */
B200_API int b200_attention_decode_shadow(const float* q, int64_t rows, int32_t tokens_per_sequence, int32_t heads,
                                          const b200_kv_cache* cache, int32_t max_length, int32_t causal, void* scratch,
                                          size_t scratch_bytes, void* out_hi, void* out_lo, void* stream);

/* No counterpart in the reference.  b200_attention_decode for callers that must not allocate and have no workspace
 * of their own to hand in: a serving loop whose device memory was budgeted once at start-up, a host runtime whose
 * device memory belongs to a pool it does not control (the reference keeps such a per-device pool), or code for
 * which the implicit device-wide synchronisation of cudaMalloc/cudaFree is not acceptable on the token path.
 * Same arguments and results as b200_attention_decode, minus the scratch: the split partials go to a fixed
 * B200_STATIC_SCRATCH_BYTES array that is part of the library image (every GPU that loads the library holds that
 * much memory until the process exits).  The call allocates nothing and frees nothing.
 *   - Shapes whose partials need more than B200_STATIC_SCRATCH_BYTES are rejected with B200_BAD_ARGUMENT and a
 *     message that states both sizes; use b200_attention_decode with your own workspace for those.
 *   - The first call on a device looks up the array's device address (once per device, with that device current);
 *     make that first call during set-up, before any stream capture is started.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Nothing in it has to
 *     start at zero: every split partial that the merge step reads was written by the same call.  Two calls that
 *     overlap on the GPU (different streams, or several host threads) race on the array: serialise them.
 *   - The KV cache object must exist before the call (creating it is where the per-device status word is allocated). */
#define B200_STATIC_SCRATCH_BYTES (8u << 20)
B200_API int b200_attention_decode_static(const float* q, int64_t rows, int32_t tokens_per_sequence, int32_t heads,
                                          const b200_kv_cache* cache, int32_t max_length, int32_t causal, float* out,
                                          void* stream);

/* dl::argmax along the last axis (src/ops/reduction.cpp:95-110; rule src/kernels/cpu/reduction.cpp:141-145:
 * first maximum wins, the first NaN wins over everything after it). */
B200_API int b200_argmax(const float* x, int64_t rows, int64_t width, int64_t* index, void* stream);

/* Temperature sampling of one index per row, the arithmetic of the reference's example loop
 * (examples/text_generate.cpp:38-39): p = softmax(x / temperature) in f32 (max, exp(v - max), sum, divide:
 * src/kernels/cpu/reduction.cpp:155-203), then the categorical draw of std::discrete_distribution for a uniform variate
 * u in [0, 1): the first index whose running sum of p (f64, index order) exceeds u times the total.  `uniform` holds one
 * u per row in device memory; the caller owns the random stream. */
B200_API int b200_sample(const float* x, int64_t rows, int64_t width, double temperature, const double* uniform, int64_t* index,
                         void* stream);

/* Takes every `stride`-th row starting at `first` of a [rows_in, width] f32 matrix (Tensor::select of the last
 * position, examples/decoder_generate.cpp:27). */
B200_API int b200_select_rows(const float* x, int64_t first, int64_t stride, int64_t rows_out, int64_t width,
                              float* out, void* stream);

/* dl::rotary_embedding (src/ops/contraction.cpp:44-49): x [outer, length, head_dim] f32, tables [length, head_dim/2];
 * adjacent pairs, each product rounded before the subtraction / addition. */
B200_API int b200_rotary(const float* x, int64_t outer, int64_t length, int64_t head_dim, const float* cosine,
                         const float* sine, float* out, void* stream);

/* in [a, b, c, d] -> out [a, c, b, d] (the transpose(1, 2) of src/nn/decoder.cpp:82,88 made dense). */
B200_API int b200_permute_0213(const float* in, int64_t a, int64_t b, int64_t c, int64_t d, float* out, void* stream);

/* Dense copy of a permuted f32 tensor (Tensor::permute + contiguous of the reference, as dl::tensordot uses it,
 * src/ops/contraction.cpp:39-41): `sizes` are the input's `rank` sizes (rank <= 8), out axis i is input axis order[i]. */
B200_API int b200_permute(const float* in, const int64_t* sizes, const int64_t* order, int32_t rank, float* out, void* stream);

/* Token feedback of the greedy loop (examples/decoder_generate.cpp:28-30) kept on the device:
 * history[counter[0] * batch + s] = next[s]; ids[s] = next[s]; counter[0] += 1. */
B200_API int b200_token_feedback(const int64_t* next, int64_t batch, int64_t* ids, int64_t* history, int64_t history_rows,
                                 int32_t* counter, void* stream);

/* y[i] = y[i] + x[i] * scale with a separate rounding for the product (the residual add of src/nn/decoder.cpp:104-105
 * with scale 1, and the adapter sum of LoRALinear::forward, src/nn/decoder.cpp:27). */
B200_API int b200_scaled_add(float* y, const float* x, float scale, int64_t count, void* stream);

/* Device-side health word: kernels that give up a bounded wait (TMA barrier) set it instead of spinning forever.
 * Returns the word and clears it (synchronises the stream). 0 = healthy. */
B200_API int b200_take_device_status(int32_t device, void* stream, int32_t* status);

/* ---- tensor-parallel sum over NVLink peer memory (no reference counterpart: the reference has no tensor parallelism) ----
 * Every rank owns a region of b200_tp_region_bytes(slot_bytes, world) bytes of its own device memory (zero-filled,
 * cudaMalloc'ed, mapped by every rank of the group, e.g. through CUDA IPC): control words and, for each of two alternating
 * sums, one slot of partial rows PER SENDER; b200_tp_slot(region, slot_bytes, world, slot, sender) is the address where
 * rank `sender` deposits its partial rows of sum `slot` in that region.  A rank's projection writes its partial rows into
 * its slot of EVERY region (b200_shadow_linear_args: y = the local one, y_copies = the peers'), so the rows cross NVLink
 * from the projection's epilogue.  b200_tp_reduce_shadow, called by every rank at the same point of its stream with
 * regions[r] = rank r's region as mapped here, then publishes "my rows are written" to all ranks, waits (bounded; on
 * expiry the device status word reads B200_DEVICE_TIMEOUT) for all ranks' signals, and writes out[rows, width] = sum over
 * senders in rank order of the slots of its OWN region (local loads only), the shadow planes of out * norm_weight and
 * per-row partial sums of squares ([b200_tp_reduce_parts(width)][rows], one partial per 1024 columns).  Callers alternate
 * slots 0 and 1 from call to call.  pull != 0: the projections deposited their rows in their own region only (no
 * y_copies) and the sum reads sender r's slot from rank r's region with peer loads instead. */
B200_API int32_t b200_tp_reduce_parts(int64_t width);
B200_API size_t b200_tp_region_bytes(size_t slot_bytes, int32_t world);
B200_API void* b200_tp_slot(void* region, size_t slot_bytes, int32_t world, int32_t slot, int32_t sender);
B200_API int b200_tp_reduce_shadow(void* const* regions, int32_t rank, int32_t world, int32_t slot, size_t slot_bytes, int32_t pull, int64_t rows,
                                   int64_t width, const void* norm_weight, int32_t norm_dtype, float* out, void* out_hi, void* out_lo,
                                   float* sumsq_out, void* stream);

/* Greedy choice with the vocabulary split over the ranks (no reference counterpart): this rank ran the logits projection
 * with B200_EPI_ARGMAX over the table rows [first_index, first_index + its slice) and holds per-tile candidates as for
 * b200_argmax_finish.  The call merges them, deposits one (value, global index) pair per row in every rank's region
 * (behind the slots: b200_tp_region_bytes covers the area; at most 1024 rows), waits (bounded) for all ranks' pairs and
 * merges those under the same rule, so every rank feeds back the same token; then the bookkeeping of b200_argmax_finish. */
B200_API int b200_tp_argmax_finish(void* const* regions, int32_t rank, int32_t world, size_t slot_bytes, int32_t first_index,
                                   const float* best_value, const int32_t* best_index, int32_t parts, int64_t rows, int64_t* next,
                                   int64_t* ids, int64_t* history, int64_t history_rows, int32_t* counter,
                                   b200_kv_cache* const* caches, int32_t cache_count, void* stream);

#ifdef __cplusplus
}
#endif
#endif
