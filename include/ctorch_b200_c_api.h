/*
 * ctorch_b200_c_api.h -- the C17 entry points of the decoder token loop, exported by libctorch_b200.so.
 *
 * Every dl_* symbol below has the name, argument list, ownership rules and error behaviour of the reference
 * declaration cited beside it (reference paths: include/dl/c_api.h, include/dl/decoder_c_api.h; implementation
 * src/api/).  A C program written against those headers for this path links against this library unchanged.
 * Differences in behaviour:
 *   - compute happens only on CUDA devices (sm_100a); an operator or module given CPU tensors returns DL_ERROR,
 *     there is no CPU fallback.  CPU tensors exist as host-side containers (dl_from_host, dl_to, state handling).
 *   - weights are f32 or bf16; activations, logits and operator results are f32 (as on the reference's CPU path).
 *   - dl_select / dl_narrow return dense tensors (copies unless the leading axis is cut), not strided views.
 * The dl_generation_* and dl_decoder_generate entry points at the end are NEW: the reference has no generate
 * call, its token loop lives in examples/decoder_generate.cpp:20-31.
 *
 * Ownership (include/dl/c_api.h:154-158): every creator writes an owning handle into *output, which is NULL on
 * failure; release functions accept NULL.  Errors: DL_ERROR plus a thread-local message from dl_last_error(),
 * valid until the thread's next status call (src/api/common.cpp:8-12, src/api/common.h:53-69).
 */
#ifndef CTORCH_B200_C_API_H
#define CTORCH_B200_C_API_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef DL_API                  /* dl/export.h defines it when the reference's include paths are used */
#if defined(__GNUC__)
#define DL_API __attribute__((visibility("default")))
#else
#define DL_API
#endif
#endif

#ifndef DL_VERSION
#define DL_VERSION "0.3.0"      /* include/dl/version.h.in */
#endif
#ifndef DL_ABI_VERSION
#define DL_ABI_VERSION 1
#endif

/* include/dl/c_api.h:15-58,72-77 */
typedef struct dl_tensor dl_tensor;
typedef struct dl_module dl_module;
typedef struct dl_state dl_state;
typedef enum dl_status { DL_OK = 0, DL_ERROR = 1 } dl_status;
typedef enum dl_dtype { DL_F32 = 0, DL_F64 = 1, DL_I64 = 2, DL_BOOL = 3, DL_F16 = 4, DL_BF16 = 5 } dl_dtype;
typedef enum dl_device_type { DL_CPU = 0, DL_CUDA = 1 } dl_device_type;
typedef struct dl_device { dl_device_type type; int32_t index; } dl_device;
typedef struct dl_shape { const int64_t* data; size_t size; } dl_shape;
typedef struct dl_tensor_options { dl_dtype dtype; dl_device device; int32_t requires_grad; } dl_tensor_options;
typedef struct dl_tensor_info {
    dl_dtype dtype;
    dl_device device;
    int64_t numel;
    int32_t contiguous, requires_grad, leaf;
} dl_tensor_info;

/* include/dl/c_api.h:159-161 */
DL_API const char* dl_version(void);
DL_API const char* dl_last_error(void);
DL_API dl_tensor_options dl_default_tensor_options(void);

/* include/dl/c_api.h:177-191 -- tensor handles */
DL_API void dl_tensor_release(dl_tensor* tensor);
DL_API dl_status dl_tensor_retain(const dl_tensor* tensor, dl_tensor** output);
DL_API dl_tensor_info dl_tensor_get_info(const dl_tensor* tensor);
DL_API dl_shape dl_tensor_shape(const dl_tensor* tensor);     /* borrowed until release */
DL_API dl_shape dl_tensor_strides(const dl_tensor* tensor);
DL_API const void* dl_tensor_data(const dl_tensor* tensor);   /* device pointer for CUDA tensors */
DL_API size_t dl_tensor_nbytes(const dl_tensor* tensor);
DL_API dl_status dl_tensor_copy_to_host(const dl_tensor* tensor, void* destination);
DL_API dl_status dl_from_host(const void* data, dl_shape shape, dl_tensor_options options, dl_tensor** output);
DL_API dl_status dl_full(dl_shape shape, double value, dl_tensor_options options, dl_tensor** output);
DL_API dl_status dl_zeros(dl_shape shape, dl_tensor_options options, dl_tensor** output);
DL_API dl_status dl_ones(dl_shape shape, dl_tensor_options options, dl_tensor** output);
/* include/dl/c_api.h:200-204,206,217-218 */
DL_API dl_status dl_clone(const dl_tensor* input, dl_tensor** output);
DL_API dl_status dl_astype(const dl_tensor* input, dl_dtype dtype, dl_tensor** output);
DL_API dl_status dl_to(const dl_tensor* input, dl_device device, dl_tensor** output);
DL_API dl_status dl_reshape(const dl_tensor* input, dl_shape shape, dl_tensor** output);
DL_API dl_status dl_select(const dl_tensor* input, int64_t axis, int64_t index, dl_tensor** output);
DL_API dl_status dl_narrow(const dl_tensor* input, int64_t axis, int64_t start, int64_t length, dl_tensor** output);

/* include/dl/c_api.h:283,306,313,378,489 -- operators on the path */
DL_API dl_status dl_argmax(const dl_tensor* input, int64_t axis, int32_t keepdim, dl_tensor** output);
DL_API dl_status dl_linear(const dl_tensor* input, const dl_tensor* weight, const dl_tensor* bias, dl_tensor** output);
DL_API dl_status dl_embedding(const dl_tensor* indices, const dl_tensor* weight, dl_tensor** output);
DL_API dl_status dl_rms_norm(const dl_tensor* input, dl_shape normalized_shape, const dl_tensor* weight,
    const double* epsilon, dl_tensor** output);
DL_API dl_status dl_synchronize(dl_device device);

/* include/dl/c_api.h:524-533,549,619,627-628,631 -- modules */
DL_API void dl_module_release(dl_module* module);
DL_API dl_status dl_module_retain(const dl_module* module, dl_module** output);
DL_API dl_status dl_linear_create(int64_t input_features, int64_t output_features, int32_t bias,
    dl_tensor_options options, dl_module** output);
DL_API dl_status dl_linear_from_tensors(const dl_tensor* weight, const dl_tensor* bias, dl_module** output);
DL_API dl_status dl_embedding_create(int64_t vocabulary, int64_t dimensions, dl_tensor_options options,
    dl_module** output);
DL_API dl_status dl_embedding_from_tensor(const dl_tensor* weight, dl_module** output);
DL_API dl_status dl_rms_norm_create(dl_shape normalized_shape, const double* epsilon, int32_t affine,
    dl_tensor_options options, dl_module** output);
DL_API dl_status dl_module_forward(dl_module* module, const dl_tensor* input, dl_tensor** output);
DL_API dl_status dl_module_train(dl_module* module, int32_t training);
DL_API int32_t dl_module_is_training(const dl_module* module);
DL_API dl_status dl_module_to(dl_module* module, dl_device device);

/* include/dl/c_api.h:637-646 -- state dictionaries */
DL_API dl_status dl_module_state(const dl_module* module, dl_state** output);
DL_API dl_status dl_module_load_state(dl_module* module, const dl_state* state);
DL_API void dl_state_release(dl_state* state);
DL_API size_t dl_state_size(const dl_state* state);
DL_API const char* dl_state_name(const dl_state* state, size_t index);   /* borrowed from the state */
DL_API dl_status dl_state_tensor(const dl_state* state, size_t index, dl_tensor** output);
/* Weight archives (".ct") in the reference's byte layout (include/dl/c_api.h:647-648, src/io/checkpoint.cpp:52-114): files
 * written by either library load in the other.  Loaded tensors live in host memory; dl_module_load_state moves them. */
DL_API dl_status dl_state_save(const char* path, const dl_state* state);
DL_API dl_status dl_state_load(const char* path, dl_state** output);
DL_API dl_status dl_state_create(const char* const* names, const dl_tensor* const* tensors, size_t count,
    dl_state** output);

/* include/dl/decoder_c_api.h:11-41 -- decoder operators, modules, cache and decode */
typedef struct dl_decoder_cache dl_decoder_cache;
/* include/dl/decoder_c_api.h:13-14 -- contraction over the given axes (f32 result; CUDA tensors only) */
DL_API dl_status dl_tensordot(const dl_tensor* a, const dl_tensor* b, dl_shape axes_a, dl_shape axes_b, dl_tensor** output);
DL_API dl_status dl_rotary_embedding(const dl_tensor* input, const dl_tensor* cosine, const dl_tensor* sine,
    dl_tensor** output);
DL_API dl_status dl_grouped_query_attention(const dl_tensor* query, const dl_tensor* key, const dl_tensor* value,
    const dl_tensor* keep_mask, dl_tensor** output);   /* keep_mask must be NULL on this path */
DL_API dl_status dl_swiglu_create(int64_t dimensions, int64_t hidden, int32_t bias, dl_tensor_options options,
    dl_module** output);
DL_API dl_status dl_lora_linear_create(const dl_module* base, int64_t rank, double alpha, dl_module** output);
DL_API dl_status dl_lora_linear_merge(const dl_module* adapter, dl_module** output);
DL_API dl_status dl_rotary_embedding_create(int64_t dimensions, int64_t capacity, double base,
    dl_tensor_options options, dl_module** output);
DL_API dl_status dl_rotary_embedding_forward(dl_module* rotary, const dl_tensor* input, int64_t offset,
    dl_tensor** output);
DL_API dl_status dl_grouped_query_attention_create(int64_t dimensions, int64_t heads, int64_t kv_heads,
    int64_t context, dl_tensor_options options, dl_module** output);
DL_API dl_status dl_transformer_decoder_create(int64_t layers, int64_t dimensions, int64_t heads, int64_t kv_heads,
    int64_t hidden, int64_t context, dl_tensor_options options, dl_module** output);
DL_API dl_status dl_decoder_cache_create(const dl_module* decoder, dl_decoder_cache** output);
DL_API void dl_decoder_cache_release(dl_decoder_cache* cache);
DL_API dl_status dl_decoder_cache_clear(dl_decoder_cache* cache);
DL_API dl_status dl_decoder_cache_truncate(dl_decoder_cache* cache, int64_t length);
DL_API dl_status dl_decoder_cache_length(const dl_decoder_cache* cache, int64_t* length);
DL_API dl_status dl_transformer_decoder_decode(dl_module* decoder, const dl_tensor* input, dl_decoder_cache* cache,
    dl_tensor** output);

/* ---- NEW entry points (no counterpart in the reference) ------------------------------------------------- */

/* Storage dtype of caches created afterwards by dl_decoder_cache_create for this decoder: DL_F32 or DL_BF16.
 * Default: DL_BF16 for bf16 decoders, DL_F32 for f32 decoders (the reference always caches f32). */
DL_API dl_status dl_transformer_decoder_set_cache_dtype(dl_module* decoder, dl_dtype dtype);
/* Precision of the activations handed from kernel to kernel in a bf16 decoder.  DL_F32 (default): f32-equivalent (two bf16
 * planes), as the reference keeps activations in f32 (src/ops/matmul.cpp:43).  DL_BF16: passes over more than 16 rows
 * (prefill, large decode batches) use one bf16 plane - about half the tensor-core work, logits still within the 2e-2 bf16
 * tolerance.  Single-token steps of up to 16 sequences are unaffected. */
DL_API dl_status dl_transformer_decoder_set_activation_dtype(dl_module* decoder, dl_dtype dtype);
/* Installs adapters (from dl_lora_linear_create) on the query and value projections of one layer; both NULL
 * removes them.  The reference can only host merged weights inside its decoder (include/dl/decoder.h:75). */
DL_API dl_status dl_transformer_decoder_set_adapters(dl_module* decoder, int64_t layer, const dl_module* query,
    const dl_module* value);

/* Greedy generation with the token loop resident on the device: the loop of examples/decoder_generate.cpp:20-31
 * (prefill the prompt, take the last position, argmax with the first-maximum rule, feed the token back) for a
 * batch.  `embedding` and `output` are the modules around the decoder (examples/decoder_model.h:15-18; pass a
 * Linear built on the embedding weight for a tied model).  The generation borrows `cache` (it must outlive it)
 * and retains the three modules. */
typedef struct dl_generation dl_generation;
DL_API dl_status dl_generation_create(dl_module* decoder, dl_module* embedding, dl_module* output,
    dl_decoder_cache* cache, int64_t batch, int64_t max_steps, dl_generation** result);
DL_API void dl_generation_release(dl_generation* generation);
/* prompt: int64 [batch, length], host or device.  Produces the first token. */
DL_API dl_status dl_generation_prefill(dl_generation* generation, const dl_tensor* prompt);
/* Enqueues `steps` more tokens (CUDA-graph replays); returns without waiting for the device. */
DL_API dl_status dl_generation_step(dl_generation* generation, int64_t steps);
/* One token with the host in the loop, as the reference example does per token: ids_in [batch] (host, may be
 * NULL to continue from the device-resident ids) is copied to the device, one step runs, the chosen ids are
 * copied back into ids_out [batch] (host) and the call waits for them. */
DL_API dl_status dl_generation_step_host(dl_generation* generation, const int64_t* ids_in, int64_t* ids_out);
/* `steps` tokens with the host in the loop, in one call: step i copies its ids [batch] from the host to the device (ids_in
 * for i = 0, the ids step i - 1 returned afterwards), runs, and copies the chosen ids back into ids_out[i * batch ...]
 * before step i + 1 starts - the loop of examples/decoder_generate.cpp:20-31 with its per-token host round trip, without
 * an interpreter between the steps.  ids_out: host, [steps, batch]. */
DL_API dl_status dl_generation_run_host(dl_generation* generation, const int64_t* ids_in, int64_t steps, int64_t* ids_out);
/* One token drawn from softmax(logits / temperature) (the sibling example's loop, examples/text_generate.cpp:37-41): the
 * caller supplies one uniform variate in [0, 1) per sequence from its own generator; the draw is the inverse of the
 * running sum in index order, as std::discrete_distribution does.  Host in the loop like dl_generation_step_host.
 * No counterpart in the reference's C API (its example samples on the host). */
DL_API dl_status dl_generation_step_sampled(dl_generation* generation, double temperature, const double* uniforms, int64_t* ids_out);
/* Tokens generated so far, int64 [batch, count] on the host (waits for the device). */
DL_API dl_status dl_generation_tokens(dl_generation* generation, dl_tensor** output);
/* Logits [batch, vocab] (f32, device) the latest token was chosen from. */
DL_API dl_status dl_generation_logits(dl_generation* generation, dl_tensor** output);
/* extensions/onnx/include/dl/onnx_c_api.h:17-18 -- the decoder as an ONNX file (opset 24) with one past_key_i / past_value_i
 * input and one present_key_i / present_value_i output per layer; embedding and output both given: int64 input_ids in,
 * logits out; both NULL: features in, hidden states out.  Host work only (weights are read back from their device). */
DL_API dl_status dl_onnx_save_decoder(const char* path, const dl_module* decoder, const dl_module* embedding, const dl_module* output);
/* Rows of the buffers in which a bf16 decoder of this width (and per-rank SwiGLU width) carries per-row partial sums of
 * squares from one kernel to the next: the largest count any of its kernels may write.  Host arithmetic only. */
DL_API int64_t dl_b200_shadow_partial_rows(int64_t dimensions, int64_t hidden);
/* Kernel launches (graph nodes) of one captured decode step. */
DL_API int64_t dl_generation_launches_per_step(const dl_generation* generation);
/* One real step run eagerly with a CUDA event after every launch (for roofline reporting): milliseconds[0] =
 * skinny-linear launches, [1] = attention launches, [2] = everything else, [3] = number of launches. */
DL_API dl_status dl_generation_profile_step(dl_generation* generation, double milliseconds[4]);
/* prefill + (steps-1) device steps; tokens int64 [batch, steps] on the prompt's device. */
DL_API dl_status dl_decoder_generate(dl_module* decoder, dl_module* embedding, dl_module* output,
    const dl_tensor* prompt, int64_t steps, dl_decoder_cache* cache, dl_tensor** tokens);

/* KV-head tensor parallelism (one process per GPU).  A group is one NCCL communicator per device: one rank asks for
 * a 128-byte id, every rank receives it by whatever transport the application has and joins.  A decoder then computes
 * slice `rank` of `world`: query heads, KV heads and SwiGLU features are split evenly; norms, the residual stream, the
 * embedding and the logits stay replicated; the partial results of the output projection and of the FFN
 * down-projection are summed over the group (all-reduce on the library's stream) before the next norm.  Caches created
 * for such a decoder hold the rank's KV heads only.  bf16 decoders only. */
DL_API dl_status dl_b200_tp_unique_id(void* id128);
DL_API dl_status dl_b200_tp_init(dl_device device, int32_t rank, int32_t world, const void* id128);
DL_API dl_status dl_b200_tp_finalize(dl_device device);
/* Optional second step: memory that the ranks read from each other over NVLink, so that the two sums per layer run as one
 * kernel that also rebuilds the next norm's input (no NCCL call on the token path).  Every rank asks for its 64-byte handle
 * (the library allocates 4 KiB + 2 * slot_bytes; a slot must hold rows * dimensions * 4 bytes of the largest step that
 * should take this path), the application gathers the handles of all ranks in rank order and passes the table to every
 * rank.  Steps whose rows do not fit a slot keep the NCCL all-reduce.  All ranks must be past their last step (a barrier of
 * the application) before any of them calls dl_b200_tp_finalize. */
DL_API dl_status dl_b200_tp_symmetric_handle(dl_device device, size_t slot_bytes, void* handle64);
DL_API dl_status dl_b200_tp_symmetric_open(dl_device device, const void* handles, int32_t world);
/* How the partial sums of the output and down projections travel once the peer memory is mapped.  push = 0 (default): a
 * projection writes its rows into its own region and the sum that follows loads the peers' rows over NVLink.  push != 0:
 * the projection's epilogue stores its rows into every peer's region and the sum reads local memory only.  Every rank of a
 * group must choose the same mode, before its first step.  The environment variable CTORCH_B200_TP_PUSH sets the default. */
DL_API dl_status dl_b200_tp_set_push(dl_device device, int32_t push);
DL_API dl_status dl_transformer_decoder_set_tensor_parallel(dl_module* decoder, int32_t rank, int32_t world);

/* CUDA-event timing on the library's compute stream of a device (benchmarks must time on the launching
 * stream).  dl_b200_timer_stop waits for the work and returns milliseconds since dl_b200_timer_start. */
DL_API dl_status dl_b200_timer_start(dl_device device);
DL_API dl_status dl_b200_timer_stop(dl_device device, double* milliseconds);
/* The library's compute stream of a device as a cudaStream_t. */
DL_API void* dl_b200_stream(dl_device device);

#ifdef __cplusplus
}
#endif
#endif
