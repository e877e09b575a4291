/* A C17 translation unit written against the reference's include paths (<dl/decoder_c_api.h>): the decoder part of the
 * reference's C ABI lifecycle test (tests/c_api.c:28-42 there) - create a decoder and its cache, decode a [1, 2, 8] chunk of
 * ones, read the cache length, clear, release - plus dl_tensordot.  argv[1] = "cuda" runs it on device 0; "cpu" checks
 * that the same handles can be created on the host and that compute on host tensors is refused (no CPU fallback). */
#include <dl/decoder_c_api.h>

#include <math.h>
#include <stdio.h>
#include <string.h>

#define OK(call)                                                                 \
    do {                                                                         \
        if ((call) != DL_OK) {                                                   \
            fprintf(stderr, "%s failed: %s\n", #call, dl_last_error());          \
            return 1;                                                            \
        }                                                                        \
    } while (0)

int main(int argc, char** argv) {
    const int cuda = argc > 1 && strcmp(argv[1], "cuda") == 0;
    if (strcmp(dl_version(), DL_VERSION) != 0 || DL_ABI_VERSION != 1) return 1;
    dl_tensor_options options = dl_default_tensor_options();
    options.device.type = cuda ? DL_CUDA : DL_CPU;
    options.device.index = 0;

    dl_module* decoder = NULL;
    dl_decoder_cache* cache = NULL;
    dl_tensor* input = NULL;
    dl_tensor* output = NULL;
    OK(dl_transformer_decoder_create(1, 8, 4, 2, 12, 16, options, &decoder));
    OK(dl_decoder_cache_create(decoder, &cache));
    const int64_t sequence_dims[] = {1, 2, 8};
    OK(dl_ones((dl_shape){sequence_dims, 3}, options, &input));
    int64_t length = -1;
    if (cuda) {
        OK(dl_transformer_decoder_decode(decoder, input, cache, &output));
        OK(dl_decoder_cache_length(cache, &length));
        if (length != 2) return 1;
        float values[16];
        if (dl_tensor_nbytes(output) != sizeof values) return 1;
        OK(dl_tensor_copy_to_host(output, values));
        for (int i = 0; i < 16; ++i)
            if (!isfinite(values[i])) return 1;
    } else {
        if (dl_transformer_decoder_decode(decoder, input, cache, &output) != DL_ERROR || output != NULL) return 1;
        if (strstr(dl_last_error(), "CUDA") == NULL) return 1;
        OK(dl_decoder_cache_length(cache, &length));
        if (length != 0) return 1;   /* a refused chunk leaves the cache where it was */
    }
    OK(dl_decoder_cache_clear(cache));
    OK(dl_decoder_cache_length(cache, &length));
    if (length != 0) return 1;
    dl_tensor_release(output);
    dl_tensor_release(input);
    dl_decoder_cache_release(cache);
    dl_module_release(decoder);

    /* dl_tensordot: a [2, 3] . b [4, 3] over the last axes = a @ b^T */
    const float a_values[] = {1, 2, 3, 4, 5, 6}, b_values[] = {1, 0, 0, 0, 1, 0, 0, 0, 1, 1, 1, 1};
    const int64_t a_dims[] = {2, 3}, b_dims[] = {4, 3}, axis[] = {1};
    dl_tensor *a = NULL, *b = NULL, *product = NULL;
    OK(dl_from_host(a_values, (dl_shape){a_dims, 2}, options, &a));
    OK(dl_from_host(b_values, (dl_shape){b_dims, 2}, options, &b));
    if (cuda) {
        OK(dl_tensordot(a, b, (dl_shape){axis, 1}, (dl_shape){axis, 1}, &product));
        float result[8];
        OK(dl_tensor_copy_to_host(product, result));
        const float want[] = {1, 2, 3, 6, 4, 5, 6, 15};
        for (int i = 0; i < 8; ++i)
            if (fabsf(result[i] - want[i]) > 1e-5f) return 1;
    } else if (dl_tensordot(a, b, (dl_shape){axis, 1}, (dl_shape){axis, 1}, &product) != DL_ERROR || product != NULL) {
        return 1;
    }
    dl_tensor_release(product);
    dl_tensor_release(b);
    dl_tensor_release(a);
    dl_tensor_release(NULL);   /* release functions accept NULL */
    puts("c17 lifecycle ok");
    return 0;
}
