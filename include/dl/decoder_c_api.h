/* dl/decoder_c_api.h -- the reference's include path for the decoder entry points (include/dl/decoder_c_api.h:11-41 there):
 * dl_tensordot, dl_rotary_embedding, dl_grouped_query_attention, the module constructors, the decoder cache and
 * dl_transformer_decoder_decode.  All of them are declared in ctorch_b200_c_api.h. */
#ifndef CTORCH_DECODER_C_API_H
#define CTORCH_DECODER_C_API_H

#include "c_api.h"

#endif
