/* dl/onnx_c_api.h -- the reference's include path for its ONNX extension (extensions/onnx/include/dl/onnx_c_api.h).  Of that
 * extension this library provides dl_onnx_save_decoder, declared in ctorch_b200_c_api.h; the generic graph exporter
 * (dl_onnx_save over a traced dl_graph) belongs to the reference's tracing layer and is not part of the decoder path. */
#ifndef CTORCH_ONNX_C_API_H
#define CTORCH_ONNX_C_API_H

#include "c_api.h"

#endif
