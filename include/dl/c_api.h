/* dl/c_api.h -- the reference's include path for the generic C entry points (include/dl/c_api.h there).  The subset the
 * decoder token loop needs is declared in ctorch_b200_c_api.h; a program written against <dl/c_api.h> for this path
 * compiles against this directory and links with -lctorch_b200 (or -lctorch, see the build script's reference names). */
#ifndef CTORCH_C_API_H
#define CTORCH_C_API_H

#include "export.h"
#include "version.h"
#include "../ctorch_b200_c_api.h"

#endif
