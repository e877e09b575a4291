/* dl/version.h -- version macros (the reference configures this header from include/dl/version.h.in). */
#ifndef DL_VERSION_H
#define DL_VERSION_H

#ifndef DL_VERSION
#define DL_VERSION "0.3.0"
#endif
#define DL_VERSION_MAJOR 0
#define DL_VERSION_MINOR 3
#define DL_VERSION_PATCH 0
#ifndef DL_ABI_VERSION
#define DL_ABI_VERSION 1
#endif

#endif
