/* dl/export.h -- export macro of the library (the reference generates this header with CMake's
 * generate_export_header: CMakeLists.txt:139-147; macro DL_API, static define CTORCH_STATIC_DEFINE). */
#ifndef DL_EXPORT_H
#define DL_EXPORT_H

#ifndef DL_API
#if defined(CTORCH_STATIC_DEFINE) || !defined(__GNUC__)
#define DL_API
#else
#define DL_API __attribute__((visibility("default")))
#endif
#endif
#ifndef DL_NO_EXPORT
#if defined(__GNUC__) && !defined(CTORCH_STATIC_DEFINE)
#define DL_NO_EXPORT __attribute__((visibility("hidden")))
#else
#define DL_NO_EXPORT
#endif
#endif
#ifndef DL_DEPRECATED
#define DL_DEPRECATED
#endif

#endif
