// Build identifier compiled into the library; the Python side compares it with the hash of the
// sources it was shipped with and refuses a stale binary.
#include "api.h"
#ifndef VG_BUILD_ID
#define VG_BUILD_ID "unknown"
#endif
extern "C" const char* vg_build_id(void) { return VG_BUILD_ID; }
