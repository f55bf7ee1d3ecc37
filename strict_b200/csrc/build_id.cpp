// The identity of the sources this library was built from: strict_b200/build.py hashes every file
// under csrc/ and the public header and passes the first 16 hex digits here, so a run can report
// whether the binary it loaded matches the sources beside it.
#include "../../include/strictb200.h"

#ifndef SB_BUILD_ID
#define SB_BUILD_ID "unstamped"
#endif

extern "C" const char* strictb200_build_id(void) { return SB_BUILD_ID " " __DATE__ " " __TIME__; }
