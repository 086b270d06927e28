/* Forwarding header: lets a driver written for the CPU runtime
 * (#include "common/rtlib.h") build against the B200 library unchanged.
 * Everything lives in fhert_b200.h. */
#ifndef FHERT_B200_COMMON_RTLIB_H
#define FHERT_B200_COMMON_RTLIB_H

#include <stdlib.h>

#include "../fhert_b200.h"

/* programs call this from their assertion macro */
static inline void Abort_location(void) { exit(1); }

#endif
