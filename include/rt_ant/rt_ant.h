/* Forwarding header: a program emitted by the compiler for the CPU runtime
 * (#include "rt_ant/rt_ant.h") builds against the B200 library unchanged.
 * The limb pointers Coeffs() returns are device addresses: the program may
 * pass them to the Hw_* entry points but must not dereference them. */
#ifndef FHERT_B200_RT_ANT_H
#define FHERT_B200_RT_ANT_H

#include <stdlib.h>
#include <string.h>

#include "../fhert_b200.h"

#endif
