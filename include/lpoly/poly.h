/* Forwarding header: code written against the CPU runtime's single-limb
 * polynomial interface (#include "lpoly/poly.h") builds against the B200
 * library unchanged. */
#ifndef FHERT_B200_LPOLY_POLY_H
#define FHERT_B200_LPOLY_POLY_H

#include <stdlib.h>
#include <string.h>

#include "../fhert_b200.h"

#endif
