/* TEST INFRASTRUCTURE ONLY.
 *
 * Programs emitted by an older compiler (all committed ResNet files) call
 * Alloc_poly(degree, level, is_ext) with a boolean third argument, while the
 * current reference runtime takes the number of special limbs there
 * (fhe-cmplr/rtlib/ant/include/poly/rns_poly.h:147).  When such a program is
 * built against the reference runtime for a twin run, this header (force-
 * included after the runtime's own) turns any non-zero third argument into
 * "all special limbs", which is what the B200 runtime's Alloc_poly does
 * itself. */
#ifndef ORACLE_OLD_PROGRAM_ADAPTER_H
#define ORACLE_OLD_PROGRAM_ADAPTER_H
#include "rt_ant/rt_ant.h" /* the runtime's own declarations first */
#define Alloc_poly(degree, num_q, is_ext) (Alloc_poly)((degree), (num_q), (is_ext) ? Get_p_cnt() : 0)
#endif
