/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * Declaration of the one BLAKE2 entry point the ANT-ACE CPU runtime calls
 * (fhe-cmplr/rtlib/ant/util/include/prng_impl.h:43): the BLAKE2Xb
 * extendable-output function with a key.  Implemented in blake2xb.c of this
 * directory from the public specifications (RFC 7693 for BLAKE2b; the BLAKE2X
 * paper for the XOF construction).  The upstream build fetches the BLAKE2
 * project at an unpinned revision; the keyed BLAKE2b core here is checked
 * against Python's hashlib, the XOF layering has no independent check.
 */
#ifndef ORACLE_SHIM_BLAKE2_H
#define ORACLE_SHIM_BLAKE2_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int blake2xb(void* out, size_t outlen, const void* in, size_t inlen,
             const void* key, size_t keylen);

/* plain (optionally keyed) BLAKE2b, exported for the hashlib cross-check */
int blake2b(void* out, size_t outlen, const void* in, size_t inlen,
            const void* key, size_t keylen);

#ifdef __cplusplus
}
#endif

#endif /* ORACLE_SHIM_BLAKE2_H */
