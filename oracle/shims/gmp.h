/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * Minimal arbitrary-precision integer with the subset of the GMP "mpz"
 * interface that the ANT-ACE CPU runtime uses (fhe-cmplr/rtlib/ant/include/
 * util/bignumber.h:35-84, util/src/number_theory.c:87, ckks/src/encoder.c:681).
 * The reference normally links the system GMP; its header is not available in
 * this build environment, so the reference sources are compiled against this
 * stand-in instead.  All results are exact integers, therefore any correct
 * implementation yields the same values as GMP.
 *
 * Representation: sign-magnitude, little-endian 32-bit limbs.
 */
#ifndef ORACLE_SHIM_GMP_H
#define ORACLE_SHIM_GMP_H

#include <stddef.h>
#include <stdint.h>
#include <stdio.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  int       _mp_alloc; /* limbs allocated */
  int       _mp_size;  /* limbs used; negative for a negative number */
  uint32_t* _mp_d;
} __mpz_struct;

typedef __mpz_struct        mpz_t[1];
typedef __mpz_struct*       mpz_ptr;
typedef const __mpz_struct* mpz_srcptr;

void mpz_init(mpz_ptr x);
void mpz_inits(mpz_ptr x, ...);
void mpz_clear(mpz_ptr x);
void mpz_clears(mpz_ptr x, ...);
void mpz_set(mpz_ptr r, mpz_srcptr a);
void mpz_set_si(mpz_ptr r, long v);
void mpz_set_ui(mpz_ptr r, unsigned long v);
int  mpz_set_str(mpz_ptr r, const char* str, int base);
void mpz_set_d(mpz_ptr r, double d);
void mpz_init_set(mpz_ptr r, mpz_srcptr a);
void mpz_init_set_si(mpz_ptr r, long v);
void mpz_init_set_ui(mpz_ptr r, unsigned long v);
void mpz_init_set_d(mpz_ptr r, double d);

void          mpz_add(mpz_ptr r, mpz_srcptr a, mpz_srcptr b);
void          mpz_add_ui(mpz_ptr r, mpz_srcptr a, unsigned long b);
void          mpz_sub(mpz_ptr r, mpz_srcptr a, mpz_srcptr b);
void          mpz_sub_ui(mpz_ptr r, mpz_srcptr a, unsigned long b);
void          mpz_mul(mpz_ptr r, mpz_srcptr a, mpz_srcptr b);
void          mpz_mul_ui(mpz_ptr r, mpz_srcptr a, unsigned long b);
void          mpz_mul_si(mpz_ptr r, mpz_srcptr a, long b);
void          mpz_addmul(mpz_ptr r, mpz_srcptr a, mpz_srcptr b);
void          mpz_addmul_ui(mpz_ptr r, mpz_srcptr a, unsigned long b);
void          mpz_fdiv_q(mpz_ptr q, mpz_srcptr n, mpz_srcptr d);
void          mpz_fdiv_r(mpz_ptr r, mpz_srcptr n, mpz_srcptr d);
unsigned long mpz_fdiv_q_ui(mpz_ptr q, mpz_srcptr n, unsigned long d);
unsigned long mpz_fdiv_r_ui(mpz_ptr r, mpz_srcptr n, unsigned long d);
void          mpz_fdiv_q_2exp(mpz_ptr q, mpz_srcptr n, unsigned long bits);
void          mpz_mul_2exp(mpz_ptr r, mpz_srcptr a, unsigned long bits);
void          mpz_powm(mpz_ptr r, mpz_srcptr b, mpz_srcptr e, mpz_srcptr m);
void          mpz_pow_ui(mpz_ptr r, mpz_srcptr b, unsigned long e);
void          mpz_sqrt(mpz_ptr r, mpz_srcptr a);
int           mpz_invert(mpz_ptr r, mpz_srcptr a, mpz_srcptr m);

int           mpz_cmp(mpz_srcptr a, mpz_srcptr b);
int           mpz_cmp_si(mpz_srcptr a, long b);
long          mpz_get_si(mpz_srcptr a);
unsigned long mpz_get_ui(mpz_srcptr a);
double        mpz_get_d(mpz_srcptr a);
double        mpz_get_d_2exp(signed long* exp, mpz_srcptr a);
int           mpz_fits_slong_p(mpz_srcptr a);
size_t        mpz_sizeinbase(mpz_srcptr a, int base);

/* printf family understanding only %Zd in addition to what vfprintf does for
 * formats without any other conversion of a bigint. */
int gmp_fprintf(FILE* fp, const char* fmt, ...);
int gmp_printf(const char* fmt, ...);

#ifdef __cplusplus
}
#endif

#endif /* ORACLE_SHIM_GMP_H */
