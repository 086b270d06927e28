/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * Determinism hooks linked into the build of the unmodified reference runtime
 * (oracle/_ref).  They live outside the reference sources:
 *
 *  - Ref_seed_prng(): pre-sets the reference's global BLAKE2 PRNG
 *    (fhe-cmplr/rtlib/ant/util/src/prng.c:13) with a caller-chosen 16-word
 *    seed and counter, so that Get_prng() never reads the clock or
 *    /dev/urandom (prng.c:62-93).
 *  - gettimeofday()/time() interposers: Srand_time()
 *    (util/src/random_sample.c:25) and Is_prime (number_theory.c:175) seed
 *    libc rand() from the wall clock; with REF_FAKE_TIME set they see a fixed
 *    instant instead.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdint.h>
#include <stdlib.h>
#include <sys/time.h>
#include <time.h>

#include "prng_impl.h"

extern BLAKE2_PRNG* Prng;
#ifdef _OPENMP
#pragma omp threadprivate(Prng) /* as the reference declares it in its OpenMP build (prng.c:13-14) */
#endif
BLAKE2_PRNG*        Alloc_blake2_prng();
void                Free_prng();

void Ref_seed_prng(const uint32_t seed[16], uint64_t counter) {
  Free_prng();
  Prng = Alloc_blake2_prng();
  for (uint32_t i = 0; i < SEED_CNT; i++) Set_ui32_value(Prng->_seed, i, seed[i]);
  Prng->_counter    = counter;
  Prng->_buffer_idx = 0;
}

static int64_t Fake_time_us = -1;

void Ref_set_fake_time(int64_t usec_since_epoch) { Fake_time_us = usec_since_epoch; }

int gettimeofday(struct timeval* restrict tv, void* restrict tz) {
  (void)tz;
  if (Fake_time_us >= 0) {
    tv->tv_sec  = Fake_time_us / 1000000;
    tv->tv_usec = Fake_time_us % 1000000;
    return 0;
  }
  struct timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  tv->tv_sec  = ts.tv_sec;
  tv->tv_usec = ts.tv_nsec / 1000;
  return 0;
}

time_t time(time_t* t) {
  time_t v;
  if (Fake_time_us >= 0) {
    v = (time_t)(Fake_time_us / 1000000);
  } else {
    struct timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    v = ts.tv_sec;
  }
  if (t) *t = v;
  return v;
}
