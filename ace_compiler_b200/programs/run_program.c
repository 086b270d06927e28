/* Driver for a program emitted by the ANT-ACE compiler, linked against the
 * B200 runtime.  It plays the part of the hand-written main() that the
 * compiler's users put around a generated file: build the context the program
 * asks for, encrypt one synthetic input tensor per image, run the program's
 * Main_graph, decrypt.  Inputs are seeded uniform[-1, 1) values; timings are
 * wall-clock around each stage with the device drained.
 *
 * usage: run_program [--shape n,c,h,w] [--seed s] [--images k] [--input name]...
 *                    [--output name] [--values m] [--pin p] [--amp a]
 * --input may be given several times for programs with several inputs (each gets
 * a tensor of the same shape, filled in turn from the one seeded stream); a name
 * followed by "=0" gets zeros.  --amp a scales the values to [-a, a).
 * --pin p seeds the library's key / encryption randomness (Fhert_seed) so that two runs
 * produce the same ciphertexts and therefore the same logits, bit for bit.
 * prints one JSON line per image:
 *   {"image": i, "encrypt_s": .., "infer_s": .., "decrypt_s": .., "logits": [..]}
 * and a final line {"setup_s": .., "images": k, "mean_infer_s": ..}.
 * FHERT_DATA_FILE=<path> replaces the weight file path compiled into the
 * program.  FHERT_REPLAY=1 captures the second image's Main_graph as one CUDA
 * graph and replays it for the following images (B200 runtime only); the final
 * line says how many runs the graph served. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "common/rtlib.h"

/* -DREFERENCE_RUNTIME builds the same driver against the reference CPU runtime
 * (its own headers and library plus the test hooks of oracle/ref_hooks.c), so
 * that a program can be run on both sides with the same pinned randomness,
 * the same input and the same weight file, and the outputs compared. */
#ifdef REFERENCE_RUNTIME
void Ref_seed_prng(const uint32_t* seed, uint64_t counter);
void Ref_set_fake_time(int64_t us);
static void Fhert_sync(void) {}
static unsigned long long Fhert_kernel_launches(void) { return 0; }
static void Fhert_seed(const uint32_t* seed, uint64_t counter, int64_t fake_us) {
  Ref_set_fake_time(fake_us);
  Ref_seed_prng(seed, counter);
}
/* the program's own hook is renamed on the command line; this one swaps in
 * the weight file named by FHERT_DATA_FILE, as the B200 runtime does itself */
RT_DATA_INFO* Program_rt_data_info(void);
RT_DATA_INFO* Get_rt_data_info(void) {
  static RT_DATA_INFO info;
  RT_DATA_INFO*       own = Program_rt_data_info();
  if (own == NULL) return NULL;
  info = *own;
  if (getenv("FHERT_DATA_FILE")) info._file_name = getenv("FHERT_DATA_FILE");
  return &info;
}
#endif

static double now_s(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

/* splitmix64: the same stream on every machine */
static uint64_t next_u64(uint64_t* s) {
  uint64_t z = (*s += 0x9E3779B97F4A7C15ull);
  z          = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z          = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

int main(int argc, char** argv) {
  size_t      shape[4] = {1, 3, 32, 32};
  uint64_t    seed     = 1;
  int         images = 1, values = 10;
  long        pin    = -1;
  const char *in_names[8] = {"input"}, *out_name = "output";
  int         n_in = 0;
  double      amp  = 1.0;
  for (int i = 1; i + 1 < argc; i += 2) {
    if (!strcmp(argv[i], "--shape"))
      sscanf(argv[i + 1], "%zu,%zu,%zu,%zu", &shape[0], &shape[1], &shape[2], &shape[3]);
    else if (!strcmp(argv[i], "--seed")) seed = strtoull(argv[i + 1], NULL, 10);
    else if (!strcmp(argv[i], "--images")) images = atoi(argv[i + 1]);
    else if (!strcmp(argv[i], "--values")) values = atoi(argv[i + 1]);
    else if (!strcmp(argv[i], "--pin")) pin = atol(argv[i + 1]);
    else if (!strcmp(argv[i], "--amp")) amp = atof(argv[i + 1]);
    else if (!strcmp(argv[i], "--input") && n_in < 8) in_names[n_in++] = argv[i + 1];
    else if (!strcmp(argv[i], "--output")) out_name = argv[i + 1];
  }
  if (pin >= 0) {
    uint32_t words[16];
    for (int k = 0; k < 16; k++) words[k] = (uint32_t)(pin * 2654435761u + 40503u * k);
    Fhert_seed(words, 0, 1700000000000000ll + pin);
  }
  double t0 = now_s();
  Prepare_context();
  Fhert_sync();
  double setup = now_s() - t0, total = 0;
  size_t count = shape[0] * shape[1] * shape[2] * shape[3];
  if (n_in == 0) n_in = 1;
  for (int img = 0; img < images; img++) {
    double enc = 0;
    for (int k_in = 0; k_in < n_in; k_in++) {
      char        name[64];
      const char* eq   = strchr(in_names[k_in], '=');
      size_t      len  = eq ? (size_t)(eq - in_names[k_in]) : strlen(in_names[k_in]);
      int         zero = eq != NULL && eq[1] == '0';
      if (len >= sizeof(name)) len = sizeof(name) - 1;
      memcpy(name, in_names[k_in], len);
      name[len] = 0;
      TENSOR* t = Alloc_tensor(shape[0], shape[1], shape[2], shape[3], NULL);
      for (size_t k = 0; k < count; k++)
        t->_vals[k] =
            zero ? 0.0 : amp * ((double)(next_u64(&seed) >> 11) / 4503599627370496.0 - 1.0);
      double a0 = now_s();
      Prepare_input(t, name);
      Fhert_sync();
      enc += now_s() - a0;
      Free_tensor(t);
    }
    double b = now_s(), a = b - enc;
    Run_main_graph();
    Fhert_sync();
    double c = now_s();
    double* out = Handle_output(out_name);
    double  d   = now_s();
    printf("{\"image\": %d, \"encrypt_s\": %.6f, \"infer_s\": %.6f, \"decrypt_s\": %.6f, "
           "\"launches\": %llu, \"logits\": [",
           img, b - a, c - b, d - c, (unsigned long long)Fhert_kernel_launches());
    for (int k = 0; k < values; k++) printf("%s%.17g", k ? ", " : "", out[k]);
    printf("]}\n");
    fflush(stdout);
    free(out);
    total += c - b;
  }
  unsigned long long replayed = 0;
  int                replay_state = 0;
  char               why[200]     = "";
#ifndef REFERENCE_RUNTIME
  uint64_t runs = 0;
  replay_state  = Fhert_replay_state(why, sizeof(why), &runs);
  replayed      = runs;
#endif
  printf("{\"setup_s\": %.3f, \"images\": %d, \"mean_infer_s\": %.6f, \"replay_state\": %d, "
         "\"replayed_runs\": %llu, \"replay_off_because\": \"%s\"}\n",
         setup, images, total / (images > 0 ? images : 1), replay_state, replayed, why);
  Finalize_context();
  return 0;
}
