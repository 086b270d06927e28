/*
 * libFHErt_b200 -- CKKS runtime for NVIDIA B200 (sm_100a) behind the C runtime
 * API that the ANT-ACE FHE compiler emits calls against.
 *
 * Every entry point below keeps the name, argument meaning and result of the
 * CPU runtime function it replaces; the comment on each group cites that
 * function as <file>:<line> inside fhe-cmplr/rtlib/ of the ANT-ACE tree.
 *
 * Data model
 *   - A polynomial is limb-major: limb i (residues modulo one RNS prime) is the
 *     N contiguous int64 words at _data + i*N.  Q limbs come first, the K
 *     special ("P") limbs sit at the end of the allocation
 *     (ant/poly/include/rns_poly_impl.h:43).  Generated code does pointer
 *     arithmetic on _data, so this layout is part of the ABI.
 *   - _data is a DEVICE pointer.  Host code may compute addresses from it but
 *     must not dereference it; use Fhert_upload / Fhert_download to move
 *     residues between host buffers and polynomials.
 *   - All work is queued on one CUDA stream owned by the library
 *     (Fhert_stream); calls return as soon as their kernels are queued.
 *     Fhert_download and Fhert_sync wait for completion.
 *   - Errors: like the CPU runtime (include/common/error.h:17-32) a failed
 *     precondition prints a message and aborts.  There is no CPU fallback: if
 *     no CUDA device is usable the first call aborts.
 */
#ifndef FHERT_B200_H
#define FHERT_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------ */
/* Types (field names are those generated programs touch directly)          */
/* ------------------------------------------------------------------------ */

/* ant/include/util/modular.h:21-26 */
typedef struct {
  int64_t           _val;
  int64_t           _br_k;
  int64_t           _br_m;
  unsigned __int128 _prec128;
} MODULUS;

/* ant/include/poly/rns_poly.h:23-32 */
typedef struct {
  uint32_t _ring_degree;
  size_t   _num_alloc_primes;
  size_t   _num_primes;
  size_t   _num_primes_p;
  bool     _is_ntt;
  int64_t* _data; /* device memory */
} POLYNOMIAL;
typedef POLYNOMIAL* POLY;
typedef POLYNOMIAL* POLY_ARR;

/* ant/include/ckks/ciphertext.h:29-35, 260-267; plaintext.h:26-31 */
typedef struct {
  POLYNOMIAL _c0_poly;
  POLYNOMIAL _c1_poly;
  uint32_t   _slots;
  double     _scaling_factor;
  uint32_t   _sf_degree;
} CIPHERTEXT;
typedef CIPHERTEXT* CIPHER;

typedef struct {
  POLYNOMIAL _c0_poly;
  POLYNOMIAL _c1_poly;
  POLYNOMIAL _c2_poly;
  uint32_t   _slots;
  double     _scaling_factor;
  uint32_t   _sf_degree;
} CIPHERTEXT3;
typedef CIPHERTEXT3* CIPHER3;

typedef struct {
  POLYNOMIAL _poly;
  uint32_t   _slots;
  double     _scaling_factor;
  uint32_t   _sf_degree;
} PLAINTEXT;
typedef PLAINTEXT* PLAIN;

/* ant/include/ckks/public_key.h:24-27, switch_key.h:27-29.  One hybrid
 * key-switch key: per digit a pair of polynomials over Q u P, NTT form. */
typedef struct {
  POLYNOMIAL _p0;
  POLYNOMIAL _p1;
} PUBLIC_KEY;
typedef struct {
  size_t      _num_parts;
  PUBLIC_KEY* _parts;
} SWITCH_KEY;
typedef SWITCH_KEY* SW_KEY;

/* include/common/common.h:73-85 */
typedef enum { LIB_ANT = 0, LIB_SEAL, LIB_OPENFHE, LIB_PHANTOM, LIB_ACE } LIB_PROV;
typedef struct {
  LIB_PROV _provider;
  uint32_t _poly_degree;
  size_t   _sec_level;
  size_t   _mul_depth;
  size_t   _input_level;
  size_t   _first_mod_size;
  size_t   _scaling_mod_size;
  size_t   _num_q_parts;
  size_t   _hamming_weight;
  size_t   _num_rot_idx;
  int32_t  _rot_idxs[];
} CKKS_PARAMS;

/* Program input/output descriptions (include/common/common.h:23-71,
 * include/common/tensor.h:22-25).  A compiled program hands these to the
 * library through the Get_*_scheme hooks below; field order is part of the
 * interface because programs initialise them positionally. */
typedef enum { NORMAL = 0, CONV, CHANNEL, DIAGONAL } MAP_KIND;
typedef enum { DE_MSG_F32 = 0, DE_MSG_F64, DE_PLAINTEXT } DATA_ENTRY_TYPE;
typedef struct {
  MAP_KIND _kind;   /* only NORMAL is handled, as in the CPU runtime */
  int      _count;  /* elements of this ciphertext; 0 = the whole tensor */
  int      _start;
  int      _pad;    /* elements repeated before and after the chunk */
  int      _stride;
} MAP_DESC;
typedef struct {
  size_t _n, _c, _h, _w;
} SHAPE;
typedef struct {
  const char* _name;
  SHAPE       _shape;
  int         _count; /* ciphertexts this tensor is split into */
  MAP_DESC*   _desc;
} DATA_SCHEME;
typedef struct {
  const char*     _file_name;
  const char*     _file_uuid;
  DATA_ENTRY_TYPE _entry_type;
} RT_DATA_INFO;
typedef struct {
  SHAPE  _shape;
  double _vals[];
} TENSOR;

#ifndef TRUE
#define TRUE 1
#endif
#ifndef FALSE
#define FALSE 0
#endif

/* ------------------------------------------------------------------------ */
/* Context  (ant/context/src/ckks_context.c:84-217, ant/util/src/crt.c)      */
/* ------------------------------------------------------------------------ */

/* Supplied by the compiled program (include/common/rt_api.h:48-80).  The
 * library carries a weak default that returns what Fhert_set_context_params
 * stored, so a host without a compiled program (tests, benchmarks) can create
 * a context too. */
CKKS_PARAMS* Get_context_params(void);
void Fhert_set_context_params(uint32_t degree, size_t num_q, size_t q0_bits,
                              size_t sf_bits, size_t num_q_parts,
                              size_t input_level, size_t hamming_weight,
                              size_t num_rot, const int32_t* rot_idxs);

/* Prepare_context builds the prime chain, the NTT and base-conversion tables
 * (same primes, roots and constants as ckks_context.c:84 -> crt.c:607) and
 * uploads them, then generates secret, public, relinearisation and rotation
 * keys in the CPU runtime's order (ant/ckks/src/key_gen.c:15-38) unless the
 * environment variable FHERT_SKIP_KEYGEN=1 is set, in which case switch keys
 * are supplied with Fhert_import_switch_key. */
void     Prepare_context(void);
void     Finalize_context(void);
uint32_t Degree(void);         /* ckks_context.c:163 */
size_t   Get_q_cnt(void);      /* number of Q primes L */
size_t   Get_p_cnt(void);      /* number of special primes K */
size_t   Get_q_parts(void);    /* dnum */
size_t   Get_part_size(void);  /* alpha = ceil(L/dnum), crt.c:419 */
MODULUS* Q_modulus(void);      /* head of contiguous MODULUS[L], crt.c:1117 */
MODULUS* P_modulus(void);      /* head of contiguous MODULUS[K], crt.c:1121 */
double   Get_default_sc(void); /* 2^sf_bits */

/* primes[0..L) = Q chain, primes[L..L+K) = P chain */
void Fhert_get_primes(int64_t* primes);
/* host copy of one prime's forward / inverse twiddles (w, floor(w*2^64/q))
 * in the bit-reversed order of ant/util/src/ntt.c:91-138 */
void Fhert_get_ntt_tables(size_t prime_idx, int64_t* rou, uint64_t* rou_prec,
                          int64_t* rou_inv, uint64_t* rou_inv_prec,
                          int64_t* degree_inv);

/* ------------------------------------------------------------------------ */
/* Memory  (ant/include/poly/rns_poly.h:109-268, ant/poly/src/rns_poly.c:1319) */
/* ------------------------------------------------------------------------ */

POLY Alloc_poly(uint32_t degree, size_t num_q, size_t num_p);
void Free_poly(POLY poly);
void Alloc_poly_data(POLY poly, uint32_t degree, size_t num_q, size_t num_p);
void Free_poly_data(POLY poly);
void Init_poly_by_size(POLY res, size_t num_q, bool is_ext);
void Copy_poly(POLY res, POLY poly); /* rns_poly.c:57-72 */
int64_t* Coeffs(POLY poly, uint32_t limb, uint32_t degree);
void     Set_coeffs(POLY poly, uint32_t limb, uint32_t degree, int64_t* src);

/* host <-> device: `limbs` consecutive limbs starting at limb `first` of the
 * allocation (P limbs are addressed by their allocation index) */
void Fhert_upload(POLY poly, size_t first, size_t limbs, const int64_t* host);
void Fhert_download(POLY poly, size_t first, size_t limbs, int64_t* host);
void Fhert_sync(void);
void* Fhert_stream(void);                /* cudaStream_t of the library */
uint64_t Fhert_kernel_launches(void);    /* kernels queued since load */
/* bytes copied host->device and device->host since the context was made */
void     Fhert_transfer_bytes(uint64_t* h2d, uint64_t* d2h);
/* Per-kernel device timing: between begin and end every kernel launch is
 * bracketed by CUDA events on the library stream; end waits for the stream and
 * writes one "name launches limbs total_ms" line per kernel into buf (limbs =
 * limbs covered by those launches). */
void   Fhert_profile_begin(void);
size_t Fhert_profile_end(char* buf, size_t cap);

/* ------------------------------------------------------------------------ */
/* Per-limb vector ops  (ant/hal/src/hal.c:15-153)                           */
/* ------------------------------------------------------------------------ */

int64_t* Hw_modadd(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree);
int64_t* Hw_modsub(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree);
int64_t* Hw_modmul(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree);
/* res += a * b */
int64_t* Hw_modmuladd(int64_t* res, int64_t* a, int64_t* b, MODULUS* m, uint32_t degree);
/* res += a * scalar                                      (hal.c:109) */
int64_t* Hw_modmuladd_scalar(int64_t* res, int64_t* a, int64_t scalar, MODULUS* m, uint32_t degree);
int64_t* Hw_modadd_scalar(int64_t* res, int64_t* a, int64_t s, MODULUS* m, uint32_t degree);
int64_t* Hw_modmul_scalar(int64_t* res, int64_t* a, int64_t s, MODULUS* m, uint32_t degree);
/* res = a - scalar                                       (hal.c:56) */
int64_t* Hw_modsub_scalar(int64_t* res, int64_t* a, int64_t s, MODULUS* m, uint32_t degree);
/* res[i] = val[order[i]]; `order` is what Auto_order returned */
int64_t* Hw_rotate(int64_t* res, int64_t* val, int64_t* order, MODULUS* m, uint32_t degree);
/* negacyclic NTT / inverse NTT of one limb of prime `mod_idx` (0..L+K-1),
 * natural -> bit-reversed order and back (ant/util/src/ntt.c:140-330) */
void Hw_ntt(int64_t* res, int64_t* val, size_t mod_idx, uint32_t degree);
void Hw_intt(int64_t* res, int64_t* val, size_t mod_idx, uint32_t degree);

/* ------------------------------------------------------------------------ */
/* RNS polynomial ops  (ant/poly/src/rns_poly.c)                             */
/* ------------------------------------------------------------------------ */

POLY   Conv_poly2ntt_inplace(POLY poly);              /* rns_poly.c:608-699 */
POLY   Conv_ntt2poly_inplace(POLY poly);
void   Conv_poly2ntt(POLY res, POLY poly);               /* rns_poly.c:637 */
void   Conv_ntt2poly(POLY res, POLY poly);               /* rns_poly_impl.c:202 */
POLY   Add_poly(POLY res, POLY a, POLY b);            /* rns_poly.c:852 */
POLY   Sub_poly(POLY res, POLY a, POLY b);            /* rns_poly.c:900 */
POLY   Mul_poly(POLY res, POLY a, POLY b);            /* rns_poly.c:950 */
POLY   Rescale(POLY res, POLY poly);                  /* rns_poly.c:310 */
POLY   Modswitch(POLY res, POLY poly);                /* rns_poly.c:406 */
size_t Num_decomp(POLY poly);                         /* crt.c:1135 */
POLY   Decomp(POLY res, POLY poly, uint32_t part);    /* rns_poly.c:74 */
POLY   Mod_up(POLY res, POLY poly, uint32_t part);    /* rns_poly.c:107 */
POLY   Decomp_modup(POLY res, POLY poly, uint32_t part); /* rns_poly.c:160 */
POLY   Mod_down(POLY res, POLY poly);                 /* rns_poly.c:260 */
POLY   Extend(POLY res, POLY poly);                   /* rns_poly.c:483 */
/* ModDown and Rescale fused, in coefficient form; res gets level-1 limbs in
 * NTT form, poly is left in coefficient form          (rns_poly.c:531) */
POLY   Mod_down_rescale(POLY res, POLY poly);
/* prints "level not match" when the shapes differ     (rns_poly.c:606) */
void   Chk_level(POLY res, POLY p0, POLY p1);
/* res = sum_{j<parts} a[j]*b[j] over Q u P limbs    (rns_poly.c:516) */
POLY   Dot_prod(POLY res, POLY a, POLY b, size_t parts);
/* res[i] = poly[order[i]] on every limb             (rns_poly.c:1056) */
POLY   Automorphism_transform(POLY res, POLY poly, int64_t* order);

/* No counterpart in the CPU runtime.  Rescale for hosts that may not allocate
 * device memory once they are running (a serving loop with a pinned-down
 * memory budget, an embedder whose policy forbids the driver allocator after
 * start-up, a process sharing the GPU with another tenant): same result as
 * Rescale, but the working storage is a 20 MiB device array built into the
 * library instead of a stream-ordered allocation.  `poly` holds `level` limbs
 * in NTT form, `res` receives level-1 limbs (both device buffers of the
 * caller, limb-major; res may alias poly).  Returns 0, or a FHERT_STATIC_*
 * code after printing why: level * N above Fhert_rescale_static_capacity()
 * words is refused, and so is a call made while earlier entry points have
 * deferred work waiting (a Rescale / Mod_down without its sibling, recorded
 * Hw_* calls): that work allocates when it runs, so finish it with Fhert_sync
 * first.  The first call on each device resolves the array's device address
 * and should therefore be made before any stream capture starts.  The entry
 * point itself calls no allocator (with Fhert_profile_begin active each launch
 * records two CUDA events, created on first use).  All calls share the one
 * array: it needs no clearing between calls, but two calls that overlap on
 * the GPU (different streams or host threads) race on it.  A failing CUDA
 * launch aborts like everywhere else in the library. */
enum {
  FHERT_STATIC_OK = 0,
  FHERT_STATIC_NO_CONTEXT = 1,
  FHERT_STATIC_BAD_ARGUMENT = 2,
  FHERT_STATIC_TOO_LARGE = 3,
  FHERT_STATIC_NO_DEVICE = 4,
  FHERT_STATIC_PENDING_WORK = 5
};
int    Fhert_rescale_static(int64_t* res, const int64_t* poly, size_t level);
size_t Fhert_rescale_static_capacity(void); /* words of built-in storage */

/* ------------------------------------------------------------------------ */
/* Keys and automorphism tables  (ant/include/ckks/key.h:25-124)             */
/* ------------------------------------------------------------------------ */

uint32_t Auto_idx(int32_t rot_idx);   /* 5^r mod 2N, number_theory.c:192 */
int64_t* Auto_order(int32_t rot_idx); /* device table, borrowed */
SW_KEY   Swk(bool is_rot, int32_t rot_idx);
POLY     Pk0_at(SW_KEY swk, uint32_t part);
POLY     Pk1_at(SW_KEY swk, uint32_t part);
void     Set_pk0(POLY pk, SW_KEY swk, uint32_t part);
void     Set_pk1(POLY pk, SW_KEY swk, uint32_t part);
/* Installs one polynomial (which = 0/1) of digit `part` of the relinearisation
 * key (is_rot = false) or of the rotation key for rot_idx; host holds L Q
 * limbs followed by K P limbs in NTT form. */
void Fhert_import_switch_key(bool is_rot, int32_t rot_idx, uint32_t part,
                             int which, const int64_t* host);

/* ------------------------------------------------------------------------ */
/* Client side: seeding, encode, encrypt, decrypt, decode                   */
/* ------------------------------------------------------------------------ */

/* Installs the 16-word key and the counter of the BLAKE2Xb generator that
 * uniform and ternary samples come from (ant/util/src/prng.c:13-93) and, when
 * fake_time_us >= 0, the clock value that seeds libc rand() for the triangle
 * error samples (ant/util/src/random_sample.c:25-29).  With the same three
 * values the CPU runtime produces the same keys and ciphertexts.  Without this
 * call the generator seeds itself from the clock and /dev/urandom as the CPU
 * runtime does.  Call before Prepare_context. */
void Fhert_seed(const uint32_t seed[16], uint64_t counter, int64_t fake_time_us);

/* ant/ckks/src/plain.c:29-102 -> encoder.c:234-325 (vectors: inverse canonical
 * embedding on the host, scaling, rounding, RNS split and NTT on the device) and
 * encoder.c:473-575 (len == 1: one scalar on every coefficient) */
void Encode_float(PLAIN plain, float* input, size_t len, uint32_t sc_degree, uint32_t level);
void Encode_double(PLAIN plain, double* input, size_t len, uint32_t sc_degree, uint32_t level);
void Encode_float_mask(PLAIN plain, float cst, size_t len, uint32_t sc_degree, uint32_t level);
void Encode_double_mask(PLAIN plain, double cst, size_t len, uint32_t sc_degree, uint32_t level);
/* input = len (re, im) pairs */
void Encode_dcmplx(PLAIN plain, double* re_im, size_t len, uint32_t sc_degree, uint32_t level);
void Free_plain_data(PLAIN plain);

CIPHER  Encrypt(CIPHER res, PLAIN plain);     /* ant/ckks/src/encryptor.c:19 */
void    Fhert_decrypt(PLAIN res, CIPHER ciph); /* ant/ckks/src/decryptor.c:19 */
/* ant/ckks/src/encoder.c:657: writes `count` (re, im) pairs */
void    Fhert_decode(PLAIN plain, double* out, size_t count);
double* Get_msg(CIPHER ciph);                 /* ant/ckks/src/cipher.c Get_msg */

/* key material as host residues: switch-key polynomials hold L Q limbs then K
 * P limbs; Fhert_export_key: 0 = secret key (coefficient form, L+K limbs),
 * 1 = secret key in NTT form, 2 / 3 = public key polynomials (L limbs) */
void Fhert_export_switch_key(bool is_rot, int32_t rot_idx, uint32_t part, int which,
                             int64_t* host);
void Fhert_export_key(int which, int64_t* host);

/* ------------------------------------------------------------------------ */
/* Ciphertext level  (ant/ckks/src/cipher.c, evaluator.c)                    */
/* ------------------------------------------------------------------------ */

/* Result shaping done by a compiled program before it fills the limbs
 * (ant/ckks/src/cipher.c:27-156, ant/include/ckks/ciphertext.h:109-238).
 * Storage that res already owns is reused when it is large enough: the
 * two-polynomial initialisers keep its contents, the ones that shape res
 * after another object clear it. */
void Init_ciph_same_scale(CIPHER res, CIPHER a, CIPHER b);          /* cipher.c:36, b may be NULL */
void Init_ciph_same_scale_plain(CIPHER res, CIPHER a, PLAIN b);     /* cipher.c:51 */
void Init_ciph_same_scale_ciph3(CIPHER res, CIPHER3 ciph);          /* cipher.c:64 */
void Init_ciph3_same_scale_ciph3(CIPHER3 res, CIPHER3 a, CIPHER3 b); /* cipher.c:77 */
void Init_ciph3_same_scale(CIPHER3 res, CIPHER3 a, CIPHER3 b);
void Init_ciph_up_scale(CIPHER res, CIPHER a, CIPHER b);            /* cipher.c:96 */
void Init_ciph_up_scale_plain(CIPHER res, CIPHER a, PLAIN b);       /* cipher.c:105 */
void Init_ciph3_up_scale(CIPHER3 res, CIPHER a, CIPHER b);          /* cipher.c:118 */
void Init_ciph_down_scale(CIPHER res, CIPHER a);                    /* cipher.c:131 */
void Init_ciph3_down_scale(CIPHER3 res, CIPHER3 a);                 /* cipher.c:144 */
void Copy_ciph(CIPHER res, CIPHER ciph);                            /* cipher.c:158 */
void Zero_ciph(CIPHER ciph);
uint32_t Sc_degree(CIPHER ciph);                                    /* cipher.c:164 */
uint32_t Get_slots(CIPHER ciph);
void     Set_slots(CIPHER ciph, uint32_t slots);
size_t   Poly_level(POLY poly);  /* ant/include/poly/rns_poly.h:41-66 */
size_t   Num_p(POLY poly);
size_t   Num_alloc(POLY poly);
size_t Level(CIPHER ciph);
void   Free_ciph_poly(CIPHER ciph, uint32_t cnt);
CIPHER  Add_ciph(CIPHER res, CIPHER a, CIPHER b);       /* evaluator.c:47 */
CIPHER  Sub_ciph(CIPHER res, CIPHER a, CIPHER b);       /* evaluator.c:118 */
CIPHER3 Mul_ciph3(CIPHER3 res, CIPHER a, CIPHER b);     /* evaluator.c:137 */
CIPHER  Relin(CIPHER res, CIPHER3 ciph);                /* evaluator.c:288 */
CIPHER  Mul_ciph(CIPHER res, CIPHER a, CIPHER b);       /* evaluator.c:177 */
CIPHER  Rescale_ciph(CIPHER res, CIPHER ciph);          /* evaluator.c:344 */
CIPHER  Rotate_ciph(CIPHER res, CIPHER ciph, int32_t rot_idx); /* evaluator.c:503-530 */
CIPHER  Conjugate_ciph(CIPHER res, CIPHER ciph);        /* evaluator.c:568 */

void    Rotate_batch_ciph(CIPHER res_arr, CIPHER ciph, const int32_t* rot_idx,
                          uint32_t count);                  /* cipher.c:460-481, digits raised once */
CIPHER  Add_plain(CIPHER res, CIPHER ciph, PLAIN plain);    /* evaluator.c:98 */
CIPHER  Mul_plain(CIPHER res, CIPHER ciph, PLAIN plain);    /* evaluator.c:192 */
void    Modswitch_ciph(CIPHER ciph);                        /* evaluator.c:401 */
CIPHER  Upscale_ciph(CIPHER res, CIPHER ciph, uint32_t mod_size);    /* evaluator.c:364 */
CIPHER  Downscale_ciph(CIPHER res, CIPHER ciph, uint32_t waterline); /* evaluator.c:380 */
CIPHER  Raise_mod(CIPHER res, CIPHER ciph, uint32_t mod_size);       /* cipher.c:417 */
CIPHER  Mul_mono_ciph(CIPHER res, CIPHER ciph, uint32_t power);      /* evaluator.c:260 */
void    Print_cipher_msg(FILE* fp, const char* name, CIPHER ciph, uint32_t len);
void    Dump_cipher_msg(const char* name, CIPHER ciph, uint32_t len);

/* Polynomial arrays and views (include/poly/rns_poly.h:169-245, include/ckks/key.h:94-118) */
POLY_ARR Alloc_polys(uint32_t cnt, uint32_t degree, size_t num_q, size_t num_p);
void     Free_polys(POLY_ARR polys);
POLY     Init_poly_by_opnd(POLY res, POLY opnd1, POLY opnd2, bool is_ext);
POLY     Swk_c0(POLY res, size_t size, bool is_rot, int32_t rot_idx);
POLY     Swk_c1(POLY res, size_t size, bool is_rot, int32_t rot_idx);
POLY_ARR Precomp(POLY_ARR res, size_t size, POLY input);   /* rns_poly.c:459 */

/* ModDown, rescale and the raise of every digit of the result in one call
 * (poly/src/rns_poly_impl.c:521-620).  poly (level Q limbs and the special
 * limbs) is brought to coefficient form in place; res, which must hold at least
 * level limbs, receives the base conversion of the special limbs (what the
 * CPU runtime leaves there) and loses one level; the value is a list of
 * ceil((level-1)/alpha) polynomials over level-1 Q limbs and the special limbs,
 * in coefficient form, digit d raised to the whole basis.  The list has the
 * layout of the CPU runtime's VALUE_LIST of pointers (include/util/type.h:64-80);
 * Free_precomp releases it together with the polynomials (rns_poly_impl.c:622). */
typedef struct VALUE_LIST {
  int    _type;   /* 0x4000: pointers */
  size_t _length;
  union {
    void**   _p;
    int64_t* _i;
  } _vals;
} VALUE_LIST;
VALUE_LIST* Reduce_and_rescale_modup(POLY res, POLY poly);
void        Free_precomp(VALUE_LIST* precomputed);

/* Single-limb polynomials of the LPOLY emit target
 * (ant/include/lpoly/poly.h:18-143, ant/lpoly/src/poly.c).  `_data` is device
 * memory, so the allocation helpers the reference keeps inline in its header
 * are entry points here; operands are passed by value as there. */
typedef struct {
  uint32_t _ring_degree;
  bool     _is_ntt;
  int64_t* _data;
} L_POLY;
typedef L_POLY* LPOLY;
typedef L_POLY* LPOLY_ARR;
static inline uint32_t Get_lpoly_degree(LPOLY poly) { return poly->_ring_degree; }
static inline int64_t* Get_lpoly_coeffs(LPOLY poly) { return poly->_data; }
static inline bool     Is_lpoly_ntt(LPOLY poly) { return poly->_is_ntt; }
static inline void     Set_lpoly_ntt(LPOLY poly, bool v) { poly->_is_ntt = v; }
static inline bool     Is_lpoly_ntt_match(LPOLY a, LPOLY b) { return a->_is_ntt == b->_is_ntt; }
void  Alloc_lpoly_data(LPOLY poly, uint32_t ring_degree);
void  Init_lpoly_data(LPOLY poly, uint32_t ring_degree, int64_t* data);
void  Free_lpoly_data(LPOLY poly);
LPOLY Alloc_lpoly(uint32_t degree);
void  Free_lpoly(LPOLY poly);
void  Zero_lpoly(LPOLY poly);
void  Copy_lpoly(LPOLY res, L_POLY poly);
LPOLY Add_lpoly(LPOLY sum, L_POLY poly1, L_POLY poly2, MODULUS* mod);
LPOLY Add_scalar(LPOLY res, L_POLY poly, int64_t scalar, MODULUS* mod);
LPOLY Sub_lpoly(LPOLY res, L_POLY poly1, L_POLY poly2, MODULUS* mod);
LPOLY Sub_scalar(LPOLY res, L_POLY poly, int64_t scalar, MODULUS* mod);
LPOLY Mul_lpoly(LPOLY res, L_POLY poly1, L_POLY poly2, MODULUS* mod);
LPOLY Mul_scalar(LPOLY res, L_POLY poly, int64_t scalar, MODULUS* mod);
LPOLY Mac_lpoly(LPOLY res, L_POLY poly1, L_POLY poly2, MODULUS* mod);   /* res += poly1 * poly2 */
LPOLY Mac_scalar(LPOLY res, L_POLY poly, int64_t scalar, MODULUS* mod); /* res += poly * scalar */
void  Ntt(LPOLY res, L_POLY poly, size_t idx);   /* idx: Q primes first, then special primes */
void  Intt(LPOLY res, L_POLY poly, size_t idx);

/* Limb-sharded ciphertext operations for single-ciphertext latency on several
 * GPUs (no reference counterpart: the CPU runtime has no distributed mode).
 * Rank r of `world` owns Q limbs [r*qb, (r+1)*qb) and special limbs
 * [r*pb, (r+1)*pb), qb = ceil(L / world), pb = ceil(K / world)
 * (Fhert_shard_blocks; the owner of a limb is the same at every level).
 * Buffers and ciphertexts use the ordinary limb-major layout with only the
 * owned limbs valid; results equal Rotate_ciph / Conjugate_ciph / Mul_ciph /
 * Rescale_ciph on the owned limbs.
 *
 * Whole operations, exchanges issued by the library as NCCL collectives on its
 * stream (one process per GPU): rank 0 obtains a 128-byte identifier with
 * Fhert_shard_comm_id and passes it to the other ranks by the host's own means;
 * every rank then calls Fhert_shard_comm_init (0 = ok; world = 1 needs neither
 * an identifier nor NCCL).  NCCL is loaded at run time (libnccl.so.2). */
void   Fhert_shard_blocks(size_t level, int world, int* q_block, int* p_block);
int    Fhert_shard_comm_id(void* id128);
int    Fhert_shard_comm_init(const void* id128, int rank, int world);
void   Fhert_shard_comm_destroy(void);
CIPHER Fhert_shard_rotate(CIPHER res, CIPHER ciph, int32_t rot_idx, int is_conj);
CIPHER Fhert_shard_mul_relin(CIPHER res, CIPHER a, CIPHER b);
CIPHER Fhert_shard_rescale(CIPHER res, CIPHER ciph);
/* The same operations as phases between which the caller runs the exchange
 * itself (used to emulate all ranks on one GPU).  Key switch of a polynomial:
 * all-gather gather_q (world*qb limbs) between begin and mid, gather_p0 /
 * gather_p1 (world*pb limbs each) between mid and end, every rank's block in
 * place.  is_conj selects the key: 0 rotation by rot_idx, 1 conjugation,
 * 2 relinearisation (no automorphism; end2 adds add0 / add1 to the two
 * results).  Rescale: the owner of the dropped limb fills bcast (2 limbs) in
 * rescale_begin (returns 1 there), everyone reads it in rescale_end. */
void* Fhert_shard_begin(const int64_t* c1, size_t level, int rank, int world, int64_t* gather_q);
void  Fhert_shard_mid(void* state, const int64_t* c1, const int64_t* gather_q, int32_t rot_idx,
                      int is_conj, int64_t* gather_p0, int64_t* gather_p1);
void  Fhert_shard_end(void* state, const int64_t* c0, const int64_t* gather_p0,
                      const int64_t* gather_p1, int32_t rot_idx, int is_conj, int64_t* out0,
                      int64_t* out1);
void  Fhert_shard_end2(void* state, const int64_t* add0, const int64_t* add1,
                       const int64_t* gather_p0, const int64_t* gather_p1, int32_t rot_idx,
                       int is_conj, int64_t* out0, int64_t* out1);
void  Fhert_shard_tensor(const int64_t* a0, const int64_t* a1, const int64_t* b0, const int64_t* b1,
                         size_t level, int rank, int world, int64_t* d0, int64_t* d1, int64_t* d2);
int   Fhert_shard_rescale_begin(const int64_t* c0, const int64_t* c1, size_t level, int rank,
                                int world, int64_t* bcast);
void  Fhert_shard_rescale_end(const int64_t* c0, const int64_t* c1, size_t level, int rank,
                              int world, const int64_t* bcast, int64_t* res0, int64_t* res1);

/* Bootstrapping (ant/ckks/src/cipher.c:565-583, bootstrap.c:1549-1830): raises
 * an exhausted ciphertext back to level_after_bts levels (0 = as many as the
 * context allows) with the reference's level budget {3, 3}, cosine series and
 * double-angle count.  Prepare_context builds the plaintexts and keys for
 * full packing when the context is deeper than the bootstrap itself, unless
 * RTLIB_DISABLE_BOOTSTRAP_PRECOM is set; other slot counts are prepared on
 * first use (context/src/ckks_context.c:239-262). */
CIPHER Bootstrap(CIPHER res, CIPHER ciph, uint32_t level_after_bts);
void   Bootstrap_precom(uint32_t num_slots);
/* the same bootstrap with an explicit slot count, and its three stages as
 * separately callable steps: CoeffsToSlots (with the raise to the full
 * modulus), EvalMod, SlotsToCoeffs.  The first stage leaves the imaginary-part
 * ciphertext of a fully packed input in a per-thread state that the second
 * stage consumes, as in the CPU runtime   (ckks/src/cipher.c:565-767) */
CIPHER Eval_bootstrap_ciph(CIPHER res, CIPHER ciph, uint32_t level_after_bts, uint32_t num_slots);
CIPHER Eval_bootstrap_coeffs_to_slots_ciph(CIPHER res, CIPHER ciph, uint32_t num_slots);
CIPHER Eval_bootstrap_eval_mod_ciph(CIPHER res, CIPHER ciph, uint32_t num_slots);
CIPHER Eval_bootstrap_slots_to_coeffs_ciph(CIPHER res, CIPHER ciph, uint32_t num_slots);
/* rotation amounts whose keys bootstrapping at this slot count uses (ascending;
 * the conjugation key comes on top); returns how many there are */
size_t Fhert_bootstrap_rotations(uint32_t slots, int32_t* out, size_t cap);
/* host copy of one linear-transform plaintext (its Q limbs, then its K special
 * limbs); returns the Q limb count, 0 when that diagonal does not exist */
size_t Fhert_export_bootstrap_plain(uint32_t slots, int encoding, uint32_t stage, uint32_t index,
                                    int64_t* host);

/* ------------------------------------------------------------------------ */
/* Program driver  (include/common/rt_api.h, ant/ckks/src/rtlib.c:164-244,   */
/* common/src/tensor.c, common/src/rt_stat.c)                                */
/* ------------------------------------------------------------------------ */

/* Hooks the compiled program defines; the library holds weak defaults. */
RT_DATA_INFO* Get_rt_data_info(void);
int           Get_input_count(void);
int           Get_output_count(void);
DATA_SCHEME*  Get_encode_scheme(int idx);
DATA_SCHEME*  Get_decode_scheme(int idx);
bool          Main_graph(void);

TENSOR* Alloc_tensor(size_t n, size_t c, size_t h, size_t w, const double* vals);
void    Free_tensor(TENSOR* tensor);
void    Print_tensor(FILE* fp, TENSOR* tensor);
static inline float* Slice(float* vec, size_t row_idx, size_t col) { return vec + row_idx * col; }

/* encode at the context's input level, encrypt, and park under name */
void       Prepare_input(TENSOR* input, const char* name);
CIPHERTEXT Get_input_data(const char* name, size_t idx); /* polynomials pass to the caller */
void       Set_output_data(const char* name, size_t idx, CIPHER data); /* copies, then frees data */
void       Run_main_graph(void);
double*    Handle_output(const char* name);              /* malloc'ed, caller frees */

/* Replay of a program run.  No counterpart in the CPU runtime.  A program
 * cannot branch on encrypted data, so every run of Main_graph issues the same
 * launches on the same device blocks.  With the mode on (this call, or
 * FHERT_REPLAY=1 in the environment), the first Run_main_graph runs as usual
 * (it fills the plaintext cache and builds the tables made on first use), the
 * second one captures its launches into one CUDA graph while the program's
 * host code runs, and every later one copies the inputs waiting from
 * Prepare_input into the captured input blocks, launches the graph and
 * registers the captured output blocks for Handle_output: one launch per run
 * from the host instead of tens of thousands.  The blocks the captured
 * launches use are kept apart from all other allocations until the mode goes
 * off.  Host data the run copies to the device (constants it encodes, weights
 * when the plaintext cache is off) are snapshotted in pinned memory at capture
 * time, up to FHERT_REPLAY_STAGE_MB (4096) MiB, and replays read the snapshots.
 * The mode goes off by itself, and the run is launched directly, when
 * something in the run cannot be captured (a copy to host memory, a
 * synchronisation, more host data than the snapshot budget);
 * Fhert_replay_state reports it.  The per-operator
 * timer lines (Tm_taken) are off while the mode is on.  Between two replayed
 * runs fetch the result (Handle_output) before the next run overwrites it. */
void Fhert_replay_mode(int on);
/* 0 off (why receives the reason when the mode went off by itself), 1 on and
 * nothing captured yet, 2 replaying; replays = runs served by the graph */
int  Fhert_replay_state(char* why, size_t cap, uint64_t* replays);
/* Shape of the captured graph.  The graph is not the chain of launches in
 * stream order: while a run is captured every launch says which memory it
 * reads and writes, and depends on exactly the launches that last wrote what it
 * reads and last wrote or read what it writes, so independent branches of the
 * program run side by side (FHERT_REPLAY_DAG=0 keeps stream order).  A launch
 * nobody described orders everything before it before everything after it. */
void Fhert_replay_graph(uint64_t* launches, uint64_t* described, uint64_t* dependences,
                        uint64_t* undescribed_barriers, uint64_t* longest_chain);

/* Weight data file named by Get_rt_data_info (message files of floats,
 * fhe-cmplr/include/fhe/core/rt_data_def.h:91-112; opened by Prepare_context)
 * and the plaintexts encoded from it (ant/porting/pt_mgr.c:179-214).
 * FHERT_PT_CACHE_MB=<n> keeps up to n MiB of encoded plaintexts resident in
 * device memory, keyed by (entry, offset, length, scale degree, level); a
 * cached plaintext is lent to the caller and Free_data leaves it alone. */
bool  Pt_mgr_init(const char* fname);
void  Pt_mgr_fini(void);
void* Pt_from_msg(void* pt, uint32_t index, size_t len, uint32_t scale, uint32_t level);
void* Pt_from_msg_ofst(void* pt, uint32_t index, size_t ofst, size_t len, uint32_t scale,
                       uint32_t level);
void  Free_data(void* poly);
void  Fhert_pt_cache_stats(size_t* entries, size_t* bytes, size_t* hits, size_t* misses);
/* on != 0: every Pt_from_msg encodes afresh (as the CPU runtime does) while the cache keeps
 * what it holds; for measuring a program with and without resident weight plaintexts. */
void  Fhert_pt_cache_bypass(int on);

/* Checks emitted by the compiler's run-time validation mode
 * (include/common/rt_validate.h:20-49, common/src/rt_validate.c:16-57) */
void Validate_impl(double* res, double* msg, uint32_t len, int32_t epsilon);
void Validate_value_range(bool within_range);
bool Within_value_range(CIPHER ciph, double* msg, uint32_t len); /* cipher.c:172 */
static inline void Validate(CIPHER ciph, double* msg, uint32_t len, int32_t epsilon) {
  double* res = Get_msg(ciph);
  Validate_impl(res, msg, len, epsilon);
  free(res);
  Validate_value_range(Within_value_range(ciph, msg, len));
}

/* Event timers that newer generated programs bracket their operators with
 * (include/common/rtlib_timing.h:111-160; the ids are the compiler's event
 * numbers and are only used as labels here).  They cost nothing unless
 * RTLIB_TIMING_OUTPUT is set (stdout, stderr or a file name); then every
 * event drains the device so that queued kernels are charged to it, and
 * Finalize_context writes count and seconds per event. */
void Fhert_tm_event(uint32_t id, uint32_t sub, int end);
void Fhert_tm_report(void);
#define RTLIB_TM_START(id, mark) Fhert_tm_event((id), 0, 0)
#define RTLIB_TM_END(id, mark)   Fhert_tm_event((id), 0, 1)
#define CMPLR_TM_START(id, s)    Fhert_tm_event((id), (s), 0)
#define CMPLR_TM_END(id, s)      Fhert_tm_event((id), (s), 1)
#define RTLIB_TM_REPORT()        Fhert_tm_report()

/* per-operator timer; prints "[RT_STAT] <msg> takes <s> seconds." after
 * draining the stream, so queued kernels are charged to their operator */
void Tm_start(const char* msg);
void Tm_taken(const char* msg);

#ifdef __cplusplus
}
#endif

#endif /* FHERT_B200_H */
