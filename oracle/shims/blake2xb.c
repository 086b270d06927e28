/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * BLAKE2b (RFC 7693) and the BLAKE2Xb extendable-output construction, written
 * from the public specifications.  See blake2.h in this directory.
 */
#include "blake2.h"

#include <string.h>

static const uint64_t kIv[8] = {
    0x6a09e667f3bcc908ULL, 0xbb67ae8584caa73bULL, 0x3c6ef372fe94f82bULL,
    0xa54ff53a5f1d36f1ULL, 0x510e527fade682d1ULL, 0x9b05688c2b3e6c1fULL,
    0x1f83d9abfb41bd6bULL, 0x5be0cd19137e2179ULL};

static const uint8_t kSigma[12][16] = {
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15},
    {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
    {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4},
    {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
    {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13},
    {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
    {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11},
    {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
    {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5},
    {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0},
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15},
    {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3}};

typedef struct {
  uint64_t h[8];
  uint64_t t[2];
  uint8_t  buf[128];
  size_t   buflen;
  size_t   outlen;
} B2B_STATE;

/* 64-byte parameter block, little-endian fields */
typedef struct {
  uint8_t  digest_length;
  uint8_t  key_length;
  uint8_t  fanout;
  uint8_t  depth;
  uint32_t leaf_length;
  uint32_t node_offset;
  uint32_t xof_length;
  uint8_t  node_depth;
  uint8_t  inner_length;
} B2B_PARAM;

static inline uint64_t Rotr64(uint64_t x, int n) {
  return (x >> n) | (x << (64 - n));
}

static inline uint64_t Load64(const uint8_t* p) {
  uint64_t v;
  memcpy(&v, p, 8); /* little-endian host */
  return v;
}

static void Compress(B2B_STATE* s, const uint8_t block[128], int last) {
  uint64_t m[16], v[16];
  for (int i = 0; i < 16; i++) m[i] = Load64(block + 8 * i);
  for (int i = 0; i < 8; i++) {
    v[i]     = s->h[i];
    v[i + 8] = kIv[i];
  }
  v[12] ^= s->t[0];
  v[13] ^= s->t[1];
  if (last) v[14] = ~v[14];
#define G(r, i, a, b, c, d)                   \
  do {                                        \
    a = a + b + m[kSigma[r][2 * i]];          \
    d = Rotr64(d ^ a, 32);                    \
    c = c + d;                                \
    b = Rotr64(b ^ c, 24);                    \
    a = a + b + m[kSigma[r][2 * i + 1]];      \
    d = Rotr64(d ^ a, 16);                    \
    c = c + d;                                \
    b = Rotr64(b ^ c, 63);                    \
  } while (0)
  for (int r = 0; r < 12; r++) {
    G(r, 0, v[0], v[4], v[8], v[12]);
    G(r, 1, v[1], v[5], v[9], v[13]);
    G(r, 2, v[2], v[6], v[10], v[14]);
    G(r, 3, v[3], v[7], v[11], v[15]);
    G(r, 4, v[0], v[5], v[10], v[15]);
    G(r, 5, v[1], v[6], v[11], v[12]);
    G(r, 6, v[2], v[7], v[8], v[13]);
    G(r, 7, v[3], v[4], v[9], v[14]);
  }
#undef G
  for (int i = 0; i < 8; i++) s->h[i] ^= v[i] ^ v[i + 8];
}

static void Init_param(B2B_STATE* s, const B2B_PARAM* p) {
  uint8_t pb[64];
  memset(pb, 0, sizeof(pb));
  pb[0] = p->digest_length;
  pb[1] = p->key_length;
  pb[2] = p->fanout;
  pb[3] = p->depth;
  memcpy(pb + 4, &p->leaf_length, 4);
  memcpy(pb + 8, &p->node_offset, 4);
  memcpy(pb + 12, &p->xof_length, 4);
  pb[16] = p->node_depth;
  pb[17] = p->inner_length;
  memset(s, 0, sizeof(*s));
  for (int i = 0; i < 8; i++) s->h[i] = kIv[i] ^ Load64(pb + 8 * i);
  s->outlen = p->digest_length;
}

static void Update(B2B_STATE* s, const uint8_t* in, size_t inlen) {
  while (inlen > 0) {
    if (s->buflen == 128) {
      /* buffer full and more input follows: compress a non-final block */
      s->t[0] += 128;
      if (s->t[0] < 128) s->t[1]++;
      Compress(s, s->buf, 0);
      s->buflen = 0;
    }
    size_t take = 128 - s->buflen;
    if (take > inlen) take = inlen;
    memcpy(s->buf + s->buflen, in, take);
    s->buflen += take;
    in += take;
    inlen -= take;
  }
}

static void Final(B2B_STATE* s, uint8_t* out, size_t outlen) {
  s->t[0] += s->buflen;
  if (s->t[0] < s->buflen) s->t[1]++;
  memset(s->buf + s->buflen, 0, 128 - s->buflen);
  Compress(s, s->buf, 1);
  uint8_t full[64];
  memcpy(full, s->h, 64);
  memcpy(out, full, outlen);
}

static void Absorb_key(B2B_STATE* s, const void* key, size_t keylen) {
  if (keylen > 0) {
    uint8_t block[128];
    memset(block, 0, sizeof(block));
    memcpy(block, key, keylen);
    Update(s, block, 128);
  }
}

int blake2b(void* out, size_t outlen, const void* in, size_t inlen,
            const void* key, size_t keylen) {
  if (outlen == 0 || outlen > 64 || keylen > 64) return -1;
  B2B_PARAM p;
  memset(&p, 0, sizeof(p));
  p.digest_length = (uint8_t)outlen;
  p.key_length    = (uint8_t)keylen;
  p.fanout        = 1;
  p.depth         = 1;
  B2B_STATE s;
  Init_param(&s, &p);
  Absorb_key(&s, key, keylen);
  Update(&s, (const uint8_t*)in, inlen);
  Final(&s, (uint8_t*)out, outlen);
  return 0;
}

int blake2xb(void* out, size_t outlen, const void* in, size_t inlen,
             const void* key, size_t keylen) {
  if (out == NULL || outlen == 0 || outlen > 0xFFFFFFFFULL) return -1;
  if (keylen > 64) return -1;
  if (in == NULL && inlen > 0) return -1;
  /* root hash: 64-byte BLAKE2b digest carrying the XOF length */
  B2B_PARAM p;
  memset(&p, 0, sizeof(p));
  p.digest_length = 64;
  p.key_length    = (uint8_t)keylen;
  p.fanout        = 1;
  p.depth         = 1;
  p.xof_length    = (uint32_t)outlen;
  B2B_STATE s;
  Init_param(&s, &p);
  Absorb_key(&s, key, keylen);
  Update(&s, (const uint8_t*)in, inlen);
  uint8_t root[64];
  Final(&s, root, 64);
  /* expansion nodes */
  B2B_PARAM q;
  memset(&q, 0, sizeof(q));
  q.leaf_length  = 64;
  q.inner_length = 64;
  q.xof_length   = (uint32_t)outlen;
  uint8_t* o     = (uint8_t*)out;
  size_t   left  = outlen;
  for (uint32_t i = 0; left > 0; i++) {
    size_t blk      = left < 64 ? left : 64;
    q.digest_length = (uint8_t)blk;
    q.node_offset   = i;
    B2B_STATE c;
    Init_param(&c, &q);
    Update(&c, root, 64);
    Final(&c, o + (size_t)i * 64, blk);
    left -= blk;
  }
  return 0;
}
