// Randomness of the key generator and the encryptor, host side.
//
// The CPU runtime draws uniform and ternary samples from a BLAKE2Xb-based
// generator (fhe-cmplr/rtlib/ant/util/include/prng_impl.h:41-93: the hash of a
// 64-bit counter under a 64-byte key yields 1024 32-bit words per refill) and
// "triangle" error samples from libc rand() re-seeded from the clock on every
// call (util/src/random_sample.c:25-29, 80-99).  Both are reproduced here so
// that identical seeds give identical keys and ciphertexts.  BLAKE2b follows
// RFC 7693, the extendable-output layering the BLAKE2X specification.
#include <fcntl.h>
#include <sys/time.h>
#include <unistd.h>

#include <cmath>
#include <cstring>

#include "runtime.h"

namespace fhert {

namespace {

// ---- BLAKE2b ----------------------------------------------------------------

const u64 kB2Iv[8] = {0x6a09e667f3bcc908ULL, 0xbb67ae8584caa73bULL, 0x3c6ef372fe94f82bULL,
                      0xa54ff53a5f1d36f1ULL, 0x510e527fade682d1ULL, 0x9b05688c2b3e6c1fULL,
                      0x1f83d9abfb41bd6bULL, 0x5be0cd19137e2179ULL};

const uint8_t kB2Sigma[10][16] = {
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15},
    {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
    {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4},
    {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
    {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13},
    {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
    {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11},
    {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
    {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5},
    {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0}};

inline u64 rotr(u64 x, int n) { return (x >> n) | (x << (64 - n)); }

// One-shot hasher for messages of at most two blocks after the key block, which
// is all the generator needs (8-byte counter, or the 64-byte root hash).
class Blake2b {
 public:
  // param words 0 and 1 carry digest/key length, fanout, depth, leaf length,
  // node offset and the XOF length; word 2 node depth and inner length
  Blake2b(uint8_t digest_len, uint8_t key_len, uint8_t fanout, uint8_t depth,
          uint32_t leaf_len, uint32_t node_offset, uint32_t xof_len, uint8_t inner_len) {
    uint8_t p[64];
    std::memset(p, 0, sizeof(p));
    p[0] = digest_len;
    p[1] = key_len;
    p[2] = fanout;
    p[3] = depth;
    std::memcpy(p + 4, &leaf_len, 4);
    std::memcpy(p + 8, &node_offset, 4);
    std::memcpy(p + 12, &xof_len, 4);
    p[17] = inner_len;
    for (int i = 0; i < 8; i++) {
      u64 w;
      std::memcpy(&w, p + 8 * i, 8);
      h_[i] = kB2Iv[i] ^ w;
    }
    t_   = 0;
    len_ = 0;
  }

  void absorb(const uint8_t* data, size_t n) {
    while (n) {
      if (len_ == 128) {
        t_ += 128;
        compress(false);
        len_ = 0;
      }
      size_t take = std::min(n, (size_t)128 - len_);
      std::memcpy(buf_ + len_, data, take);
      len_ += take;
      data += take;
      n -= take;
    }
  }

  void absorb_key(const uint8_t* key, size_t n) {
    if (!n) return;
    uint8_t block[128];
    std::memset(block, 0, sizeof(block));
    std::memcpy(block, key, n);
    absorb(block, 128);
  }

  void finish(uint8_t* out, size_t n) {
    t_ += len_;
    std::memset(buf_ + len_, 0, 128 - len_);
    compress(true);
    std::memcpy(out, h_, n);
  }

 private:
  void compress(bool last) {
    u64 m[16], v[16];
    std::memcpy(m, buf_, 128);
    for (int i = 0; i < 8; i++) {
      v[i]     = h_[i];
      v[i + 8] = kB2Iv[i];
    }
    v[12] ^= t_;
    if (last) v[14] = ~v[14];
    auto g = [&](int r, int i, int a, int b, int c, int d) {
      v[a] = v[a] + v[b] + m[kB2Sigma[r % 10][2 * i]];
      v[d] = rotr(v[d] ^ v[a], 32);
      v[c] = v[c] + v[d];
      v[b] = rotr(v[b] ^ v[c], 24);
      v[a] = v[a] + v[b] + m[kB2Sigma[r % 10][2 * i + 1]];
      v[d] = rotr(v[d] ^ v[a], 16);
      v[c] = v[c] + v[d];
      v[b] = rotr(v[b] ^ v[c], 63);
    };
    for (int r = 0; r < 12; r++) {
      g(r, 0, 0, 4, 8, 12);
      g(r, 1, 1, 5, 9, 13);
      g(r, 2, 2, 6, 10, 14);
      g(r, 3, 3, 7, 11, 15);
      g(r, 4, 0, 5, 10, 15);
      g(r, 5, 1, 6, 11, 12);
      g(r, 6, 2, 7, 8, 13);
      g(r, 7, 3, 4, 9, 14);
    }
    for (int i = 0; i < 8; i++) h_[i] ^= v[i] ^ v[i + 8];
  }

  u64     h_[8];
  u64     t_;  // byte counter (messages here stay far below 2^64 bytes)
  uint8_t buf_[128];
  size_t  len_;
};

// BLAKE2Xb: root hash over (key block, message) carrying the requested length,
// then one 64-byte BLAKE2b output block per node offset over the root hash.
void blake2xb(uint8_t* out, size_t out_len, const uint8_t* msg, size_t msg_len,
              const uint8_t* key, size_t key_len) {
  Blake2b root(64, (uint8_t)key_len, 1, 1, 0, 0, (uint32_t)out_len, 0);
  root.absorb_key(key, key_len);
  root.absorb(msg, msg_len);
  uint8_t h0[64];
  root.finish(h0, 64);
  uint32_t node = 0;
  for (size_t done = 0; done < out_len; done += 64, node++) {
    size_t  blk = std::min((size_t)64, out_len - done);
    Blake2b leaf((uint8_t)blk, 0, 0, 0, 64, node, (uint32_t)out_len, 64);
    leaf.absorb(h0, 64);
    leaf.finish(out + done, blk);
  }
}

// ---- generator state (util/src/prng.c) ----------------------------------------

constexpr int      kSeedWords = 16;
constexpr int      kBufWords  = 1024;
constexpr uint32_t kMaxU32    = 0xffffffffu;

struct Prng {
  u64      counter = 0;
  uint32_t seed[kSeedWords];
  uint32_t buf[kBufWords];
  int      idx = 0;

  uint32_t next() {
    if (idx == kBufWords) idx = 0;
    if (idx == 0) {
      blake2xb((uint8_t*)buf, sizeof(buf), (const uint8_t*)&counter, sizeof(counter),
               (const uint8_t*)seed, sizeof(seed));
      counter++;
    }
    return buf[idx++];
  }

  // prng_impl.h:67-88
  uint32_t uniform(uint32_t lo, uint32_t hi) {
    uint32_t range = hi - lo, ret;
    if (range < kMaxU32) {
      range += 1;
      uint32_t scaling = kMaxU32 / range, past = range * scaling;
      do ret = next();
      while (ret >= past);
      ret /= scaling;
    } else {
      ret = next();
    }
    return ret + lo;
  }
};

Prng*   g_prng = nullptr;
int64_t g_fake_time_us = -1;

void wall_clock(struct timeval* tv) {
  if (g_fake_time_us >= 0) {
    tv->tv_sec  = g_fake_time_us / 1000000;
    tv->tv_usec = g_fake_time_us % 1000000;
  } else {
    gettimeofday(tv, nullptr);
  }
}

uint32_t random_device_word() {
  uint32_t v  = 0;
  int      fd = open("/dev/urandom", O_RDONLY);
  FHERT_ASSERT(fd >= 0, "Failed to open /dev/urandom");
  ssize_t n = read(fd, &v, sizeof(v));
  FHERT_ASSERT(n == (ssize_t)sizeof(v), "Failed to read from /dev/urandom");
  close(fd);
  return v;
}

// prng.c:62-93: unless a seed was installed, seed from a clock-seeded generator
// plus the random device
Prng* prng() {
  if (g_prng) return g_prng;
  g_prng = new Prng();
  Prng gen;
  std::memset(gen.seed, 0, sizeof(gen.seed));
  struct timeval tv;
  wall_clock(&tv);
  gen.seed[0] = (uint32_t)((u64)tv.tv_sec >> 32);
  gen.seed[1] = (uint32_t)tv.tv_usec;
  void* probe = std::malloc(1);
  gen.counter = (uint32_t)(intptr_t)probe;
  std::free(probe);
  for (int i = 0; i < kSeedWords; i++)
    g_prng->seed[i] = gen.uniform(0, kMaxU32) + random_device_word();
  return g_prng;
}

}  // namespace

void seed_prng(const uint32_t seed[16], u64 counter, int64_t fake_time_us) {
  delete g_prng;
  g_prng = new Prng();
  std::memcpy(g_prng->seed, seed, sizeof(g_prng->seed));
  g_prng->counter = counter;
  g_fake_time_us  = fake_time_us;
}

void release_prng() {
  delete g_prng;
  g_prng = nullptr;
}

// random_sample.c:41-78 (PRNG branch): 32-bit chunks, last chunk bounded,
// rejection until below the bound
void sample_uniform(int64_t* out, size_t n, u64 upper_bound) {
  Prng*    p           = prng();
  uint32_t full_chunks = (uint32_t)std::log2((double)upper_bound) / 32;
  uint32_t shift_chunk = full_chunks * 32;
  uint32_t last_bound  = (uint32_t)(upper_bound >> shift_chunk);
  for (size_t i = 0; i < n; i++) {
    for (;;) {
      u64 r = 0;
      for (uint32_t k = 0, sh = 0; k < full_chunks; k++, sh += 32)
        r += (u64)p->uniform(0, kMaxU32) << sh;
      r += (u64)p->uniform(0, last_bound) << shift_chunk;
      if (r < upper_bound) {
        out[i] = (int64_t)r;
        break;
      }
    }
  }
}

// random_sample.c:101-154 (PRNG branch)
void sample_ternary(int64_t* out, size_t n, size_t hamming_weight) {
  Prng* p = prng();
  if (hamming_weight == 0) {
    for (size_t i = 0; i < n; i++) out[i] = (int64_t)(int32_t)p->uniform((uint32_t)-1, 1);
    return;
  }
  if (hamming_weight > n) hamming_weight = n;
  int64_t hw      = (int64_t)hamming_weight;
  int32_t one_cnt = 0;
  while (one_cnt < hw / 2 - 1 || one_cnt > hw / 2 + 1) {
    one_cnt = 0;
    std::memset(out, 0, n * sizeof(int64_t));
    int64_t total = 0;
    while (total < hw) {
      uint32_t index = p->uniform(0, (uint32_t)n - 1);
      if (out[index] == 0) {
        if ((int32_t)p->uniform(0, 1) == 0) {
          out[index] = -1;
        } else {
          out[index] = 1;
          one_cnt++;
        }
        total++;
      }
    }
  }
}

// random_sample.c:25-35, 80-99: libc rand() re-seeded from the clock
void sample_triangle(int64_t* out, size_t n) {
  struct timeval tv;
  wall_clock(&tv);
  srand((unsigned)(tv.tv_usec * tv.tv_sec));
  for (size_t i = 0; i < n; i++) {
    int64_t r = rand() % 4;
    out[i]    = r == 0 ? -1 : (r == 1 ? 1 : 0);
  }
}

}  // namespace fhert
