// Portable BLAKE3 (hash mode, 32-byte output), written from the public specification.
// Used for the content address of a plan / artifact directory and for cache keys, as the reference
// uses the blake3 crate (crates/skein_ir/src/plan.rs:140, crates/skein_compile/src/search_cache.rs:36-55).
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace skein {
namespace blake3_detail {

constexpr uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                            0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
constexpr int MSG_PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
enum : uint32_t { CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8 };
constexpr size_t BLOCK = 64, CHUNK = 1024;

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

inline void g(uint32_t* s, int a, int b, int c, int d, uint32_t mx, uint32_t my) {
  s[a] = s[a] + s[b] + mx; s[d] = rotr(s[d] ^ s[a], 16);
  s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 12);
  s[a] = s[a] + s[b] + my; s[d] = rotr(s[d] ^ s[a], 8);
  s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 7);
}

inline void round_fn(uint32_t* s, const uint32_t* m) {
  g(s, 0, 4, 8, 12, m[0], m[1]);   g(s, 1, 5, 9, 13, m[2], m[3]);
  g(s, 2, 6, 10, 14, m[4], m[5]);  g(s, 3, 7, 11, 15, m[6], m[7]);
  g(s, 0, 5, 10, 15, m[8], m[9]);  g(s, 1, 6, 11, 12, m[10], m[11]);
  g(s, 2, 7, 8, 13, m[12], m[13]); g(s, 3, 4, 9, 14, m[14], m[15]);
}

// out: 16 words (first 8 = chaining value)
inline void compress(const uint32_t cv[8], const uint32_t block_words[16], uint64_t counter, uint32_t block_len,
                     uint32_t flags, uint32_t out[16]) {
  uint32_t s[16] = {cv[0], cv[1], cv[2], cv[3], cv[4], cv[5], cv[6], cv[7],
                    IV[0], IV[1], IV[2], IV[3], (uint32_t)counter, (uint32_t)(counter >> 32), block_len, flags};
  uint32_t m[16];
  memcpy(m, block_words, sizeof m);
  for (int r = 0; r < 7; ++r) {
    round_fn(s, m);
    if (r < 6) {
      uint32_t p[16];
      for (int i = 0; i < 16; ++i) p[i] = m[MSG_PERM[i]];
      memcpy(m, p, sizeof m);
    }
  }
  for (int i = 0; i < 8; ++i) { s[i] ^= s[i + 8]; s[i + 8] ^= cv[i]; }
  memcpy(out, s, sizeof s);
}

inline void words_from_bytes(const uint8_t* b, size_t len, uint32_t w[16]) {
  uint8_t buf[64] = {0};
  memcpy(buf, b, len);
  for (int i = 0; i < 16; ++i)
    w[i] = (uint32_t)buf[4 * i] | ((uint32_t)buf[4 * i + 1] << 8) | ((uint32_t)buf[4 * i + 2] << 16) | ((uint32_t)buf[4 * i + 3] << 24);
}

struct Output {
  uint32_t cv[8];
  uint32_t block[16];
  uint64_t counter;
  uint32_t block_len;
  uint32_t flags;
  void chaining_value(uint32_t out[8]) const {
    uint32_t o[16];
    compress(cv, block, counter, block_len, flags, o);
    memcpy(out, o, 32);
  }
  void root_bytes(uint8_t out[32]) const {
    uint32_t o[16];
    compress(cv, block, 0, block_len, flags | ROOT, o);
    for (int i = 0; i < 8; ++i) {
      out[4 * i] = (uint8_t)o[i]; out[4 * i + 1] = (uint8_t)(o[i] >> 8);
      out[4 * i + 2] = (uint8_t)(o[i] >> 16); out[4 * i + 3] = (uint8_t)(o[i] >> 24);
    }
  }
};

// Output of one chunk (up to 1024 bytes) numbered `chunk_counter`.
inline Output chunk_output(const uint8_t* data, size_t len, uint64_t chunk_counter) {
  uint32_t cv[8];
  memcpy(cv, IV, sizeof cv);
  size_t nblocks = len == 0 ? 1 : (len + BLOCK - 1) / BLOCK;
  Output o{};
  for (size_t b = 0; b < nblocks; ++b) {
    size_t off = b * BLOCK;
    size_t bl = len - off < BLOCK ? len - off : BLOCK;
    if (len == 0) bl = 0;
    uint32_t w[16];
    words_from_bytes(data + off, bl, w);
    uint32_t flags = (b == 0 ? CHUNK_START : 0) | (b + 1 == nblocks ? CHUNK_END : 0);
    if (b + 1 == nblocks) {
      memcpy(o.cv, cv, sizeof cv);
      memcpy(o.block, w, sizeof w);
      o.counter = chunk_counter; o.block_len = (uint32_t)bl; o.flags = flags;
    } else {
      uint32_t out[16];
      compress(cv, w, chunk_counter, (uint32_t)bl, flags, out);
      memcpy(cv, out, sizeof cv);
    }
  }
  return o;
}

inline Output parent_output(const uint32_t left[8], const uint32_t right[8]) {
  Output o{};
  memcpy(o.cv, IV, sizeof o.cv);
  memcpy(o.block, left, 32);
  memcpy(o.block + 8, right, 32);
  o.counter = 0; o.block_len = BLOCK; o.flags = PARENT;
  return o;
}

// Hash of the subtree over data[0..len) whose first chunk is numbered `first_chunk`.
inline Output subtree(const uint8_t* data, size_t len, uint64_t first_chunk) {
  if (len <= CHUNK) return chunk_output(data, len, first_chunk);
  // the left subtree takes the largest power-of-two number of chunks that leaves at least one byte on the right
  size_t full_chunks = (len - 1) / CHUNK;
  size_t left_chunks = 1;
  while (left_chunks * 2 <= full_chunks) left_chunks *= 2;
  size_t left_len = left_chunks * CHUNK;
  uint32_t l[8], r[8];
  subtree(data, left_len, first_chunk).chaining_value(l);
  subtree(data + left_len, len - left_len, first_chunk + left_chunks).chaining_value(r);
  return parent_output(l, r);
}

}  // namespace blake3_detail

inline std::vector<uint8_t> blake3(const void* data, size_t len) {
  std::vector<uint8_t> out(32);
  blake3_detail::subtree(static_cast<const uint8_t*>(data), len, 0).root_bytes(out.data());
  return out;
}

inline std::string blake3_hex(const std::string& s) {
  auto h = blake3(s.data(), s.size());
  static const char* d = "0123456789abcdef";
  std::string hex;
  for (uint8_t b : h) { hex += d[b >> 4]; hex += d[b & 15]; }
  return hex;
}

}  // namespace skein
