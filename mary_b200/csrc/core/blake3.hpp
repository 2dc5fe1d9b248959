// BLAKE3-256 (unkeyed hash mode), portable C++17.
//
// Content addresses of every blob in a pile are BLAKE3 digests (the reference
// validates blobs with BLAKE3 on first read: src/models/inkling/pile.rs:700-701,
// 816-821).  This is a from-the-specification implementation: 1024-byte chunks,
// 64-byte blocks, 7-round compression, binary tree with the left subtree holding
// the largest power-of-two number of chunks.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace mary {

struct Blake3 {
  static constexpr uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                                     0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
  enum : uint32_t { CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8 };

  static inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

  static inline void g(uint32_t* s, int a, int b, int c, int d, uint32_t mx, uint32_t my) {
    s[a] = s[a] + s[b] + mx; s[d] = rotr(s[d] ^ s[a], 16);
    s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 12);
    s[a] = s[a] + s[b] + my; s[d] = rotr(s[d] ^ s[a], 8);
    s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 7);
  }

  // Full 16-word compression output.
  static void compress(const uint32_t cv[8], const uint32_t block[16], uint64_t counter,
                       uint32_t block_len, uint32_t flags, uint32_t out[16]) {
    static const uint8_t PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
    uint32_t s[16] = {cv[0], cv[1], cv[2], cv[3], cv[4], cv[5], cv[6], cv[7],
                      IV[0], IV[1], IV[2], IV[3],
                      (uint32_t)counter, (uint32_t)(counter >> 32), block_len, flags};
    uint32_t m[16];
    std::memcpy(m, block, 64);
    for (int r = 0; r < 7; ++r) {
      g(s, 0, 4, 8, 12, m[0], m[1]);   g(s, 1, 5, 9, 13, m[2], m[3]);
      g(s, 2, 6, 10, 14, m[4], m[5]);  g(s, 3, 7, 11, 15, m[6], m[7]);
      g(s, 0, 5, 10, 15, m[8], m[9]);  g(s, 1, 6, 11, 12, m[10], m[11]);
      g(s, 2, 7, 8, 13, m[12], m[13]); g(s, 3, 4, 9, 14, m[14], m[15]);
      if (r < 6) {
        uint32_t t[16];
        for (int i = 0; i < 16; ++i) t[i] = m[PERM[i]];
        std::memcpy(m, t, 64);
      }
    }
    for (int i = 0; i < 8; ++i) { out[i] = s[i] ^ s[i + 8]; out[i + 8] = s[i + 8] ^ cv[i]; }
  }

  static inline void load_block(const uint8_t* p, size_t n, uint32_t w[16]) {
    uint8_t buf[64];
    if (n < 64) { std::memset(buf, 0, 64); if (n) std::memcpy(buf, p, n); p = buf; }
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t)p[4 * i] | ((uint32_t)p[4 * i + 1] << 8) | ((uint32_t)p[4 * i + 2] << 16) |
             ((uint32_t)p[4 * i + 3] << 24);
  }

  // A node whose final compression has not been applied yet, so that ROOT can be
  // added when it turns out to be the top of the tree.
  struct Output { uint32_t cv[8]; uint32_t block[16]; uint64_t counter; uint32_t block_len, flags; };

  static void chaining_value(const Output& o, uint32_t cv[8]) {
    uint32_t out[16];
    compress(o.cv, o.block, o.counter, o.block_len, o.flags, out);
    std::memcpy(cv, out, 32);
  }

  static Output chunk_output(const uint8_t* p, size_t n, uint64_t chunk_index) {
    uint32_t cv[8];
    std::memcpy(cv, IV, 32);
    size_t nblocks = n == 0 ? 1 : (n + 63) / 64;
    Output o;
    for (size_t b = 0; b < nblocks; ++b) {
      size_t off = b * 64, len = (n - off) < 64 ? (n - off) : 64;
      if (n == 0) len = 0;
      uint32_t w[16];
      load_block(p + off, len, w);
      uint32_t flags = (b == 0 ? CHUNK_START : 0);
      if (b + 1 == nblocks) {
        std::memcpy(o.cv, cv, 32); std::memcpy(o.block, w, 64);
        o.counter = chunk_index; o.block_len = (uint32_t)len; o.flags = flags | CHUNK_END;
        return o;
      }
      uint32_t out[16];
      compress(cv, w, chunk_index, 64, flags, out);
      std::memcpy(cv, out, 32);
    }
    return o;  // unreachable
  }

  static Output parent_output(const uint32_t l[8], const uint32_t r[8]) {
    Output o;
    std::memcpy(o.cv, IV, 32);
    std::memcpy(o.block, l, 32); std::memcpy(o.block + 8, r, 32);
    o.counter = 0; o.block_len = 64; o.flags = PARENT;
    return o;
  }

  // Subtree over p[0..n), whose first chunk has index chunk0.
  static Output subtree(const uint8_t* p, size_t n, uint64_t chunk0) {
    if (n <= 1024) return chunk_output(p, n, chunk0);
    size_t chunks = (n + 1023) / 1024;
    size_t left = 1;
    while (left * 2 < chunks) left *= 2;
    uint32_t l[8], r[8];
    chaining_value(subtree(p, left * 1024, chunk0), l);
    chaining_value(subtree(p + left * 1024, n - left * 1024, chunk0 + left), r);
    return parent_output(l, r);
  }

  static void hash(const void* data, size_t n, uint8_t out[32]) {
    Output o = subtree((const uint8_t*)data, n, 0);
    uint32_t w[16];
    compress(o.cv, o.block, 0, o.block_len, o.flags | ROOT, w);
    // counter of the root compression is 0 for the first 64 output bytes; for a
    // single chunk o.counter is 0 as well.
    for (int i = 0; i < 8; ++i) {
      out[4 * i] = (uint8_t)w[i]; out[4 * i + 1] = (uint8_t)(w[i] >> 8);
      out[4 * i + 2] = (uint8_t)(w[i] >> 16); out[4 * i + 3] = (uint8_t)(w[i] >> 24);
    }
  }
};

}  // namespace mary
