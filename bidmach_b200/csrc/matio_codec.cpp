// Byte codecs for BIDMat's compressed matrix files (host code, no CUDA).
//
// The reference reads its corpora and writes its checkpoints through BIDMat's
// loadMat / saveMat, with the compression chosen by the file extension
// (scripts/getw2vdata.ssc writes "*.imat.lz4"; models/Model.scala:259 writes
// "modelmat%02d.lz4").  BIDMat itself is an un-vendored dependency of the
// reference (pom.xml: BIDMat 2.1.11-cuda9.2), and so is the lz4-java library it
// streams through, so both layers are restated here from their published
// formats:
//   * the LZ4 block format (sequences of token / literals / 16-bit offset /
//     match length, matches at least 4 bytes, the last 5 bytes literals, the
//     last match starting at least 12 bytes before the end);
//   * XXH32, the 32-bit xxHash;
// and, in matio.py, lz4-java's block-stream container around them.
// Pinning: the uncompressed and ".gz" layouts by the reference's own C writers
// (src/main/C/newparse/utils.cpp:350-362); the container and the checksum by
// the one ".lz4" matrix file in the BIDMach checkout
// (scripts/networks/modelmat_test.fmat.lz4, raw blocks only); XXH32 by its
// published test values; the block codec by interoperation with another LZ4
// implementation in the tests.
#include <stdint.h>
#include <string.h>

#include "../../include/bidmach_b200.h"

namespace {

inline uint32_t read32(const uint8_t *p) {
  uint32_t v;
  memcpy(&v, p, 4);
  return v;
}

inline uint32_t rotl(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }

constexpr uint32_t P1 = 2654435761u, P2 = 2246822519u, P3 = 3266489917u, P4 = 668265263u,
                   P5 = 374761393u;

// writes a length >= 15 (or >= 19 for matches) tail: bytes of 255 and a remainder
inline uint8_t *put_length(uint8_t *op, int len) {
  while (len >= 255) {
    *op++ = 255;
    len -= 255;
  }
  *op++ = (uint8_t)len;
  return op;
}

}  // namespace

extern "C" {

uint32_t bidmach_xxh32(const void *data, int64_t len, uint32_t seed) {
  const uint8_t *p = (const uint8_t *)data, *end = p + len;
  uint32_t h;
  if (len >= 16) {
    uint32_t v1 = seed + P1 + P2, v2 = seed + P2, v3 = seed, v4 = seed - P1;
    const uint8_t *limit = end - 16;
    do {
      v1 = rotl(v1 + read32(p) * P2, 13) * P1;
      v2 = rotl(v2 + read32(p + 4) * P2, 13) * P1;
      v3 = rotl(v3 + read32(p + 8) * P2, 13) * P1;
      v4 = rotl(v4 + read32(p + 12) * P2, 13) * P1;
      p += 16;
    } while (p <= limit);
    h = rotl(v1, 1) + rotl(v2, 7) + rotl(v3, 12) + rotl(v4, 18);
  } else {
    h = seed + P5;
  }
  h += (uint32_t)len;
  while (p + 4 <= end) {
    h = rotl(h + read32(p) * P3, 17) * P4;
    p += 4;
  }
  while (p < end) {
    h = rotl(h + (*p) * P5, 11) * P1;
    p++;
  }
  h ^= h >> 15;
  h *= P2;
  h ^= h >> 13;
  h *= P3;
  h ^= h >> 16;
  return h;
}

int64_t bidmach_lz4_compress_bound(int64_t n) { return n + n / 255 + 16; }

// Greedy single-pass compressor: a hash table of the latest position of every
// 4-byte prefix.  Returns the compressed size, or -1 when dst is too small.
int64_t bidmach_lz4_compress(const void *src_, int64_t n, void *dst_, int64_t cap) {
  const uint8_t *src = (const uint8_t *)src_;
  uint8_t *dst = (uint8_t *)dst_, *op = dst;
  if (n < 0 || cap < bidmach_lz4_compress_bound(n)) return -1;
  constexpr int kHashBits = 14;
  static thread_local int32_t table[1 << kHashBits];
  for (int i = 0; i < (1 << kHashBits); i++) table[i] = -1;
  int64_t anchor = 0, ip = 0;
  const int64_t match_limit = n - 12;  // a match may not start past here
  const int64_t copy_limit = n - 5;    // nor extend past here
  while (ip < match_limit) {
    const uint32_t seq = read32(src + ip);
    const uint32_t h = (seq * 2654435761u) >> (32 - kHashBits);
    const int64_t ref = table[h];
    table[h] = (int32_t)ip;
    if (ref < 0 || ip - ref > 65535 || read32(src + ref) != seq) {
      ip++;
      continue;
    }
    int64_t len = 4;
    while (ip + len < copy_limit && src[ref + len] == src[ip + len]) len++;
    const int64_t lit = ip - anchor;
    uint8_t *token = op++;
    if (lit >= 15) {
      *token = 15 << 4;
      op = put_length(op, (int)(lit - 15));
    } else {
      *token = (uint8_t)(lit << 4);
    }
    memcpy(op, src + anchor, (size_t)lit);
    op += lit;
    const uint16_t off = (uint16_t)(ip - ref);
    *op++ = (uint8_t)(off & 255);
    *op++ = (uint8_t)(off >> 8);
    if (len - 4 >= 15) {
      *token |= 15;
      op = put_length(op, (int)(len - 4 - 15));
    } else {
      *token |= (uint8_t)(len - 4);
    }
    ip += len;
    anchor = ip;
  }
  const int64_t lit = n - anchor;  // the rest goes out as literals
  uint8_t *token = op++;
  if (lit >= 15) {
    *token = 15 << 4;
    op = put_length(op, (int)(lit - 15));
  } else {
    *token = (uint8_t)(lit << 4);
  }
  memcpy(op, src + anchor, (size_t)lit);
  op += lit;
  return op - dst;
}

// Returns the decompressed size, or -1 for a malformed block or a dst that is
// too small.  Never reads outside [src, src+n) nor writes outside [dst, dst+cap).
int64_t bidmach_lz4_decompress(const void *src_, int64_t n, void *dst_, int64_t cap) {
  const uint8_t *ip = (const uint8_t *)src_, *iend = ip + n;
  uint8_t *dst = (uint8_t *)dst_, *op = dst, *oend = dst + cap;
  if (n == 0) return 0;
  for (;;) {
    if (ip >= iend) return -1;
    const unsigned token = *ip++;
    int64_t lit = token >> 4;
    if (lit == 15) {
      unsigned b;
      do {
        if (ip >= iend) return -1;
        b = *ip++;
        lit += b;
      } while (b == 255);
    }
    if (lit > iend - ip || lit > oend - op) return -1;
    memcpy(op, ip, (size_t)lit);
    ip += lit;
    op += lit;
    if (ip == iend) break;  // the last sequence has no match
    if (iend - ip < 2) return -1;
    const int64_t off = ip[0] | (ip[1] << 8);
    ip += 2;
    if (off == 0 || off > op - dst) return -1;
    int64_t len = (token & 15);
    if (len == 15) {
      unsigned b;
      do {
        if (ip >= iend) return -1;
        b = *ip++;
        len += b;
      } while (b == 255);
    }
    len += 4;
    if (len > oend - op) return -1;
    const uint8_t *from = op - off;
    if (off >= len) {
      memcpy(op, from, (size_t)len);
      op += len;
    } else {
      for (int64_t k = 0; k < len; k++) *op++ = from[k];  // overlapping copy repeats the pattern
    }
  }
  return op - dst;
}

}  // extern "C"
