// Engram n-gram memory, host side: the prime-bucket layout, the XOR-multiplicative n-gram hash, and the
// packed per-rank table files.  Reference: crates/sparkflash-engram/src/{hash,primes,packer,paged}.rs;
// docs/architecture/04-engram.md sections 3-5 and 7 (layout: primes strictly increasing above vocab-1 and never
// reused across (layer, order, head); hash = XOR over shifts of token*multiplier, reduced modulo the bucket
// prime; look-back stops at a dead position and at the sequence start; rows sharded by range over ranks).
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <vector>

namespace {

bool is_prime(int64_t n) {
  if (n < 2) return false;
  if (n % 2 == 0) return n == 2;
  for (int64_t d = 3; d * d <= n; d += 2)
    if (n % d == 0) return false;
  return true;
}

}  // namespace

extern "C" {

// primes[layer][order][head]: walk upwards from `vocab - 1`, restarting at vocab - 1 for every (layer, order)
// but never re-using a prime (the global seen set makes the sequence strictly increasing overall).
void sfb_engram_primes(int64_t vocab, int n_layers, int n_orders, int n_heads, int64_t* out) {
  std::vector<int64_t> seen;
  int k = 0;
  for (int l = 0; l < n_layers; ++l)
    for (int o = 0; o < n_orders; ++o) {
      int64_t cur = vocab - 1;
      for (int h = 0; h < n_heads; ++h) {
        for (;;) {
          ++cur;
          if (!is_prime(cur)) continue;
          bool dup = false;
          for (int64_t s : seen) if (s == cur) { dup = true; break; }
          if (!dup) break;
        }
        seen.push_back(cur);
        out[k++] = cur;
      }
    }
}

// Hash ids of `n` positions of one sequence.  cache: compressed token ids of the sequence (dead positions = -1),
// valid for [0, max(pos)].  multipliers[max_ngram]; primes / offsets for this layer: [n_orders][n_heads] and
// [n_orders] with n_orders = max_ngram - 1.  out: [n, n_orders * n_heads] row ids inside the layer's table.
void sfb_engram_hash(const int64_t* cache, const int32_t* positions, int n, int max_ngram, int n_heads, int64_t pad_id,
                     const int64_t* multipliers, const int64_t* primes, const int64_t* offsets, int64_t* out) {
  const int orders = max_ngram - 1;
  for (int r = 0; r < n; ++r) {
    const int64_t p = positions[r];
    bool blocked = false;
    int64_t rolling = 0;
    for (int s = 0; s < max_ngram; ++s) {
      int64_t src = cache[p - s < 0 ? 0 : p - s];
      blocked = blocked || p < s || src == -1;
      int64_t tok = blocked ? pad_id : src;
      int64_t prod = (int64_t)((uint64_t)tok * (uint64_t)multipliers[s]);
      rolling = s == 0 ? prod : (rolling ^ prod);
      if (s >= 1)
        for (int h = 0; h < n_heads; ++h) {
          int64_t pr = primes[(s - 1) * n_heads + h];
          int64_t m = rolling % pr;            // floor-mod semantics for a (never expected) negative value
          if (m < 0) m += pr;
          out[(size_t)r * orders * n_heads + (s - 1) * n_heads + h] = m + offsets[(s - 1) * n_heads + h];
        }
    }
  }
}

// Pack one rank's row range: rows interleaved as 256 e4m3 bytes + 8 ue8m0 bytes + 8 zero bytes = 272-byte stride
// (16-byte aligned for vector loads).  The tail shard is padded with weight 0 and scale code 127 (= 1.0).
int sfb_engram_pack(const uint8_t* weight, const uint8_t* scale, int64_t rows, int width, int64_t first, int64_t count,
                    uint8_t* out, int stride) {
  const int sb = width / 32;
  if (stride < width + sb) return 1;
  for (int64_t i = 0; i < count; ++i) {
    uint8_t* dst = out + (size_t)i * stride;
    memset(dst, 0, stride);
    int64_t r = first + i;
    if (r < rows) { memcpy(dst, weight + (size_t)r * width, width); memcpy(dst + width, scale + (size_t)r * sb, sb); }
    else memset(dst + width, 127, sb);
  }
  return 0;
}

}  // extern "C"
