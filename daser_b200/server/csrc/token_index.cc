// Native part of the control-plane index: token hashing and the digest table.
//
// The reference hashes in Python through the xxhash wheel and re-hashes every candidate prefix
// of a prompt from scratch (daser/retrieval/prefix.py:63-72: quadratic in the prompt length).
// Here one streaming pass produces the XXH3-128 digest of every block-aligned prefix, or of
// every aligned block, and an open-addressing table keyed by (model tag, digest) answers
// "longest stored prefix" and "which aligned blocks are anchors of stored chunks" in one call,
// with no Python object per probe.
//
// Digests are bit-identical to xxhash's canonical XXH3-128 (seed 0) over little-endian int32
// token ids: the hash itself comes from the system's libxxhash (resolved with dlopen, so the
// library loads and reports "unavailable" where libxxhash is missing, and the Python
// implementation takes over).
#include <dlfcn.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <vector>

#define DASER_API extern "C" __attribute__((visibility("default")))

namespace {

struct XXH128 {
  uint64_t low64, high64;
};
typedef void* (*CreateFn)(void);
typedef int (*FreeFn)(void*);
typedef int (*ResetFn)(void*);
typedef int (*UpdateFn)(void*, const void*, size_t);
typedef XXH128 (*DigestFn)(const void*);
typedef XXH128 (*OneShotFn)(const void*, size_t);

struct Xxh {
  CreateFn create = nullptr;
  FreeFn release = nullptr;
  ResetFn reset = nullptr;
  UpdateFn update = nullptr;
  DigestFn digest = nullptr;
  OneShotFn oneshot = nullptr;
  bool ok = false;
};

const Xxh& xxh() {
  static Xxh x;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = nullptr;
    for (const char* name : {"libxxhash.so.0", "libxxhash.so"}) {
      h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
      if (h) break;
    }
    if (!h) return;
    x.create = (CreateFn)dlsym(h, "XXH3_createState");
    x.release = (FreeFn)dlsym(h, "XXH3_freeState");
    x.reset = (ResetFn)dlsym(h, "XXH3_128bits_reset");
    x.update = (UpdateFn)dlsym(h, "XXH3_128bits_update");
    x.digest = (DigestFn)dlsym(h, "XXH3_128bits_digest");
    x.oneshot = (OneShotFn)dlsym(h, "XXH3_128bits");
    x.ok = x.create && x.release && x.reset && x.update && x.digest && x.oneshot;
  });
  return x;
}

// canonical form: high64 then low64, big-endian (what hexdigest() of the wheel prints)
inline void canonical(const XXH128& d, uint8_t out[16]) {
  for (int i = 0; i < 8; ++i) {
    out[i] = (uint8_t)(d.high64 >> (56 - 8 * i));
    out[8 + i] = (uint8_t)(d.low64 >> (56 - 8 * i));
  }
}

struct Key {
  uint64_t tag;
  uint8_t digest[16];
};
inline bool same(const Key& a, uint64_t tag, const uint8_t* digest) {
  return a.tag == tag && memcmp(a.digest, digest, 16) == 0;
}
inline uint64_t mix(uint64_t tag, const uint8_t* digest) {
  uint64_t a, b;
  memcpy(&a, digest, 8);
  memcpy(&b, digest + 8, 8);
  uint64_t h = a ^ (b * 0x9E3779B97F4A7C15ull) ^ (tag * 0xC2B2AE3D27D4EB4Full);
  h ^= h >> 29;
  h *= 0xBF58476D1CE4E5B9ull;
  h ^= h >> 32;
  return h;
}

enum : uint8_t { EMPTY = 0, FULL = 1, TOMB = 2 };

}  // namespace

// Open addressing, linear probing, tombstones; grows at 70 % load (tombstones included).
struct daser_table {
  std::vector<Key> keys;
  std::vector<int64_t> values;
  std::vector<uint8_t> state;
  int64_t live = 0, used = 0;  // used = live + tombstones
  std::mutex mu;

  explicit daser_table(int64_t hint) {
    int64_t cap = 64;
    while (cap * 7 < hint * 10) cap <<= 1;
    keys.resize(cap);
    values.resize(cap);
    state.assign(cap, EMPTY);
  }
  int64_t find(uint64_t tag, const uint8_t* digest) const {
    const int64_t mask = (int64_t)state.size() - 1;
    for (int64_t i = (int64_t)(mix(tag, digest) & (uint64_t)mask);; i = (i + 1) & mask) {
      if (state[i] == EMPTY) return -1;
      if (state[i] == FULL && same(keys[i], tag, digest)) return i;
    }
  }
  void rehash(int64_t cap) {
    std::vector<Key> ok(std::move(keys));
    std::vector<int64_t> ov(std::move(values));
    std::vector<uint8_t> os(std::move(state));
    keys.assign(cap, Key());
    values.assign(cap, 0);
    state.assign(cap, EMPTY);
    live = used = 0;
    for (size_t i = 0; i < os.size(); ++i)
      if (os[i] == FULL) put(ok[i].tag, ok[i].digest, ov[i]);
  }
  void put(uint64_t tag, const uint8_t* digest, int64_t value) {
    if ((used + 1) * 10 > (int64_t)state.size() * 7) rehash(live * 10 > (int64_t)state.size() * 3 ? (int64_t)state.size() * 2 : (int64_t)state.size());
    const int64_t mask = (int64_t)state.size() - 1;
    int64_t slot = -1;
    for (int64_t i = (int64_t)(mix(tag, digest) & (uint64_t)mask);; i = (i + 1) & mask) {
      if (state[i] == FULL && same(keys[i], tag, digest)) { values[i] = value; return; }
      if (state[i] == TOMB && slot < 0) slot = i;
      if (state[i] == EMPTY) { if (slot < 0) { slot = i; ++used; } break; }
    }
    keys[slot].tag = tag;
    memcpy(keys[slot].digest, digest, 16);
    values[slot] = value;
    state[slot] = FULL;
    ++live;
  }
  bool del(uint64_t tag, const uint8_t* digest) {
    const int64_t i = find(tag, digest);
    if (i < 0) return false;
    state[i] = TOMB;
    --live;
    return true;
  }
};

DASER_API int daser_index_available(void) { return xxh().ok ? 1 : 0; }

// out: 16 bytes, canonical digest of the n tokens.
DASER_API int daser_hash_tokens(const int32_t* tokens, int64_t n, uint8_t* out) {
  if (!xxh().ok || n < 0 || (!tokens && n) || !out) return -1;
  canonical(xxh().oneshot(tokens, (size_t)n * 4), out);
  return 0;
}

// out: 16 bytes per block-aligned prefix tokens[0 : (i + 1) * block]; returns their number.
DASER_API int64_t daser_prefix_digests(const int32_t* tokens, int64_t n, int32_t block, uint8_t* out) {
  if (!xxh().ok || block <= 0 || n < 0 || (!tokens && n) || !out) return -1;
  const int64_t nb = n / block;
  if (nb == 0) return 0;
  void* st = xxh().create();
  if (!st) return -1;
  xxh().reset(st);
  for (int64_t i = 0; i < nb; ++i) {
    xxh().update(st, tokens + i * block, (size_t)block * 4);
    canonical(xxh().digest(st), out + 16 * i);
  }
  xxh().release(st);
  return nb;
}

// out: 16 bytes per aligned block tokens[i * block : (i + 1) * block]; returns their number.
DASER_API int64_t daser_block_digests(const int32_t* tokens, int64_t n, int32_t block, uint8_t* out) {
  if (!xxh().ok || block <= 0 || n < 0 || (!tokens && n) || !out) return -1;
  const int64_t nb = n / block;
  for (int64_t i = 0; i < nb; ++i) canonical(xxh().oneshot(tokens + i * block, (size_t)block * 4), out + 16 * i);
  return nb;
}

// out: 16 bytes per window tokens[i : i + block], i = 0 .. n - block (every token offset: anchors
// of chunks that sit at offsets which are not multiples of the block size); returns their number.
DASER_API int64_t daser_window_digests(const int32_t* tokens, int64_t n, int32_t block, uint8_t* out) {
  if (!xxh().ok || block <= 0 || n < 0 || (!tokens && n) || !out) return -1;
  const int64_t nw = n >= block ? n - block + 1 : 0;
  for (int64_t i = 0; i < nw; ++i) canonical(xxh().oneshot(tokens + i, (size_t)block * 4), out + 16 * i);
  return nw;
}

DASER_API daser_table* daser_table_new(int64_t capacity_hint) { return new daser_table(capacity_hint < 0 ? 0 : capacity_hint); }
DASER_API void daser_table_free(daser_table* t) { delete t; }
DASER_API int64_t daser_table_size(daser_table* t) {
  std::lock_guard<std::mutex> g(t->mu);
  return t->live;
}
DASER_API int daser_table_put(daser_table* t, uint64_t tag, const uint8_t* digest, int64_t value) {
  if (!t || !digest) return -1;
  std::lock_guard<std::mutex> g(t->mu);
  t->put(tag, digest, value);
  return 0;
}
DASER_API int daser_table_del(daser_table* t, uint64_t tag, const uint8_t* digest) {
  if (!t || !digest) return -1;
  std::lock_guard<std::mutex> g(t->mu);
  return t->del(tag, digest) ? 1 : 0;
}
// returns the value, or `missing`
DASER_API int64_t daser_table_get(daser_table* t, uint64_t tag, const uint8_t* digest, int64_t missing) {
  if (!t || !digest) return missing;
  std::lock_guard<std::mutex> g(t->mu);
  const int64_t i = t->find(tag, digest);
  return i < 0 ? missing : t->values[i];
}

// Longest block-aligned prefix of `tokens` stored under `tag`: returns its value and writes the
// prefix length in tokens; returns `missing` (and 0 tokens) when no prefix is stored.
DASER_API int64_t daser_table_longest_prefix(daser_table* t, uint64_t tag, const int32_t* tokens, int64_t n,
                                             int32_t block, int64_t missing, int64_t* matched_tokens) {
  if (matched_tokens) *matched_tokens = 0;
  if (!t || !xxh().ok || block <= 0 || n < block) return missing;
  const int64_t nb = n / block;
  std::vector<uint8_t> dig((size_t)nb * 16);
  if (daser_prefix_digests(tokens, n, block, dig.data()) != nb) return missing;
  std::lock_guard<std::mutex> g(t->mu);
  for (int64_t i = nb - 1; i >= 0; --i) {
    const int64_t slot = t->find(tag, dig.data() + 16 * i);
    if (slot >= 0) {
      if (matched_tokens) *matched_tokens = (i + 1) * block;
      return t->values[slot];
    }
  }
  return missing;
}

// Aligned blocks of `tokens` whose digest is stored under `tag` (anchors of stored chunks):
// writes up to max_hits (block index, value) pairs, returns how many there are in total.
DASER_API int64_t daser_table_scan_blocks(daser_table* t, uint64_t tag, const int32_t* tokens, int64_t n, int32_t block,
                                          int64_t* block_index, int64_t* values, int64_t max_hits) {
  if (!t || !xxh().ok || block <= 0 || n < 0) return -1;
  const int64_t nb = n / block;
  int64_t hits = 0;
  std::lock_guard<std::mutex> g(t->mu);
  for (int64_t i = 0; i < nb; ++i) {
    uint8_t d[16];
    canonical(xxh().oneshot(tokens + i * block, (size_t)block * 4), d);
    const int64_t slot = t->find(tag, d);
    if (slot >= 0) {
      if (hits < max_hits && block_index && values) {
        block_index[hits] = i;
        values[hits] = t->values[slot];
      }
      ++hits;
    }
  }
  return hits;
}
