// Stand-alone exerciser of the token index, built with -fsanitize=address,undefined and with
// -fsanitize=thread by the tests: concurrent writers and readers on one table, growth and
// tombstone reuse, digest passes from several threads.  Exit code 0 = everything matched.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <thread>
#include <vector>

struct daser_table;
extern "C" {
int daser_index_available(void);
int daser_hash_tokens(const int32_t*, int64_t, uint8_t*);
int64_t daser_prefix_digests(const int32_t*, int64_t, int32_t, uint8_t*);
int64_t daser_block_digests(const int32_t*, int64_t, int32_t, uint8_t*);
daser_table* daser_table_new(int64_t);
void daser_table_free(daser_table*);
int64_t daser_table_size(daser_table*);
int daser_table_put(daser_table*, uint64_t, const uint8_t*, int64_t);
int daser_table_del(daser_table*, uint64_t, const uint8_t*);
int64_t daser_table_get(daser_table*, uint64_t, const uint8_t*, int64_t);
int64_t daser_table_longest_prefix(daser_table*, uint64_t, const int32_t*, int64_t, int32_t, int64_t, int64_t*);
int64_t daser_table_scan_blocks(daser_table*, uint64_t, const int32_t*, int64_t, int32_t, int64_t*, int64_t*, int64_t);
}

int main() {
  if (!daser_index_available()) {
    printf("libxxhash unavailable: skipped\nSELFTEST_OK\n");
    return 0;
  }
  const int kTokens = 16 * 200, kBlock = 16, kThreads = 4;
  std::vector<int32_t> tokens(kTokens);
  for (int i = 0; i < kTokens; ++i) tokens[i] = (int32_t)(i * 2654435761u);
  std::vector<uint8_t> prefix(16 * (kTokens / kBlock)), blocks(16 * (kTokens / kBlock));
  if (daser_prefix_digests(tokens.data(), kTokens, kBlock, prefix.data()) != kTokens / kBlock) return 1;
  if (daser_block_digests(tokens.data(), kTokens, kBlock, blocks.data()) != kTokens / kBlock) return 1;
  uint8_t one[16];
  daser_hash_tokens(tokens.data(), kBlock, one);
  if (memcmp(one, prefix.data(), 16) != 0 || memcmp(one, blocks.data(), 16) != 0) { fprintf(stderr, "first block digests differ\n"); return 1; }

  daser_table* t = daser_table_new(4);
  std::atomic<int> bad{0};
  std::vector<std::thread> threads;
  for (int th = 0; th < kThreads; ++th) {
    threads.emplace_back([&, th] {
      // every thread owns a tag; inserts all prefixes, deletes the odd ones, queries throughout
      const uint64_t tag = 100 + th;
      for (int i = 0; i < kTokens / kBlock; ++i) daser_table_put(t, tag, prefix.data() + 16 * i, i);
      for (int i = 1; i < kTokens / kBlock; i += 2) if (daser_table_del(t, tag, prefix.data() + 16 * i) != 1) bad++;
      for (int i = 0; i < kTokens / kBlock; ++i) {
        const int64_t v = daser_table_get(t, tag, prefix.data() + 16 * i, -1);
        if (v != ((i & 1) ? -1 : i)) bad++;
      }
      int64_t matched = 0;
      const int64_t v = daser_table_longest_prefix(t, tag, tokens.data(), kTokens, kBlock, -1, &matched);
      // the last prefix has an odd index (199): the longest survivor is index 198
      if (v != 198 || matched != 199 * kBlock) bad++;
      std::vector<uint8_t> mine(16 * (kTokens / kBlock));
      if (daser_prefix_digests(tokens.data(), kTokens, kBlock, mine.data()) != kTokens / kBlock || mine != prefix) bad++;
    });
  }
  for (auto& th : threads) th.join();
  if (daser_table_size(t) != (int64_t)kThreads * (kTokens / kBlock / 2)) bad++;
  // anchors: block digests of two positions under a fresh tag
  daser_table_put(t, 7, blocks.data() + 16 * 10, 1000);
  daser_table_put(t, 7, blocks.data() + 16 * 150, 1001);
  int64_t idx[8], val[8];
  const int64_t hits = daser_table_scan_blocks(t, 7, tokens.data(), kTokens, kBlock, idx, val, 8);
  if (hits != 2 || idx[0] != 10 || val[0] != 1000 || idx[1] != 150 || val[1] != 1001) bad++;
  daser_table_free(t);
  printf(bad.load() == 0 ? "SELFTEST_OK\n" : "SELFTEST_FAIL\n");
  return bad.load() == 0 ? 0 : 1;
}
