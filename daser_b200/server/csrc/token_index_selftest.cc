// Stand-alone exerciser of the token index and of the lookup thread, built with -fsanitize=address,undefined and with
// -fsanitize=thread by the tests: concurrent writers and readers on one table, growth and
// tombstone reuse, digest passes from several threads.  Exit code 0 = everything matched.
#include <arpa/inet.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <string>
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

struct daser_fast;
extern "C" {
daser_fast* daser_fast_start(const char*, int64_t);
void daser_fast_stop(daser_fast*);
int daser_fast_put(daser_fast*, const char*, const char*, int64_t, int64_t, int64_t, int64_t);
int daser_fast_del(daser_fast*, const char*);
void daser_fast_stats(daser_fast*, int64_t*);
}

// One framed request on a fresh connection: {"op": "lookup_chunks", "keys": [key], "model_id": "m"};
// returns 1 for a hit (the reply's only array element is a map), 0 for a miss (nil), -1 on error.
static int fast_probe(int fd, const char* key) {
  std::string b;
  b.push_back((char)0x83);
  auto str = [&b](const char* t) { b.push_back((char)(0xA0 | strlen(t))); b.append(t); };
  str("op"); str("lookup_chunks");
  str("keys"); b.push_back((char)0x91); str(key);
  str("model_id"); str("m");
  const uint32_t n = htonl((uint32_t)b.size());
  std::string out((const char*)&n, 4);
  out += b;
  if (send(fd, out.data(), out.size(), MSG_NOSIGNAL) != (ssize_t)out.size()) return -1;
  uint8_t hdr[4];
  size_t got = 0;
  while (got < 4) { const ssize_t r = recv(fd, hdr + got, 4 - got, 0); if (r <= 0) return -1; got += (size_t)r; }
  uint32_t len;
  memcpy(&len, hdr, 4);
  len = ntohl(len);
  std::vector<uint8_t> body(len);
  got = 0;
  while (got < len) { const ssize_t r = recv(fd, body.data() + got, len - got, 0); if (r <= 0) return -1; got += (size_t)r; }
  // {"chunks": [x]}: 0x81, fixstr "chunks" (7 bytes), 0x91, then x
  if (len < 10 || body[0] != 0x81 || body[8] != 0x91) return -1;
  return body[9] == 0xC0 ? 0 : ((body[9] & 0xF0) == 0x80 ? 1 : -1);
}

static int fast_connect(const char* path) {
  sockaddr_un a{};
  a.sun_family = AF_UNIX;
  strcpy(a.sun_path, path);
  const int fd = socket(AF_UNIX, SOCK_STREAM, 0);
  if (fd < 0 || connect(fd, (sockaddr*)&a, sizeof a) != 0) { if (fd >= 0) close(fd); return -1; }
  return fd;
}

// The lookup thread under concurrent clients while the owner adds and removes records.
static int fast_lookup_selftest() {
  char path[64];
  snprintf(path, sizeof path, "/tmp/daser_fast_selftest_%d.sock", (int)getpid());
  daser_fast* f = daser_fast_start(path, 4096);
  if (!f) return 1;
  std::atomic<int> bad{0};
  daser_fast_put(f, "stay", "m", 1, 2, 32, 0);
  std::vector<std::thread> clients;
  for (int c = 0; c < 4; ++c) {
    clients.emplace_back([&] {
      const int fd = fast_connect(path);
      if (fd < 0) { bad++; return; }
      for (int i = 0; i < 500; ++i) {
        if (fast_probe(fd, "stay") != 1) bad++;
        if (fast_probe(fd, "never") != 0) bad++;
        if (fast_probe(fd, "flip") < 0) bad++;  // present or not, depending on the owner's progress
      }
      close(fd);
    });
  }
  for (int i = 0; i < 2000; ++i) {
    daser_fast_put(f, "flip", "m", i, 1, 16, 0);
    daser_fast_del(f, "flip");
  }
  for (auto& t : clients) t.join();
  // garbage and an oversized length: the connection is dropped, the thread lives on
  int fd = fast_connect(path);
  const uint8_t junk[8] = {0xFF, 0xFF, 0xFF, 0xFF, 1, 2, 3, 4};
  if (fd < 0 || send(fd, junk, 8, MSG_NOSIGNAL) != 8) bad++;
  uint8_t one;
  if (fd >= 0 && recv(fd, &one, 1, 0) != 0) bad++;  // orderly close from the server
  if (fd >= 0) close(fd);
  fd = fast_connect(path);
  if (fd < 0 || fast_probe(fd, "stay") != 1) bad++;
  if (fd >= 0) close(fd);
  int64_t st[5];
  daser_fast_stats(f, st);
  if (st[0] != 1 || st[2] < 2001) bad++;
  daser_fast_stop(f);
  if (access(path, F_OK) == 0) bad++;
  return bad.load();
}

int main() {
  if (fast_lookup_selftest() != 0) {
    printf("SELFTEST_FAIL (lookup thread)\n");
    return 1;
  }
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
