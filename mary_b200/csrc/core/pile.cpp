// Append-only, memory-mapped, content-addressed pile file (C ABI, loaded with ctypes).
//
// Role of the reference's external `triblespace` Pile (usage: src/persist.rs:744-799,
// src/leaf.rs:40-49): every record carries a uniform 256-byte header and its payload is
// padded to a multiple of 256 bytes, so each blob starts at a 256-byte aligned file offset
// and can be handed to the GPU copy engine (or registered as pinned memory) without a
// staging copy (src/persist.rs:2068-2073, src/format.rs:161-162).  Handles are 32-byte
// BLAKE3 digests.  The file is never truncated implicitly: a torn tail makes open/refresh
// fail, and repair is the explicit pile_amputate() (src/persist.rs:143-151).
//
// Record header (256 bytes, little endian):
//   [0,8)    magic "MARYPIL3"
//   [8,12)   kind: 1 = blob, 2 = branch head
//   [12,16)  reserved
//   [16,24)  payload length in bytes
//   [24,32)  timestamp, ns since the epoch
//   [32,64)  BLAKE3(payload)
//   [64,80)  branch id (kind 2), else zero
//   [80,224) reserved (zero)
//   [224,256) BLAKE3(header[0,224))
// The mapping reserves 1 TiB of address space so that blob pointers stay valid while the
// file grows (src/models/inkling/pile.rs:143-149).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <array>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "blake3.hpp"

namespace {

constexpr size_t HDR = 256;
constexpr size_t RESERVE = size_t(1) << 40;
const char MAGIC[8] = {'M', 'A', 'R', 'Y', 'P', 'I', 'L', '3'};

struct Key {
  uint8_t b[32];
  bool operator==(const Key& o) const { return std::memcmp(b, o.b, 32) == 0; }
};
struct KeyHash {
  size_t operator()(const Key& k) const { size_t v; std::memcpy(&v, k.b, sizeof v); return v; }
};

struct Record {
  uint64_t offset;  // of the header
  uint64_t len;
  uint32_t kind;
  uint64_t ts;
  Key hash;
  uint8_t branch[16];
  bool validated;
};

struct Pile {
  int fd = -1;
  uint8_t* map = nullptr;
  uint64_t size = 0;  // bytes of the file that were scanned and accepted
  std::vector<Record> recs;
  std::unordered_map<Key, uint32_t, KeyHash> index;
  std::mutex mu;
  std::string err;
  bool validate = true;
  uint64_t bytes_put = 0, bytes_dedup = 0;
};

size_t pad256(size_t n) { return (n + 255) & ~size_t(255); }

// Parallel BLAKE3 over large payloads: the tree is split at power-of-two chunk
// boundaries, so subtrees can be hashed independently and joined with parent nodes.
void hash_payload(const uint8_t* p, size_t n, uint8_t out[32]) {
  using B = mary::Blake3;
  constexpr size_t MIN_PAR = size_t(8) << 20;
  unsigned hw = std::thread::hardware_concurrency();
  if (n < MIN_PAR || hw < 2) { B::hash(p, n, out); return; }
  // Pick leaf subtrees of 2^k chunks such that the whole input is a left-complete tree of them.
  size_t chunks = (n + 1023) / 1024;
  size_t leaf = 1;
  while (leaf * 64 < chunks) leaf *= 2;  // at most ~64..128 leaves
  size_t nleaf = (chunks + leaf - 1) / leaf;
  std::vector<std::array<uint32_t, 8>> cvs(nleaf);
  std::atomic<size_t> next{0};
  auto work = [&] {
    for (;;) {
      size_t i = next.fetch_add(1);
      if (i >= nleaf) return;
      size_t off = i * leaf * 1024, len = std::min(n - off, leaf * 1024);
      B::Output o = B::subtree(p + off, len, i * leaf);
      B::chaining_value(o, cvs[i].data());
    }
  };
  unsigned nt = std::min<unsigned>(hw, 16);
  std::vector<std::thread> th;
  for (unsigned t = 1; t < nt; ++t) th.emplace_back(work);
  work();
  for (auto& t : th) t.join();
  // Join leaves [lo,hi) following the same "largest power of two on the left" rule.
  struct J {
    static B::Output join(std::vector<std::array<uint32_t, 8>>& cv, size_t lo, size_t hi) {
      size_t cnt = hi - lo, left = 1;
      while (left * 2 < cnt) left *= 2;
      uint32_t l[8], r[8];
      if (left == 1) std::memcpy(l, cv[lo].data(), 32);
      else B::chaining_value(join(cv, lo, lo + left), l);
      if (cnt - left == 1) std::memcpy(r, cv[lo + left].data(), 32);
      else B::chaining_value(join(cv, lo + left, hi), r);
      return B::parent_output(l, r);
    }
  };
  B::Output root = J::join(cvs, 0, nleaf);
  uint32_t w[16];
  B::compress(root.cv, root.block, 0, root.block_len, root.flags | B::ROOT, w);
  std::memcpy(out, w, 32);
}

bool parse_header(const uint8_t* h, Record& r) {
  if (std::memcmp(h, MAGIC, 8) != 0) return false;
  uint8_t chk[32];
  mary::Blake3::hash(h, 224, chk);
  if (std::memcmp(chk, h + 224, 32) != 0) return false;
  std::memcpy(&r.kind, h + 8, 4);
  std::memcpy(&r.len, h + 16, 8);
  std::memcpy(&r.ts, h + 24, 8);
  std::memcpy(r.hash.b, h + 32, 32);
  std::memcpy(r.branch, h + 64, 16);
  r.validated = false;
  return true;
}

// Scan records from p->size to the end of the file.  Returns 0, or -1 with p->err set
// when the tail is torn (a partial header or payload, or a header that fails its checksum).
int scan(Pile* p) {
  struct stat st;
  if (fstat(p->fd, &st) != 0) { p->err = "fstat failed"; return -1; }
  uint64_t end = (uint64_t)st.st_size;
  uint64_t off = p->size;
  while (off < end) {
    if (end - off < HDR) { p->err = "torn tail: partial record header at offset " + std::to_string(off); return -1; }
    Record r;
    if (!parse_header(p->map + off, r)) {
      p->err = "torn tail: bad record header at offset " + std::to_string(off);
      return -1;
    }
    uint64_t total = HDR + pad256(r.len);
    if (end - off < total) { p->err = "torn tail: partial payload at offset " + std::to_string(off); return -1; }
    r.offset = off;
    uint32_t idx = (uint32_t)p->recs.size();
    p->recs.push_back(r);
    if (r.kind == 1) p->index.emplace(r.hash, idx);
    off += total;
    p->size = off;
  }
  return 0;
}

}  // namespace

extern "C" {

void* pile_open(const char* path, int create, int validate) {
  Pile* p = new Pile();
  p->validate = validate != 0;
  p->fd = ::open(path, create ? (O_RDWR | O_CREAT) : O_RDWR, 0644);
  if (p->fd < 0) {
    p->fd = ::open(path, O_RDONLY);
    if (p->fd < 0) { delete p; return nullptr; }
  }
  void* m = mmap(nullptr, RESERVE, PROT_READ, MAP_SHARED | MAP_NORESERVE, p->fd, 0);
  if (m == MAP_FAILED) { ::close(p->fd); delete p; return nullptr; }
  p->map = (uint8_t*)m;
  scan(p);  // an error stays in p->err; the caller checks pile_error()
  return p;
}

const char* pile_error(void* h) { return ((Pile*)h)->err.c_str(); }

void pile_close(void* h) {
  Pile* p = (Pile*)h;
  if (!p) return;
  if (p->map) munmap(p->map, RESERVE);
  if (p->fd >= 0) ::close(p->fd);
  delete p;
}

int pile_refresh(void* h) {
  Pile* p = (Pile*)h;
  std::lock_guard<std::mutex> g(p->mu);
  p->err.clear();
  return scan(p);
}

void pile_hash(const void* data, uint64_t len, uint8_t* out32) { hash_payload((const uint8_t*)data, len, out32); }

// Append one record.  Blobs dedupe on their content hash.  Returns the record index or -1.
int64_t pile_put(void* h, uint32_t kind, const void* data, uint64_t len, const uint8_t* branch16, uint8_t* out_hash32) {
  Pile* p = (Pile*)h;
  uint8_t hash[32];
  hash_payload((const uint8_t*)data, len, hash);
  if (out_hash32) std::memcpy(out_hash32, hash, 32);
  std::lock_guard<std::mutex> g(p->mu);
  if (!p->err.empty()) return -1;  // refuse to write behind a torn tail
  Key k;
  std::memcpy(k.b, hash, 32);
  if (kind == 1) {
    auto it = p->index.find(k);
    if (it != p->index.end()) { p->bytes_dedup += len; return it->second; }
  }
  uint8_t hdr[HDR];
  std::memset(hdr, 0, HDR);
  std::memcpy(hdr, MAGIC, 8);
  std::memcpy(hdr + 8, &kind, 4);
  std::memcpy(hdr + 16, &len, 8);
  uint64_t ts = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
                    std::chrono::system_clock::now().time_since_epoch()).count();
  std::memcpy(hdr + 24, &ts, 8);
  std::memcpy(hdr + 32, hash, 32);
  if (branch16) std::memcpy(hdr + 64, branch16, 16);
  mary::Blake3::hash(hdr, 224, hdr + 224);
  uint64_t off = p->size;
  uint64_t padded = pad256(len);
  if (pwrite(p->fd, hdr, HDR, off) != (ssize_t)HDR) { p->err = "pwrite header failed"; return -1; }
  uint64_t done = 0;
  while (done < len) {
    ssize_t w = pwrite(p->fd, (const uint8_t*)data + done, len - done, off + HDR + done);
    if (w <= 0) { p->err = "pwrite payload failed"; return -1; }
    done += (uint64_t)w;
  }
  if (padded > len) {
    static const uint8_t zeros[256] = {0};
    if (pwrite(p->fd, zeros, padded - len, off + HDR + len) != (ssize_t)(padded - len)) {
      p->err = "pwrite padding failed"; return -1;
    }
  }
  Record r;
  r.offset = off; r.len = len; r.kind = kind; r.ts = ts; r.hash = k; r.validated = true;
  std::memset(r.branch, 0, 16);
  if (branch16) std::memcpy(r.branch, branch16, 16);
  uint32_t idx = (uint32_t)p->recs.size();
  p->recs.push_back(r);
  if (kind == 1) p->index.emplace(k, idx);
  p->size = off + HDR + padded;
  p->bytes_put += len;
  return idx;
}

// Look a blob up by hash.  The pointer aims into the mapping (256-byte aligned file offset).
// On the first read of a record its payload is re-hashed (src/persist.rs:945-949).
int pile_get(void* h, const uint8_t* hash32, const uint8_t** ptr, uint64_t* len) {
  Pile* p = (Pile*)h;
  Key k;
  std::memcpy(k.b, hash32, 32);
  // Everything needed from the record is copied while the lock is held: a concurrent put may grow `recs` and move it.
  size_t slot;
  uint64_t offset, rlen;
  bool validated;
  {
    std::lock_guard<std::mutex> g(p->mu);
    auto it = p->index.find(k);
    if (it == p->index.end()) return -1;
    slot = it->second;
    const Record& r = p->recs[slot];
    offset = r.offset; rlen = r.len; validated = r.validated;
  }
  const uint8_t* data = p->map + offset + HDR;
  if (p->validate && !validated) {
    uint8_t chk[32];
    hash_payload(data, rlen, chk);                   // the payload itself never moves (append-only mapping)
    if (std::memcmp(chk, k.b, 32) != 0) return -2;
    std::lock_guard<std::mutex> g(p->mu);
    p->recs[slot].validated = true;
  }
  *ptr = data;
  *len = rlen;
  return 0;
}

int64_t pile_count(void* h) { return (int64_t)((Pile*)h)->recs.size(); }
uint64_t pile_size(void* h) { return ((Pile*)h)->size; }

int pile_record(void* h, int64_t i, uint32_t* kind, uint64_t* offset, uint64_t* len, uint64_t* ts,
                uint8_t* hash32, uint8_t* branch16) {
  Pile* p = (Pile*)h;
  if (i < 0 || (size_t)i >= p->recs.size()) return -1;
  const Record& r = p->recs[(size_t)i];
  *kind = r.kind; *offset = r.offset + HDR; *len = r.len; *ts = r.ts;
  std::memcpy(hash32, r.hash.b, 32);
  std::memcpy(branch16, r.branch, 16);
  return 0;
}

const uint8_t* pile_base(void* h) { return ((Pile*)h)->map; }

void pile_stats(void* h, uint64_t* put, uint64_t* dedup) {
  *put = ((Pile*)h)->bytes_put; *dedup = ((Pile*)h)->bytes_dedup;
}

int pile_flush(void* h) { return fsync(((Pile*)h)->fd); }

// Explicit repair: cut the file back to the last record that scans cleanly.
// Returns the number of bytes removed, or -1.
int64_t pile_amputate(const char* path) {
  Pile* p = (Pile*)pile_open(path, 0, 0);
  if (!p) return -1;
  struct stat st;
  fstat(p->fd, &st);
  int64_t cut = (int64_t)st.st_size - (int64_t)p->size;
  int rc = 0;
  if (cut > 0) rc = ftruncate(p->fd, (off_t)p->size);
  pile_close(p);
  return rc == 0 ? cut : -1;
}

// Advise the kernel that a blob's pages will not be needed again (after its bytes were
// copied to the device), mirroring the reference's SourceRelease (pile.rs:119-207).
int pile_release(void* h, const uint8_t* ptr, uint64_t len) {
  (void)h;
  uintptr_t a = (uintptr_t)ptr & ~uintptr_t(4095);
  uintptr_t e = ((uintptr_t)ptr + len + 4095) & ~uintptr_t(4095);
  return madvise((void*)a, e - a, MADV_DONTNEED);
}

}  // extern "C"
