// Cold tier for KV blocks and state snapshots on a local NVMe file system.
//
// One slab file of fixed-size pages, opened with O_DIRECT when the file system allows it (page-aligned bounce
// buffers; falls back to buffered IO on tmpfs and the like).  A blob (the bytes of one KV block chain or one
// recurrent-state snapshot, keyed by its 64-bit prefix hash) occupies one or more pages.  Every page starts with a
// 64-byte header -- magic "DGPPNVM2", key, index of the page within the blob, blob length, payload length, CRC-32C of
// the payload -- so a page can be validated on its own and the index can be rebuilt by scanning the slab.
// Writes go through one IO thread (put_async -> ticket, wait / flush); reads are synchronous and verify every
// page's CRC, a mismatch makes the blob disappear instead of returning wrong bytes.  When the slab is full the
// least recently used blob is dropped.  commit() writes the index atomically (temp file + rename) with its own CRC
// so that a restarted server adopts the slab; commit_digest() is what ranks compare before they agree that a commit
// is the same everywhere.
// (reference counterparts: src/engine/nvme_tier.hpp O_DIRECT slab, CRC-32C pages, async IO thread, adoption at warm
//  start; src/sched/disk_cache.cpp DGPPNVM2 envelope and commit agreement; src/common/cache_storage.cpp mount checks.)
#pragma once
#include <fcntl.h>
#include <sys/stat.h>
#include <sys/statvfs.h>
#include <unistd.h>

#include <condition_variable>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <list>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "rt/core_util.h"

namespace dgpp {

struct DiskTierStats {
  uint64_t puts = 0, gets = 0, hits = 0, misses = 0, evictions = 0, crc_failures = 0, bytes_written = 0, bytes_read = 0;
};

// What the start-up check reports about the directory the tier is asked to use.
struct CacheStorageInfo {
  bool exists = false, writable = false, direct_io = false;
  uint64_t free_bytes = 0, total_bytes = 0;
};

inline CacheStorageInfo probe_cache_storage(const std::string& dir) {
  CacheStorageInfo info;
  struct stat st;
  if (::stat(dir.c_str(), &st) != 0 || !S_ISDIR(st.st_mode)) return info;
  info.exists = true;
  struct statvfs vs;
  if (::statvfs(dir.c_str(), &vs) == 0) {
    info.free_bytes = static_cast<uint64_t>(vs.f_bavail) * vs.f_frsize;
    info.total_bytes = static_cast<uint64_t>(vs.f_blocks) * vs.f_frsize;
  }
  const std::string probe = dir + "/.dgpp_probe";
  int fd = ::open(probe.c_str(), O_CREAT | O_WRONLY | O_TRUNC, 0600);
  if (fd >= 0) {
    info.writable = true;
    ::close(fd);
    fd = ::open(probe.c_str(), O_WRONLY | O_DIRECT);
    if (fd >= 0) { info.direct_io = true; ::close(fd); }
    ::unlink(probe.c_str());
  }
  return info;
}

class DiskTier {
 public:
  static constexpr size_t kHeaderBytes = 64;
  static constexpr char kMagic[9] = "DGPPNVM2";

  DiskTier(const std::string& dir, size_t page_bytes, size_t pages, bool try_direct = true, bool adopt = true)
      : dir_(dir), page_bytes_(page_bytes), pages_(pages) {
    if (page_bytes < 4096 || page_bytes % 4096 != 0) throw std::invalid_argument("disk tier: page size must be a multiple of 4096");
    if (pages == 0) throw std::invalid_argument("disk tier: no pages");
    const std::string slab = dir + "/slab.bin";
    if (try_direct) fd_ = ::open(slab.c_str(), O_CREAT | O_RDWR | O_DIRECT, 0600);
    direct_ = fd_ >= 0;
    if (fd_ < 0) fd_ = ::open(slab.c_str(), O_CREAT | O_RDWR, 0600);
    if (fd_ < 0) throw std::runtime_error("disk tier: cannot open " + slab);
    if (::ftruncate(fd_, static_cast<off_t>(page_bytes_ * pages_)) != 0) throw std::runtime_error("disk tier: cannot size the slab");
    if (posix_memalign(reinterpret_cast<void**>(&wbuf_), 4096, page_bytes_) != 0 ||
        posix_memalign(reinterpret_cast<void**>(&rbuf_), 4096, page_bytes_) != 0)
      throw std::bad_alloc();
    for (size_t p = pages_; p-- > 0;) free_.push_back(static_cast<uint32_t>(p));
    if (adopt) adopt_index();
    io_ = std::thread([this] { io_loop(); });
  }
  ~DiskTier() {
    {
      std::lock_guard<std::mutex> g(qmu_);
      stop_ = true;
    }
    qcv_.notify_all();
    if (io_.joinable()) io_.join();
    if (fd_ >= 0) ::close(fd_);
    free(wbuf_);
    free(rbuf_);
  }
  DiskTier(const DiskTier&) = delete;
  DiskTier& operator=(const DiskTier&) = delete;

  bool direct_io() const { return direct_; }
  size_t payload_per_page() const { return page_bytes_ - kHeaderBytes; }
  size_t free_pages() const { std::lock_guard<std::mutex> g(mu_); return free_.size(); }
  size_t blobs() const { std::lock_guard<std::mutex> g(mu_); return index_.size(); }
  DiskTierStats stats() const { std::lock_guard<std::mutex> g(mu_); return stats_; }
  bool contains(uint64_t key) const { std::lock_guard<std::mutex> g(mu_); return index_.count(key) != 0; }

  // Queue a write; the bytes are copied.  Returns a ticket for wait().
  uint64_t put_async(uint64_t key, const void* data, size_t len) {
    Job j;
    j.key = key;
    j.bytes.assign(static_cast<const char*>(data), len);
    std::lock_guard<std::mutex> g(qmu_);
    j.ticket = ++issued_;
    queue_.push_back(std::move(j));
    qcv_.notify_all();
    return issued_;
  }
  bool put(uint64_t key, const void* data, size_t len) {
    wait(put_async(key, data, len));
    return contains(key);
  }
  void wait(uint64_t ticket) {
    std::unique_lock<std::mutex> g(qmu_);
    done_cv_.wait(g, [&] { return done_ >= ticket; });
  }
  void flush() {
    uint64_t t;
    { std::lock_guard<std::mutex> g(qmu_); t = issued_; }
    wait(t);
  }
  // Reads the blob; false when it is absent or failed its checks (then it is dropped from the index).
  bool get(uint64_t key, std::string* out) {
    std::vector<uint32_t> pages;
    size_t len = 0;
    {
      std::lock_guard<std::mutex> g(mu_);
      ++stats_.gets;
      auto it = index_.find(key);
      if (it == index_.end()) { ++stats_.misses; return false; }
      pages = it->second.pages;
      len = it->second.len;
      lru_.splice(lru_.begin(), lru_, it->second.lru);
    }
    out->clear();
    out->reserve(len);
    std::lock_guard<std::mutex> rg(rmu_);
    for (size_t i = 0; i < pages.size(); ++i) {
      Header h;
      if (!read_page(pages[i], &h) || h.key != key || h.part != i || h.blob_len != len ||
          h.payload_len > payload_per_page() || crc32c(rbuf_ + kHeaderBytes, h.payload_len) != h.crc) {
        std::lock_guard<std::mutex> g(mu_);
        ++stats_.crc_failures;
        ++stats_.misses;
        drop_locked(key);
        out->clear();
        return false;
      }
      out->append(reinterpret_cast<const char*>(rbuf_ + kHeaderBytes), h.payload_len);
    }
    std::lock_guard<std::mutex> g(mu_);
    if (out->size() != len) { ++stats_.crc_failures; ++stats_.misses; drop_locked(key); out->clear(); return false; }
    ++stats_.hits;
    stats_.bytes_read += len;
    return true;
  }
  void erase(uint64_t key) { std::lock_guard<std::mutex> g(mu_); drop_locked(key); }

  // FNV-1a over the sorted (key, length) pairs: equal on two ranks iff they hold the same set of blobs.
  uint64_t commit_digest() const {
    std::lock_guard<std::mutex> g(mu_);
    std::map<uint64_t, uint64_t> sorted;
    for (const auto& kv : index_) sorted[kv.first] = kv.second.len;
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](uint64_t v) { for (int i = 0; i < 8; ++i) { h ^= (v >> (8 * i)) & 0xff; h *= 1099511628211ull; } };
    for (const auto& kv : sorted) { mix(kv.first); mix(kv.second); }
    return h;
  }
  // Persist the index: "DGPPNVM2" + page size + count + entries + CRC-32C, written to a temp file and renamed.
  void commit() {
    flush();
    std::string body(kMagic, 8);
    auto put64 = [&](uint64_t v) { body.append(reinterpret_cast<const char*>(&v), 8); };
    {
      std::lock_guard<std::mutex> g(mu_);
      put64(page_bytes_);
      put64(pages_);
      put64(index_.size());
      for (auto it = lru_.rbegin(); it != lru_.rend(); ++it) {   // oldest first, so adoption rebuilds the LRU order
        const Entry& e = index_.at(*it);
        put64(*it);
        put64(e.len);
        put64(e.pages.size());
        for (uint32_t p : e.pages) put64(p);
      }
    }
    const uint32_t crc = crc32c(body.data(), body.size());
    body.append(reinterpret_cast<const char*>(&crc), 4);
    const std::string tmp = dir_ + "/index.tmp", fin = dir_ + "/index.bin";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) throw std::runtime_error("disk tier: cannot write " + tmp);
    const bool ok = fwrite(body.data(), 1, body.size(), f) == body.size() && fflush(f) == 0 && fsync(fileno(f)) == 0;
    fclose(f);
    if (!ok || ::rename(tmp.c_str(), fin.c_str()) != 0) throw std::runtime_error("disk tier: commit failed");
    if (!direct_) fsync(fd_);
  }
  // Test hook: flip one payload byte of the blob's first page on disk.
  bool corrupt_for_test(uint64_t key) {
    uint32_t page;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = index_.find(key);
      if (it == index_.end()) return false;
      page = it->second.pages[0];
    }
    std::lock_guard<std::mutex> rg(rmu_);
    Header h;
    if (!read_page(page, &h)) return false;
    rbuf_[kHeaderBytes] ^= 0x5a;
    return ::pwrite(fd_, rbuf_, page_bytes_, static_cast<off_t>(page) * static_cast<off_t>(page_bytes_)) == static_cast<ssize_t>(page_bytes_);
  }

 private:
  struct Header {
    char magic[8];
    uint64_t key, blob_len;
    uint32_t part, payload_len, crc, pad;
    char reserved[24];
  };
  static_assert(sizeof(Header) == kHeaderBytes, "page header is 64 bytes");
  struct Entry {
    std::vector<uint32_t> pages;
    size_t len = 0;
    std::list<uint64_t>::iterator lru;
  };
  struct Job {
    uint64_t key = 0, ticket = 0;
    std::string bytes;
  };

  bool read_page(uint32_t page, Header* h) {
    const ssize_t n = ::pread(fd_, rbuf_, page_bytes_, static_cast<off_t>(page) * static_cast<off_t>(page_bytes_));
    if (n != static_cast<ssize_t>(page_bytes_)) return false;
    memcpy(h, rbuf_, sizeof(Header));
    return memcmp(h->magic, kMagic, 8) == 0;
  }
  void drop_locked(uint64_t key) {
    auto it = index_.find(key);
    if (it == index_.end()) return;
    for (uint32_t p : it->second.pages) free_.push_back(p);
    lru_.erase(it->second.lru);
    index_.erase(it);
  }
  void write_blob(const Job& j) {
    const size_t per = payload_per_page();
    const size_t need = j.bytes.empty() ? 1 : (j.bytes.size() + per - 1) / per;
    std::vector<uint32_t> pages;
    {
      std::lock_guard<std::mutex> g(mu_);
      ++stats_.puts;
      drop_locked(j.key);
      if (need > pages_) return;
      while (free_.size() < need && !lru_.empty()) {
        ++stats_.evictions;
        drop_locked(lru_.back());
      }
      if (free_.size() < need) return;
      for (size_t i = 0; i < need; ++i) { pages.push_back(free_.back()); free_.pop_back(); }
    }
    bool ok = true;
    for (size_t i = 0; i < need && ok; ++i) {
      const size_t off = i * per, n = std::min(per, j.bytes.size() - std::min(off, j.bytes.size()));
      Header h;
      memset(&h, 0, sizeof(h));
      memcpy(h.magic, kMagic, 8);
      h.key = j.key;
      h.blob_len = j.bytes.size();
      h.part = static_cast<uint32_t>(i);
      h.payload_len = static_cast<uint32_t>(n);
      memset(wbuf_, 0, page_bytes_);
      if (n) memcpy(wbuf_ + kHeaderBytes, j.bytes.data() + off, n);
      h.crc = crc32c(wbuf_ + kHeaderBytes, n);
      memcpy(wbuf_, &h, sizeof(h));
      ok = ::pwrite(fd_, wbuf_, page_bytes_, static_cast<off_t>(pages[i]) * static_cast<off_t>(page_bytes_)) == static_cast<ssize_t>(page_bytes_);
    }
    std::lock_guard<std::mutex> g(mu_);
    if (!ok) { for (uint32_t p : pages) free_.push_back(p); return; }
    Entry e;
    e.pages = std::move(pages);
    e.len = j.bytes.size();
    lru_.push_front(j.key);
    e.lru = lru_.begin();
    index_[j.key] = std::move(e);
    stats_.bytes_written += j.bytes.size();
  }
  void io_loop() {
    for (;;) {
      Job j;
      {
        std::unique_lock<std::mutex> g(qmu_);
        qcv_.wait(g, [&] { return stop_ || !queue_.empty(); });
        if (queue_.empty()) return;
        j = std::move(queue_.front());
        queue_.pop_front();
      }
      write_blob(j);
      {
        std::lock_guard<std::mutex> g(qmu_);
        done_ = j.ticket;
      }
      done_cv_.notify_all();
    }
  }
  // Adopt a committed index when it matches this geometry and its CRC; every blob's first page is checked.
  void adopt_index() {
    FILE* f = fopen((dir_ + "/index.bin").c_str(), "rb");
    if (!f) return;
    std::string body;
    char tmp[65536];
    size_t n;
    while ((n = fread(tmp, 1, sizeof(tmp), f)) > 0) body.append(tmp, n);
    fclose(f);
    if (body.size() < 8 + 24 + 4 || memcmp(body.data(), kMagic, 8) != 0) return;
    uint32_t crc;
    memcpy(&crc, body.data() + body.size() - 4, 4);
    if (crc32c(body.data(), body.size() - 4) != crc) return;
    size_t off = 8;
    auto get64 = [&](uint64_t* v) {
      if (off + 8 > body.size() - 4) return false;
      memcpy(v, body.data() + off, 8);
      off += 8;
      return true;
    };
    uint64_t pb, np, count;
    if (!get64(&pb) || !get64(&np) || !get64(&count) || pb != page_bytes_ || np != pages_) return;
    std::vector<bool> used(pages_, false);
    for (uint64_t i = 0; i < count; ++i) {
      uint64_t key, len, cnt;
      if (!get64(&key) || !get64(&len) || !get64(&cnt) || cnt == 0 || cnt > pages_) return;
      Entry e;
      e.len = len;
      bool ok = true;
      for (uint64_t k = 0; k < cnt; ++k) {
        uint64_t p;
        if (!get64(&p)) return;
        if (p >= pages_ || used[p]) ok = false;
        else e.pages.push_back(static_cast<uint32_t>(p));
      }
      Header h;
      if (!ok || !read_page(e.pages[0], &h) || h.key != key || h.part != 0 || h.blob_len != len) continue;
      for (uint32_t p : e.pages) used[p] = true;
      lru_.push_front(key);
      e.lru = lru_.begin();
      index_[key] = std::move(e);
    }
    free_.clear();
    for (size_t p = pages_; p-- > 0;)
      if (!used[p]) free_.push_back(static_cast<uint32_t>(p));
  }

  std::string dir_;
  size_t page_bytes_, pages_;
  int fd_ = -1;
  bool direct_ = false;
  unsigned char* wbuf_ = nullptr;
  unsigned char* rbuf_ = nullptr;
  mutable std::mutex mu_;   // index, free list, LRU, stats
  std::mutex rmu_;          // read bounce buffer
  std::unordered_map<uint64_t, Entry> index_;
  std::list<uint64_t> lru_;
  std::vector<uint32_t> free_;
  DiskTierStats stats_;
  std::mutex qmu_;
  std::condition_variable qcv_, done_cv_;
  std::deque<Job> queue_;
  uint64_t issued_ = 0, done_ = 0;
  bool stop_ = false;
  std::thread io_;
};

}  // namespace dgpp
