#include "pcache.h"

#include <dirent.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <sys/types.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdlib>
#include <cstring>

#include "sha256.h"

namespace spark_rt {

namespace {
constexpr uint64_t kMagic = 0x53504b5043314130ull;   // "SPKPC1A0"
struct Header {
  uint64_t magic;
  int64_t tokens, bytes, chunks;
  uint64_t table_sum;
  char pad[4096 - 40];
};
static_assert(sizeof(Header) == 4096, "header is one direct-I/O block");

uint64_t fnv64(const void* p, size_t n) {
  const uint8_t* b = static_cast<const uint8_t*>(p);
  uint64_t h = 1469598103934665603ull;
  // 8 bytes at a time: fast enough to keep up with NVMe, still catches torn / truncated chunks
  size_t i = 0;
  for (; i + 8 <= n; i += 8) { uint64_t v; memcpy(&v, b + i, 8); h = (h ^ v) * 1099511628211ull; }
  for (; i < n; ++i) h = (h ^ b[i]) * 1099511628211ull;
  return h;
}

void mkdirs(const std::string& p) {
  std::string cur;
  for (size_t i = 0; i <= p.size(); ++i) {
    if (i == p.size() || p[i] == '/') { if (!cur.empty()) mkdir(cur.c_str(), 0755); }
    if (i < p.size()) cur += p[i];
  }
}

struct Aligned {
  void* p = nullptr;
  explicit Aligned(size_t n) { if (posix_memalign(&p, 4096, n)) p = nullptr; }
  ~Aligned() { free(p); }
};

bool write_all(int fd, const void* buf, size_t n, off_t off) {
  const char* b = static_cast<const char*>(buf);
  while (n) {
    ssize_t w = pwrite(fd, b, n, off);
    if (w <= 0) { if (errno == EINTR) continue; return false; }
    b += w; n -= w; off += w;
  }
  return true;
}
bool read_all(int fd, void* buf, size_t n, off_t off) {
  char* b = static_cast<char*>(buf);
  while (n) {
    ssize_t r = pread(fd, b, n, off);
    if (r <= 0) { if (r < 0 && errno == EINTR) continue; return false; }
    b += r; n -= r; off += r;
  }
  return true;
}
}  // namespace

std::string Pcache::identity_dir(const std::vector<std::string>& parts) {
  Sha256 s;
  for (auto& p : parts) { s.update(p.data(), p.size()); uint8_t z = 0; s.update(&z, 1); }
  return s.hex().substr(0, 32);
}

std::string Pcache::prefix_key(const int32_t* ids, int64_t n) {
  Sha256 s;
  s.update(ids, static_cast<size_t>(n) * 4);
  return s.hex().substr(0, 40);
}

Pcache::Pcache(const std::string& root, const std::string& identity, int64_t byte_budget, bool direct_io)
    : dir_(root + "/" + identity), budget_(byte_budget), direct_(direct_io) {
  mkdirs(dir_);
  reconcile();
  writer_ = std::thread([this] { writer_loop(); });
}

Pcache::~Pcache() {
  { std::lock_guard<std::mutex> l(mu_); stop_ = true; }
  cv_.notify_all();
  if (writer_.joinable()) writer_.join();
}

int Pcache::reconcile() {
  std::lock_guard<std::mutex> l(mu_);
  index_.clear();
  int dropped = 0;
  DIR* d = opendir(dir_.c_str());
  if (!d) return 0;
  while (dirent* e = readdir(d)) {
    std::string name = e->d_name;
    const std::string full = dir_ + "/" + name;
    if (name.size() > 4 && name.substr(name.size() - 4) == ".tmp") { unlink(full.c_str()); ++dropped; continue; }
    if (name.size() <= 3 || name.substr(name.size() - 3) != ".pc") continue;
    int fd = open(full.c_str(), O_RDONLY);
    Header h;
    bool ok = fd >= 0 && read_all(fd, &h, sizeof(h), 0) && h.magic == kMagic && h.bytes >= 0 && h.chunks == (h.bytes + kChunk - 1) / kChunk;
    struct stat st;
    if (ok) {
      const int64_t padded = (h.bytes + 4095) / 4096 * 4096;
      const int64_t table = (h.chunks * 8 + 4095) / 4096 * 4096;
      ok = fstat(fd, &st) == 0 && st.st_size == static_cast<off_t>(sizeof(Header) + padded + table);
      if (ok && h.chunks) {
        std::vector<uint64_t> sums(h.chunks);
        ok = read_all(fd, sums.data(), h.chunks * 8, sizeof(Header) + padded) && fnv64(sums.data(), h.chunks * 8) == h.table_sum;
      }
    }
    if (fd >= 0) close(fd);
    if (!ok) { unlink(full.c_str()); ++dropped; ++st_.corrupt; continue; }
    PcacheEntry pe; pe.key = name.substr(0, name.size() - 3); pe.tokens = h.tokens; pe.bytes = h.bytes; pe.last_use = ++clock_;
    index_[pe.key] = pe;
  }
  closedir(d);
  return dropped;
}

void Pcache::evict_to_budget(int64_t incoming) {
  int64_t used = 0;
  for (auto& kv : index_) used += kv.second.bytes;
  while (used + incoming > budget_ && !index_.empty()) {
    auto victim = std::min_element(index_.begin(), index_.end(), [](auto& a, auto& b) { return a.second.last_use < b.second.last_use; });
    used -= victim->second.bytes;
    unlink(path(victim->first).c_str());
    index_.erase(victim);
    ++st_.evictions;
  }
}

bool Pcache::save(const std::string& key, int64_t tokens, const void* data, int64_t bytes) {
  if (bytes > budget_) return false;
  { std::lock_guard<std::mutex> l(mu_); evict_to_budget(bytes); }
  const std::string tmp = path(key) + ".tmp";
  int flags = O_WRONLY | O_CREAT | O_TRUNC;
  int fd = -1;
  bool direct = direct_;
  if (direct) fd = open(tmp.c_str(), flags | O_DIRECT, 0644);
  if (fd < 0) { direct = false; fd = open(tmp.c_str(), flags, 0644); }
  if (fd < 0) return false;
  const int64_t chunks = (bytes + kChunk - 1) / kChunk;
  std::vector<uint64_t> sums(chunks);
  Aligned bounce(kChunk);
  bool ok = bounce.p != nullptr;
  off_t off = sizeof(Header);
  for (int64_t c = 0; ok && c < chunks; ++c) {
    const int64_t n = std::min<int64_t>(kChunk, bytes - c * kChunk);
    const char* src = static_cast<const char*>(data) + c * kChunk;
    sums[c] = fnv64(src, n);
    const int64_t padded = (n + 4095) / 4096 * 4096;
    memcpy(bounce.p, src, n);
    if (padded > n) memset(static_cast<char*>(bounce.p) + n, 0, padded - n);
    ok = write_all(fd, bounce.p, padded, off);
    off += padded;
  }
  if (ok) {
    const int64_t table = (chunks * 8 + 4095) / 4096 * 4096;
    if (table) {
      memset(bounce.p, 0, table);
      memcpy(bounce.p, sums.data(), chunks * 8);
      ok = write_all(fd, bounce.p, table, off);
    }
    Header* h = static_cast<Header*>(bounce.p);
    memset(h, 0, sizeof(Header));
    h->magic = kMagic; h->tokens = tokens; h->bytes = bytes; h->chunks = chunks; h->table_sum = fnv64(sums.data(), chunks * 8);
    ok = ok && write_all(fd, h, sizeof(Header), 0);
  }
  ok = ok && fdatasync(fd) == 0;
  close(fd);
  if (!ok) { unlink(tmp.c_str()); return false; }
  if (rename(tmp.c_str(), path(key).c_str()) != 0) { unlink(tmp.c_str()); return false; }
  std::lock_guard<std::mutex> l(mu_);
  PcacheEntry pe; pe.key = key; pe.tokens = tokens; pe.bytes = bytes; pe.last_use = ++clock_;
  index_[key] = pe;
  ++st_.saves;
  return true;
}

int64_t Pcache::load(const std::string& key, void* out, int64_t cap) {
  {
    std::lock_guard<std::mutex> l(mu_);
    auto it = index_.find(key);
    if (it == index_.end()) { ++st_.misses; return -1; }
    it->second.last_use = ++clock_;
  }
  int fd = -1;
  if (direct_) fd = open(path(key).c_str(), O_RDONLY | O_DIRECT);
  if (fd < 0) fd = open(path(key).c_str(), O_RDONLY);
  if (fd < 0) return -1;
  Aligned bounce(kChunk);
  Header h;
  bool ok = bounce.p && read_all(fd, bounce.p, sizeof(Header), 0);
  if (ok) memcpy(&h, bounce.p, sizeof(h));
  ok = ok && h.magic == kMagic && h.bytes <= cap;
  std::vector<uint64_t> sums;
  if (ok && h.chunks) {
    const int64_t padded_total = (h.bytes + 4095) / 4096 * 4096;
    const int64_t table = (h.chunks * 8 + 4095) / 4096 * 4096;
    ok = read_all(fd, bounce.p, table, sizeof(Header) + padded_total);
    if (ok) { sums.assign(static_cast<uint64_t*>(bounce.p), static_cast<uint64_t*>(bounce.p) + h.chunks); }
  }
  off_t off = sizeof(Header);
  for (int64_t c = 0; ok && c < h.chunks; ++c) {
    const int64_t n = std::min<int64_t>(kChunk, h.bytes - c * kChunk);
    const int64_t padded = (n + 4095) / 4096 * 4096;
    ok = read_all(fd, bounce.p, padded, off) && fnv64(bounce.p, n) == sums[c];
    if (ok) memcpy(static_cast<char*>(out) + c * kChunk, bounce.p, n);
    off += padded;
  }
  close(fd);
  std::lock_guard<std::mutex> l(mu_);
  if (!ok) { ++st_.corrupt; index_.erase(key); unlink(path(key).c_str()); return -1; }
  ++st_.loads; ++st_.hits;
  return h.bytes;
}

void Pcache::save_async(const std::string& key, int64_t tokens, const void* data, int64_t bytes, std::function<void(bool)> done) {
  { std::lock_guard<std::mutex> l(mu_); jobs_.push_back(Job{key, tokens, data, bytes, std::move(done)}); ++inflight_; }
  cv_.notify_one();
}

void Pcache::writer_loop() {
  for (;;) {
    Job j;
    {
      std::unique_lock<std::mutex> l(mu_);
      cv_.wait(l, [this] { return stop_ || !jobs_.empty(); });
      if (jobs_.empty()) { if (stop_) return; continue; }
      j = std::move(jobs_.front());
      jobs_.pop_front();
    }
    const bool ok = save(j.key, j.tokens, j.data, j.bytes);
    if (j.done) j.done(ok);
    { std::lock_guard<std::mutex> l(mu_); --inflight_; }
    idle_cv_.notify_all();
  }
}

void Pcache::drain() {
  std::unique_lock<std::mutex> l(mu_);
  idle_cv_.wait(l, [this] { return inflight_ == 0; });
}

int64_t Pcache::longest_prefix(const int32_t* ids, int64_t n, int64_t granule, std::string* key_out) {
  for (int64_t t = n / granule * granule; t > 0; t -= granule) {
    const std::string k = prefix_key(ids, t);
    std::lock_guard<std::mutex> l(mu_);
    auto it = index_.find(k);
    if (it != index_.end() && it->second.tokens == t) { if (key_out) *key_out = k; return t; }
  }
  return 0;
}

bool Pcache::contains(const std::string& key) { std::lock_guard<std::mutex> l(mu_); return index_.count(key) != 0; }
void Pcache::remove(const std::string& key) { std::lock_guard<std::mutex> l(mu_); if (index_.erase(key)) unlink(path(key).c_str()); }
std::vector<PcacheEntry> Pcache::entries() { std::lock_guard<std::mutex> l(mu_); std::vector<PcacheEntry> v; for (auto& kv : index_) v.push_back(kv.second); return v; }
void Pcache::keep_only(const std::vector<std::string>& keys) {
  std::lock_guard<std::mutex> l(mu_);
  for (auto it = index_.begin(); it != index_.end();) {
    if (std::find(keys.begin(), keys.end(), it->first) == keys.end()) { unlink(path(it->first).c_str()); it = index_.erase(it); }
    else ++it;
  }
}
int64_t Pcache::bytes_used() { std::lock_guard<std::mutex> l(mu_); int64_t s = 0; for (auto& kv : index_) s += kv.second.bytes; return s; }
Pcache::Stats Pcache::stats() { std::lock_guard<std::mutex> l(mu_); return st_; }

}  // namespace spark_rt
