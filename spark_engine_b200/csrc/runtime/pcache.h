// Persistent prefix cache on NVMe: sequence-state checkpoints that survive restarts.
//
// An entry is keyed by the token prefix it covers and stored as ONE file: a header, the payload (whatever the
// model runner serialised: KV rows up to the boundary, linear-attention states, conv tails, indexer pools, last
// logits) written in chunks, and a table of per-chunk checksums.  Files are written to `<name>.tmp`, fdatasync'ed
// and renamed, so a crash never leaves a half-written entry under its final name.  Writers and readers run on
// their own threads with O_DIRECT when the file system supports it (aligned bounce buffers) so that cache I/O does
// not go through, or evict, the page cache.  The directory name is a SHA-256 over everything that determines the
// bytes (binary hash, model paths, numerics flags): a stale cache is never read.  A byte budget is enforced by
// evicting least-recently-used entries; at start-up the directory is scanned and entries with a bad header or
// checksum table are dropped ("reconciliation"), and under tensor parallelism the ranks keep only the
// intersection of valid entries (`agree`).
// Reference: engine-rs/src/pcache_core.rs:1-26,249-765, pcache.rs:1-29.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace spark_rt {

struct PcacheEntry {
  std::string key;        // hex digest of the token prefix
  int64_t tokens = 0;     // prefix length
  int64_t bytes = 0;      // payload bytes
  uint64_t last_use = 0;
};

class Pcache {
 public:
  static constexpr int64_t kChunk = 16ll << 20;
  Pcache(const std::string& root, const std::string& identity, int64_t byte_budget, bool direct_io = true);
  ~Pcache();
  static std::string identity_dir(const std::vector<std::string>& parts);        // SHA-256 hex of the parts
  static std::string prefix_key(const int32_t* ids, int64_t n);                  // SHA-256 hex of the token ids
  // Synchronous API (called from writer/reader threads or directly).
  bool save(const std::string& key, int64_t tokens, const void* data, int64_t bytes);
  int64_t load(const std::string& key, void* out, int64_t cap);                  // bytes read, -1 missing/corrupt
  // Asynchronous save: copies nothing, the caller keeps `data` alive until `done` runs on the writer thread.
  void save_async(const std::string& key, int64_t tokens, const void* data, int64_t bytes, std::function<void(bool)> done);
  void drain();
  // Longest cached prefix of ids[0:n] among boundaries that are multiples of `granule`; returns tokens (0 = none).
  int64_t longest_prefix(const int32_t* ids, int64_t n, int64_t granule, std::string* key_out);
  bool contains(const std::string& key);
  void remove(const std::string& key);
  std::vector<PcacheEntry> entries();
  void keep_only(const std::vector<std::string>& keys);                          // `agree`: intersection across ranks
  int64_t bytes_used();
  int reconcile();                                                               // returns dropped files
  std::string dir() const { return dir_; }
  struct Stats { int64_t saves = 0, loads = 0, hits = 0, misses = 0, evictions = 0, corrupt = 0; };
  Stats stats();

 private:
  std::string path(const std::string& key) const { return dir_ + "/" + key + ".pc"; }
  void evict_to_budget(int64_t incoming);
  void writer_loop();
  std::string dir_;
  int64_t budget_;
  bool direct_;
  std::mutex mu_;
  std::map<std::string, PcacheEntry> index_;
  uint64_t clock_ = 0;
  Stats st_;
  struct Job { std::string key; int64_t tokens; const void* data; int64_t bytes; std::function<void(bool)> done; };
  std::deque<Job> jobs_;
  std::condition_variable cv_, idle_cv_;
  bool stop_ = false;
  int inflight_ = 0;
  std::thread writer_;
};

}  // namespace spark_rt
