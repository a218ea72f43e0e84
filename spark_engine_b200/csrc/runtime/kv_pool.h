// KV pool: one pool of token rows per GPU, leased to sequence slots in granules.
// Contiguous first-fit placement (a sequence never moves; its region can grow in place while the following
// granules are free) with LRU eviction candidates for idle stores.  The same bookkeeping drives the CUDA-VMM
// backend (vmm.cpp), where a region keeps its virtual address and physical granules are mapped behind it.
// Reference: engine-rs/src/kv_pool.rs:1-19,53-241 (pool, leases, per-array {div,width,kind} layout),
// shim/vmm.cpp:28-86.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace spark_rt {

struct Lease {
  int id = -1;
  int64_t base = 0;      // first token row
  int64_t cap = 0;       // rows reserved (multiple of the granule)
  int64_t used = 0;      // rows holding committed tokens
  uint64_t last_use = 0; // LRU stamp
  bool pinned = false;   // running sequences cannot be evicted
};

struct ArrayLayout {     // one cached array of a layer: rows = tokens / div, row width in bytes
  std::string name;
  int div = 1;
  int width = 0;
  int kind = 0;
};

class KvPool {
 public:
  KvPool(int64_t total_tokens, int64_t granule);
  // Reserve room for `tokens` rows.  Returns lease id or -1 (nothing is modified on failure: capacity checks
  // fail before any state is written).
  int acquire(int64_t tokens);
  bool grow(int id, int64_t tokens);          // in place; false if the following granules are taken
  void shrink(int id, int64_t tokens);
  void release(int id);
  void touch(int id);
  void pin(int id, bool on);
  void set_used(int id, int64_t used);
  const Lease* get(int id) const;
  int lru_victim() const;                     // idle lease with the oldest stamp, -1 if none
  int64_t free_tokens() const;
  int64_t largest_free_run() const;
  int64_t allocated_tokens() const;
  int64_t active_tokens() const;
  int64_t total() const { return total_; }
  int64_t granule() const { return granule_; }
  int64_t bytes_per_token(const std::vector<ArrayLayout>& arrays, int layers) const;

 private:
  int64_t round_up(int64_t t) const { return (t + granule_ - 1) / granule_ * granule_; }
  int64_t total_, granule_;
  std::map<int64_t, int> by_base_;            // base -> lease id
  std::map<int, Lease> leases_;
  int next_id_ = 0;
  uint64_t clock_ = 0;
};

}  // namespace spark_rt
