#include "kv_pool.h"

#include <algorithm>
#include <stdexcept>

namespace spark_rt {

KvPool::KvPool(int64_t total_tokens, int64_t granule) : total_(total_tokens / granule * granule), granule_(granule) {
  if (granule <= 0 || total_ <= 0) throw std::invalid_argument("KvPool: bad size");
}

int KvPool::acquire(int64_t tokens) {
  const int64_t need = round_up(std::max<int64_t>(tokens, 1));
  int64_t cursor = 0;
  for (auto it = by_base_.begin();; ++it) {
    const int64_t gap_end = (it == by_base_.end()) ? total_ : it->first;
    if (gap_end - cursor >= need) {
      Lease l;
      l.id = next_id_++; l.base = cursor; l.cap = need; l.last_use = ++clock_;
      leases_[l.id] = l;
      by_base_[l.base] = l.id;
      return l.id;
    }
    if (it == by_base_.end()) break;
    cursor = it->first + leases_.at(it->second).cap;
  }
  return -1;
}

bool KvPool::grow(int id, int64_t tokens) {
  auto it = leases_.find(id);
  if (it == leases_.end()) return false;
  Lease& l = it->second;
  const int64_t need = round_up(tokens);
  if (need <= l.cap) return true;
  auto nxt = by_base_.upper_bound(l.base);
  const int64_t limit = (nxt == by_base_.end()) ? total_ : nxt->first;
  if (l.base + need > limit) return false;
  l.cap = need;
  return true;
}

void KvPool::shrink(int id, int64_t tokens) {
  auto it = leases_.find(id);
  if (it == leases_.end()) return;
  Lease& l = it->second;
  const int64_t keep = round_up(std::max<int64_t>({tokens, l.used, 1}));
  if (keep < l.cap) l.cap = keep;
}

void KvPool::release(int id) {
  auto it = leases_.find(id);
  if (it == leases_.end()) return;
  by_base_.erase(it->second.base);
  leases_.erase(it);
}

void KvPool::touch(int id) { auto it = leases_.find(id); if (it != leases_.end()) it->second.last_use = ++clock_; }
void KvPool::pin(int id, bool on) { auto it = leases_.find(id); if (it != leases_.end()) it->second.pinned = on; }
void KvPool::set_used(int id, int64_t used) {
  auto it = leases_.find(id);
  if (it == leases_.end()) return;
  if (used > it->second.cap) throw std::out_of_range("sequence capacity exceeded");
  it->second.used = used;
}
const Lease* KvPool::get(int id) const { auto it = leases_.find(id); return it == leases_.end() ? nullptr : &it->second; }

int KvPool::lru_victim() const {
  int best = -1; uint64_t stamp = ~0ull;
  for (auto& kv : leases_) if (!kv.second.pinned && kv.second.last_use < stamp) { stamp = kv.second.last_use; best = kv.first; }
  return best;
}
int64_t KvPool::allocated_tokens() const { int64_t s = 0; for (auto& kv : leases_) s += kv.second.cap; return s; }
int64_t KvPool::active_tokens() const { int64_t s = 0; for (auto& kv : leases_) s += kv.second.used; return s; }
int64_t KvPool::free_tokens() const { return total_ - allocated_tokens(); }
int64_t KvPool::largest_free_run() const {
  int64_t cursor = 0, best = 0;
  for (auto& kv : by_base_) { best = std::max(best, kv.first - cursor); cursor = kv.first + leases_.at(kv.second).cap; }
  return std::max(best, total_ - cursor);
}
int64_t KvPool::bytes_per_token(const std::vector<ArrayLayout>& arrays, int layers) const {
  double b = 0;
  for (auto& a : arrays) b += static_cast<double>(a.width) / a.div;
  return static_cast<int64_t>(b * layers + 0.5);
}

}  // namespace spark_rt
