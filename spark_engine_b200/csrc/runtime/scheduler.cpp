#include "scheduler.h"

#include <algorithm>

namespace spark_rt {

Scheduler::Scheduler(int n_slots, int64_t kv_budget_tokens, int64_t slot_tokens, int prefill_chunk, int max_batch)
    : n_slots_(n_slots), kv_budget_(kv_budget_tokens), slot_tokens_(slot_tokens), chunk_(prefill_chunk),
      max_batch_(max_batch), slots_(n_slots) {
  st_.kv_budget = kv_budget_tokens;
}

int64_t Scheduler::common_prefix(const std::vector<int32_t>& a, const std::vector<int32_t>& b) {
  const size_t n = std::min(a.size(), b.size());
  size_t i = 0;
  while (i < n && a[i] == b[i]) ++i;
  return static_cast<int64_t>(i);
}

void Scheduler::submit(const Request& r) { queue_.push_back(r); }

bool Scheduler::cancel(int64_t id) {
  for (auto it = queue_.begin(); it != queue_.end(); ++it)
    if (it->id == id) { queue_.erase(it); ++st_.cancelled; return true; }
  for (auto& s : slots_)
    if (s.busy && s.request_id == id) { s.cancelled = true; return true; }
  return false;
}

void Scheduler::set_checkpoint(int index, const std::vector<int32_t>& tokens) { checkpoints_[index] = tokens; }
void Scheduler::drop_checkpoint(int index) { checkpoints_.erase(index); }

const Request* Scheduler::request(int64_t id) const {
  auto it = live_.find(id);
  return it == live_.end() ? nullptr : &it->second;
}

// Choose where the request runs and which cached prefix it starts from.  A usable prefix must leave at least one
// prompt token to prefill (the last prompt token's logits are needed).
AdmitPlan Scheduler::plan(const Request& r, int64_t disk_prefix_tokens) {
  AdmitPlan p;
  p.request_id = r.id;
  const int64_t limit = static_cast<int64_t>(r.prompt.size()) - 1;
  // 1. an idle store whose history is a prefix of the prompt: continue it in place (no copy at all)
  int best_slot = -1; int64_t best = 0;
  for (int i = 0; i < n_slots_; ++i) {
    if (slots_[i].busy) continue;
    const int64_t c = std::min(common_prefix(slots_[i].tokens, r.prompt), limit);
    if (c == static_cast<int64_t>(slots_[i].tokens.size()) && c > best) { best = c; best_slot = i; }
  }
  // 2. checkpoints / other stores whose prefix matches (restored or cloned into a free slot)
  int ck = -1; int64_t ck_len = 0;
  for (auto& kv : checkpoints_) {
    const int64_t c = common_prefix(kv.second, r.prompt);
    if (c == static_cast<int64_t>(kv.second.size()) && c <= limit && c > ck_len) { ck_len = c; ck = kv.first; }
  }
  int free_slot = -1, lru_slot = -1; uint64_t lru = ~0ull;
  for (int i = 0; i < n_slots_; ++i) {
    if (slots_[i].busy) continue;
    if (slots_[i].tokens.empty() && free_slot < 0) free_slot = i;
    if (slots_[i].last_use < lru) { lru = slots_[i].last_use; lru_slot = i; }
  }
  const int target = free_slot >= 0 ? free_slot : lru_slot;
  if (best_slot >= 0 && best >= ck_len && best >= disk_prefix_tokens && best > 0) {
    p.slot = best_slot; p.kind = ReuseKind::ContinueStore; p.source = best_slot; p.reuse_tokens = best;
    return p;
  }
  if (target < 0) return p;                                    // no slot: stay queued
  p.slot = target;
  if (free_slot < 0) p.evict_slot = target;                    // an idle store with history is overwritten
  if (ck >= 0 && ck_len >= disk_prefix_tokens && ck_len > 0) { p.kind = ReuseKind::Checkpoint; p.source = ck; p.reuse_tokens = ck_len; }
  else if (disk_prefix_tokens > 0 && disk_prefix_tokens <= limit) { p.kind = ReuseKind::Disk; p.reuse_tokens = disk_prefix_tokens; }
  return p;
}

Step Scheduler::next(int64_t disk_prefix_tokens) {
  Step s;
  // cancellations first
  for (int i = 0; i < n_slots_; ++i)
    if (slots_[i].busy && slots_[i].cancelled) { s.kind = Step::Cancel; s.slot = i; return s; }
  // admission: FIFO, needs a slot and KV room for prompt + max_new
  if (!queue_.empty()) {
    const Request& r = queue_.front();
    const int64_t need = static_cast<int64_t>(r.prompt.size()) + r.max_new;
    int64_t active = 0;
    for (auto& sl : slots_) if (sl.busy) active += sl.prompt_len + sl.max_new;
    if (need <= slot_tokens_ && active + need <= kv_budget_) {
      AdmitPlan p = plan(r, disk_prefix_tokens);
      if (p.slot >= 0) { s.kind = Step::Admit; s.admit = p; return s; }
    } else if (need > slot_tokens_) {
      // can never fit: reject by admitting with slot -1 (executor reports the error)
      s.kind = Step::Admit; s.admit.request_id = r.id; s.admit.slot = -1; return s;
    }
  }
  std::vector<int> pre, dec;
  for (int i = 0; i < n_slots_; ++i) {
    if (!slots_[i].busy) continue;
    (slots_[i].prefilled < slots_[i].prompt_len ? pre : dec).push_back(i);
  }
  // alternate one prefill chunk with one batched decode round so that running streams keep their cadence
  const bool do_prefill = !pre.empty() && (dec.empty() || !last_was_prefill_);
  if (do_prefill) {
    const int n = static_cast<int>(pre.size()), first = rr_++ % n;
    s.kind = Step::Prefill;
    // equal shares of the chunk budget; what a sequence with few tokens left does not use goes to the others (two passes:
    // sequences that fit their share first, then the rest split what remains)
    std::vector<int64_t> want(n), give(n, 0);
    int64_t budget = chunk_;
    int open = n;
    for (int k = 0; k < n; ++k) { const int i = pre[(first + k) % n]; want[k] = slots_[i].prompt_len - slots_[i].prefilled; }
    for (int pass = 0; pass < 2 && open > 0; ++pass) {
      const int64_t share = std::max<int64_t>(1, budget / open);
      for (int k = 0; k < n; ++k) {
        if (give[k] > 0) continue;
        if (pass == 0 && want[k] > share) continue;             // the long ones wait for the second pass
        give[k] = std::min(want[k], std::max<int64_t>(share, 1));
        budget -= give[k];
        --open;
      }
      if (budget < open) budget = open;                            // every sequence advances by at least one token
    }
    for (int k = 0; k < n; ++k) {
      const int i = pre[(first + k) % n];
      PrefillPart p;
      p.slot = i;
      p.begin = slots_[i].prefilled;
      p.end = p.begin + give[k];
      s.parts.push_back(p);
    }
    s.slot = s.parts[0].slot; s.chunk_begin = s.parts[0].begin; s.chunk_end = s.parts[0].end;
    last_was_prefill_ = true;
    return s;
  }
  if (!dec.empty()) {
    if (static_cast<int>(dec.size()) > max_batch_) {            // rotate so that nobody starves
      std::rotate(dec.begin(), dec.begin() + (rr_++ % dec.size()), dec.end());
      dec.resize(max_batch_);
      std::sort(dec.begin(), dec.end());
    }
    s.kind = Step::Decode; s.decode_slots = dec;
    last_was_prefill_ = false;
    return s;
  }
  return s;
}

void Scheduler::on_admitted(const AdmitPlan& p) {
  if (queue_.empty() || queue_.front().id != p.request_id) return;
  Request r = queue_.front();
  queue_.pop_front();
  if (p.slot < 0) { ++st_.finished; return; }
  SlotState& s = slots_[p.slot];
  s.busy = true; s.request_id = r.id; s.cancelled = false;
  s.prompt_len = static_cast<int64_t>(r.prompt.size());
  s.prefilled = p.reuse_tokens; s.generated = 0; s.max_new = r.max_new;
  s.tokens = r.prompt;
  s.last_use = ++clock_;
  live_[r.id] = std::move(r);
  ++st_.admitted;
  st_.prefix_hit_tokens += p.reuse_tokens;
}

void Scheduler::on_prefilled(int slot, int64_t upto) { slots_[slot].prefilled = upto; slots_[slot].last_use = ++clock_; }

void Scheduler::on_tokens(int slot, const std::vector<int32_t>& toks, bool finished) {
  SlotState& s = slots_[slot];
  s.tokens.insert(s.tokens.end(), toks.begin(), toks.end());
  s.generated += static_cast<int>(toks.size());
  s.last_use = ++clock_;
  if (finished) on_finished(slot);
}

void Scheduler::on_finished(int slot) {
  SlotState& s = slots_[slot];
  if (!s.busy) return;
  live_.erase(s.request_id);
  s.busy = false; s.request_id = -1;
  if (s.cancelled) { ++st_.cancelled; s.cancelled = false; } else ++st_.finished;
}

SchedStats Scheduler::stats() const {
  SchedStats st = st_;
  st.waiting = static_cast<int64_t>(queue_.size());
  for (auto& s : slots_) {
    if (!s.busy) continue;
    ++st.running;
    if (s.prefilled < s.prompt_len) ++st.prefilling; else ++st.decoding;
    st.kv_active += static_cast<int64_t>(s.tokens.size());
  }
  return st;
}

}  // namespace spark_rt
