// Host scheduler core: request queue, admission with KV budget and prefix reuse planning, round-robin between one
// prefill chunk and one batched decode round, cancellation, statistics.  Pure host logic (no CUDA): rank 0 runs it
// and replicates the chosen step to the other ranks, which execute identical steps (lockstep graphs).
// Reference: engine-rs/src/spec_probe.rs:2407-2708 (rank-0 loop: socket -> queue -> admission -> unit of work),
// :2482-2603 (admission planner: continue store / restore checkpoint / clone / library / NVMe / cold),
// qwen/serve.rs:158-470, ds41/serve.rs:448-1051.
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <string>
#include <vector>

namespace spark_rt {

struct Request {
  int64_t id = 0;
  std::vector<int32_t> prompt;
  int max_new = 256;
  std::vector<int32_t> stop;
  float temperature = 0.f;
  uint64_t seed = 0;
  double t_arrive = 0;
};

enum class ReuseKind : int { Cold = 0, ContinueStore = 1, Checkpoint = 2, CloneStore = 3, Library = 4, Disk = 5 };

struct AdmitPlan {
  int64_t request_id = -1;
  int slot = -1;
  ReuseKind kind = ReuseKind::Cold;
  int source = -1;             // store / checkpoint index the prefix comes from
  int64_t reuse_tokens = 0;    // tokens that need no prefill
  int evict_slot = -1;         // idle store to evict first (-1 none)
};

struct SlotState {
  bool busy = false;           // running a request
  int64_t request_id = -1;
  std::vector<int32_t> tokens; // history of the store (prompt + generated) for prefix matching
  int64_t prefilled = 0;       // prompt tokens already processed
  int64_t prompt_len = 0;
  int generated = 0;
  int max_new = 0;
  bool cancelled = false;
  uint64_t last_use = 0;
};

struct PrefillPart { int slot = -1; int64_t begin = 0, end = 0; };

struct Step {
  enum Kind : int { Idle = 0, Admit = 1, Prefill = 2, Decode = 3, Cancel = 4 } kind = Idle;
  AdmitPlan admit;
  int slot = -1;                       // Prefill (first part) / Cancel
  int64_t chunk_begin = 0, chunk_end = 0;
  // Prefill: every sequence that still has prompt tokens gets a share of the chunk budget in the same forward (one
  // segment each), so a layer's weights are read once for all of them; parts[0] repeats slot / chunk_begin / chunk_end
  std::vector<PrefillPart> parts;
  std::vector<int> decode_slots;       // Decode: sequences batched into this round
};

struct SchedStats {
  int64_t waiting = 0, running = 0, decoding = 0, prefilling = 0, admitted = 0, finished = 0, cancelled = 0;
  int64_t prefix_hit_tokens = 0, kv_budget = 0, kv_active = 0;
};

class Scheduler {
 public:
  Scheduler(int n_slots, int64_t kv_budget_tokens, int64_t slot_tokens, int prefill_chunk, int max_batch);
  void submit(const Request& r);
  bool cancel(int64_t request_id);
  // checkpoints: (index, tokens covered); disk: longest cached prefix callback result supplied by the caller
  void set_checkpoint(int index, const std::vector<int32_t>& tokens);
  void drop_checkpoint(int index);
  Step next(int64_t disk_prefix_tokens = 0);      // decide one unit of work
  // feedback from the executor
  void on_admitted(const AdmitPlan& p);
  void on_prefilled(int slot, int64_t upto);
  void on_tokens(int slot, const std::vector<int32_t>& toks, bool finished);
  void on_finished(int slot);
  const SlotState& slot(int i) const { return slots_[i]; }
  const Request* request(int64_t id) const;
  SchedStats stats() const;
  // anything queued or running (a step may still turn out idle, e.g. a queued request waiting for KV room)
  bool has_work() const {
    if (!queue_.empty()) return true;
    for (auto& s : slots_) if (s.busy) return true;
    return false;
  }
  static int64_t common_prefix(const std::vector<int32_t>& a, const std::vector<int32_t>& b);

 private:
  AdmitPlan plan(const Request& r, int64_t disk_prefix_tokens);
  int n_slots_;
  int64_t kv_budget_, slot_tokens_;
  int chunk_, max_batch_;
  std::deque<Request> queue_;
  std::map<int64_t, Request> live_;
  std::vector<SlotState> slots_;
  std::map<int, std::vector<int32_t>> checkpoints_;
  uint64_t clock_ = 0;
  bool last_was_prefill_ = false;
  int rr_ = 0;
  SchedStats st_;
};

}  // namespace spark_rt
