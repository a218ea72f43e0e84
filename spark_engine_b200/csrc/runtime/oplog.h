// Replicated op log between the ranks of one box: rank 0 decides a step and appends it; the other ranks (one
// process per GPU) read the same sequence and execute identical steps.  A single-producer ring in POSIX shared
// memory with a futex-free spin/yield wait bounded by a deadline; a heartbeat op keeps followers' deadlines alive,
// and a follower that sees no op before its deadline reports the leader as lost (fail-stop).
// Reference: engine-rs/src/spec_probe.rs:1515,1741-1758,2355-2383 (OP_* log, doorbell, followers),
// ds41/serve.rs:266-300 (JSON step per round on a TCP control channel); on one NVSwitch box shared memory replaces TCP.
#pragma once
#include <atomic>
#include <cstdint>
#include <string>
#include <vector>

namespace spark_rt {

struct OpRecord {
  uint64_t seq;
  int32_t kind;
  int32_t n;
  int32_t payload[1018];
};

class OpLog {
 public:
  static constexpr int kSlots = 64;
  // Leader: create = true, n_followers = how many readers must acknowledge a record before its slot is reused.
  // Follower: create = false, follower_index in [0, n_followers).
  OpLog(const std::string& name, bool create, int n_followers = 0, int follower_index = -1);
  ~OpLog();
  // leader
  // Appends a record; waits (bounded by timeout_ms) while the slowest follower is a whole ring behind.
  // Returns the sequence number, or 0 if a follower did not catch up in time (follower lost).
  uint64_t append(int kind, const std::vector<int32_t>& payload, int timeout_ms = 5000);
  // follower: waits up to timeout_ms for the record after `last_seq`; returns false on timeout (leader lost)
  bool next(uint64_t last_seq, int timeout_ms, int* kind, std::vector<int32_t>* payload);
  uint64_t head() const;
  // leader: waits up to timeout_ms until every follower has read record `seq`; returns the index of the first follower
  // that has not (a follower that stopped), or -1 when all have.  Called before a step whose collectives need every rank.
  int wait_acked(uint64_t seq, int timeout_ms) const;
  static void unlink_name(const std::string& name);

 private:
  struct Shared { std::atomic<uint64_t> head; std::atomic<uint64_t> acks[7]; OpRecord ring[kSlots]; };
  int n_followers_ = 0, index_ = -1;
  std::string name_;
  Shared* sh_ = nullptr;
  bool owner_;
};

}  // namespace spark_rt
