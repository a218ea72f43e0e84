#include "oplog.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace spark_rt {

OpLog::OpLog(const std::string& name, bool create, int n_followers, int follower_index)
    : name_(name), owner_(create), n_followers_(n_followers), index_(follower_index) {
  if (n_followers > 7 || follower_index >= 7) throw std::invalid_argument("oplog: at most 7 followers");
  int fd = shm_open(name.c_str(), create ? (O_CREAT | O_RDWR) : O_RDWR, 0600);
  if (fd < 0) throw std::runtime_error("oplog: shm_open failed for " + name);
  if (create && ftruncate(fd, sizeof(Shared)) != 0) { close(fd); throw std::runtime_error("oplog: ftruncate failed"); }
  void* p = mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) throw std::runtime_error("oplog: mmap failed");
  sh_ = static_cast<Shared*>(p);
  if (create) { memset(p, 0, sizeof(Shared)); sh_->head.store(0, std::memory_order_release); }
}

OpLog::~OpLog() {
  if (sh_) munmap(sh_, sizeof(Shared));
  if (owner_) shm_unlink(name_.c_str());
}

void OpLog::unlink_name(const std::string& name) { shm_unlink(name.c_str()); }

uint64_t OpLog::append(int kind, const std::vector<int32_t>& payload, int timeout_ms) {
  if (payload.size() > 1018) throw std::length_error("oplog: payload too long");
  const uint64_t seq = sh_->head.load(std::memory_order_relaxed) + 1;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (int f = 0; f < n_followers_; ++f) {           // flow control: never overwrite a record a follower still needs
    while (seq - sh_->acks[f].load(std::memory_order_acquire) > static_cast<uint64_t>(kSlots - 1)) {
      if (std::chrono::steady_clock::now() > deadline) return 0;
      std::this_thread::yield();
    }
  }
  OpRecord& r = sh_->ring[seq % kSlots];
  r.kind = kind; r.n = static_cast<int32_t>(payload.size());
  if (!payload.empty()) memcpy(r.payload, payload.data(), payload.size() * 4);
  r.seq = seq;
  sh_->head.store(seq, std::memory_order_release);
  return seq;
}

int OpLog::wait_acked(uint64_t seq, int timeout_ms) const {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (int f = 0; f < n_followers_; ++f) {
    int spins = 0;
    while (sh_->acks[f].load(std::memory_order_acquire) < seq) {
      if (std::chrono::steady_clock::now() > deadline) return f;
      if (++spins < 200) std::this_thread::yield(); else std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
  return -1;
}

uint64_t OpLog::head() const { return sh_->head.load(std::memory_order_acquire); }

bool OpLog::next(uint64_t last_seq, int timeout_ms, int* kind, std::vector<int32_t>* payload) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  int spins = 0;
  while (sh_->head.load(std::memory_order_acquire) <= last_seq) {
    if (std::chrono::steady_clock::now() > deadline) return false;
    if (++spins < 200) std::this_thread::yield(); else std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  const uint64_t want = last_seq + 1;
  const OpRecord& r = sh_->ring[want % kSlots];
  if (r.seq != want) throw std::runtime_error("oplog: follower fell more than one ring behind");
  *kind = r.kind;
  payload->assign(r.payload, r.payload + r.n);
  if (index_ >= 0) sh_->acks[index_].store(want, std::memory_order_release);
  return true;
}

}  // namespace spark_rt
