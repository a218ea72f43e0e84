#pragma once
#include <atomic>
#include <cstdint>
#include <functional>
#include <string>
#include <thread>

namespace spark_rt {
int64_t mem_available_bytes(const char* meminfo_path = nullptr);
int64_t allocator_cap(int64_t reserved_bytes, int64_t margin_bytes, const char* meminfo_path = nullptr);
void trim_host_memory();
bool drop_file_cache(const char* path);

class MemWatch {
 public:
  MemWatch(int64_t threshold_bytes, int period_ms, std::function<void(int64_t)> on_low, const std::string& meminfo = "");
  ~MemWatch();
  int fired() const { return fired_.load(); }
 private:
  int64_t threshold_; int period_ms_;
  std::function<void(int64_t)> on_low_;
  std::string meminfo_;
  std::atomic<bool> stop_{false};
  std::atomic<int> fired_{0};
  std::thread th_;
};
}  // namespace spark_rt
