// Host memory guard: reads MemAvailable, answers "how much may the allocator use" (reserved + available - margin),
// trims malloc arenas and drops this process's file cache pages.  A watch thread calls a callback when available
// memory falls below a threshold so the engine can shed load before the OOM killer acts.
// Reference: engine-rs/src/ds41/mem.rs:48-163, host_memory.rs:22-104, serve/start-qwen.sh:20-29.
#include "memguard.h"

#include <fcntl.h>
#include <malloc.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>

namespace spark_rt {

int64_t mem_available_bytes(const char* meminfo_path) {
  FILE* f = fopen(meminfo_path ? meminfo_path : "/proc/meminfo", "r");
  if (!f) return -1;
  char line[256];
  int64_t kb = -1;
  while (fgets(line, sizeof(line), f))
    if (strncmp(line, "MemAvailable:", 13) == 0) { long long v; if (sscanf(line + 13, "%lld", &v) == 1) kb = v; break; }
  fclose(f);
  return kb < 0 ? -1 : kb * 1024;
}

int64_t allocator_cap(int64_t reserved_bytes, int64_t margin_bytes, const char* meminfo_path) {
  const int64_t avail = mem_available_bytes(meminfo_path);
  if (avail < 0) return -1;
  const int64_t cap = reserved_bytes + avail - margin_bytes;
  return cap > 0 ? cap : 0;
}

void trim_host_memory() { malloc_trim(0); }

bool drop_file_cache(const char* path) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) return false;
  const bool ok = posix_fadvise(fd, 0, 0, POSIX_FADV_DONTNEED) == 0;
  close(fd);
  return ok;
}

MemWatch::MemWatch(int64_t threshold_bytes, int period_ms, std::function<void(int64_t)> on_low, const std::string& meminfo)
    : threshold_(threshold_bytes), period_ms_(period_ms), on_low_(std::move(on_low)), meminfo_(meminfo) {
  th_ = std::thread([this] {
    while (!stop_.load()) {
      const int64_t a = mem_available_bytes(meminfo_.empty() ? nullptr : meminfo_.c_str());
      if (a >= 0 && a < threshold_) { ++fired_; if (on_low_) on_low_(a); }
      for (int i = 0; i < period_ms_ / 10 && !stop_.load(); ++i) std::this_thread::sleep_for(std::chrono::milliseconds(10));
    }
  });
}
MemWatch::~MemWatch() { stop_.store(true); if (th_.joinable()) th_.join(); }

}  // namespace spark_rt
