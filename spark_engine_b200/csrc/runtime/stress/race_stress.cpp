// Concurrency stress of the host runtime, meant to be built with -fsanitize=thread (data races) and
// -fsanitize=address (lifetime / bounds) and run on a machine without a GPU:
//   prefix cache   several threads save (sync and async), load, list, look up and remove entries while the writer
//                  thread runs and the byte budget evicts
//   op log         one leader appends records with checked payloads, two followers read them through their own
//                  mappings of the shared ring and acknowledge
//   memory watch   the watch thread fires on a fake meminfo file while the owner reads the counter, then is joined
//   fast load      reader threads fill pinned staging buffers that the issuing thread hands to the (fake) driver
// Exit code 0 and no sanitizer report = pass.  The reference has no sanitizer builds (engine-rs/build.rs:80-93).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <thread>
#include <vector>
#include <unistd.h>

#include "../devmem.h"
#include "../memguard.h"
#include "../oplog.h"
#include "../pcache.h"

using namespace spark_rt;

static int failures = 0;
#define EXPECT(c) do { if (!(c)) { std::fprintf(stderr, "FAILED %s:%d %s\n", __FILE__, __LINE__, #c); ++failures; } } while (0)

static void stress_pcache(const std::string& root) {
  Pcache pc(root, Pcache::identity_dir({"race", "stress"}), 6ll << 20, /*direct_io=*/false);
  std::atomic<int> done_cb{0};
  std::atomic<int> bad{0};
  std::vector<std::thread> th;
  for (int w = 0; w < 4; ++w) {
    th.emplace_back([&, w] {
      std::vector<std::vector<char>> keep;                    // async payloads stay alive until drain()
      keep.reserve(16);
      for (int i = 0; i < 12; ++i) {
        std::vector<int32_t> ids(64 + i, w * 1000 + i);
        const std::string key = Pcache::prefix_key(ids.data(), static_cast<int64_t>(ids.size()));
        keep.emplace_back(200000 + 1000 * i, static_cast<char>(w * 16 + i));
        auto& buf = keep.back();
        if (i & 1) pc.save_async(key, static_cast<int64_t>(ids.size()), buf.data(), static_cast<int64_t>(buf.size()),
                                 [&done_cb](bool) { done_cb.fetch_add(1); });
        else pc.save(key, static_cast<int64_t>(ids.size()), buf.data(), static_cast<int64_t>(buf.size()));
        std::vector<char> out(buf.size());
        const int64_t n = pc.load(key, out.data(), static_cast<int64_t>(out.size()));
        if (n >= 0 && (n != static_cast<int64_t>(buf.size()) || out[0] != buf[0] || out.back() != buf.back())) bad.fetch_add(1);
        pc.contains(key);
        pc.entries();
        pc.bytes_used();
        std::string k2;
        pc.longest_prefix(ids.data(), static_cast<int64_t>(ids.size()), 16, &k2);
        if (i % 5 == 4) pc.remove(key);
      }
      pc.drain();
    });
  }
  for (auto& t : th) t.join();
  pc.drain();
  EXPECT(bad.load() == 0);
  EXPECT(done_cb.load() == 4 * 6);
  EXPECT(pc.bytes_used() <= (6ll << 20));
  EXPECT(pc.stats().saves > 0);
}

static void stress_oplog() {
  const std::string name = "/spark_race_" + std::to_string(::getpid());
  OpLog::unlink_name(name);
  {
    OpLog leader(name, true, 2);
    constexpr int N = 400;
    std::atomic<int> wrong{0};
    std::vector<std::thread> fol;
    for (int f = 0; f < 2; ++f) {
      fol.emplace_back([&, f] {
        OpLog me(name, false, 2, f);
        uint64_t last = 0;
        for (int i = 0; i < N; ++i) {
          int kind = -1;
          std::vector<int32_t> p;
          if (!me.next(last, 5000, &kind, &p)) { wrong.fetch_add(1000); return; }
          ++last;
          if (kind != (i % 7) || static_cast<int>(p.size()) != 1 + i % 50 || p[0] != i || p.back() != i + static_cast<int>(p.size()) - 1)
            wrong.fetch_add(1);
        }
      });
    }
    for (int i = 0; i < N; ++i) {
      std::vector<int32_t> p(1 + i % 50);
      for (size_t j = 0; j < p.size(); ++j) p[j] = i + static_cast<int>(j);
      EXPECT(leader.append(i % 7, p, 5000) == static_cast<uint64_t>(i + 1));
    }
    EXPECT(leader.wait_acked(N, 5000) == -1);
    for (auto& t : fol) t.join();
    EXPECT(wrong.load() == 0);
  }
  OpLog::unlink_name(name);
}

static void stress_memwatch(const std::string& root) {
  const std::string mi = root + "/meminfo";
  { std::ofstream f(mi); f << "MemTotal:       1000000 kB\nMemAvailable:     100000 kB\n"; }
  std::atomic<int64_t> seen{0};
  {
    MemWatch w(1ll << 30, 2, [&seen](int64_t avail) { seen.store(avail); }, mi);
    for (int i = 0; i < 200 && w.fired() == 0; ++i) ::usleep(1000);
    EXPECT(w.fired() > 0);
  }
  EXPECT(seen.load() == 100000ll * 1024);
}

static void stress_fast_load(const std::string& root) {
  const DriverApi* api = fake_driver_api();
  const std::string path = root + "/blob.bin";
  const size_t n = 3 * (1 << 20) + 12345;
  std::vector<unsigned char> src(n);
  for (size_t i = 0; i < n; ++i) src[i] = static_cast<unsigned char>(i * 131 + 7);
  { std::ofstream f(path, std::ios::binary); f.write(reinterpret_cast<const char*>(src.data()), static_cast<std::streamsize>(n)); }
  std::vector<unsigned char> dst(n, 0);                       // the fake driver's "device memory" is host memory
  const LoadStats st = fast_load(api, path, 0, static_cast<int64_t>(n), reinterpret_cast<uint64_t>(dst.data()), 0, 256 << 10, 3, 3);
  EXPECT(st.bytes == static_cast<int64_t>(n));
  EXPECT(std::memcmp(src.data(), dst.data(), n) == 0);
  // the same through O_DIRECT reads at an unaligned offset (falls back to buffered reads where the flag is refused)
  std::vector<unsigned char> dst2(n - 4099, 0);
  const LoadStats st2 = fast_load(api, path, 4099, static_cast<int64_t>(n - 4099), reinterpret_cast<uint64_t>(dst2.data()), 0, 300001, 2, 3, true);
  EXPECT(st2.bytes == static_cast<int64_t>(n - 4099));
  EXPECT(std::memcmp(src.data() + 4099, dst2.data(), n - 4099) == 0);
}

int main(int argc, char** argv) {
  const std::string root = argc > 1 ? argv[1] : "/tmp";
  stress_pcache(root);
  stress_oplog();
  stress_memwatch(root);
  stress_fast_load(root);
  if (failures) { std::fprintf(stderr, "%d expectation(s) failed\n", failures); return 1; }
  std::puts("race_stress ok");
  return 0;
}
