#include "devmem.h"

#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <thread>

// ------------------------------------------------------------------------------------------------ real driver
namespace {
struct CuProp { int type; int requestedHandleTypes; struct { int type; int id; } location; void* win32; struct { unsigned char c; unsigned char g; unsigned short u; unsigned char r[4]; } flags; };
struct CuAccess { struct { int type; int id; } location; int flags; };
typedef int (*fn_init)(unsigned);
typedef int (*fn_gran)(size_t*, const CuProp*, int);
typedef int (*fn_reserve)(uint64_t*, size_t, size_t, uint64_t, unsigned long long);
typedef int (*fn_addrfree)(uint64_t, size_t);
typedef int (*fn_create)(uint64_t*, size_t, const CuProp*, unsigned long long);
typedef int (*fn_release)(uint64_t);
typedef int (*fn_map)(uint64_t, size_t, size_t, uint64_t, unsigned long long);
typedef int (*fn_unmap)(uint64_t, size_t);
typedef int (*fn_access)(uint64_t, size_t, const CuAccess*, size_t);
typedef int (*fn_hreg)(void*, size_t, unsigned);
typedef int (*fn_hunreg)(void*);
typedef int (*fn_h2d)(uint64_t, const void*, size_t, void*);
typedef int (*fn_ssync)(void*);
typedef int (*fn_ctx)(void**, int);
typedef int (*fn_setctx)(void*);

struct Real {
  fn_gran gran; fn_reserve reserve; fn_addrfree addrfree; fn_create create; fn_release release; fn_map map; fn_unmap unmap;
  fn_access access; fn_hreg hreg; fn_hunreg hunreg; fn_h2d h2d; fn_ssync ssync; fn_ctx ctx_retain; fn_setctx ctx_set;
} R;

CuProp prop_for(int device) {
  CuProp p;
  std::memset(&p, 0, sizeof(p));
  p.type = 1;              // pinned device memory
  p.location.type = 1;     // device
  p.location.id = device;
  return p;
}
void ensure_ctx(int device) {      // worker threads need the primary context current
  void* ctx = nullptr;
  if (R.ctx_retain && R.ctx_retain(&ctx, device) == 0 && ctx) R.ctx_set(ctx);
}
int r_gran(int device, size_t* out) { CuProp p = prop_for(device); return R.gran(out, &p, 0); }
int r_reserve(uint64_t* ptr, size_t size, size_t align) { return R.reserve(ptr, size, align, 0, 0); }
int r_addrfree(uint64_t ptr, size_t size) { return R.addrfree(ptr, size); }
int r_create(uint64_t* h, size_t size, int device) { CuProp p = prop_for(device); return R.create(h, size, &p, 0); }
int r_release(uint64_t h) { return R.release(h); }
int r_map(uint64_t ptr, size_t size, uint64_t h) { return R.map(ptr, size, 0, h, 0); }
int r_unmap(uint64_t ptr, size_t size) { return R.unmap(ptr, size); }
int r_access(uint64_t ptr, size_t size, int device) {
  CuAccess a; a.location.type = 1; a.location.id = device; a.flags = 3;   // read + write
  return R.access(ptr, size, &a, 1);
}
int r_hreg(void* p, size_t n) { return R.hreg(p, n, 1 /* portable */); }
int r_hunreg(void* p) { return R.hunreg(p); }
int r_h2d(uint64_t dst, const void* src, size_t n, uint64_t stream) { return R.h2d(dst, src, n, reinterpret_cast<void*>(stream)); }
int r_ssync(uint64_t stream) { return R.ssync(reinterpret_cast<void*>(stream)); }
}  // namespace

const DriverApi* cuda_driver_api() {
  static DriverApi api;
  static int state = 0;      // 0 unknown, 1 ok, -1 unavailable
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  if (state == 0) {
    void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    state = -1;
    if (h) {
      auto sym = [&](const char* n) { return dlsym(h, n); };
      fn_init init = reinterpret_cast<fn_init>(sym("cuInit"));
      R.gran = reinterpret_cast<fn_gran>(sym("cuMemGetAllocationGranularity"));
      R.reserve = reinterpret_cast<fn_reserve>(sym("cuMemAddressReserve"));
      R.addrfree = reinterpret_cast<fn_addrfree>(sym("cuMemAddressFree"));
      R.create = reinterpret_cast<fn_create>(sym("cuMemCreate"));
      R.release = reinterpret_cast<fn_release>(sym("cuMemRelease"));
      R.map = reinterpret_cast<fn_map>(sym("cuMemMap"));
      R.unmap = reinterpret_cast<fn_unmap>(sym("cuMemUnmap"));
      R.access = reinterpret_cast<fn_access>(sym("cuMemSetAccess"));
      R.hreg = reinterpret_cast<fn_hreg>(sym("cuMemHostRegister_v2"));
      R.hunreg = reinterpret_cast<fn_hunreg>(sym("cuMemHostUnregister"));
      R.h2d = reinterpret_cast<fn_h2d>(sym("cuMemcpyHtoDAsync_v2"));
      R.ssync = reinterpret_cast<fn_ssync>(sym("cuStreamSynchronize"));
      R.ctx_retain = reinterpret_cast<fn_ctx>(sym("cuDevicePrimaryCtxRetain"));
      R.ctx_set = reinterpret_cast<fn_setctx>(sym("cuCtxSetCurrent"));
      if (init && R.gran && R.reserve && R.addrfree && R.create && R.release && R.map && R.unmap && R.access && R.hreg &&
          R.hunreg && R.h2d && R.ssync && init(0) == 0) {
        api = DriverApi{r_gran, r_reserve, r_addrfree, r_create, r_release, r_map, r_unmap, r_access, r_hreg, r_hunreg, r_h2d,
                        r_ssync, true};
        state = 1;
      }
    }
  }
  return state == 1 ? &api : nullptr;
}

// ------------------------------------------------------------------------------------------------ fake driver
namespace {
std::mutex fake_mu;
std::map<uint64_t, size_t> fake_ranges;          // reserved ranges (backed by one anonymous mapping each)
std::map<uint64_t, size_t> fake_handles;
std::map<uint64_t, size_t> fake_mapped;
uint64_t fake_next_handle = 1;
std::atomic<int64_t> fake_bytes{0};

int f_gran(int, size_t* out) { *out = 64 * 1024; return 0; }
int f_reserve(uint64_t* ptr, size_t size, size_t) {
  void* p = mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (p == MAP_FAILED) return 2;
  std::lock_guard<std::mutex> lk(fake_mu);
  fake_ranges[reinterpret_cast<uint64_t>(p)] = size;
  *ptr = reinterpret_cast<uint64_t>(p);
  return 0;
}
int f_addrfree(uint64_t ptr, size_t size) {
  std::lock_guard<std::mutex> lk(fake_mu);
  fake_ranges.erase(ptr);
  return munmap(reinterpret_cast<void*>(ptr), size);
}
int f_create(uint64_t* h, size_t size, int) { std::lock_guard<std::mutex> lk(fake_mu); *h = fake_next_handle++; fake_handles[*h] = size; return 0; }
int f_release(uint64_t h) { std::lock_guard<std::mutex> lk(fake_mu); return fake_handles.erase(h) ? 0 : 1; }
int f_map(uint64_t ptr, size_t size, uint64_t h) {
  std::lock_guard<std::mutex> lk(fake_mu);
  if (!fake_handles.count(h) || fake_handles[h] != size || fake_mapped.count(ptr)) return 1;
  fake_mapped[ptr] = size;
  fake_bytes += static_cast<int64_t>(size);
  return 0;
}
int f_unmap(uint64_t ptr, size_t size) {
  std::lock_guard<std::mutex> lk(fake_mu);
  auto it = fake_mapped.find(ptr);
  if (it == fake_mapped.end() || it->second != size) return 1;
  fake_mapped.erase(it);
  fake_bytes -= static_cast<int64_t>(size);
  madvise(reinterpret_cast<void*>(ptr), size, MADV_DONTNEED);      // contents are gone, like real unmapped memory
  return 0;
}
int f_access(uint64_t, size_t, int) { return 0; }
int f_hreg(void*, size_t) { return 0; }
int f_hunreg(void*) { return 0; }
int f_h2d(uint64_t dst, const void* src, size_t n, uint64_t) { std::memcpy(reinterpret_cast<void*>(dst), src, n); return 0; }
int f_ssync(uint64_t) { return 0; }
}  // namespace

const DriverApi* fake_driver_api() {
  static DriverApi api{f_gran, f_reserve, f_addrfree, f_create, f_release, f_map, f_unmap, f_access, f_hreg, f_hunreg, f_h2d,
                       f_ssync, false};
  return &api;
}
int64_t fake_driver_mapped_bytes() { return fake_bytes.load(); }

// ------------------------------------------------------------------------------------------------ VmmRegion
static void check(int rc, const char* what) {
  if (rc != 0) throw std::runtime_error(std::string(what) + " failed with driver code " + std::to_string(rc));
}

VmmRegion::VmmRegion(const DriverApi* api, int device, size_t max_bytes) : api_(api), device_(device) {
  if (!api) throw std::runtime_error("no CUDA driver on this host");
  check(api_->mem_granularity(device, &gran_), "cuMemGetAllocationGranularity");
  cap_ = (max_bytes + gran_ - 1) / gran_ * gran_;
  check(api_->address_reserve(&base_, cap_, gran_), "cuMemAddressReserve");
}

VmmRegion::~VmmRegion() {
  try { resize(0); } catch (...) {}
  if (base_) api_->address_free(base_, cap_);
}

size_t VmmRegion::resize(size_t bytes) {
  if (bytes > cap_) throw std::runtime_error("VmmRegion: request exceeds the reserved range");
  const size_t want = (bytes + gran_ - 1) / gran_;
  while (chunks_.size() < want) {
    uint64_t h = 0;
    check(api_->mem_create(&h, gran_, device_), "cuMemCreate");
    const uint64_t at = base_ + chunks_.size() * gran_;
    int rc = api_->mem_map(at, gran_, h);
    if (rc == 0) rc = api_->set_access(at, gran_, device_);
    if (rc != 0) { api_->mem_release(h); check(rc, "cuMemMap/cuMemSetAccess"); }
    chunks_.push_back(h);
  }
  while (chunks_.size() > want) {
    const uint64_t at = base_ + (chunks_.size() - 1) * gran_;
    check(api_->mem_unmap(at, gran_), "cuMemUnmap");
    check(api_->mem_release(chunks_.back()), "cuMemRelease");
    chunks_.pop_back();
  }
  return size();
}

// ------------------------------------------------------------------------------------------------ PinnedBuffer
PinnedBuffer::PinnedBuffer(const DriverApi* api, size_t bytes, bool huge_pages) : api_(api) {
  const size_t page = huge_pages ? (2u << 20) : 4096u;
  n_ = (bytes + page - 1) / page * page;
  p_ = mmap(nullptr, n_, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (p_ == MAP_FAILED) { p_ = nullptr; throw std::runtime_error("PinnedBuffer: mmap failed"); }
  if (huge_pages) madvise(p_, n_, MADV_HUGEPAGE);
  std::memset(p_, 0, n_);                                   // touch: pages exist before they are locked
  registered_ = api_ && api_->host_register(p_, n_) == 0;
}

PinnedBuffer::~PinnedBuffer() {
  if (p_) {
    if (registered_) api_->host_unregister(p_);
    munmap(p_, n_);
  }
}

// ------------------------------------------------------------------------------------------------ fast_load
LoadStats fast_load(const DriverApi* api, const std::string& path, int64_t offset, int64_t size, uint64_t dst, uint64_t stream,
                    size_t chunk, int n_buffers, int n_threads, bool direct) {
  if (!api) throw std::runtime_error("no CUDA driver on this host");
  LoadStats st;
  const auto t0 = std::chrono::steady_clock::now();
  constexpr int64_t kAlign = 4096;
  int fd = -1;
  if (direct) fd = open(path.c_str(), O_RDONLY | O_DIRECT);
  st.direct = fd >= 0;
  if (fd < 0) fd = open(path.c_str(), O_RDONLY);
  if (fd < 0) throw std::runtime_error("fast_load: cannot open " + path);
  if (!st.direct) posix_fadvise(fd, offset, size, POSIX_FADV_SEQUENTIAL);
  n_buffers = std::max(2, n_buffers);
  n_threads = std::max(1, n_threads);
  std::vector<std::unique_ptr<PinnedBuffer>> bufs;
  // direct reads start and end on 4 KiB boundaries of the file: room for the widened head and tail
  const size_t buf_bytes = chunk + (st.direct ? 2 * static_cast<size_t>(kAlign) : 0);
  for (int i = 0; i < n_buffers; ++i) bufs.emplace_back(new PinnedBuffer(api, buf_bytes, buf_bytes >= (2u << 20)));
  std::vector<size_t> head(n_buffers, 0);             // where a chunk's first byte sits inside its buffer
  const int64_t n_chunks = (size + static_cast<int64_t>(chunk) - 1) / static_cast<int64_t>(chunk);
  // chunk c uses buffer c % n_buffers; a buffer is free again once the copy of chunk c - n_buffers was synchronised
  std::mutex mu;
  std::condition_variable cv;
  std::vector<int64_t> filled(n_buffers, -1);        // chunk index whose data the buffer holds (ready to copy)
  int64_t copied = 0;                                // chunks whose copy has been issued and synchronised
  std::atomic<int64_t> next{0};
  std::atomic<bool> failed{false};
  std::atomic<int64_t> read_ns{0};
  auto reader = [&]() {
    for (;;) {
      const int64_t c = next.fetch_add(1);
      if (c >= n_chunks || failed) return;
      const int b = static_cast<int>(c % n_buffers);
      {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait(lk, [&] { return failed || c - copied < n_buffers; });       // the buffer's previous chunk is done
        if (failed) return;
      }
      const int64_t off = c * static_cast<int64_t>(chunk);
      const size_t n = static_cast<size_t>(std::min<int64_t>(chunk, size - off));
      const auto r0 = std::chrono::steady_clock::now();
      const int64_t fo = offset + off;                                      // file position of the chunk
      const int64_t a0 = st.direct ? fo / kAlign * kAlign : fo;             // where the read starts
      const size_t h = static_cast<size_t>(fo - a0);
      const size_t want = st.direct ? (h + n + kAlign - 1) / kAlign * kAlign : n;   // may reach past the end of the file
      size_t got = 0;
      while (got < h + n) {
        const ssize_t k = pread(fd, static_cast<char*>(bufs[b]->data()) + got, want - got, a0 + static_cast<int64_t>(got));
        if (k <= 0) { failed = true; cv.notify_all(); return; }
        got += static_cast<size_t>(k);
        if (st.direct && (got % kAlign) != 0 && got < h + n) { failed = true; cv.notify_all(); return; }   // short, unaligned, not at the end
      }
      head[b] = h;
      read_ns += std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - r0).count();
      {
        std::lock_guard<std::mutex> lk(mu);
        filled[b] = c;
      }
      cv.notify_all();
    }
  };
  std::vector<std::thread> threads;
  for (int i = 0; i < n_threads; ++i) threads.emplace_back(reader);
  for (int64_t c = 0; c < n_chunks && !failed; ++c) {
    const int b = static_cast<int>(c % n_buffers);
    {
      std::unique_lock<std::mutex> lk(mu);
      cv.wait(lk, [&] { return failed || filled[b] == c; });
      if (failed) break;
    }
    const int64_t off = c * static_cast<int64_t>(chunk);
    const size_t n = static_cast<size_t>(std::min<int64_t>(chunk, size - off));
    if (api->memcpy_htod_async(dst + static_cast<uint64_t>(off), static_cast<char*>(bufs[b]->data()) + head[b], n, stream) != 0 ||
        api->stream_sync(stream) != 0) {
      failed = true;
    }
    {
      std::lock_guard<std::mutex> lk(mu);
      copied = c + 1;
    }
    cv.notify_all();
    st.copies++;
    st.bytes += static_cast<int64_t>(n);
  }
  cv.notify_all();
  for (auto& t : threads) t.join();
  close(fd);
  if (failed) throw std::runtime_error("fast_load: read or copy failed for " + path);
  st.reads = n_chunks;
  st.read_s = read_ns.load() * 1e-9;
  st.total_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  return st;
}
