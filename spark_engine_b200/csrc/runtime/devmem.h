// Device-memory plumbing of the host runtime, on the CUDA *driver* API resolved at run time (dlopen of libcuda):
//   VmmRegion   a growable device buffer with a stable address: one virtual range reserved up front, physical
//               chunks mapped / unmapped at its end (KV stores grow and shrink in place, no copy, no pointer change).
//   PinnedBuffer  page-locked host staging memory: mmap (optionally huge-page advised) + host registration, which
//               survives compaction unlike a plain pinned allocation; falls back to ordinary memory without a GPU.
//   FastLoader  file -> device streaming: reader threads pread() file ranges into a ring of pinned staging buffers
//               while the caller's stream copies finished buffers to the device (two stages overlapped).
// All driver entry points go through a function table, so CPU tests run the same logic against an in-process fake.
// Reference: engine-rs/shim/vmm.cpp:28-86, host_pin.cuh:17-35, engine-rs/src/weights.rs:194-283 (fast load),
// readahead.rs:79-170, kv_pool.rs:53-241 (VMM backend).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

struct DriverApi {
  // all return 0 on success
  int (*mem_granularity)(int device, size_t* out);
  int (*address_reserve)(uint64_t* ptr, size_t size, size_t align);
  int (*address_free)(uint64_t ptr, size_t size);
  int (*mem_create)(uint64_t* handle, size_t size, int device);
  int (*mem_release)(uint64_t handle);
  int (*mem_map)(uint64_t ptr, size_t size, uint64_t handle);
  int (*mem_unmap)(uint64_t ptr, size_t size);
  int (*set_access)(uint64_t ptr, size_t size, int device);
  int (*host_register)(void* p, size_t size);
  int (*host_unregister)(void* p);
  int (*memcpy_htod_async)(uint64_t dst, const void* src, size_t size, uint64_t stream);
  int (*stream_sync)(uint64_t stream);
  bool real;
};

const DriverApi* cuda_driver_api();      // nullptr when libcuda cannot be loaded (no GPU on this host)
const DriverApi* fake_driver_api();      // host-memory emulation (tests)
int64_t fake_driver_mapped_bytes();      // bytes currently "mapped" by the fake

class VmmRegion {
 public:
  VmmRegion(const DriverApi* api, int device, size_t max_bytes);
  ~VmmRegion();
  VmmRegion(const VmmRegion&) = delete;
  uint64_t ptr() const { return base_; }
  size_t size() const { return chunks_.size() * gran_; }
  size_t capacity() const { return cap_; }
  size_t granularity() const { return gran_; }
  // map or unmap chunks so that at least `bytes` are backed; returns the backed size; throws on failure
  size_t resize(size_t bytes);

 private:
  const DriverApi* api_;
  int device_;
  size_t gran_ = 0, cap_ = 0;
  uint64_t base_ = 0;
  std::vector<uint64_t> chunks_;
};

class PinnedBuffer {
 public:
  PinnedBuffer(const DriverApi* api, size_t bytes, bool huge_pages);
  ~PinnedBuffer();
  PinnedBuffer(const PinnedBuffer&) = delete;
  void* data() const { return p_; }
  size_t size() const { return n_; }
  bool registered() const { return registered_; }

 private:
  const DriverApi* api_;
  void* p_ = nullptr;
  size_t n_ = 0;
  bool registered_ = false;
};

struct LoadStats { int64_t bytes = 0, reads = 0, copies = 0; double read_s = 0, total_s = 0; bool direct = false; };

// Copy file[offset, offset+size) to device memory at dst through `n_buffers` pinned staging buffers of `chunk` bytes,
// `n_threads` reader threads.  Blocks until every copy has been issued and the stream is synchronised.
// `direct`: read with O_DIRECT (no page cache: a checkpoint larger than host memory does not evict everything else and
// is not copied twice); reads are widened to 4 KiB boundaries inside the staging buffer.  Falls back to buffered reads
// when the file system refuses the flag (LoadStats::direct tells which).
LoadStats fast_load(const DriverApi* api, const std::string& path, int64_t offset, int64_t size, uint64_t dst, uint64_t stream,
                    size_t chunk, int n_buffers, int n_threads, bool direct = false);
