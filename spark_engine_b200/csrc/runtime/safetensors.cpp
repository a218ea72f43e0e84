// safetensors reader: 8-byte little-endian header length, JSON header, raw tensor bytes.  The file is mmap'ed;
// `read_into` preads a tensor into a caller buffer (pinned staging for the upload thread).
// Reference: engine-rs/src/safetensors.rs (header scan + mmap), weights.rs:217-247 (pread -> pinned -> device).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "safetensors.h"

namespace spark_rt {

namespace {
// Tiny JSON walker for the flat header: {"name": {"dtype": "...", "shape": [...], "data_offsets": [a, b]}, ...}
struct Cur {
  const char* p; const char* e;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  std::string str() {
    ws();
    if (p >= e || *p != '"') throw std::runtime_error("safetensors: expected string");
    ++p; std::string s;
    while (p < e && *p != '"') { if (*p == '\\' && p + 1 < e) ++p; s += *p++; }
    ++p; return s;
  }
  int64_t num() { ws(); int64_t v = 0; bool any = false; while (p < e && *p >= '0' && *p <= '9') { v = v * 10 + (*p++ - '0'); any = true; } if (!any) throw std::runtime_error("safetensors: expected number"); return v; }
  void skip_value() {
    ws();
    if (p < e && *p == '"') { str(); return; }
    if (p < e && (*p == '{' || *p == '[')) {
      int depth = 0;
      do { if (*p == '"') { str(); continue; } if (*p == '{' || *p == '[') ++depth; if (*p == '}' || *p == ']') --depth; ++p; } while (p < e && depth > 0);
      return;
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
  }
};
// bits per element of the dtypes the format defines (0 = unknown: size not checked)
int dtype_bits(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 64;
  if (d == "F32" || d == "I32" || d == "U32") return 32;
  if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 16;
  if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2" || d == "F8_E8M0") return 8;
  if (d == "F4" || d == "F4_E2M1") return 4;
  return 0;
}

}  // namespace

SafeTensors::SafeTensors(const std::string& path) : path_(path) {
  fd_ = open(path.c_str(), O_RDONLY);
  if (fd_ < 0) throw std::runtime_error("safetensors: cannot open " + path);
  struct stat st;
  fstat(fd_, &st);
  size_ = st.st_size;
  if (size_ < 8) throw std::runtime_error("safetensors: file too small");
  map_ = static_cast<const uint8_t*>(mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0));
  if (map_ == MAP_FAILED) throw std::runtime_error("safetensors: mmap failed");
  uint64_t hl;
  memcpy(&hl, map_, 8);
  if (8 + hl > static_cast<uint64_t>(size_)) throw std::runtime_error("safetensors: bad header length");
  data_off_ = 8 + hl;
  Cur c{reinterpret_cast<const char*>(map_ + 8), reinterpret_cast<const char*>(map_ + 8 + hl)};
  if (!c.eat('{')) throw std::runtime_error("safetensors: bad header");
  while (!c.eat('}')) {
    std::string name = c.str();
    c.eat(':');
    if (name == "__metadata__") { c.skip_value(); c.eat(','); continue; }
    TensorInfo ti;
    c.eat('{');
    while (!c.eat('}')) {
      std::string k = c.str();
      c.eat(':');
      if (k == "dtype") ti.dtype = c.str();
      else if (k == "shape") { c.eat('['); while (!c.eat(']')) { ti.shape.push_back(c.num()); c.eat(','); } }
      else if (k == "data_offsets") { c.eat('['); ti.begin = c.num(); c.eat(','); ti.end = c.num(); c.eat(']'); }
      else c.skip_value();
      c.eat(',');
    }
    c.eat(',');
    // a truncated or crafted file must not make data() / read_into() reach past the mapping
    const int64_t payload = static_cast<int64_t>(size_) - static_cast<int64_t>(data_off_);
    if (ti.begin < 0 || ti.end < ti.begin || ti.end > payload)
      throw std::runtime_error("safetensors: data_offsets of " + name + " are outside the file");
    int64_t numel = 1;
    for (int64_t d : ti.shape) {
      if (d < 0) throw std::runtime_error("safetensors: negative dimension in " + name);
      numel *= d;
    }
    const int bits = dtype_bits(ti.dtype);
    if (bits > 0 && (numel * bits + 7) / 8 != ti.end - ti.begin)
      throw std::runtime_error("safetensors: byte count of " + name + " does not match its shape and dtype");
    tensors_[name] = ti;
  }
}

SafeTensors::~SafeTensors() {
  if (map_ && map_ != MAP_FAILED) munmap(const_cast<uint8_t*>(map_), size_);
  if (fd_ >= 0) close(fd_);
}

const TensorInfo& SafeTensors::info(const std::string& name) const {
  auto it = tensors_.find(name);
  if (it == tensors_.end()) throw std::out_of_range("safetensors: no tensor " + name);
  return it->second;
}

std::vector<std::string> SafeTensors::names() const { std::vector<std::string> v; for (auto& kv : tensors_) v.push_back(kv.first); return v; }

const uint8_t* SafeTensors::data(const std::string& name) const { return map_ + data_off_ + info(name).begin; }

int64_t SafeTensors::read_into(const std::string& name, void* dst, int64_t cap) const {
  const TensorInfo& ti = info(name);
  const int64_t n = ti.end - ti.begin;
  if (n > cap) throw std::length_error("safetensors: destination too small");
  int64_t done = 0;
  while (done < n) {
    ssize_t r = pread(fd_, static_cast<char*>(dst) + done, n - done, data_off_ + ti.begin + done);
    if (r <= 0) throw std::runtime_error("safetensors: short read");
    done += r;
  }
  return n;
}

void SafeTensors::prefetch(const std::string& name) const {
  const TensorInfo& ti = info(name);
  posix_fadvise(fd_, data_off_ + ti.begin, ti.end - ti.begin, POSIX_FADV_WILLNEED);
}

}  // namespace spark_rt
