#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace spark_rt {

struct TensorInfo {
  std::string dtype;
  std::vector<int64_t> shape;
  int64_t begin = 0, end = 0;
};

class SafeTensors {
 public:
  explicit SafeTensors(const std::string& path);
  ~SafeTensors();
  const TensorInfo& info(const std::string& name) const;
  std::vector<std::string> names() const;
  const uint8_t* data(const std::string& name) const;                 // mmap'ed bytes
  int64_t read_into(const std::string& name, void* dst, int64_t cap) const;
  void prefetch(const std::string& name) const;                        // page-cache read-ahead hint
  bool has(const std::string& name) const { return tensors_.count(name) != 0; }
  int64_t data_offset() const { return data_off_; }                    // file offset of the first tensor byte
  const std::string& path() const { return path_; }

 private:
  std::string path_;
  int fd_ = -1;
  int64_t size_ = 0, data_off_ = 0;
  const uint8_t* map_ = nullptr;
  std::map<std::string, TensorInfo> tensors_;
};

}  // namespace spark_rt
