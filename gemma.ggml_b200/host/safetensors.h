// safetensors.h — reader of a .safetensors file: 8 bytes little-endian header length, that many bytes of JSON
// (name -> dtype, shape, data_offsets), then the data.  The file is read into memory once; tensors are views into it
// (data may start at any byte: copy before use where alignment matters).
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

struct st_tensor {
    std::string dtype; // "BF16", "F32", "I32", ...
    std::vector<int64_t> shape;
    const uint8_t *data = nullptr;
    size_t nbytes = 0;
    int64_t numel() const {
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        return n;
    }
};

class safetensors_file {
  public:
    int open(const std::string &path, std::string *err);
    const st_tensor *find(const std::string &name) const {
        auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }
    const std::map<std::string, st_tensor> &tensors() const { return tensors_; }

  private:
    std::vector<uint8_t> bytes_;
    std::map<std::string, st_tensor> tensors_;
};
