// Minimal GGUF reader for the engine's loader: header, metadata scalars/strings, tensor
// infos, and a read-only mapping of the tensor data section. Format facts follow the
// reference reader (gguf_parser.cpp:123-806): little-endian; magic 0x46554747; strings are
// uint64 length + bytes; the data section starts at the next multiple of general.alignment
// (default 32) after the tensor infos; tensor offsets are relative to it.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace b200 {

struct GgufTensor {
  std::string name;
  int type = 0;
  std::vector<uint64_t> shape;  // shape[0] = input dimension (ne0)
  uint64_t offset = 0;          // relative to the data section
  uint64_t bytes = 0;
  const uint8_t* data = nullptr;
};

struct GgufFile {
  std::map<std::string, double> numbers;      // every scalar metadata value
  std::map<std::string, std::string> strings;
  std::vector<GgufTensor> tensors;
  const uint8_t* map_base = nullptr;
  size_t map_size = 0;
  int fd = -1;
  ~GgufFile();
  GgufFile() = default;
  GgufFile(const GgufFile&) = delete;
  GgufFile& operator=(const GgufFile&) = delete;
  double number(const std::string& key, double dflt) const {
    auto it = numbers.find(key);
    return it == numbers.end() ? dflt : it->second;
  }
};

// Throws std::runtime_error on malformed input.
void gguf_open(const std::string& path, GgufFile& out);

}  // namespace b200
