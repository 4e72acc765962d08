#include "gguf.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

namespace b200 {
namespace {

struct Cursor {
  const uint8_t* p;
  const uint8_t* end;
  template <typename T>
  T get() {
    if (p + sizeof(T) > end) throw std::runtime_error("GGUF: truncated file");
    T v;
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string str() {
    uint64_t n = get<uint64_t>();
    if (n > (uint64_t)(end - p)) throw std::runtime_error("GGUF: string runs past end of file");
    std::string s(reinterpret_cast<const char*>(p), (size_t)n);
    p += n;
    return s;
  }
};

// GGUF metadata value types (reference ggml_types.h: GGUFValueType)
enum { VT_U8 = 0, VT_I8, VT_U16, VT_I16, VT_U32, VT_I32, VT_F32, VT_BOOL, VT_STR, VT_ARR, VT_U64, VT_I64, VT_F64 };

bool read_scalar(Cursor& c, uint32_t t, double& out) {
  switch (t) {
    case VT_U8: out = c.get<uint8_t>(); return true;
    case VT_I8: out = c.get<int8_t>(); return true;
    case VT_U16: out = c.get<uint16_t>(); return true;
    case VT_I16: out = c.get<int16_t>(); return true;
    case VT_U32: out = c.get<uint32_t>(); return true;
    case VT_I32: out = c.get<int32_t>(); return true;
    case VT_F32: out = c.get<float>(); return true;
    case VT_BOOL: out = c.get<uint8_t>(); return true;
    case VT_U64: out = (double)c.get<uint64_t>(); return true;
    case VT_I64: out = (double)c.get<int64_t>(); return true;
    case VT_F64: out = c.get<double>(); return true;
    default: return false;
  }
}

uint64_t type_bytes(int type, uint64_t n) {
  switch (type) {
    case 0: return n * 4;
    case 1: return n * 2;
    case 8: return n / 32 * 34;
    case 12: return n / 256 * 144;
    case 14: return n / 256 * 210;
    case 30: return n * 2;
    default: return 0;
  }
}

}  // namespace

GgufFile::~GgufFile() {
  if (map_base) munmap(const_cast<uint8_t*>(map_base), map_size);
  if (fd >= 0) close(fd);
}

void gguf_open(const std::string& path, GgufFile& out) {
  out.fd = open(path.c_str(), O_RDONLY);
  if (out.fd < 0) throw std::runtime_error("GGUF: cannot open " + path);
  struct stat st;
  if (fstat(out.fd, &st) != 0 || st.st_size < 24) throw std::runtime_error("GGUF: cannot stat " + path);
  out.map_size = (size_t)st.st_size;
  void* m = mmap(nullptr, out.map_size, PROT_READ, MAP_PRIVATE, out.fd, 0);
  if (m == MAP_FAILED) throw std::runtime_error("GGUF: mmap failed for " + path);
  out.map_base = static_cast<const uint8_t*>(m);
  Cursor c{out.map_base, out.map_base + out.map_size};
  if (c.get<uint32_t>() != 0x46554747u) throw std::runtime_error("GGUF: bad magic in " + path);
  c.get<uint32_t>();  // version
  const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
  for (uint64_t i = 0; i < n_kv; ++i) {
    std::string key = c.str();
    uint32_t t = c.get<uint32_t>();
    double v;
    if (t == VT_STR) {
      out.strings[key] = c.str();
    } else if (t == VT_ARR) {
      uint32_t et = c.get<uint32_t>();
      uint64_t n = c.get<uint64_t>();
      for (uint64_t k = 0; k < n; ++k) {
        if (et == VT_STR) c.str();
        else if (!read_scalar(c, et, v)) throw std::runtime_error("GGUF: unsupported array element type in " + key);
      }
    } else if (read_scalar(c, t, v)) {
      out.numbers[key] = v;
    } else {
      throw std::runtime_error("GGUF: unsupported metadata type for " + key);
    }
  }
  out.tensors.resize((size_t)n_tensors);
  for (auto& t : out.tensors) {
    t.name = c.str();
    uint32_t nd = c.get<uint32_t>();
    if (nd > 4) throw std::runtime_error("GGUF: tensor " + t.name + " has too many dimensions");
    t.shape.resize(nd);
    uint64_t n = 1;
    for (auto& d : t.shape) { d = c.get<uint64_t>(); n *= d; }
    t.type = (int)c.get<uint32_t>();
    t.offset = c.get<uint64_t>();
    t.bytes = type_bytes(t.type, n);
    if (t.bytes == 0 && n > 0) throw std::runtime_error("GGUF: tensor " + t.name + " has unsupported type " + std::to_string(t.type));
  }
  const uint64_t align = (uint64_t)out.number("general.alignment", 32);
  uint64_t pos = (uint64_t)(c.p - out.map_base);
  const uint64_t data_start = (pos + align - 1) / align * align;
  for (auto& t : out.tensors) {
    if (data_start + t.offset + t.bytes > out.map_size) throw std::runtime_error("GGUF: tensor " + t.name + " runs past end of file");
    t.data = out.map_base + data_start + t.offset;
  }
}

}  // namespace b200
