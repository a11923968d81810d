// Read-only memory mapping of one safetensors file with a validated header.
//
// File layout: an 8-byte little-endian header length N, N bytes of JSON
// ({"name": {"dtype": "BF16", "shape": [..], "data_offsets": [begin, end]}, ..., "__metadata__": {..}})
// and the raw tensor bytes. Everything the header claims is checked against the file before a byte is
// handed out: header length, dtype names, offset order, byte counts against shapes, ranges against the
// file size. A truncated or corrupted checkpoint fails with a message that names the tensor.
// A mapping is immutable after construction, so any number of threads may read from it.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "check.hpp"

namespace cosmos {
namespace host {

// A JSON reader for the subset the header uses: objects, arrays, strings, non-negative integers.
struct JsonCursor {
  const char* p;
  const char* end;
  const std::string& file;

  [[noreturn]] void bad(const char* what) const { fail("safetensors header of ", file, " is not valid JSON: ", what); }
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  char peek() {
    ws();
    if (p >= end) bad("unexpected end");
    return *p;
  }
  void expect(char c) {
    if (peek() != c) bad("unexpected character");
    ++p;
  }
  std::string str() {
    expect('"');
    std::string out;
    while (true) {
      if (p >= end) bad("unterminated string");
      char c = *p++;
      if (c == '"') break;
      if (c != '\\') {
        out.push_back(c);
        continue;
      }
      if (p >= end) bad("unterminated escape");
      char e = *p++;
      switch (e) {
        case 'n': out.push_back('\n'); break;
        case 't': out.push_back('\t'); break;
        case 'r': out.push_back('\r'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'u':  // kept verbatim; tensor names and metadata are ASCII in practice
          if (end - p < 4) bad("short unicode escape");
          out.append("\\u").append(p, 4);
          p += 4;
          break;
        default: out.push_back(e);  // \" \\ \/
      }
    }
    return out;
  }
  int64_t integer() {
    ws();
    if (p >= end || *p < '0' || *p > '9') bad("expected a non-negative integer");
    int64_t v = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      if (v > (INT64_MAX - 9) / 10) bad("integer overflow");
      v = v * 10 + (*p++ - '0');
    }
    return v;
  }
  std::vector<int64_t> int_array() {
    std::vector<int64_t> out;
    expect('[');
    if (peek() == ']') {
      ++p;
      return out;
    }
    while (true) {
      out.push_back(integer());
      if (peek() == ',') {
        ++p;
        continue;
      }
      expect(']');
      return out;
    }
  }
  // Skips any value (keys this reader does not know); nesting depth is bounded.
  void skip(int depth = 0) {
    if (depth > 64) bad("nesting too deep");
    char c = peek();
    if (c == '"') {
      str();
      return;
    }
    if (c == '[' || c == '{') {
      const char close = c == '[' ? ']' : '}';
      ++p;
      if (peek() == close) {
        ++p;
        return;
      }
      while (true) {
        if (c == '{') {
          str();
          expect(':');
        }
        skip(depth + 1);
        if (peek() == ',') {
          ++p;
          continue;
        }
        expect(close);
        return;
      }
    }
    const char* start = p;
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;  // number / true / false / null
    if (p == start) bad("empty value");
  }
};

struct TensorEntry {
  std::string dtype;  // the file's spelling: F32, BF16, I64, ...
  int64_t elem_size = 0;
  std::vector<int64_t> shape;
  int64_t begin = 0, end = 0;  // byte range inside the data section
  int64_t numel = 0;
};

inline int64_t dtype_size(const std::string& s) {
  static const std::map<std::string, int64_t> table = {{"F64", 8}, {"F32", 4}, {"F16", 2}, {"BF16", 2}, {"I64", 8},
                                                       {"I32", 4}, {"I16", 2}, {"I8", 1},  {"U8", 1},   {"BOOL", 1}};
  auto it = table.find(s);
  return it == table.end() ? 0 : it->second;
}

class SafetensorsMap {
 public:
  explicit SafetensorsMap(std::string path) : path_(std::move(path)) {
    fd_ = ::open(path_.c_str(), O_RDONLY);
    if (fd_ < 0) fail("cannot open ", path_, ": ", std::strerror(errno));
    try {
      struct stat st {};
      if (::fstat(fd_, &st) != 0) fail("cannot stat ", path_);
      size_ = (int64_t)st.st_size;
      if (size_ < 8) fail(path_, " is too short to be a safetensors file (", size_, " bytes)");
      void* m = ::mmap(nullptr, (size_t)size_, PROT_READ, MAP_PRIVATE, fd_, 0);
      if (m == MAP_FAILED) fail("cannot map ", path_, ": ", std::strerror(errno));
      map_ = static_cast<const uint8_t*>(m);
      parse();
    } catch (...) {
      close_all();
      throw;
    }
  }
  ~SafetensorsMap() { close_all(); }
  SafetensorsMap(const SafetensorsMap&) = delete;
  SafetensorsMap& operator=(const SafetensorsMap&) = delete;

  const std::string& path() const { return path_; }
  const std::vector<std::string>& keys() const { return order_; }
  const std::map<std::string, std::string>& metadata() const { return meta_; }
  bool has(const std::string& name) const { return entries_.count(name) != 0; }

  const TensorEntry& find(const std::string& name) const {
    auto it = entries_.find(name);
    if (it == entries_.end()) fail(path_, " has no tensor '", name, "'");
    return it->second;
  }

  // First byte of elements [elem_offset, elem_offset + count) of a tensor, after a range check.
  const uint8_t* data(const std::string& name, int64_t elem_offset = 0, int64_t count = -1) const {
    const TensorEntry& e = find(name);
    if (count < 0) count = e.numel - elem_offset;
    check(elem_offset >= 0 && count >= 0 && elem_offset <= e.numel && count <= e.numel - elem_offset, "elements [", elem_offset,
          ", ", elem_offset + count, ") are outside tensor '", name, "' of ", e.numel, " elements");
    return map_ + data_start_ + e.begin + elem_offset * e.elem_size;
  }

 private:
  void close_all() {
    if (map_) ::munmap(const_cast<uint8_t*>(map_), (size_t)size_);
    map_ = nullptr;
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
  }

  void parse() {
    uint64_t n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | map_[i];
    check(n >= 2 && n <= (uint64_t)(size_ - 8), "header of ", path_, " claims ", n, " bytes but the file has ", size_ - 8,
          " after the length field (truncated or not a safetensors file)");
    data_start_ = 8 + (int64_t)n;
    const int64_t data_bytes = size_ - data_start_;
    const char* h = reinterpret_cast<const char*>(map_ + 8);
    JsonCursor c{h, h + n, path_};
    c.expect('{');
    if (c.peek() != '}') {
      while (true) {
        std::string name = c.str();
        c.expect(':');
        if (name == "__metadata__") {
          parse_metadata(c);
        } else {
          parse_tensor(c, name, data_bytes);
        }
        if (c.peek() == ',') {
          ++c.p;
          continue;
        }
        break;
      }
    }
    c.expect('}');
  }

  void parse_metadata(JsonCursor& c) {
    c.expect('{');
    if (c.peek() != '}') {
      while (true) {
        std::string k = c.str();
        c.expect(':');
        if (c.peek() == '"') {
          meta_[k] = c.str();
        } else {
          c.skip();
        }
        if (c.peek() == ',') {
          ++c.p;
          continue;
        }
        break;
      }
    }
    c.expect('}');
  }

  void parse_tensor(JsonCursor& c, const std::string& name, int64_t data_bytes) {
    TensorEntry e;
    std::vector<int64_t> offs;
    bool has_shape = false;
    c.expect('{');
    if (c.peek() != '}') {
      while (true) {
        std::string k = c.str();
        c.expect(':');
        if (k == "dtype") {
          e.dtype = c.str();
        } else if (k == "shape") {
          e.shape = c.int_array();
          has_shape = true;
        } else if (k == "data_offsets") {
          offs = c.int_array();
        } else {
          c.skip();
        }
        if (c.peek() == ',') {
          ++c.p;
          continue;
        }
        break;
      }
    }
    c.expect('}');
    check(has_shape && offs.size() == 2 && !e.dtype.empty(), path_, ": tensor '", name, "' lacks dtype, shape or data_offsets");
    e.elem_size = dtype_size(e.dtype);
    check(e.elem_size > 0, path_, ": tensor '", name, "' has unsupported dtype ", e.dtype);
    e.begin = offs[0];
    e.end = offs[1];
    e.numel = 1;
    for (int64_t d : e.shape) {
      check(d >= 0 && (d == 0 || e.numel <= INT64_MAX / d), path_, ": tensor '", name, "' has a bad shape");
      e.numel *= d;
    }
    check(e.numel <= INT64_MAX / e.elem_size, path_, ": tensor '", name, "' has a bad shape");
    check(e.begin >= 0 && e.begin <= e.end, path_, ": tensor '", name, "' has offsets out of order");
    check(e.end - e.begin == e.numel * e.elem_size, path_, ": tensor '", name, "' spans ", e.end - e.begin,
          " bytes but its shape and dtype need ", e.numel * e.elem_size);
    check(e.end <= data_bytes, path_, ": tensor '", name, "' ends at byte ", e.end, " of the data section, which has only ",
          data_bytes, " (file truncated?)");
    check(entries_.emplace(name, e).second, path_, ": duplicate tensor '", name, "'");
    order_.push_back(name);
  }

  std::string path_;
  int fd_ = -1;
  const uint8_t* map_ = nullptr;
  int64_t size_ = 0, data_start_ = 0;
  std::map<std::string, TensorEntry> entries_;
  std::vector<std::string> order_;
  std::map<std::string, std::string> meta_;
};

}  // namespace host
}  // namespace cosmos
