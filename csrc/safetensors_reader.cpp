// Memory-mapped safetensors reader (host runtime, C++).
//
// A safetensors file is an 8-byte little-endian header length N, N bytes of JSON
// ({"name": {"dtype": "BF16", "shape": [..], "data_offsets": [begin, end]}, ..., "__metadata__": {..}})
// and the raw tensor bytes. The file is mapped read-only once; a tensor (or any element range of
// it) is copied straight from the mapping into the destination tensor, so a rank that owns a shard
// of a flat parameter reads exactly its slice and nothing is staged in between. Everything the
// header claims is checked against the file before any byte is copied: header length, dtype names,
// offset order, byte counts against shapes, ranges against the file size. A truncated or corrupted
// checkpoint therefore fails with a message that names the tensor, not with a fault.
#include "runtime.h"

#include <ATen/ATen.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <torch/custom_class.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace cosmos {
namespace {

// ---- a JSON reader for the subset the header uses: objects, arrays, strings, non-negative integers
struct JsonCursor {
  const char* p;
  const char* end;
  const std::string& file;

  [[noreturn]] void fail(const char* what) const {
    TORCH_CHECK(false, "safetensors header of ", file, " is not valid JSON: ", what);
  }
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  char peek() {
    ws();
    if (p >= end) fail("unexpected end");
    return *p;
  }
  void expect(char c) {
    if (peek() != c) fail("unexpected character");
    ++p;
  }
  std::string str() {
    expect('"');
    std::string out;
    while (true) {
      if (p >= end) fail("unterminated string");
      char c = *p++;
      if (c == '"') break;
      if (c == '\\') {
        if (p >= end) fail("unterminated escape");
        char e = *p++;
        switch (e) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {  // keep the escape verbatim; tensor names and metadata are ASCII in practice
            if (end - p < 4) fail("short unicode escape");
            out.append("\\u").append(p, 4);
            p += 4;
            break;
          }
          default: out.push_back(e);  // \" \\ \/
        }
      } else {
        out.push_back(c);
      }
    }
    return out;
  }
  int64_t integer() {
    ws();
    if (p >= end || *p < '0' || *p > '9') fail("expected a non-negative integer");
    int64_t v = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      if (v > (INT64_MAX - 9) / 10) fail("integer overflow");
      v = v * 10 + (*p++ - '0');
    }
    return v;
  }
  std::vector<int64_t> int_array() {
    std::vector<int64_t> out;
    expect('[');
    if (peek() == ']') { ++p; return out; }
    while (true) {
      out.push_back(integer());
      if (peek() == ',') { ++p; continue; }
      expect(']');
      return out;
    }
  }
  // skips any value (used for keys this reader does not know)
  void skip() {
    char c = peek();
    if (c == '"') { str(); return; }
    if (c == '[' || c == '{') {
      const char close = c == '[' ? ']' : '}';
      ++p;
      if (peek() == close) { ++p; return; }
      while (true) {
        if (c == '{') { str(); expect(':'); }
        skip();
        if (peek() == ',') { ++p; continue; }
        expect(close);
        return;
      }
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;  // number / true / false / null
  }
};

struct Entry {
  at::ScalarType dtype;
  int64_t elem_size;
  std::vector<int64_t> shape;
  int64_t begin, end;  // byte range inside the data section
  int64_t numel;
};

bool dtype_of(const std::string& s, at::ScalarType& t, int64_t& size) {
  static const std::map<std::string, std::pair<at::ScalarType, int64_t>> table = {
      {"F64", {at::kDouble, 8}}, {"F32", {at::kFloat, 4}}, {"F16", {at::kHalf, 2}}, {"BF16", {at::kBFloat16, 2}},
      {"I64", {at::kLong, 8}},   {"I32", {at::kInt, 4}},   {"I16", {at::kShort, 2}}, {"I8", {at::kChar, 1}},
      {"U8", {at::kByte, 1}},    {"BOOL", {at::kBool, 1}}};
  auto it = table.find(s);
  if (it == table.end()) return false;
  t = it->second.first;
  size = it->second.second;
  return true;
}

}  // namespace

struct SafetensorsFile : torch::CustomClassHolder {
  std::string path;
  int fd = -1;
  const uint8_t* map = nullptr;
  int64_t file_size = 0, data_start = 0;
  std::map<std::string, Entry> entries;
  std::vector<std::string> order;
  std::map<std::string, std::string> meta;

  explicit SafetensorsFile(std::string path_) : path(std::move(path_)) {
    fd = ::open(path.c_str(), O_RDONLY);
    TORCH_CHECK(fd >= 0, "cannot open ", path, ": ", std::strerror(errno));
    struct stat st {};
    if (::fstat(fd, &st) != 0) { close_all(); TORCH_CHECK(false, "cannot stat ", path); }
    file_size = (int64_t)st.st_size;
    if (file_size < 8) { close_all(); TORCH_CHECK(false, path, " is too short to be a safetensors file (", file_size, " bytes)"); }
    void* m = ::mmap(nullptr, (size_t)file_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (m == MAP_FAILED) { close_all(); TORCH_CHECK(false, "cannot map ", path, ": ", std::strerror(errno)); }
    map = static_cast<const uint8_t*>(m);
    try {
      parse();
    } catch (...) {
      close_all();
      throw;
    }
  }
  ~SafetensorsFile() override { close_all(); }

  void close_all() {
    if (map) ::munmap(const_cast<uint8_t*>(map), (size_t)file_size);
    map = nullptr;
    if (fd >= 0) ::close(fd);
    fd = -1;
  }

  void parse() {
    uint64_t n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | map[i];
    TORCH_CHECK(n >= 2 && n <= (uint64_t)(file_size - 8), "header of ", path, " claims ", n, " bytes but the file has ",
                file_size - 8, " after the length field (truncated or not a safetensors file)");
    data_start = 8 + (int64_t)n;
    const int64_t data_bytes = file_size - data_start;
    const char* h = reinterpret_cast<const char*>(map + 8);
    JsonCursor c{h, h + n, path};
    c.expect('{');
    if (c.peek() != '}') {
      while (true) {
        std::string name = c.str();
        c.expect(':');
        if (name == "__metadata__") {
          c.expect('{');
          if (c.peek() != '}') {
            while (true) {
              std::string k = c.str();
              c.expect(':');
              if (c.peek() == '"') meta[k] = c.str(); else c.skip();
              if (c.peek() == ',') { ++c.p; continue; }
              break;
            }
          }
          c.expect('}');
        } else {
          Entry e{};
          std::string dt;
          std::vector<int64_t> offs;
          bool has_shape = false;
          c.expect('{');
          while (true) {
            std::string k = c.str();
            c.expect(':');
            if (k == "dtype") dt = c.str();
            else if (k == "shape") { e.shape = c.int_array(); has_shape = true; }
            else if (k == "data_offsets") offs = c.int_array();
            else c.skip();
            if (c.peek() == ',') { ++c.p; continue; }
            break;
          }
          c.expect('}');
          TORCH_CHECK(has_shape && offs.size() == 2 && !dt.empty(), path, ": tensor '", name,
                      "' lacks dtype, shape or data_offsets");
          TORCH_CHECK(dtype_of(dt, e.dtype, e.elem_size), path, ": tensor '", name, "' has unsupported dtype ", dt);
          e.begin = offs[0];
          e.end = offs[1];
          e.numel = 1;
          for (int64_t d : e.shape) {
            TORCH_CHECK(d >= 0 && (d == 0 || e.numel <= INT64_MAX / (d > 0 ? d : 1)), path, ": tensor '", name, "' has a bad shape");
            e.numel *= d;
          }
          TORCH_CHECK(e.begin >= 0 && e.begin <= e.end, path, ": tensor '", name, "' has offsets out of order");
          TORCH_CHECK(e.end - e.begin == e.numel * e.elem_size, path, ": tensor '", name, "' spans ", e.end - e.begin,
                      " bytes but its shape and dtype need ", e.numel * e.elem_size);
          TORCH_CHECK(e.end <= data_bytes, path, ": tensor '", name, "' ends at byte ", e.end, " of the data section, which has only ",
                      data_bytes, " (file truncated?)");
          TORCH_CHECK(entries.emplace(name, e).second, path, ": duplicate tensor '", name, "'");
          order.push_back(name);
        }
        if (c.peek() == ',') { ++c.p; continue; }
        break;
      }
    }
    c.expect('}');
  }

  const Entry& find(const std::string& name) const {
    auto it = entries.find(name);
    TORCH_CHECK(it != entries.end(), path, " has no tensor '", name, "'");
    return it->second;
  }

  std::vector<std::string> keys() const { return order; }
  bool has(std::string name) const { return entries.count(name) != 0; }
  std::vector<int64_t> shape(std::string name) const { return find(name).shape; }
  int64_t numel(std::string name) const { return find(name).numel; }
  std::string dtype(std::string name) const { return c10::toString(find(name).dtype); }
  std::string metadata(std::string key) const {
    auto it = meta.find(key);
    return it == meta.end() ? std::string() : it->second;
  }
  std::vector<std::string> metadata_keys() const {
    std::vector<std::string> out;
    for (auto& kv : meta) out.push_back(kv.first);
    return out;
  }

  // A new CPU tensor with the stored dtype and shape (one copy out of the mapping).
  at::Tensor get(std::string name) const {
    const Entry& e = find(name);
    at::Tensor t = at::empty(e.shape, at::TensorOptions().dtype(e.dtype).device(at::kCPU));
    if (e.numel > 0) std::memcpy(t.data_ptr(), map + data_start + e.begin, (size_t)(e.end - e.begin));
    return t;
  }

  // Copies elements [elem_offset, elem_offset + dst.numel()) of the stored tensor (flattened, row-major)
  // into `dst` (contiguous; CPU or CUDA; same dtype, or any floating dtype when the stored one is floating).
  void read_into(std::string name, at::Tensor dst, int64_t elem_offset) const {
    const Entry& e = find(name);
    const int64_t n = dst.numel();
    TORCH_CHECK(dst.is_contiguous(), "read_into: destination for '", name, "' must be contiguous");
    TORCH_CHECK(elem_offset >= 0 && elem_offset + n <= e.numel, "read_into: elements [", elem_offset, ", ", elem_offset + n,
                ") are outside tensor '", name, "' of ", e.numel, " elements");
    if (n == 0) return;
    at::Tensor view = at::from_blob(const_cast<uint8_t*>(map + data_start + e.begin + elem_offset * e.elem_size), {n},
                                    at::TensorOptions().dtype(e.dtype).device(at::kCPU));
    const bool same = dst.scalar_type() == e.dtype;
    TORCH_CHECK(same || (at::isFloatingType(dst.scalar_type()) && at::isFloatingType(e.dtype)), "read_into: '", name, "' is ",
                c10::toString(e.dtype), ", destination is ", c10::toString(dst.scalar_type()));
    dst.view({n}).copy_(view);  // converts and / or crosses to the device as needed
  }
};

void register_safetensors(torch::Library& m) {
  m.class_<SafetensorsFile>("SafetensorsFile")
      .def(torch::init<std::string>())
      .def("keys", &SafetensorsFile::keys)
      .def("has", &SafetensorsFile::has)
      .def("shape", &SafetensorsFile::shape)
      .def("numel", &SafetensorsFile::numel)
      .def("dtype", &SafetensorsFile::dtype)
      .def("metadata", &SafetensorsFile::metadata)
      .def("metadata_keys", &SafetensorsFile::metadata_keys)
      .def("get", &SafetensorsFile::get)
      .def("read_into", &SafetensorsFile::read_into);
}

}  // namespace cosmos
