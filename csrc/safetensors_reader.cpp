// Torch binding of the memory-mapped safetensors reader (host/safetensors_map.hpp).
//
// The file is mapped read-only once; a tensor (or any element range of it) is copied straight from the
// mapping into the destination tensor, so a rank that owns a shard of a flat parameter reads exactly its
// slice and nothing is staged in between. Header validation lives in the mapping class.
#include "runtime.h"

#include <ATen/ATen.h>
#include <torch/custom_class.h>

#include <cstring>

#include "host/safetensors_map.hpp"

namespace cosmos {
namespace {

at::ScalarType scalar_type_of(const std::string& s) {
  static const std::map<std::string, at::ScalarType> table = {
      {"F64", at::kDouble}, {"F32", at::kFloat}, {"F16", at::kHalf}, {"BF16", at::kBFloat16}, {"I64", at::kLong},
      {"I32", at::kInt},    {"I16", at::kShort}, {"I8", at::kChar},  {"U8", at::kByte},       {"BOOL", at::kBool}};
  auto it = table.find(s);
  TORCH_CHECK(it != table.end(), "unsupported safetensors dtype ", s);
  return it->second;
}

}  // namespace

struct SafetensorsFile : torch::CustomClassHolder {
  host::SafetensorsMap map;

  explicit SafetensorsFile(std::string path) : map(std::move(path)) {}

  std::vector<std::string> keys() const { return map.keys(); }
  bool has(std::string name) const { return map.has(name); }
  std::vector<int64_t> shape(std::string name) const { return map.find(name).shape; }
  int64_t numel(std::string name) const { return map.find(name).numel; }
  std::string dtype(std::string name) const { return c10::toString(scalar_type_of(map.find(name).dtype)); }
  std::string metadata(std::string key) const {
    auto it = map.metadata().find(key);
    return it == map.metadata().end() ? std::string() : it->second;
  }
  std::vector<std::string> metadata_keys() const {
    std::vector<std::string> out;
    for (auto& kv : map.metadata()) out.push_back(kv.first);
    return out;
  }

  // A new CPU tensor with the stored dtype and shape (one copy out of the mapping).
  at::Tensor get(std::string name) const {
    const host::TensorEntry& e = map.find(name);
    at::Tensor t = at::empty(e.shape, at::TensorOptions().dtype(scalar_type_of(e.dtype)).device(at::kCPU));
    if (e.numel > 0) std::memcpy(t.data_ptr(), map.data(name), (size_t)(e.end - e.begin));
    return t;
  }

  // Copies elements [elem_offset, elem_offset + dst.numel()) of the stored tensor (flattened, row-major)
  // into `dst` (contiguous; CPU or CUDA; same dtype, or any floating dtype when the stored one is floating).
  void read_into(std::string name, at::Tensor dst, int64_t elem_offset) const {
    const host::TensorEntry& e = map.find(name);
    const at::ScalarType st = scalar_type_of(e.dtype);
    const int64_t n = dst.numel();
    TORCH_CHECK(dst.is_contiguous(), "read_into: destination for '", name, "' must be contiguous");
    TORCH_CHECK(elem_offset >= 0 && elem_offset + n <= e.numel, "read_into: elements [", elem_offset, ", ", elem_offset + n,
                ") are outside tensor '", name, "' of ", e.numel, " elements");
    if (n == 0) return;
    at::Tensor view = at::from_blob(const_cast<uint8_t*>(map.data(name, elem_offset, n)), {n},
                                    at::TensorOptions().dtype(st).device(at::kCPU));
    const bool same = dst.scalar_type() == st;
    TORCH_CHECK(same || (at::isFloatingType(dst.scalar_type()) && at::isFloatingType(st)), "read_into: '", name, "' is ",
                c10::toString(st), ", destination is ", c10::toString(dst.scalar_type()));
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
