// Torch binding of the paged KV-cache block allocator (host/paged_allocator.hpp): the Reasoner's engine
// holds one by reference, and growing a sequence by one token touches no Python list.
#include "runtime.h"

#include <ATen/ATen.h>
#include <torch/custom_class.h>

#include "host/paged_allocator.hpp"

namespace cosmos {

struct PagedKVAllocator : torch::CustomClassHolder {
  host::PagedAllocator core;

  PagedKVAllocator(int64_t num_blocks, int64_t block_size, int64_t max_blocks_per_seq)
      : core(num_blocks, block_size, max_blocks_per_seq) {}

  int64_t num_free() const { return core.num_free(); }
  bool can_allocate(int64_t tokens) const { return core.can_allocate(tokens); }
  bool extend(int64_t seq, int64_t tokens) { return core.extend(seq, tokens); }
  void release(int64_t seq) { core.release(seq); }
  int64_t length(int64_t seq) const { return core.length(seq); }

  std::vector<int64_t> blocks(int64_t seq) const {
    const auto* b = core.blocks(seq);
    return b ? std::vector<int64_t>(b->begin(), b->end()) : std::vector<int64_t>();
  }

  // Rows of the block table and the sequence lengths for `seqs` (in order) into CPU int32 tensors
  // [n, max_blocks_per_seq] / [n]; unused entries are -1.
  void fill_tables(std::vector<int64_t> seqs, at::Tensor table, at::Tensor lens) const {
    TORCH_CHECK(table.device().is_cpu() && table.scalar_type() == at::kInt && table.is_contiguous());
    TORCH_CHECK(lens.device().is_cpu() && lens.scalar_type() == at::kInt && lens.is_contiguous());
    TORCH_CHECK(table.dim() == 2 && table.size(0) >= (int64_t)seqs.size() && table.size(1) == core.max_blocks_per_seq());
    TORCH_CHECK(lens.numel() >= (int64_t)seqs.size());
    core.fill_tables(seqs.data(), (int64_t)seqs.size(), table.data_ptr<int32_t>(), lens.data_ptr<int32_t>());
  }
};

void register_runtime_ops(torch::Library& m) {
  m.class_<PagedKVAllocator>("PagedKVAllocator")
      .def(torch::init<int64_t, int64_t, int64_t>())
      .def("num_free", &PagedKVAllocator::num_free)
      .def("can_allocate", &PagedKVAllocator::can_allocate)
      .def("extend", &PagedKVAllocator::extend)
      .def("release", &PagedKVAllocator::release)
      .def("length", &PagedKVAllocator::length)
      .def("blocks", &PagedKVAllocator::blocks)
      .def("fill_tables", &PagedKVAllocator::fill_tables);
}

}  // namespace cosmos
