// Paged KV-cache block allocator (free-list + per-sequence block tables) in C++.
// The Reasoner keeps K/V in fixed-size pages; each sequence owns a list of page ids.
// The allocator fills an int32 block-table tensor [max_seqs, max_blocks_per_seq] that the
// decode-attention kernel reads, so growing a sequence by one token touches no Python list.
#include "runtime.h"

#include <ATen/ATen.h>
#include <torch/custom_class.h>

#include <unordered_map>
#include <vector>

namespace cosmos {

struct PagedKVAllocator : torch::CustomClassHolder {
  int64_t num_blocks, block_size, max_blocks_per_seq;
  std::vector<int32_t> free_list;
  std::unordered_map<int64_t, std::vector<int32_t>> tables;  // seq id -> blocks
  std::unordered_map<int64_t, int64_t> lengths;              // seq id -> tokens

  PagedKVAllocator(int64_t num_blocks_, int64_t block_size_, int64_t max_blocks_per_seq_)
      : num_blocks(num_blocks_), block_size(block_size_), max_blocks_per_seq(max_blocks_per_seq_) {
    TORCH_CHECK(num_blocks > 0 && block_size > 0 && max_blocks_per_seq > 0, "bad allocator sizes");
    free_list.reserve(num_blocks);
    for (int64_t i = num_blocks - 1; i >= 0; --i) free_list.push_back((int32_t)i);
  }

  int64_t num_free() const { return (int64_t)free_list.size(); }

  bool can_allocate(int64_t tokens) const {
    return (tokens + block_size - 1) / block_size <= (int64_t)free_list.size();
  }

  // Reserves room for `tokens` more tokens of sequence `seq`; returns false (and changes
  // nothing) when the pool or the per-sequence table is exhausted.
  bool extend(int64_t seq, int64_t tokens) {
    auto& tab = tables[seq];
    int64_t& len = lengths[seq];
    const int64_t need = (len + tokens + block_size - 1) / block_size - (int64_t)tab.size();
    if (need > (int64_t)free_list.size() || (int64_t)tab.size() + need > max_blocks_per_seq) {
      if (tab.empty() && len == 0) { tables.erase(seq); lengths.erase(seq); }
      return false;
    }
    for (int64_t i = 0; i < need; ++i) {
      tab.push_back(free_list.back());
      free_list.pop_back();
    }
    len += tokens;
    return true;
  }

  void release(int64_t seq) {
    auto it = tables.find(seq);
    if (it == tables.end()) return;
    for (auto b : it->second) free_list.push_back(b);
    tables.erase(it);
    lengths.erase(seq);
  }

  int64_t length(int64_t seq) const {
    auto it = lengths.find(seq);
    return it == lengths.end() ? 0 : it->second;
  }

  std::vector<int64_t> blocks(int64_t seq) const {
    std::vector<int64_t> out;
    auto it = tables.find(seq);
    if (it != tables.end()) out.assign(it->second.begin(), it->second.end());
    return out;
  }

  // Writes rows of the block table and the sequence lengths for `seqs` (in order) into CPU
  // int32 tensors [n, max_blocks_per_seq] / [n]; unused entries are -1.
  void fill_tables(std::vector<int64_t> seqs, at::Tensor table, at::Tensor lens) const {
    TORCH_CHECK(table.device().is_cpu() && table.scalar_type() == at::kInt && table.is_contiguous());
    TORCH_CHECK(lens.device().is_cpu() && lens.scalar_type() == at::kInt && lens.is_contiguous());
    TORCH_CHECK(table.size(0) >= (int64_t)seqs.size() && table.size(1) == max_blocks_per_seq);
    int32_t* t = table.data_ptr<int32_t>();
    int32_t* l = lens.data_ptr<int32_t>();
    for (size_t i = 0; i < seqs.size(); ++i) {
      int32_t* row = t + i * max_blocks_per_seq;
      std::fill(row, row + max_blocks_per_seq, -1);
      auto it = tables.find(seqs[i]);
      if (it != tables.end()) std::copy(it->second.begin(), it->second.end(), row);
      l[i] = (int32_t)length(seqs[i]);
    }
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
