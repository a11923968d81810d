// Paged KV-cache block allocator: a free list of fixed-size pages and a page list per sequence.
// The Reasoner keeps K/V in pages; a sequence that grows by one token takes a new page only when it
// crosses a page boundary. `fill_tables` writes the int32 block table the decode-attention kernel reads.
// One thread (the engine's step loop) owns an allocator; it is not synchronised internally.
#pragma once
#include <algorithm>
#include <cstdint>
#include <unordered_map>
#include <vector>

#include "check.hpp"

namespace cosmos {
namespace host {

class PagedAllocator {
 public:
  PagedAllocator(int64_t num_blocks, int64_t block_size, int64_t max_blocks_per_seq)
      : num_blocks_(num_blocks), block_size_(block_size), max_blocks_per_seq_(max_blocks_per_seq) {
    check(num_blocks > 0 && block_size > 0 && max_blocks_per_seq > 0, "bad allocator sizes");
    free_.reserve((size_t)num_blocks);
    for (int64_t i = num_blocks - 1; i >= 0; --i) free_.push_back((int32_t)i);
  }

  int64_t num_blocks() const { return num_blocks_; }
  int64_t block_size() const { return block_size_; }
  int64_t max_blocks_per_seq() const { return max_blocks_per_seq_; }
  int64_t num_free() const { return (int64_t)free_.size(); }
  int64_t num_sequences() const { return (int64_t)tables_.size(); }

  bool can_allocate(int64_t tokens) const { return blocks_for(tokens) <= (int64_t)free_.size(); }

  // Reserves room for `tokens` more tokens of sequence `seq`; returns false (and changes nothing) when
  // the pool or the per-sequence table is exhausted.
  bool extend(int64_t seq, int64_t tokens) {
    check(tokens >= 0, "extend: negative token count");
    auto it = tables_.find(seq);
    const int64_t have = it == tables_.end() ? 0 : (int64_t)it->second.blocks.size();
    const int64_t len = it == tables_.end() ? 0 : it->second.length;
    const int64_t need = blocks_for(len + tokens) - have;
    if (need > (int64_t)free_.size() || have + need > max_blocks_per_seq_) return false;
    Seq& s = it == tables_.end() ? tables_[seq] : it->second;
    for (int64_t i = 0; i < need; ++i) {
      s.blocks.push_back(free_.back());
      free_.pop_back();
    }
    s.length = len + tokens;
    return true;
  }

  void release(int64_t seq) {
    auto it = tables_.find(seq);
    if (it == tables_.end()) return;
    for (int32_t b : it->second.blocks) free_.push_back(b);
    tables_.erase(it);
  }

  int64_t length(int64_t seq) const {
    auto it = tables_.find(seq);
    return it == tables_.end() ? 0 : it->second.length;
  }

  const std::vector<int32_t>* blocks(int64_t seq) const {
    auto it = tables_.find(seq);
    return it == tables_.end() ? nullptr : &it->second.blocks;
  }

  // Rows of the block table and the sequence lengths for `seqs`, in order: table [n, max_blocks_per_seq]
  // (unused entries -1) and lens [n]. A sequence the allocator does not know gives an empty row.
  void fill_tables(const int64_t* seqs, int64_t n, int32_t* table, int32_t* lens) const {
    for (int64_t i = 0; i < n; ++i) {
      int32_t* row = table + i * max_blocks_per_seq_;
      std::fill(row, row + max_blocks_per_seq_, (int32_t)-1);
      auto it = tables_.find(seqs[i]);
      if (it != tables_.end()) std::copy(it->second.blocks.begin(), it->second.blocks.end(), row);
      lens[i] = it == tables_.end() ? 0 : (int32_t)it->second.length;
    }
  }

 private:
  struct Seq {
    std::vector<int32_t> blocks;
    int64_t length = 0;
  };
  int64_t blocks_for(int64_t tokens) const { return (tokens + block_size_ - 1) / block_size_; }

  int64_t num_blocks_, block_size_, max_blocks_per_seq_;
  std::vector<int32_t> free_;
  std::unordered_map<int64_t, Seq> tables_;
};

}  // namespace host
}  // namespace cosmos
