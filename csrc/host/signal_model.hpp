// Host model of the signal-pad protocol that the device code in comm.cu runs between GPUs, written
// with std::atomic so that a thread sanitizer can check its ordering. One thread stands for one rank.
//
// Protocol: pad[slot][src] of rank r is written by rank src only. A barrier of epoch e on a slot is:
// store-release e into every peer's pad[slot][me], then load-acquire my own pad[slot][p] for every p
// until it shows e or a later value. Epochs only grow, so no word is ever reset and a fast rank may run
// one barrier ahead of a slow one. Every wait is bounded: after `limit` polls it records ST_TIMEOUT_PEER
// in the rank's status word (first writer wins) and gives up.
//
// The one-shot all-reduce brackets its peer reads with two barriers (epochs 2k+1 and 2k+2 of call k):
// the first makes every rank's input visible, the second keeps a fast rank from overwriting its input
// while a slow one still reads it. The input and output buffers are plain (non-atomic) memory, which
// is what makes a missing or mis-ordered barrier show up as a data race.
#pragma once
#include <atomic>
#include <cstdint>
#include <memory>
#include <thread>
#include <vector>

namespace cosmos {
namespace host {

constexpr int kSignalSlots = 64;
constexpr int kSignalRow = 64;
constexpr int kStatusOk = 0;
constexpr int kStatusTimeoutPeer = 5;

struct SignalWorld {
  int world;
  std::vector<std::unique_ptr<std::atomic<int>[]>> pads;      // [rank][slot * 64 + src]
  std::vector<std::unique_ptr<std::atomic<int>>> status;      // one word per rank
  std::vector<std::vector<int>> counters;                     // per rank: epoch kept per slot (rank-local)
  std::vector<std::vector<int64_t>> inputs;                   // per rank: all-reduce input buffer

  SignalWorld(int world_, size_t n_elems) : world(world_) {
    for (int r = 0; r < world; ++r) {
      pads.emplace_back(new std::atomic<int>[kSignalSlots * kSignalRow]);
      for (int i = 0; i < kSignalSlots * kSignalRow; ++i) pads.back()[i].store(0, std::memory_order_relaxed);
      status.emplace_back(new std::atomic<int>(kStatusOk));
      counters.emplace_back(kSignalSlots, 0);
      inputs.emplace_back(n_elems, 0);
    }
  }
};

// Returns false after a timeout. `skip_signal` models a peer that never arrives.
inline bool barrier(SignalWorld& w, int rank, int slot, int epoch, int64_t limit, bool skip_signal = false) {
  if (!skip_signal)
    for (int p = 0; p < w.world; ++p) w.pads[p][slot * kSignalRow + rank].store(epoch, std::memory_order_release);
  for (int p = 0; p < w.world; ++p) {
    int64_t polls = 0;
    while (w.pads[rank][slot * kSignalRow + p].load(std::memory_order_acquire) < epoch) {
      if (++polls > limit) {
        int expected = kStatusOk;
        w.status[rank]->compare_exchange_strong(expected, kStatusTimeoutPeer);
        return false;
      }
      std::this_thread::yield();
    }
  }
  return true;
}

// One call of the one-shot all-reduce on `rank`: out[i] = sum over ranks of inputs[r][i].
// The epoch comes from the rank's own counter for the slot, as in the graph-capturable device path.
inline bool allreduce_oneshot(SignalWorld& w, int rank, int slot, std::vector<int64_t>& out, int64_t limit,
                              bool with_trailing_barrier = true) {
  const int epoch = w.counters[rank][slot] + 1;
  if (!barrier(w, rank, slot, epoch, limit)) return false;
  const size_t n = w.inputs[rank].size();
  out.assign(n, 0);
  for (int r = 0; r < w.world; ++r)
    for (size_t i = 0; i < n; ++i) out[i] += w.inputs[r][i];
  bool ok = true;
  if (with_trailing_barrier) ok = barrier(w, rank, slot, epoch + 1, limit);
  w.counters[rank][slot] = epoch + 1;
  return ok;
}

}  // namespace host
}  // namespace cosmos
