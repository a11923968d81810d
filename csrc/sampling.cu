// Token sampling for the decode step in two launches (no [B, V] intermediate, no library top-k):
//
//   sample_topk_kernel  one CTA per sequence. Reads the bf16 logits of this rank's vocabulary shard once per pass,
//                       applies the repetition and presence penalties on the fly (the "seen" flags of the token
//                       consumed by this step are set here as well), finds the 64 largest penalised logits with a
//                       radix select over order-preserving keys (histogram passes of 12 + 12 + 8 bits; the row
//                       stays in L2 between passes), sorts them and writes (value, global token id) pairs.
//   sample_pick_kernel  one warp per sequence. Merges the candidates of all vocabulary shards (the pairs of every
//                       rank, gathered by the caller), then temperature, top-k, top-p and the Gumbel-max draw with
//                       the caller's uniform noise; temperature 0 takes the best candidate.
//
// Same arithmetic as the eager definition in serve/decoder.py (`_penalise`, `_sample`); reference behaviour:
// the sampling parameters of cosmos_framework/inference/omni_vllm.py (temperature, top_k, top_p, presence and
// repetition penalties of the Reasoner requests).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>

#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace cb {

constexpr int SK = 64;             // candidates kept per sequence and shard
constexpr int S_CAP = 2048;        // capacity of the candidate list that is sorted
constexpr int S_THREADS = 512;
constexpr int S_BINS = 4096;

__device__ __forceinline__ uint32_t f2key(float x) {
  if (!(x == x)) x = -INFINITY;  // NaN sorts last
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ float penalised(float l, uint32_t any, uint32_t out, float rep, float presence) {
  if (any) l = l > 0.f ? __fdiv_rn(l, rep) : l * rep;
  return out ? l - presence : l;
}

// Calls f(index, key) for every element of the row; 8 elements per 16-byte load when the row allows it.
template <typename F>
// (the flag rows are written by this kernel before they are read, so they are not declared read-only)
__device__ __forceinline__ void for_each_key(const bf16* __restrict__ row, const uint8_t* any, const uint8_t* out,
                                             int V, bool vec, float rep, float presence, F f) {
  if (vec) {
    const int nv = V >> 3;
    for (int v = threadIdx.x; v < nv; v += S_THREADS) {
      const uint4 lv = reinterpret_cast<const uint4*>(row)[v];
      const uint2 av = any ? reinterpret_cast<const uint2*>(any)[v] : make_uint2(0u, 0u);
      const uint2 ov = out ? reinterpret_cast<const uint2*>(out)[v] : make_uint2(0u, 0u);
      const uint32_t lw[4] = {lv.x, lv.y, lv.z, lv.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t bits = (e & 1) ? (lw[e >> 1] & 0xffff0000u) : (lw[e >> 1] << 16);
        const uint32_t a = ((e < 4 ? av.x : av.y) >> (8 * (e & 3))) & 0xffu;
        const uint32_t o = ((e < 4 ? ov.x : ov.y) >> (8 * (e & 3))) & 0xffu;
        f(v * 8 + e, f2key(penalised(__uint_as_float(bits), a, o, rep, presence)));
      }
    }
    for (int i = (nv << 3) + threadIdx.x; i < V; i += S_THREADS)
      f(i, f2key(penalised(__bfloat162float(row[i]), any ? any[i] : 0, out ? out[i] : 0, rep, presence)));
  } else {
    for (int i = threadIdx.x; i < V; i += S_THREADS)
      f(i, f2key(penalised(__bfloat162float(row[i]), any ? any[i] : 0, out ? out[i] : 0, rep, presence)));
  }
}

// Descending bitonic sort of n (a power of two) 64-bit keys in shared memory by all threads of the block.
__device__ __forceinline__ void bitonic_desc(unsigned long long* a, int n, int nthreads) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += nthreads) {
        const int x = i ^ j;
        if (x > i) {
          const unsigned long long u = a[i], w = a[x];
          const bool desc = (i & k) == 0;
          if (desc ? (u < w) : (u > w)) {
            a[i] = w;
            a[x] = u;
          }
        }
      }
      __syncthreads();
    }
  }
}

// cand[b, r] = (penalised logit, global token id as int bits) of the r-th largest entry of row b, r < 64.
__global__ void __launch_bounds__(S_THREADS)
sample_topk_kernel(const bf16* __restrict__ logits, long long ld, int V, uint8_t* seen_any, uint8_t* seen_out,
                   const long long* __restrict__ tokens, const float* __restrict__ presence,
                   const float* __restrict__ repetition, int vocab_offset, float2* __restrict__ cand) {
  __shared__ int hist[S_BINS];
  __shared__ unsigned long long list[S_CAP];
  __shared__ int scan[S_THREADS];
  __shared__ int sh_bin, sh_above, sh_count;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  const bf16* row = logits + (long long)b * ld;
  uint8_t* any = seen_any ? seen_any + (long long)b * V : nullptr;
  uint8_t* out = seen_out ? seen_out + (long long)b * V : nullptr;
  const float rep = repetition ? repetition[b] : 1.f, pres = presence ? presence[b] : 0.f;
  // the token consumed by this step counts as generated (and as seen) from now on
  if (tid == 0 && tokens && any && out) {
    const long long loc = tokens[b] - vocab_offset;
    if (loc >= 0 && loc < V) {
      any[loc] = 1;
      out[loc] = 1;
    }
    __threadfence_block();
  }
  __syncthreads();
  const bool vec = (V >= 8) && (reinterpret_cast<uintptr_t>(row) % 16 == 0) &&
                   (!any || (reinterpret_cast<uintptr_t>(any) % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0));

  // ---- radix select: after each level `prefix` holds the leading `done` bits of the key of the 64th largest
  // element, `need` how many of the 64 lie inside that prefix bin
  uint32_t prefix = 0;
  int done = 0, need = SK < V ? SK : V;
  const int level_bits[3] = {12, 12, 8};
  int in_bin = V;
  for (int lv = 0; lv < 3 && in_bin > S_CAP - SK; ++lv) {
    const int bits = level_bits[lv], shift = 32 - done - bits;
    const uint32_t mask = (1u << bits) - 1u;
    for (int i = tid; i < S_BINS; i += S_THREADS) hist[i] = 0;
    __syncthreads();
    for_each_key(row, any, out, V, vec, rep, pres, [&](int, uint32_t key) {
      if (done == 0 || (key >> (32 - done)) == prefix) atomicAdd(&hist[(key >> shift) & mask], 1);
    });
    __syncthreads();
    // suffix sums over the bins: thread t owns bins [8t, 8t + 8)
    int own = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) own += hist[tid * 8 + e];
    scan[tid] = own;
    __syncthreads();
    for (int off = 1; off < S_THREADS; off <<= 1) {
      const int add = tid + off < S_THREADS ? scan[tid + off] : 0;
      __syncthreads();
      scan[tid] += add;
      __syncthreads();
    }
    const int above_mine = scan[tid] - own;  // elements in bins above this thread's eight
    if (above_mine < need && need <= above_mine + own) {
      int above = above_mine;
      for (int e = 7; e >= 0; --e) {
        const int h = hist[tid * 8 + e];
        if (need <= above + h) {
          sh_bin = tid * 8 + e;
          sh_above = above;
          break;
        }
        above += h;
      }
    }
    __syncthreads();
    prefix = (prefix << bits) | uint32_t(sh_bin);
    need -= sh_above;
    in_bin = hist[sh_bin];
    done += bits;
    __syncthreads();
  }

  // ---- collect: the elements above the threshold bin (fewer than 64) go to the first 64 slots, the bin's own
  // elements behind them while the list has room (only exact ties can overflow it, and any of them will do)
  if (tid == 0) {
    sh_count = 0;
    sh_above = 0;
  }
  if (tid < SK) list[tid] = 0ull;
  __syncthreads();
  for_each_key(row, any, out, V, vec, rep, pres, [&](int i, uint32_t key) {
    const uint32_t hi = done == 0 ? 0u : (key >> (32 - done));
    const unsigned long long e = ((unsigned long long)key << 32) | (0xffffffffu - uint32_t(i));
    if (done != 0 && hi > prefix) {
      const int pos = atomicAdd(&sh_above, 1);
      if (pos < SK) list[pos] = e;
    } else if (done == 0 || hi == prefix) {
      const int pos = atomicAdd(&sh_count, 1);
      if (pos < S_CAP - SK) list[SK + pos] = e;
    }
  });
  __syncthreads();
  const int n = SK + (sh_count < S_CAP - SK ? sh_count : S_CAP - SK);
  int n2 = SK;
  while (n2 < n) n2 <<= 1;
  for (int i = n + tid; i < n2; i += S_THREADS) list[i] = 0ull;
  __syncthreads();
  bitonic_desc(list, n2, S_THREADS);
  if (tid < SK) {
    float2 o;
    const unsigned long long e = list[tid];
    if (e != 0ull) {
      o.x = key2f(uint32_t(e >> 32));
      o.y = __int_as_float(int(0xffffffffu - uint32_t(e)) + vocab_offset);
    } else {
      o.x = -INFINITY;
      o.y = __int_as_float(vocab_offset);
    }
    cand[(long long)b * SK + tid] = o;
  }
}

// One warp per sequence: merge of the shards' candidates, then the draw. cand is [n_src, B, 64] pairs.
constexpr int PICK_MAX = 1024;  // n_src * 64 rounded up to a power of two
__global__ void __launch_bounds__(128)
sample_pick_kernel(const float2* __restrict__ cand, int n_src, int B, const float* __restrict__ temperature,
                   const long long* __restrict__ top_k, const float* __restrict__ top_p,
                   const float* __restrict__ noise, long long noise_ld, int vocab_size,
                   long long* __restrict__ tokens_out) {
  extern __shared__ unsigned long long pick_list[];  // [4 warps][n2]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * 4 + warp;
  int n2 = SK;
  while (n2 < n_src * SK) n2 <<= 1;
  unsigned long long* a = pick_list + warp * n2;
  const bool live = b < B;
  // (value key, source slot) pairs: the slot finds the token id again after the sort
  for (int i = lane; i < n2; i += 32) {
    unsigned long long e = 0ull;
    if (live && i < n_src * SK) {
      const int src = i / SK, r = i - src * SK;
      const float2 c = cand[((long long)src * B + b) * SK + r];
      // equal values: the smaller token id first, whatever shard it came from
      e = ((unsigned long long)f2key(c.x) << 32) | (0xffffffffu - uint32_t(__float_as_int(c.y)));
    }
    a[i] = e;
  }
  __syncwarp();
  if (n_src > 1) {
    for (int k = 2; k <= n2; k <<= 1) {
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int i = lane; i < n2; i += 32) {
          const int x = i ^ j;
          if (x > i) {
            const unsigned long long u = a[i], w = a[x];
            const bool desc = (i & k) == 0;
            if (desc ? (u < w) : (u > w)) {
              a[i] = w;
              a[x] = u;
            }
          }
        }
        __syncwarp();
      }
    }
  }
  if (!live) return;
  const float t = temperature[b];
  int tk = (int)top_k[b];
  tk = tk < 1 ? 1 : (tk > SK ? SK : tk);
  const float tp = top_p[b];
  const float inv_t = t > 0.f ? t : 1.f;
  // two candidates per lane: r = lane and lane + 32 (sorted, best first)
  float z[2];
  int id[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = lane + 32 * h;
    const unsigned long long e = a[r];
    z[h] = (r < tk && e != 0ull) ? __fdiv_rn(key2f(uint32_t(e >> 32)), inv_t) : -INFINITY;
    id[h] = int(0xffffffffu - uint32_t(e));
  }
  const float zmax = __shfl_sync(0xffffffffu, z[0], 0);
  float p[2] = {expf(z[0] - zmax), expf(z[1] - zmax)};
  float sum = p[0] + p[1];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  p[0] /= sum;
  p[1] /= sum;
  // exclusive prefix sums in candidate order
  float inc0 = p[0];
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, inc0, o);
    if (lane >= o) inc0 += v;
  }
  const float first_half = __shfl_sync(0xffffffffu, inc0, 31);
  float inc1 = p[1];
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, inc1, o);
    if (lane >= o) inc1 += v;
  }
  inc1 += first_half;
  const float exc[2] = {inc0 - p[0], inc1 - p[1]};
  float best = -INFINITY;
  int best_r = 0x7fffffff;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = lane + 32 * h;
    if (exc[h] < tp && z[h] > -INFINITY) {
      const float u = noise[(long long)b * noise_ld + r];
      const float g = -logf(-logf(u));
      const float s = z[h] + g;
      if (s > best || (s == best && r < best_r)) {
        best = s;
        best_r = r;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int orr = __shfl_xor_sync(0xffffffffu, best_r, o);
    if (ob > best || (ob == best && orr < best_r)) {
      best = ob;
      best_r = orr;
    }
  }
  if (best_r > SK - 1) best_r = 0;
  const int pick = t > 0.f ? best_r : 0;
  const int tok_lo = __shfl_sync(0xffffffffu, id[0], pick & 31);
  const int tok_hi = __shfl_sync(0xffffffffu, id[1], pick & 31);
  if (lane == 0) {
    int tok = pick < 32 ? tok_lo : tok_hi;
    if (tok > vocab_size - 1) tok = vocab_size - 1;
    if (tok < 0) tok = 0;
    tokens_out[b] = tok;
  }
}

}  // namespace cb

namespace cosmos {

void sample_topk(const void* logits, long long ld, int B, int V, void* seen_any, void* seen_out,
                 const long long* tokens, const float* presence, const float* repetition, int vocab_offset,
                 void* cand, cudaStream_t s) {
  if (B <= 0) return;
  if (V < 1) throw std::runtime_error("sample_topk: empty vocabulary shard");
  cb::sample_topk_kernel<<<B, cb::S_THREADS, 0, s>>>((const bf16*)logits, ld, V, (uint8_t*)seen_any,
                                                     (uint8_t*)seen_out, tokens, presence, repetition, vocab_offset,
                                                     (float2*)cand);
}

void sample_pick(const void* cand, int n_src, int B, const float* temperature, const long long* top_k,
                 const float* top_p, const float* noise, long long noise_ld, int vocab_size, long long* tokens_out,
                 cudaStream_t s) {
  if (B <= 0) return;
  if (n_src < 1 || n_src * cb::SK > cb::PICK_MAX)
    throw std::runtime_error("sample_pick: between 1 and 16 candidate sources");
  int n2 = cb::SK;
  while (n2 < n_src * cb::SK) n2 <<= 1;
  cb::sample_pick_kernel<<<(B + 3) / 4, 128, 4 * n2 * sizeof(unsigned long long), s>>>(
      (const float2*)cand, n_src, B, temperature, top_k, top_p, noise, noise_ld, vocab_size, tokens_out);
}

}  // namespace cosmos
