// Decode attention over the paged KV cache on the tensor cores (head_dim 128, bf16, GQA).
//
// Decode attention reads every cached K/V byte once per step, so the kernel is built around the
// copy engine: one thread streams whole cache pages with TMA into a 3-stage ring of 128-token
// K/V tiles (128-byte swizzle), and both products run as tcgen05 MMAs straight from that shared
// memory, so no thread ever touches a K or V element:
//     S^T[token, head] = K_tile . Q^T          M = 128 tokens, N = 16 (the GQA group, zero padded), K = 128
//     O^T[dim, head]  += V_tile^T . P^T        M = 128 dims,   N = 16, K = 128 tokens (V read MN-major)
// The transposed products put tokens (then output dims) on the 128 TMEM lanes, so the softmax
// threads hold one token each: 16 scores per tile, a running max per head shared through shared
// memory, exp2, and a 2-byte store of P into the swizzled B-operand buffer of the second product.
// The running max is refreshed lazily (only when it grows by more than 2^8), so O^T is rescaled
// rarely; every thread keeps its own partial row sums and they are added once at the end.
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 softmax + epilogue.
// Long sequences are split along kv exactly as in paged_decode.cu (same partial format, same merge
// kernel). The kernel is persistent: one CTA per SM walks over the (sequence, kv head, kv split)
// items, and ring, barriers and tile counter run on across items, so the next item's first tiles are
// already in flight while the current one finishes. Every wait is bounded.
//
//   k_cache / v_cache [num_pages, Hkv, page_size, 128] bf16, page_size in {8, 16, 32, 64, 128}
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace cb {

constexpr int PT_THREADS = 192;
constexpr int PT_TILE = 128;
constexpr int PT_NST = 3;
constexpr int PT_TILE_BYTES = PT_TILE * 128 * 2;    // 32 KB (K or V of one tile)
constexpr int PT_HALF = PT_TILE_BYTES / 2;
constexpr int PT_OPB = 16 * 128 * 2;                // one 16-row B operand (Q^T or P^T): 4 KB
constexpr int PT_NQ = 4;                            // Q^T buffers (ring over items)
constexpr int PT_NOPB = PT_NQ + 2;                  // + P^T x 2 (tiles)
constexpr int PT_SMEM = PT_NST * 2 * PT_TILE_BYTES + PT_NOPB * PT_OPB + 2048 + 1024;

// barrier indices
constexpr int PB_FULL = 0;                 // + stage
constexpr int PB_EMPTY = PT_NST;           // + stage
constexpr int PB_S = 2 * PT_NST;           // + (tile & 1): scores ready
// One P barrier per P buffer. With a single barrier the 128 softmax threads could complete the phases of tiles t
// and t + 1 back to back (the scores of t + 1 are issued before the issuer waits for P of t) and an issuer that
// looked late would see the parity of t "not completed" again and wait for good. A buffer's barrier completes a
// second time only after the product that read the buffer, which the issuer starts after it has seen the first.
constexpr int PB_P = 2 * PT_NST + 2;       // + (tile & 1): P of that tile written (128 arrivals)
constexpr int PB_PV = 2 * PT_NST + 4;      // + (tile & 1): second product of that tile done
constexpr int PB_COUNT = 2 * PT_NST + 6;

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
      "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

// Byte offset of element (row, col) in a K-major 16-row x 128-column bf16 operand stored as two
// 64-column halves of 128-byte rows with the 128-byte swizzle (chunk index xor row % 8).
__device__ __forceinline__ uint32_t opb_offset(int row, int col) {
  const int half = col >> 6, c = (col & 63) >> 3;
  return uint32_t(half * 2048 + row * 128 + ((c ^ (row & 7)) << 4) + (col & 7) * 2);
}

__device__ __forceinline__ float pt_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void pt_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct PtItem {
  int split, kvh, b, kv_begin, kv_end, n_tiles;
};

__device__ __forceinline__ PtItem pt_item(int it, int n_splits, int Hkv, const int* __restrict__ seq_lens) {
  PtItem I;
  I.split = it % n_splits;
  I.kvh = (it / n_splits) % Hkv;
  I.b = it / (n_splits * Hkv);
  const int len = seq_lens[I.b];
  const int chunk = ((len + n_splits - 1) / n_splits + PT_TILE - 1) / PT_TILE * PT_TILE;
  I.kv_begin = I.split * chunk;
  I.kv_end = min(len, I.kv_begin + chunk);
  I.n_tiles = I.kv_end > I.kv_begin ? (I.kv_end - I.kv_begin + PT_TILE - 1) / PT_TILE : 0;
  return I;
}

// Persistent: CTA c works on items c, c + gridDim.x, ... (item = one (sequence, kv head, kv split)); the
// K/V ring, the barriers and the global tile counter `gt` run on across items, so the copies of the
// next item's first tiles are in flight while the current item finishes.
template <int GROUP>
__global__ void __launch_bounds__(PT_THREADS, 1)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const bf16* __restrict__ q, const int* __restrict__ table, const int* __restrict__ seq_lens,
                       int max_pages, int page_size, int num_pages, int n_seqs, int Hq, int Hkv, int n_splits,
                       float scale_log2, float* __restrict__ part_acc, float* __restrict__ part_ml,
                       bf16* __restrict__ out, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  auto k_smem = [&](int s) { return base + uint32_t(s) * 2 * PT_TILE_BYTES; };
  auto v_smem = [&](int s) { return base + uint32_t(s) * 2 * PT_TILE_BYTES + PT_TILE_BYTES; };
  const uint32_t ring_bytes = PT_NST * 2 * PT_TILE_BYTES;
  // 16-row operands: a ring of PT_NQ Q^T buffers (one per item), then P^T of even / odd tiles
  auto q_smem = [&](int i) { return base + ring_bytes + PT_OPB * i; };
  auto p_smem = [&](int i) { return base + ring_bytes + PT_OPB * (PT_NQ + i); };
  uint8_t* opb_gen = gen + ring_bytes;
  float* red = reinterpret_cast<float*>(gen + ring_bytes + PT_NOPB * PT_OPB);  // [3][4][GROUP]
  const uint32_t bar = base + ring_bytes + PT_NOPB * PT_OPB + 1024;
  auto B = [&](int i) { return bar + 8u * i; };
  const uint32_t tmem_slot = bar + 8u * PB_COUNT;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(gen + ring_bytes + PT_NOPB * PT_OPB + 1024 + 8 * PB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot_ptr + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = n_splits * Hkv * n_seqs;

  // ---- setup: barriers, TMEM, operand buffers zeroed (rows >= GROUP of Q^T / P^T stay zero for good)
  if (threadIdx.x == 0) {
    for (int s = 0; s < PT_NST; ++s) {
      mbar_init(B(PB_FULL + s), 1);
      mbar_init(B(PB_EMPTY + s), 1);
    }
    mbar_init(B(PB_S), 1);
    mbar_init(B(PB_S + 1), 1);
    mbar_init(B(PB_P), 128);
    mbar_init(B(PB_P + 1), 128);
    mbar_init(B(PB_PV), 1);
    mbar_init(B(PB_PV + 1), 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i < PT_NOPB * PT_OPB / 16; i += PT_THREADS)
    reinterpret_cast<uint4*>(opb_gen)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // set-up done: the next kernel may start its own, and this one waits for the kernel that wrote q and the
  // newest cache row (no-ops unless launched as a programmatic dependent)
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t T_S0 = tmem_base, T_O = tmem_base + 32;  // scores of global tile g at T_S0 + 16 * (g & 1)

  if (warp == 0) {
    // ---------------- producer warp: Q^T operand of the item, then one TMA box (page_size rows x 64 columns)
    // per page, tensor and half. Copy `op` of a tile is (page op / 4, K lo | K hi | V lo | V hi); lane l
    // takes ops l and l + 32; the page ids of the next tile are loaded one tile ahead.
    const int pages_per_tile = PT_TILE / page_size;
    const int n_ops = 4 * pages_per_tile;  // 4 .. 64
    int gt = 0, io = 0;
    bool ok = true;
    int issued_lo = 0;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
      const PtItem I = pt_item(it, n_splits, Hkv, seq_lens);
      if (I.n_tiles == 0) continue;
      // Q^T buffer of this item: a ring of PT_NQ. It is written below after the wait for the ring slot of
      // the item's first tile T0, which returns once tile T0 - PT_NST has been consumed; the previous user of
      // the buffer is PT_NQ items back, and every item has at least one tile, so its last tile is at most
      // T0 - PT_NQ <= T0 - PT_NST and (MMAs complete in order) has been consumed as well.
      static_assert(PT_NQ >= PT_NST, "the Q^T ring must cover the K/V ring's run-ahead");
      const int qb = io % PT_NQ;
      auto page_of = [&](int j, int op) {
        // pages past the end of the sequence are read from an out-of-range page index: zero fill
        const int tok = I.kv_begin + j * PT_TILE + (op >> 2) * page_size;
        int page = num_pages;
        if (j < I.n_tiles && op < n_ops && tok < I.kv_end) {
          page = table[(long long)I.b * max_pages + tok / page_size];
          if (page < 0 || page >= num_pages) {
#ifdef COSMOS_BOUNDS_CHECK
            if (status) atomicCAS(status, 0, ST_BAD_INDEX | (SITE_PAGED_DECODE_TC_PAGE << 8));
#endif
            page = num_pages;
          }
        }
        return page;
      };
      int pg0 = page_of(0, lane), pg1 = page_of(0, lane + 32);
      for (int j = 0; j < I.n_tiles; ++j, ++gt) {
        const int s = gt % PT_NST;
        const int cur0 = pg0, cur1 = pg1;
        pg0 = page_of(j + 1, lane);
        pg1 = page_of(j + 1, lane + 32);
        const uint32_t full = B(PB_FULL + s);
        int good = 1;
        if (lane == 0)
          good = mbar_wait(B(PB_EMPTY + s), ((gt / PT_NST) & 1) ^ 1, abort_flag, status, ST_TIMEOUT_TMA) ? 1 : 0;
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) {
          ok = false;
          break;
        }
        if (j == 0) {
          for (int i = lane; i < GROUP * 128; i += 32) {
            const int g = i >> 7, d = i & 127;
            *reinterpret_cast<bf16*>(opb_gen + PT_OPB * qb + opb_offset(g, d)) =
                q[((long long)I.b * Hq + I.kvh * GROUP + g) * 128 + d];
          }
          fence_proxy_async();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_expect_tx(full, 2 * PT_TILE_BYTES);
        __syncwarp();
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int op = lane + 32 * r;
          if (op < n_ops) {
            const int which = op & 3;
            const uint32_t dst = ((which & 2) ? v_smem(s) : k_smem(s)) + ((which & 1) ? PT_HALF : 0) +
                                 uint32_t((op >> 2) * page_size) * 128u;
            tma_load_4d(dst, (which & 2) ? &tmV : &tmK, full, (which & 1) ? 64 : 0, 0, I.kvh, r ? cur1 : cur0);
          }
        }
        issued_lo = gt + 1;
      }
      ++io;
    }
    if (!ok && lane == 0) {
      volatile int no_abort = 0;
      const int first = issued_lo > PT_NST ? issued_lo - PT_NST : 0;
      for (int i = first; i < issued_lo; ++i)
        mbar_wait(B(PB_FULL + i % PT_NST), (i / PT_NST) & 1, &no_abort, nullptr, 0);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 16, 0, 0);
    constexpr uint32_t idesc_o = make_idesc_bf16(128, 16, 1, 0);
    int gt = 0, io = 0;
    bool ok = true;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
      const PtItem I = pt_item(it, n_splits, Hkv, seq_lens);
      if (I.n_tiles == 0) continue;
      const uint64_t q_desc = make_smem_desc_sw128(q_smem(io % PT_NQ), 16, 1024);
      auto issue_s = [&](int g) {
        const uint64_t k_desc = make_smem_desc_sw128(k_smem(g % PT_NST), 16, 1024);
        const uint32_t d = T_S0 + 16 * (g & 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t ka = (kk >> 2) * (PT_HALF >> 4) + 2 * (kk & 3);
          const uint32_t kb = (kk >> 2) * (2048 >> 4) + 2 * (kk & 3);
          mma_ss(d, k_desc + ka, q_desc + kb, idesc_s, kk > 0 ? 1u : 0u);
        }
      };
      ok = mbar_wait(B(PB_FULL + gt % PT_NST), (gt / PT_NST) & 1, abort_flag, status, ST_TIMEOUT_MMA);
      if (!ok) break;
      tc_fence_after();
      issue_s(gt);
      tc_commit(B(PB_S + (gt & 1)));
      for (int j = 0; j < I.n_tiles && ok; ++j, ++gt) {
        const int s = gt % PT_NST;
        if (j + 1 < I.n_tiles) {
          // scores of the next tile while the softmax threads work on this one
          ok = mbar_wait(B(PB_FULL + (gt + 1) % PT_NST), ((gt + 1) / PT_NST) & 1, abort_flag, status, ST_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_s(gt + 1);
          tc_commit(B(PB_S + ((gt + 1) & 1)));
        }
        ok = mbar_wait(B(PB_P + (gt & 1)), (gt >> 1) & 1, abort_flag, status, ST_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint64_t v_desc = make_smem_desc_sw128(v_smem(s), PT_HALF, 1024);
        const uint64_t p_desc = make_smem_desc_sw128(p_smem(gt & 1), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t kb = (kk >> 2) * (2048 >> 4) + 2 * (kk & 3);
          mma_ss(T_O, v_desc + uint64_t(kk * (2048 >> 4)), p_desc + kb, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(B(PB_EMPTY + s));
        tc_commit(B(PB_PV + (gt & 1)));
      }
      ++io;
    }
  } else if (warp >= 2) {
    // ---------------- softmax: this thread owns token t of every tile (TMEM lane t), then output dim t
    const int quad = warp & 3;
    const int t = quad * 32 + lane;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    int gt = 0;
    bool ok = true;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
      const PtItem I = pt_item(it, n_splits, Hkv, seq_lens);
      float m_used[GROUP], l_part[GROUP];
#pragma unroll
      for (int g = 0; g < GROUP; ++g) { m_used[g] = -1e30f; l_part[g] = 0.f; }
      for (int j = 0; j < I.n_tiles; ++j, ++gt) {
        if (!mbar_wait(B(PB_S + (gt & 1)), (gt >> 1) & 1, abort_flag, status, ST_TIMEOUT_SOFTMAX)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t sv[16];
        tmem_ld16(T_S0 + 16 * (gt & 1) + lane_addr, sv);
        tmem_wait_ld();
        const bool valid = I.kv_begin + j * PT_TILE + t < I.kv_end;
        float x[GROUP], tm[GROUP];
        float* rbuf = red + (gt & 1) * 4 * GROUP;
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
          x[g] = valid ? __uint_as_float(sv[g]) * scale_log2 : -1e30f;
          float v = x[g];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
          if (lane == 0) rbuf[quad * GROUP + g] = v;
        }
        pt_bar_sync();
        bool need = false;
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
          tm[g] = fmaxf(fmaxf(rbuf[g], rbuf[GROUP + g]), fmaxf(rbuf[2 * GROUP + g], rbuf[3 * GROUP + g]));
          tm[g] = fmaxf(tm[g], m_used[g]);
          need |= tm[g] > m_used[g] + 8.f;
        }
        if (j == 0) {
#pragma unroll
          for (int g = 0; g < GROUP; ++g) m_used[g] = tm[g];
        } else if (need) {
          // the running max moved by more than 2^8 for some head: rescale O^T once every earlier product is done
          if (!mbar_wait(B(PB_PV + ((gt - 1) & 1)), ((gt - 1) >> 1) & 1, abort_flag, status, ST_TIMEOUT_SOFTMAX)) {
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t ov[16];
          tmem_ld16(T_O + lane_addr, ov);
          tmem_wait_ld();
#pragma unroll
          for (int g = 0; g < GROUP; ++g) {
            if (tm[g] > m_used[g] + 8.f) {
              const float sc = pt_ex2(m_used[g] - tm[g]);
              ov[g] = __float_as_uint(__uint_as_float(ov[g]) * sc);
              l_part[g] *= sc;
              m_used[g] = tm[g];
            }
          }
          tmem_st16(T_O + lane_addr, ov);
          tmem_wait_st();
          tc_fence_before();
        }
        // P buffer (gt & 1) was last read by the second product of global tile gt - 2
        if (gt >= 2 && !mbar_wait(B(PB_PV + (gt & 1)), ((gt >> 1) - 1) & 1, abort_flag, status, ST_TIMEOUT_SOFTMAX)) {
          ok = false;
          break;
        }
        uint8_t* pbuf = opb_gen + PT_OPB * (PT_NQ + (gt & 1));
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
          const float p = pt_ex2(x[g] - m_used[g]);
          l_part[g] += p;
          *reinterpret_cast<bf16*>(pbuf + opb_offset(g, t)) = __float2bfloat16(p);
        }
        fence_proxy_async();
        mbar_arrive(B(PB_P + (gt & 1)));
      }
      if (!ok) break;
      // ---- item epilogue: row sums over the 128 threads, then this thread's output dim for every head
      uint32_t ov[16];
#pragma unroll
      for (int g = 0; g < 16; ++g) ov[g] = 0u;
      float l[GROUP];
#pragma unroll
      for (int g = 0; g < GROUP; ++g) l[g] = 0.f;
      if (I.n_tiles > 0) {
        float* rbuf = red + 2 * 4 * GROUP;  // third slice, not used by the tile loop
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
          float v = l_part[g];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) rbuf[quad * GROUP + g] = v;
        }
        pt_bar_sync();
#pragma unroll
        for (int g = 0; g < GROUP; ++g) l[g] = rbuf[g] + rbuf[GROUP + g] + rbuf[2 * GROUP + g] + rbuf[3 * GROUP + g];
        if (!mbar_wait(B(PB_PV + ((gt - 1) & 1)), ((gt - 1) >> 1) & 1, abort_flag, status, ST_TIMEOUT_SOFTMAX)) {
          ok = false;
          break;
        }
        tc_fence_after();
        tmem_ld16(T_O + lane_addr, ov);
        tmem_wait_ld();
        tc_fence_before();  // the next item's first product overwrites O^T only after every thread's arrive below
      }
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
        const int h = I.kvh * GROUP + g;
        const float a = __uint_as_float(ov[g]);
        if (n_splits == 1) {
          out[((long long)I.b * Hq + h) * 128 + t] = __float2bfloat16(l[g] > 0.f ? a / l[g] : 0.f);
        } else {
          const long long pb = ((long long)I.b * Hq + h) * n_splits + I.split;
          part_acc[pb * 128 + t] = a;
          if (t == 0) {
            part_ml[pb * 2] = m_used[g];
            part_ml[pb * 2 + 1] = l[g];
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
}

}  // namespace cb

namespace cosmos {

// Splits along kv for the tensor-core kernel (persistent, one CTA per SM, items handed out round-robin):
// the count that minimises the tiles of the busiest CTA plus a small per-item cost.
int paged_decode_tc_pick_splits(int B, int Hkv, int max_len) {
  const long long pairs = (long long)B * Hkv;
  const int tiles = (max_len + cb::PT_TILE - 1) / cb::PT_TILE;
  int best = 1;
  double best_cost = 1e30;
  for (int ns = 1; ns <= 32 && ns <= tiles; ++ns) {
    const long long items_per_cta = (pairs * ns + 147) / 148;
    const int per = (tiles + ns - 1) / ns;
    const double cost = (double)items_per_cta * (per + 0.3);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = ns;
    }
  }
  return best;
}

bool paged_decode_tc_supported(const PagedDecodeArgs& a) {
  const int g = a.Hkv > 0 ? a.Hq / a.Hkv : 0;
  const int ps = a.page_size;
  return a.num_pages > 0 && (g == 1 || g == 2 || g == 4 || g == 8) &&
         (ps == 8 || ps == 16 || ps == 32 || ps == 64 || ps == 128);
}

static CUtensorMap cache_map(const void* base, int num_pages, int Hkv, int page_size) {
  const uint64_t dims[4] = {128, (uint64_t)page_size, (uint64_t)Hkv, (uint64_t)num_pages};
  const uint64_t strides[3] = {256, (uint64_t)page_size * 256, (uint64_t)Hkv * page_size * 256};
  const uint32_t box[4] = {64, (uint32_t)page_size, 1, 1};
  return cbh::make_tmap_bf16(base, 4, dims, strides, box, true);
}

template <int GROUP>
static void launch_tc(const PagedDecodeArgs& a, float* pa, float* pm, cudaStream_t s) {
  static thread_local bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(cb::paged_decode_tc_kernel<GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, cb::PT_SMEM);
    configured = true;
  }
  CUtensorMap tk = cache_map(a.k_cache, a.num_pages, a.Hkv, a.page_size);
  CUtensorMap tv = cache_map(a.v_cache, a.num_pages, a.Hkv, a.page_size);
  // persistent: one CTA per SM walks over the (sequence, kv head, split) items
  static thread_local int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const long long items = (long long)a.n_splits * a.Hkv * a.B;
  const int grid = (int)std::min<long long>(items, sms);
  launch_pdl(cb::paged_decode_tc_kernel<GROUP>, dim3(grid), dim3(cb::PT_THREADS), cb::PT_SMEM, s,
      tk, tv, (const bf16*)a.q, a.block_table, a.seq_lens, a.max_pages, a.page_size, a.num_pages, a.B, a.Hq, a.Hkv,
      a.n_splits, a.scale * 1.4426950408889634f, pa, pm, (bf16*)a.out, a.status);
}

// Launches the tensor-core kernel (partials into pa / pm when n_splits > 1; the caller merges them: a merge by the
// CTA that finishes a head's last split was measured slower, 12.81 against 12.45 ms per decode step at batch 32,
// because every item then pays a device-scope fence on the softmax threads' path).
// The caller has checked paged_decode_tc_supported().
void paged_decode_tc_launch(const PagedDecodeArgs& a, float* pa, float* pm, cudaStream_t s) {
  switch (a.Hq / a.Hkv) {
    case 1: launch_tc<1>(a, pa, pm, s); break;
    case 2: launch_tc<2>(a, pa, pm, s); break;
    case 4: launch_tc<4>(a, pa, pm, s); break;
    case 8: launch_tc<8>(a, pa, pm, s); break;
    default: throw std::runtime_error("paged_decode_tc: Hq / Hkv must be 1, 2, 4 or 8");
  }
}

}  // namespace cosmos
