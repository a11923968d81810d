// Flash attention backward (head_dim 128, bf16, GQA) on tcgen05 tensor cores, as two kernels that
// need no atomics and no O(S^2) memory:
//
//   dK/dV kernel: one CTA owns a 128-row K/V tile (stationary in shared memory) and streams the
//   Q / dO tiles of every query head of its GQA group through a 2-stage TMA ring. Per tile pair
//       S^T  = K Q^T          (SS MMA)          dP^T = V dO^T             (SS MMA)
//       P^T  = exp2(S^T * scale*log2e - lse)    dS^T = P^T (dP^T - D) scale   (registers -> TMEM, bf16)
//       dV  += P^T dO         (TS MMA)          dK  += dS^T Q             (TS MMA)
//   The transposed products put the K/V rows on the TMEM lanes, so P^T and dS^T can feed the
//   accumulating MMAs straight from tensor memory (they alias S^T and dP^T), and dK / dV
//   accumulate in TMEM over the whole loop: 4 x 128 columns = the full 512.
//
//   dQ kernel: one CTA owns a 128-row Q / dO tile and streams K/V tiles:
//       S = Q K^T, dP = dO V^T (SS), dS = P (dP - D) scale -> TMEM (bf16), dQ += dS K (TS).
//
// Warp roles (384 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 4..11 element-wise math
// and epilogue: two warpgroups, each thread owns one TMEM lane (a K/V row resp. a Q row) and one
// 64-column half of the score tile; a warpgroup writes its bf16 P / dS into the first half of its
// own fp32 score columns, so the two never touch each other's inputs.
// D = rowsum(dO * O) and the log-sum-exp of the forward pass come in as [B, Hq, Sq] fp32.
// Masks as in the forward kernel (full, causal, Mixture-of-Transformers block mask).
// Every wait is bounded; on expiry the kernel records a status code and unwinds.
#include "common.cuh"
#include "kernels.h"

namespace cb {

constexpr int BWD_THREADS = 384;
constexpr int BT = 128;                         // tile rows (queries and keys), = head_dim
constexpr int BTILE_BYTES = BT * 128 * 2;       // 32 KB
constexpr int BHALF_BYTES = BTILE_BYTES / 2;    // one 64-column half
constexpr int BWD_NST = 2;                      // streamed stages (two tiles each)
constexpr int BWD_SMEM = 2 * BTILE_BYTES + BWD_NST * 2 * BTILE_BYTES + 4 * BT * 4 + 256 + 1024;

struct AttnBwdParams {
  int Sq, Skv, Hq, Hkv, group;
  int mask, n_ar;
  float scale, scale_log2;
  const float* lse;    // [B, Hq, Sq] natural log
  const float* delta;  // [B, Hq, Sq]
  bf16* dQ;            // [B, Sq, Hq, 128] contiguous
  bf16* dK;            // [B, Skv, Hkv, 128] contiguous
  bf16* dV;
  int* status;
};

__device__ __forceinline__ float bwd_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ bool bwd_masked(int kv, int q, const AttnBwdParams& p) {
  if (kv >= p.Skv) return true;
  if (p.mask == MASK_CAUSAL) return kv > q + (p.Skv - p.Sq);
  if (p.mask == MASK_MOT) return q < p.n_ar && kv > q;
  return false;
}

// True when some (kv, q) pair of the 128 x 128 tile pair is masked.
__device__ __forceinline__ bool bwd_tile_needs_mask(int kv0, int q0, const AttnBwdParams& p) {
  if (kv0 + BT > p.Skv) return true;
  if (p.mask == MASK_CAUSAL) return kv0 + BT - 1 > q0 + (p.Skv - p.Sq);
  if (p.mask == MASK_MOT) return q0 < p.n_ar && kv0 + BT - 1 > q0;
  return false;
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

struct BwdSmem {
  uint32_t base;         // 1024-aligned shared address of the tile area
  uint8_t* gen;          // generic pointer to the same byte
  uint32_t bar;          // first barrier
  __device__ uint32_t fixed(int t) const { return base + t * BTILE_BYTES; }                       // two stationary tiles
  __device__ uint32_t stream(int s, int t) const { return base + (2 + 2 * s + t) * BTILE_BYTES; }  // stage s, tile t
};

constexpr int BWD_TILES = 2 + 2 * BWD_NST;
// barrier indices
constexpr int BB_FIXED = 0;                 // stationary tiles landed
constexpr int BB_FULL = 1;                  // + s
constexpr int BB_EMPTY = 1 + BWD_NST;       // + s
// The score tile is handled as two 64-column halves, one per element-wise warpgroup, each with its own pair of
// barriers: while a warpgroup turns its half into P / dS the tensor pipe runs the other half's products, and a
// half's next scores are issued as soon as the gradient products that read its P / dS have been issued.
constexpr int BB_S = 1 + 2 * BWD_NST;       // + half: scores of that half ready (tcgen05.commit)
constexpr int BB_P = 3 + 2 * BWD_NST;       // + half: P / dS of that half written (128 arrivals)
constexpr int BB_DONE = 5 + 2 * BWD_NST;    // accumulators final
constexpr int BB_COUNT = 6 + 2 * BWD_NST;
constexpr uint32_t HALF_ROWS_DESC = (64 * 128) >> 4;  // descriptor offset of rows 64.. of a K-major tile

__device__ __forceinline__ BwdSmem bwd_smem_setup(uint8_t* raw) {
  BwdSmem s;
  s.base = (smem_u32(raw) + 1023u) & ~1023u;
  s.gen = raw + (s.base - smem_u32(raw));
  s.bar = s.base + BWD_TILES * BTILE_BYTES + 4 * BT * 4;
  return s;
}

__device__ __forceinline__ void bwd_init_barriers(const BwdSmem& sm, volatile int* abort_flag) {
  mbar_init(sm.bar + 8u * BB_FIXED, 1);
  for (int s = 0; s < BWD_NST; ++s) {
    mbar_init(sm.bar + 8u * (BB_FULL + s), 1);
    mbar_init(sm.bar + 8u * (BB_EMPTY + s), 1);
  }
  mbar_init(sm.bar + 8u * BB_S, 1);
  mbar_init(sm.bar + 8u * (BB_S + 1), 1);
  mbar_init(sm.bar + 8u * BB_P, 128);
  mbar_init(sm.bar + 8u * (BB_P + 1), 128);
  mbar_init(sm.bar + 8u * BB_DONE, 1);
  *abort_flag = 0;
  fence_barrier_init();
}

// Loads one 128 x 128 tile (two 64-column halves) of a [B, S, H, 128] tensor.
__device__ __forceinline__ void bwd_load_tile(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int head, int row0,
                                              int batch) {
  tma_load_4d(dst, tm, bar, 0, head, row0, batch);
  tma_load_4d(dst + BHALF_BYTES, tm, bar, 64, head, row0, batch);
}

// The producer's exit path after a failed wait: its own copies in flight must land before the
// CTA's shared memory is released.
__device__ __forceinline__ void bwd_drain(const BwdSmem& sm, bool fixed_issued, int issued) {
  volatile int no_abort = 0;
  if (fixed_issued) mbar_wait(sm.bar + 8u * BB_FIXED, 0, &no_abort, nullptr, 0);
  const int first = issued > BWD_NST ? issued - BWD_NST : 0;
  for (int i = first; i < issued; ++i)
    mbar_wait(sm.bar + 8u * (BB_FULL + i % BWD_NST), (i / BWD_NST) & 1, &no_abort, nullptr, 0);
}

// fp32 accumulator row (this thread's TMEM lane, columns [c_begin, c_end) at `taddr`) -> bf16 at dst.
__device__ __forceinline__ void bwd_store_row(uint32_t taddr, bf16* dst, bool row_ok, int c_begin, int c_end) {
#pragma unroll 1
  for (int c = c_begin; c < c_end; c += 32) {
    uint32_t o[32];
    tmem_ld32(taddr + c, o);
    tmem_wait_ld();
    if (row_ok) {
      uint4* d4 = reinterpret_cast<uint4*>(dst + c);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 v;
        v.x = pack_bf16(__uint_as_float(o[q * 8 + 0]), __uint_as_float(o[q * 8 + 1]));
        v.y = pack_bf16(__uint_as_float(o[q * 8 + 2]), __uint_as_float(o[q * 8 + 3]));
        v.z = pack_bf16(__uint_as_float(o[q * 8 + 4]), __uint_as_float(o[q * 8 + 5]));
        v.w = pack_bf16(__uint_as_float(o[q * 8 + 6]), __uint_as_float(o[q * 8 + 7]));
        d4[q] = v;
      }
    }
  }
}

// ====================================================================== dK / dV
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                           const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                           const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const BwdSmem sm = bwd_smem_setup(smem_raw);
  float* lse_s = reinterpret_cast<float*>(sm.gen + BWD_TILES * BTILE_BYTES);  // [2][128]
  float* dlt_s = lse_s + 2 * BT;                                              // [2][128]
  const uint32_t tmem_slot = sm.bar + 8u * BB_COUNT;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(sm.gen + BWD_TILES * BTILE_BYTES + 4 * BT * 4 + 8 * BB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot_ptr + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv0 = blockIdx.x * BT, kvh = blockIdx.y, batch = blockIdx.z;
  const int n_qt_all = (p.Sq + BT - 1) / BT;
  // leading query tiles that the mask removes completely for this K/V tile
  int i0 = 0;
  if (p.mask == MASK_CAUSAL) i0 = max(0, kv0 - (p.Skv - p.Sq)) / BT;
  if (p.mask == MASK_MOT) i0 = min(p.n_ar, kv0) / BT;
  i0 = min(i0, n_qt_all);
  const int n_qt = n_qt_all - i0;
  const int n_it = n_qt * p.group;

  if (threadIdx.x == 0) {
    bwd_init_barriers(sm, abort_flag);
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmdO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t T_ST = tmem_base, T_DPT = tmem_base + 128, T_DV = tmem_base + 256, T_DK = tmem_base + 384;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer
    bool fixed_issued = false;
    int issued = 0;
    bool ok = true;
    if (n_it > 0) {
      mbar_arrive_expect_tx(sm.bar + 8u * BB_FIXED, 2 * BTILE_BYTES);
      bwd_load_tile(sm.fixed(0), &tmK, sm.bar + 8u * BB_FIXED, kvh, kv0, batch);
      bwd_load_tile(sm.fixed(1), &tmV, sm.bar + 8u * BB_FIXED, kvh, kv0, batch);
      fixed_issued = true;
    }
    for (int it = 0; it < n_it; ++it) {
      const int s = it % BWD_NST;
      if (!mbar_wait(sm.bar + 8u * (BB_EMPTY + s), ((it / BWD_NST) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMA)) {
        ok = false;
        break;
      }
      const int head = kvh * p.group + it / n_qt;
      const int q0 = (i0 + it % n_qt) * BT;
      const uint32_t full = sm.bar + 8u * (BB_FULL + s);
      mbar_arrive_expect_tx(full, 2 * BTILE_BYTES);
      bwd_load_tile(sm.stream(s, 0), &tmQ, full, head, q0, batch);
      bwd_load_tile(sm.stream(s, 1), &tmdO, full, head, q0, batch);
      issued = it + 1;
    }
    if (!ok) bwd_drain(sm, fixed_issued, issued);
  } else if (warp == 1) {
    // ---------------- MMA issuer: the whole warp walks the loop (barrier phases and descriptors are warp-uniform
    // values), one elected lane issues the tcgen05 instructions
    const bool issuer = elect_one();
    auto wait_all = [&](uint32_t bar, uint32_t phase) {
      return __all_sync(0xffffffffu, mbar_wait(bar, phase, abort_flag, p.status, ST_TIMEOUT_MMA)) != 0;
    };
    constexpr uint32_t idesc_ss = make_idesc_bf16(BT, 64, 0, 0);   // one 64-column half of the score tile
    constexpr uint32_t idesc_ts = make_idesc_bf16(BT, 128, 0, 1);
    const uint64_t k_desc = make_smem_desc_sw128(sm.fixed(0), 16, 1024);
    const uint64_t v_desc = make_smem_desc_sw128(sm.fixed(1), 16, 1024);
    // S^T and dP^T of query columns [64 h, 64 h + 64) of the tile pair in stage st
    auto scores = [&](int st, int h) {
      const uint64_t q_k = make_smem_desc_sw128(sm.stream(st, 0), 16, 1024) + uint64_t(h * HALF_ROWS_DESC);
      const uint64_t do_k = make_smem_desc_sw128(sm.stream(st, 1), 16, 1024) + uint64_t(h * HALF_ROWS_DESC);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * (BHALF_BYTES >> 4) + 2 * (kk & 3);
        mma_ss(T_ST + 64 * h, k_desc + off, q_k + off, idesc_ss, kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * (BHALF_BYTES >> 4) + 2 * (kk & 3);
        mma_ss(T_DPT + 64 * h, v_desc + off, do_k + off, idesc_ss, kk > 0 ? 1u : 0u);
      }
      tc_commit(sm.bar + 8u * (BB_S + h));
    };
    // dV += P^T dO and dK += dS^T Q over the 64 queries of half h (bf16 P^T / dS^T of those columns sit at
    // 32-bit columns [64 h, 64 h + 32) of the score buffers)
    auto grads = [&](int st, int h, bool first) {
      const uint64_t q_mn = make_smem_desc_sw128(sm.stream(st, 0), BHALF_BYTES, 1024);
      const uint64_t do_mn = make_smem_desc_sw128(sm.stream(st, 1), BHALF_BYTES, 1024);
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        const int kk = 4 * h + k4;
        mma_ts(T_DV, T_ST + h * 64 + k4 * 8, do_mn + uint64_t(kk * (2048 >> 4)), idesc_ts, (first && k4 == 0) ? 0u : 1u);
      }
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        const int kk = 4 * h + k4;
        mma_ts(T_DK, T_DPT + h * 64 + k4 * 8, q_mn + uint64_t(kk * (2048 >> 4)), idesc_ts, (first && k4 == 0) ? 0u : 1u);
      }
    };
    bool ok = n_it == 0 || wait_all(sm.bar + 8u * BB_FIXED, 0);
    if (ok && n_it > 0) {
      ok = wait_all(sm.bar + 8u * BB_FULL, 0);
      if (ok) {
        tc_fence_after();
        if (issuer) {
          scores(0, 0);
          scores(0, 1);
        }
        __syncwarp();
      }
    }
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it % BWD_NST;
      const bool more = it + 1 < n_it;
      const int sn = (it + 1) % BWD_NST;
      if (more) {
        ok = wait_all(sm.bar + 8u * (BB_FULL + sn), ((it + 1) / BWD_NST) & 1);
        if (!ok) break;
      }
      ok = wait_all(sm.bar + 8u * BB_P, it & 1);
      if (!ok) break;
      tc_fence_after();
      if (issuer) {
        grads(s, 0, it == 0);
        if (more) scores(sn, 0);   // in issue order behind the products that read this half's P^T / dS^T
      }
      __syncwarp();
      ok = wait_all(sm.bar + 8u * (BB_P + 1), it & 1);
      if (!ok) break;
      tc_fence_after();
      if (issuer) {
        grads(s, 1, false);
        tc_commit(sm.bar + 8u * (BB_EMPTY + s));
        if (more) scores(sn, 1);
      }
      __syncwarp();
    }
    if (ok && n_it > 0 && issuer) tc_commit(sm.bar + 8u * BB_DONE);
    __syncwarp();
  } else if (warp >= 4) {
    // ---------------- element-wise math: this thread owns K/V row kv0 + r (TMEM lane r)
    const int quad = warp & 3;
    const int wg = (warp - 4) >> 2;  // which 64-column half of the score tile
    const int r = quad * 32 + lane;
    const int kv = kv0 + r;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int head = kvh * p.group + it / n_qt;
      const int q0 = (i0 + it % n_qt) * BT;
      const int buf = it & 1;
      if (r < 64) {
        // log-sum-exp and D of this warpgroup's 64 query columns (double-buffered; the warpgroup's own barrier
        // of the next iteration separates the reads of this buffer from its rewrite two iterations later)
        const int qc = 64 * wg + r;
        const int qi = q0 + qc;
        const long long off = ((long long)batch * p.Hq + head) * p.Sq + qi;
        lse_s[buf * BT + qc] = qi < p.Sq ? p.lse[off] * 1.4426950408889634f : INFINITY;
        dlt_s[buf * BT + qc] = qi < p.Sq ? p.delta[off] : 0.f;
      }
      named_bar_sync(1 + wg, 128);
      if (!mbar_wait(sm.bar + 8u * (BB_S + wg), it & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool need_mask = bwd_tile_needs_mask(kv0, q0, p);
      const float* ls = lse_s + buf * BT;
      const float* dl = dlt_s + buf * BT;
      {
        const int c = wg;  // this warpgroup's 64 query columns
        uint32_t pk[32], dsk[32];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int col0 = c * 64 + hh * 32;
          uint32_t s[32], dp[32];
          tmem_ld32(T_ST + lane_addr + col0, s);
          tmem_ld32(T_DPT + lane_addr + col0, dp);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int col = col0 + 2 * i;
            const float2 l2 = *reinterpret_cast<const float2*>(ls + col);
            const float2 d2 = *reinterpret_cast<const float2*>(dl + col);
            float p0 = bwd_ex2(fmaf(__uint_as_float(s[2 * i]), p.scale_log2, -l2.x));
            float p1 = bwd_ex2(fmaf(__uint_as_float(s[2 * i + 1]), p.scale_log2, -l2.y));
            if (need_mask) {
              if (bwd_masked(kv, q0 + col, p)) p0 = 0.f;
              if (bwd_masked(kv, q0 + col + 1, p)) p1 = 0.f;
            }
            const float ds0 = p0 * (__uint_as_float(dp[2 * i]) - d2.x) * p.scale;
            const float ds1 = p1 * (__uint_as_float(dp[2 * i + 1]) - d2.y) * p.scale;
            pk[hh * 16 + i] = pack_bf16(p0, p1);
            dsk[hh * 16 + i] = pack_bf16(ds0, ds1);
          }
        }
        // bf16 P^T / dS^T alias the fp32 scores: the 64 columns of this warpgroup become 32 32-bit
        // columns at 64 * c, which only covers score columns that this thread already holds
        tmem_st32(T_ST + lane_addr + 64 * c, pk);
        tmem_st32(T_DPT + lane_addr + 64 * c, dsk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(sm.bar + 8u * (BB_P + wg));
    }
    const bool row_ok = kv < p.Skv;
    bf16* dk_row = p.dK + (((long long)batch * p.Skv + kv) * p.Hkv + kvh) * 128;
    bf16* dv_row = p.dV + (((long long)batch * p.Skv + kv) * p.Hkv + kvh) * 128;
    if (n_it == 0) {
      if (row_ok) {
        for (int c = 0; c < 16; ++c) reinterpret_cast<uint4*>(wg == 0 ? dv_row : dk_row)[c] = make_uint4(0, 0, 0, 0);
      }
    } else {
      if (ok) ok = mbar_wait(sm.bar + 8u * BB_DONE, 0, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
      if (ok) {
        tc_fence_after();
        // one accumulator per warpgroup
        if (wg == 0) bwd_store_row(T_DV + lane_addr, dv_row, row_ok, 0, 128);
        else bwd_store_row(T_DK + lane_addr, dk_row, row_ok, 0, 128);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ====================================================================== dQ
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                         const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const BwdSmem sm = bwd_smem_setup(smem_raw);
  const uint32_t tmem_slot = sm.bar + 8u * BB_COUNT;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(sm.gen + BWD_TILES * BTILE_BYTES + 4 * BT * 4 + 8 * BB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot_ptr + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BT, head = blockIdx.y, batch = blockIdx.z;
  const int kvh = head / p.group;
  int n_blocks;
  {
    const int last_row = min(p.Sq - 1, q0 + BT - 1);
    int lim = p.Skv;
    if (p.mask == MASK_CAUSAL) lim = min(p.Skv, last_row + 1 + (p.Skv - p.Sq));
    if (p.mask == MASK_MOT) lim = (last_row >= p.n_ar) ? p.Skv : last_row + 1;
    n_blocks = (max(lim, 1) + BT - 1) / BT;
  }

  if (threadIdx.x == 0) {
    bwd_init_barriers(sm, abort_flag);
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmdO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t T_S = tmem_base, T_DP = tmem_base + 128, T_DQ = tmem_base + 256;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer
    int issued = 0;
    bool ok = true;
    mbar_arrive_expect_tx(sm.bar + 8u * BB_FIXED, 2 * BTILE_BYTES);
    bwd_load_tile(sm.fixed(0), &tmQ, sm.bar + 8u * BB_FIXED, head, q0, batch);
    bwd_load_tile(sm.fixed(1), &tmdO, sm.bar + 8u * BB_FIXED, head, q0, batch);
    for (int j = 0; j < n_blocks; ++j) {
      const int s = j % BWD_NST;
      if (!mbar_wait(sm.bar + 8u * (BB_EMPTY + s), ((j / BWD_NST) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMA)) {
        ok = false;
        break;
      }
      const uint32_t full = sm.bar + 8u * (BB_FULL + s);
      mbar_arrive_expect_tx(full, 2 * BTILE_BYTES);
      bwd_load_tile(sm.stream(s, 0), &tmK, full, kvh, j * BT, batch);
      bwd_load_tile(sm.stream(s, 1), &tmV, full, kvh, j * BT, batch);
      issued = j + 1;
    }
    if (!ok) bwd_drain(sm, true, issued);
  } else if (warp == 1) {
    // ---------------- MMA issuer (whole warp walks the loop, one elected lane issues)
    const bool issuer = elect_one();
    auto wait_all = [&](uint32_t bar, uint32_t phase) {
      return __all_sync(0xffffffffu, mbar_wait(bar, phase, abort_flag, p.status, ST_TIMEOUT_MMA)) != 0;
    };
    constexpr uint32_t idesc_ss = make_idesc_bf16(BT, 64, 0, 0);   // one 64-key half of the score tile
    constexpr uint32_t idesc_ts = make_idesc_bf16(BT, 128, 0, 1);
    const uint64_t q_desc = make_smem_desc_sw128(sm.fixed(0), 16, 1024);
    const uint64_t do_desc = make_smem_desc_sw128(sm.fixed(1), 16, 1024);
    // S and dP against keys [64 h, 64 h + 64) of the K/V tiles in stage st
    auto scores = [&](int st, int h) {
      const uint64_t k_k = make_smem_desc_sw128(sm.stream(st, 0), 16, 1024) + uint64_t(h * HALF_ROWS_DESC);
      const uint64_t v_k = make_smem_desc_sw128(sm.stream(st, 1), 16, 1024) + uint64_t(h * HALF_ROWS_DESC);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * (BHALF_BYTES >> 4) + 2 * (kk & 3);
        mma_ss(T_S + 64 * h, q_desc + off, k_k + off, idesc_ss, kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * (BHALF_BYTES >> 4) + 2 * (kk & 3);
        mma_ss(T_DP + 64 * h, do_desc + off, v_k + off, idesc_ss, kk > 0 ? 1u : 0u);
      }
      tc_commit(sm.bar + 8u * (BB_S + h));
    };
    // dQ += dS K over the 64 keys of half h
    auto grads = [&](int st, int h, bool first) {
      const uint64_t k_mn = make_smem_desc_sw128(sm.stream(st, 0), BHALF_BYTES, 1024);
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        const int kk = 4 * h + k4;
        mma_ts(T_DQ, T_S + h * 64 + k4 * 8, k_mn + uint64_t(kk * (2048 >> 4)), idesc_ts, (first && k4 == 0) ? 0u : 1u);
      }
    };
    bool ok = wait_all(sm.bar + 8u * BB_FIXED, 0);
    if (ok) {
      ok = wait_all(sm.bar + 8u * BB_FULL, 0);
      if (ok) {
        tc_fence_after();
        if (issuer) {
          scores(0, 0);
          scores(0, 1);
        }
        __syncwarp();
      }
    }
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int s = j % BWD_NST;
      const bool more = j + 1 < n_blocks;
      const int sn = (j + 1) % BWD_NST;
      if (more) {
        ok = wait_all(sm.bar + 8u * (BB_FULL + sn), ((j + 1) / BWD_NST) & 1);
        if (!ok) break;
      }
      ok = wait_all(sm.bar + 8u * BB_P, j & 1);
      if (!ok) break;
      tc_fence_after();
      if (issuer) {
        grads(s, 0, j == 0);
        if (more) scores(sn, 0);
      }
      __syncwarp();
      ok = wait_all(sm.bar + 8u * (BB_P + 1), j & 1);
      if (!ok) break;
      tc_fence_after();
      if (issuer) {
        grads(s, 1, false);
        tc_commit(sm.bar + 8u * (BB_EMPTY + s));
        if (more) scores(sn, 1);
      }
      __syncwarp();
    }
    if (ok && issuer) tc_commit(sm.bar + 8u * BB_DONE);
    __syncwarp();
  } else if (warp >= 4) {
    // ---------------- element-wise math: this thread owns query row q0 + r (TMEM lane r)
    const int quad = warp & 3;
    const int wg = (warp - 4) >> 2;  // which 64-column half of the score tile
    const int r = quad * 32 + lane;
    const int qi = q0 + r;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    const bool row_ok = qi < p.Sq;
    const long long off = ((long long)batch * p.Hq + head) * p.Sq + qi;
    const float lse2 = row_ok ? p.lse[off] * 1.4426950408889634f : INFINITY;
    const float dlt = row_ok ? p.delta[off] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      if (!mbar_wait(sm.bar + 8u * (BB_S + wg), j & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int kv0 = j * BT;
      const bool need_mask = bwd_tile_needs_mask(kv0, q0, p);
      {
        const int c = wg;  // this warpgroup's 64 key columns
        uint32_t dsk[32];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int col0 = c * 64 + hh * 32;
          uint32_t s[32], dp[32];
          tmem_ld32(T_S + lane_addr + col0, s);
          tmem_ld32(T_DP + lane_addr + col0, dp);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int col = col0 + 2 * i;
            float p0 = bwd_ex2(fmaf(__uint_as_float(s[2 * i]), p.scale_log2, -lse2));
            float p1 = bwd_ex2(fmaf(__uint_as_float(s[2 * i + 1]), p.scale_log2, -lse2));
            if (need_mask) {
              if (bwd_masked(kv0 + col, qi, p)) p0 = 0.f;
              if (bwd_masked(kv0 + col + 1, qi, p)) p1 = 0.f;
            }
            const float ds0 = p0 * (__uint_as_float(dp[2 * i]) - dlt) * p.scale;
            const float ds1 = p1 * (__uint_as_float(dp[2 * i + 1]) - dlt) * p.scale;
            dsk[hh * 16 + i] = pack_bf16(ds0, ds1);
          }
        }
        tmem_st32(T_S + lane_addr + 64 * c, dsk);  // bf16 dS aliases score columns this thread already holds
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(sm.bar + 8u * (BB_P + wg));
    }
    if (ok) ok = mbar_wait(sm.bar + 8u * BB_DONE, 0, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
    if (ok) {
      tc_fence_after();
      bf16* dq_row = p.dQ + (((long long)batch * p.Sq + qi) * p.Hq + head) * 128;
      bwd_store_row(T_DQ + lane_addr, dq_row, row_ok, 64 * wg, 64 * wg + 64);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace cb

namespace cosmos {

static CUtensorMap bwd_map(const void* base, int B, int S, int H, long long sb, long long ss, long long sh) {
  const uint64_t dims[4] = {128, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)sh * 2, (uint64_t)ss * 2, (uint64_t)(sb > 0 ? sb : ss * S) * 2};
  const uint32_t box[4] = {64, 1, 128, 1};
  return cbh::make_tmap_bf16(base, 4, dims, strides, box, true);
}

void flash_attn_bwd(const AttnBwdArgs& a, cudaStream_t stream) {
  if (a.Hkv <= 0 || a.Hq % a.Hkv != 0) throw std::runtime_error("flash_attn_bwd: Hq % Hkv != 0");
  if (a.Sq <= 0 || a.Skv <= 0 || a.B <= 0) return;
  if (a.mask == MASK_CAUSAL && a.Skv < a.Sq) throw std::runtime_error("flash_attn_bwd: causal mask needs Skv >= Sq");
  if (a.mask == MASK_MOT && a.Skv != a.Sq) throw std::runtime_error("flash_attn_bwd: MoT mask needs Skv == Sq");
  static thread_local bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(cb::flash_attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, cb::BWD_SMEM);
    cudaFuncSetAttribute(cb::flash_attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, cb::BWD_SMEM);
    configured = true;
  }
  CUtensorMap tq = bwd_map(a.Q, a.B, a.Sq, a.Hq, a.q_stride_b, a.q_stride_s, a.q_stride_h);
  CUtensorMap tk = bwd_map(a.K, a.B, a.Skv, a.Hkv, a.k_stride_b, a.k_stride_s, a.k_stride_h);
  CUtensorMap tv = bwd_map(a.V, a.B, a.Skv, a.Hkv, a.v_stride_b, a.v_stride_s, a.v_stride_h);
  CUtensorMap tdo = bwd_map(a.dO, a.B, a.Sq, a.Hq, a.do_stride_b, a.do_stride_s, a.do_stride_h);
  cb::AttnBwdParams p{};
  p.Sq = a.Sq; p.Skv = a.Skv; p.Hq = a.Hq; p.Hkv = a.Hkv; p.group = a.Hq / a.Hkv;
  p.mask = a.mask; p.n_ar = a.n_ar;
  p.scale = a.scale; p.scale_log2 = a.scale * 1.4426950408889634f;
  p.lse = a.lse; p.delta = a.delta;
  p.dQ = reinterpret_cast<bf16*>(a.dQ); p.dK = reinterpret_cast<bf16*>(a.dK); p.dV = reinterpret_cast<bf16*>(a.dV);
  p.status = a.status;
  dim3 grid_kv((a.Skv + cb::BT - 1) / cb::BT, a.Hkv, a.B);
  cb::flash_attn_bwd_dkdv_kernel<<<grid_kv, cb::BWD_THREADS, cb::BWD_SMEM, stream>>>(tq, tk, tv, tdo, p);
  dim3 grid_q((a.Sq + cb::BT - 1) / cb::BT, a.Hq, a.B);
  cb::flash_attn_bwd_dq_kernel<<<grid_q, cb::BWD_THREADS, cb::BWD_SMEM, stream>>>(tq, tk, tv, tdo, p);
}

}  // namespace cosmos
