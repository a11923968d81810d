// K7: flash attention forward (head_dim 128, bf16, GQA) on tcgen05 tensor cores.
//
// One CTA owns 256 query rows of one head as two 128-row tiles and streams 128-row K/V
// blocks through a 5-slot TMA ring. Both GEMMs of a block run on the tensor cores with
// accumulators in tensor memory (512 columns: S0 | S1 | O0 | O1):
//     S_t  = Q_t K_j^T                    (A, B from shared memory)
//     O_t += P_t V_j                      (A = P_t in tensor memory, aliasing S_t; B = V_j in smem)
// Warp roles (384 threads):
//     warp 0        TMA producer (Q once, then K_0, V_0, K_1, V_1, ...)
//     warp 1        MMA issuer (one thread); the two tiles are interleaved so that the
//                   tensor cores work on tile 1 while the softmax of tile 0 runs and vice versa
//     warps 4..7    softmax + output epilogue of tile 0 (one query row per thread)
//     warps 8..11   softmax + output epilogue of tile 1
// The running max is only refreshed (and O rescaled) when it grows by more than 2^8, so the
// rescale is rare and stays in the softmax warps; the final 1/l normalisation uses the same
// stale max, which keeps the result exact.
// Masks: full, causal, and the Mixture-of-Transformers block mask (AR rows causal over AR
// keys, DM rows see everything). Output rows can be routed to per-destination buffers
// (peer GPUs) to fuse the head->sequence all-to-all of Ulysses context parallelism.
#include "common.cuh"
#include "kernels.h"

namespace cb {

constexpr int ATT_THREADS = 384;
constexpr int TQ = 128, TKV = 128, HD = 128;
constexpr int NSLOT = 5;
constexpr int TILE_BYTES = TQ * HD * 2;        // 32 KB
constexpr int HALF_BYTES = TILE_BYTES / 2;     // one 64-column half, 16 KB
constexpr int ATT_SMEM = 2 * TILE_BYTES + NSLOT * TILE_BYTES + 1024 + 256;

struct AttnParams {
  int Sq, Skv, Hq, Hkv, group;  // group = Hq / Hkv
  int mask, n_ar;
  float scale_log2;  // softmax scale * log2(e)
  bf16* O;
  long long o_stride_b, o_stride_s, o_stride_h;
  float* lse;  // [B, Hq, Sq]
  const long long* dest_ptr;
  int rows_per_dest;
  int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// exp2 on the FMA/ALU pipes: round-to-nearest split x = n + f, f in [-0.5, 0.5], degree-3 minimax
// polynomial for 2^f (max relative error 7.5e-5, far below bf16 rounding of P), exponent add for 2^n.
// Used for a fixed share of the softmax elements to take load off the 16-lane MUFU pipe, which
// otherwise needs as many cycles per score tile as the tensor cores.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -126.f);
  const float magic = 12582912.f;  // 1.5 * 2^23: the integer part lands in the low mantissa bits
  const float t = x + magic;
  const float n = t - magic;
  const float f = x - n;
  float p = fmaf(0.0551716648f, f, 0.2426111251f);
  p = fmaf(p, f, 0.6932609677f);
  p = fmaf(p, f, 0.9999280572f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

template <int EMU>
__device__ __forceinline__ float ex2_mix(float x, int i) {
  if (EMU > 0 && (i % EMU) == EMU - 1) return ex2_poly(x);
  return ex2(x);
}

__device__ __forceinline__ int kv_limit(int qi, const AttnParams& p) {
  if (p.mask == MASK_CAUSAL) return min(p.Skv, qi + 1 + (p.Skv - p.Sq));
  if (p.mask == MASK_MOT) return qi < p.n_ar ? qi + 1 : p.Skv;
  return p.Skv;
}

template <int EMU>
__global__ void __launch_bounds__(ATT_THREADS, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;
  const uint32_t kv_smem = smem_base + 2 * TILE_BYTES;
  const uint32_t bar_base = kv_smem + NSLOT * TILE_BYTES;
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + NSLOT + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (1 + 2 * NSLOT + t); };
  auto p_full = [&](int t, int h) { return bar_base + 8u * (3 + 2 * NSLOT + 2 * t + h); };
  auto o_final = [&](int t) { return bar_base + 8u * (7 + 2 * NSLOT + t); };
  constexpr int NBAR = 9 + 2 * NSLOT;
  const uint32_t tmem_slot = bar_base + 8u * NBAR;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(gen_base + 7 * TILE_BYTES + 8 * NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + 7 * TILE_BYTES + 8 * NBAR + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = (p.mask == MASK_FULL) ? blockIdx.x : (gridDim.x - 1 - blockIdx.x);
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / p.group;
  const int q0 = qt * 2 * TQ;

  // Number of K/V blocks this CTA visits.
  int n_blocks;
  {
    const int last_row = min(p.Sq - 1, q0 + 2 * TQ - 1);
    int lim = p.Skv;
    if (p.mask == MASK_CAUSAL) lim = kv_limit(last_row, p);
    if (p.mask == MASK_MOT) lim = (last_row >= p.n_ar) ? p.Skv : last_row + 1;
    n_blocks = (max(lim, 1) + TKV - 1) / TKV;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t, 0), 128);
      mbar_init(p_full(t, 1), 128);
      mbar_init(o_final(t), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // Register re-partitioning: the CTA owns 384 x 168 registers; 128 x 56 + 256 x 224 uses
  // exactly that many. A split that needs more would block in setmaxnreg.inc forever.
  static_assert(128 * 56 + 256 * 224 <= ATT_THREADS * 168, "setmaxnreg split exceeds the CTA's registers");
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0 && lane == 0) {
      // ---------------- TMA producer
      mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_4d(q_smem + t * TILE_BYTES + h * HALF_BYTES, &tmQ, q_full, h * 64, head,
                      q0 + t * TQ, batch);
      int issued = 0;
      bool ok = true;
      for (int i = 0; i < 2 * n_blocks; ++i) {
        const int s = i % NSLOT;
        const uint32_t ph = (i / NSLOT) & 1;
        if (!mbar_wait(kv_empty(s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMA)) {
          ok = false;
          break;
        }
        const int j = i >> 1;
        const CUtensorMap* tm = (i & 1) ? &tmV : &tmK;
        const uint32_t dst = kv_smem + s * TILE_BYTES;
        mbar_arrive_expect_tx(kv_full(s), TILE_BYTES);
        tma_load_4d(dst, tm, kv_full(s), 0, kv_head, j * TKV, batch);
        tma_load_4d(dst + HALF_BYTES, tm, kv_full(s), 64, kv_head, j * TKV, batch);
        issued = i + 1;
      }
      if (!ok) {
        volatile int no_abort = 0;
        mbar_wait(q_full, 0, &no_abort, nullptr, 0);
        const int first = issued > NSLOT ? issued - NSLOT : 0;
        for (int i = first; i < issued; ++i)
          mbar_wait(kv_full(i % NSLOT), (i / NSLOT) & 1, &no_abort, nullptr, 0);
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer
      constexpr uint32_t idesc_qk = make_idesc_bf16(TQ, TKV, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(TQ, HD, 0, 1);
      // Descriptors differ only in their 14-bit start-address field, so they are built as
      // one 64-bit constant plus a small address offset (in 16-byte units).
      const uint64_t q_desc0 = make_smem_desc_sw128(q_smem, 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(kv_smem, 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(kv_smem, HALF_BYTES, 1024);
      auto issue_qk = [&](int t, int slot) {
        const uint32_t d = tmem_base + t * 128;
        const uint64_t a0 = q_desc0 + uint64_t(t * (TILE_BYTES >> 4));
        const uint64_t b0 = k_desc0 + uint64_t(slot * (TILE_BYTES >> 4));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * (HALF_BYTES >> 4) + 2 * (kk & 3);
          mma_ss(d, a0 + off, b0 + off, idesc_qk, kk > 0 ? 1u : 0u);
        }
      };
      // P is handed over in two halves of 64 keys, so the first four k-steps of PV run while the
      // softmax warps still compute the exponentials of the second half.
      auto issue_pv = [&](int t, int slot, bool acc, int half) {
        const uint32_t d = tmem_base + 256 + t * 128;
        const uint32_t a0 = tmem_base + t * 128;
        const uint64_t b0 = v_desc0 + uint64_t(slot * (TILE_BYTES >> 4));
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const int kk = half * 4 + k4;
          mma_ts(d, a0 + kk * 8, b0 + uint64_t(kk * (2048 >> 4)), idesc_pv, (acc || kk > 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok) ok = mbar_wait(kv_full(0), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        tc_commit(s_full(0));
        issue_qk(1, 0);
        tc_commit(s_full(1));
        tc_commit(kv_empty(0));
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int iv = 2 * j + 1, ik = 2 * j + 2;
        const int sv = iv % NSLOT, sk = ik % NSLOT;
        const bool more = (j + 1 < n_blocks);
        ok = mbar_wait(kv_full(sv), (iv / NSLOT) & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (ok && more)
          ok = mbar_wait(kv_full(sk), (ik / NSLOT) & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (!ok) break;
#pragma unroll 1
        for (int t = 0; t < 2; ++t) {
          ok = mbar_wait(p_full(t, 0), j & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_pv(t, sv, j > 0, 0);
          ok = mbar_wait(p_full(t, 1), j & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_pv(t, sv, j > 0, 1);
          if (more) {
            issue_qk(t, sk);
            tc_commit(s_full(t));
          } else {
            tc_commit(o_final(t));
          }
        }
        if (!ok) break;
        tc_commit(kv_empty(sv));
        if (more) tc_commit(kv_empty(sk));
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ---------------- softmax + epilogue, one query row per thread
    const int t = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int qi = q0 + t * TQ + row;
    const int limit = kv_limit(min(qi, p.Sq - 1), p);
    const uint32_t lane_addr = tmem_base + (uint32_t(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + t * 128;
    const uint32_t o_addr = lane_addr + 256 + t * 128;
    const float sl2 = p.scale_log2;
    float m_used = -1e30f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      if (!mbar_wait(s_full(t), j & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[128];
      tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld32(s_addr + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
      tmem_ld32(s_addr + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
      tmem_wait_ld();
      const int kv0 = j * TKV;
      if (kv0 + TKV > limit) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (kv0 + i >= limit) s[i] = 0xff800000u;  // -inf
      }
      float mx = __uint_as_float(s[0]);
#pragma unroll
      for (int i = 1; i < 128; ++i) mx = fmaxf(mx, __uint_as_float(s[i]));
      const float m_new = fmaxf(m_used, mx * sl2);
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool need = m_new > m_used + 8.f;
        if (__any_sync(0xffffffffu, need)) {
          const float sc = need ? ex2(m_used - m_new) : 1.f;
#pragma unroll 1
          for (int c = 0; c < 128; c += 32) {
            uint32_t o[32];
            tmem_ld32(o_addr + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * sc);
            tmem_st32(o_addr + c, o);
          }
          tmem_wait_st();
          l *= sc;
          if (need) m_used = m_new;
        }
      }
      float lsum = 0.f;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int e = half * 64 + 2 * i;
          const float p0 = ex2_mix<EMU>(fmaf(__uint_as_float(s[e]), sl2, -m_used), e);
          const float p1 = ex2_mix<EMU>(fmaf(__uint_as_float(s[e + 1]), sl2, -m_used), e + 1);
          lsum += p0 + p1;
          pk[i] = pack_bf16(p0, p1);
        }
        tmem_st32(s_addr + half * 32, pk);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(p_full(t, half));
      }
      l += lsum;
    }
    if (ok) ok = mbar_wait(o_final(t), 0, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qi < p.Sq;
      bf16* dst = nullptr;
      if (row_ok) {
        if (p.dest_ptr) {
          const int r = qi / p.rows_per_dest;
          dst = reinterpret_cast<bf16*>(p.dest_ptr[r]) + (long long)batch * p.o_stride_b +
                (long long)(qi - r * p.rows_per_dest) * p.o_stride_s + (long long)head * p.o_stride_h;
        } else {
          dst = p.O + (long long)batch * p.o_stride_b + (long long)qi * p.o_stride_s +
                (long long)head * p.o_stride_h;
        }
        if (p.lse)
          p.lse[((long long)batch * p.Hq + head) * p.Sq + qi] =
              l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t o[32];
        tmem_ld32(o_addr + c, o);
        tmem_wait_ld();
        if (row_ok) {
          uint4* d4 = reinterpret_cast<uint4*>(dst + c);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[q * 8 + 0]) * inv, __uint_as_float(o[q * 8 + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(o[q * 8 + 2]) * inv, __uint_as_float(o[q * 8 + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(o[q * 8 + 4]) * inv, __uint_as_float(o[q * 8 + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(o[q * 8 + 6]) * inv, __uint_as_float(o[q * 8 + 7]) * inv);
            d4[q] = v;
          }
        }
      }
    }
  }

  // ---------------- common tail
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// Second-generation pipeline: keys are consumed in sub-blocks of 64 and every query tile has TWO
// score sub-buffers in tensor memory (columns [0,64) and [64,128) of its S region; the bf16
// probabilities of a sub-block alias the first 32 columns of the sub-buffer they came from).
// While the softmax warps work on sub-block b of a tile, the tensor cores already compute the
// scores of sub-block b+1 of the SAME tile into the other sub-buffer, and PV of sub-block b-1;
// the tile's own softmax -> PV -> next-QK dependency chain, which bounded the first-generation
// kernel at ~63 % tensor-pipe utilisation, is cut in half.
//   MMA issue order per sub-block b and tile t:  wait P_t(b) -> PV_t(b) -> QK_t(b+2) (same sub-buffer)
//   O rescale (rare, lazy) additionally waits for PV_t(b-1) through its own barrier.
__global__ void __launch_bounds__(ATT_THREADS, 1)
flash_attn_fwd_kernel_v2(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int SUB = 64;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;
  const uint32_t kv_smem = smem_base + 2 * TILE_BYTES;
  const uint32_t bar_base = kv_smem + NSLOT * TILE_BYTES;
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + NSLOT + s); };
  auto s_full = [&](int t, int u) { return bar_base + 8u * (1 + 2 * NSLOT + 2 * t + u); };
  auto p_full = [&](int t, int u) { return bar_base + 8u * (5 + 2 * NSLOT + 2 * t + u); };
  auto pv_done = [&](int t) { return bar_base + 8u * (9 + 2 * NSLOT + t); };
  auto o_final = [&](int t) { return bar_base + 8u * (11 + 2 * NSLOT + t); };
  constexpr int NBAR = 13 + 2 * NSLOT;
  const uint32_t tmem_slot = bar_base + 8u * NBAR;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(gen_base + 7 * TILE_BYTES + 8 * NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + 7 * TILE_BYTES + 8 * NBAR + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = (p.mask == MASK_FULL) ? blockIdx.x : (gridDim.x - 1 - blockIdx.x);
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / p.group;
  const int q0 = qt * 2 * TQ;

  int n_sub;
  {
    const int last_row = min(p.Sq - 1, q0 + 2 * TQ - 1);
    int lim = p.Skv;
    if (p.mask == MASK_CAUSAL) lim = kv_limit(last_row, p);
    if (p.mask == MASK_MOT) lim = (last_row >= p.n_ar) ? p.Skv : last_row + 1;
    n_sub = (max(lim, 1) + SUB - 1) / SUB;
  }
  const int n_blocks = (n_sub + 1) / 2;  // 128-row K/V tiles

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      for (int u = 0; u < 2; ++u) {
        mbar_init(s_full(t, u), 1);
        mbar_init(p_full(t, u), 128);
      }
      mbar_init(pv_done(t), 1);
      mbar_init(o_final(t), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  static_assert(128 * 56 + 256 * 224 <= ATT_THREADS * 168, "setmaxnreg split exceeds the CTA's registers");
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0 && lane == 0) {
      // ---------------- TMA producer (identical item order: K_0, V_0, K_1, V_1, ...)
      mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_4d(q_smem + t * TILE_BYTES + h * HALF_BYTES, &tmQ, q_full, h * 64, head,
                      q0 + t * TQ, batch);
      int issued = 0;
      bool ok = true;
      for (int i = 0; i < 2 * n_blocks; ++i) {
        const int s = i % NSLOT;
        const uint32_t ph = (i / NSLOT) & 1;
        if (!mbar_wait(kv_empty(s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMA)) {
          ok = false;
          break;
        }
        const int j = i >> 1;
        const CUtensorMap* tm = (i & 1) ? &tmV : &tmK;
        const uint32_t dst = kv_smem + s * TILE_BYTES;
        mbar_arrive_expect_tx(kv_full(s), TILE_BYTES);
        tma_load_4d(dst, tm, kv_full(s), 0, kv_head, j * TKV, batch);
        tma_load_4d(dst + HALF_BYTES, tm, kv_full(s), 64, kv_head, j * TKV, batch);
        issued = i + 1;
      }
      if (!ok) {
        volatile int no_abort = 0;
        mbar_wait(q_full, 0, &no_abort, nullptr, 0);
        const int first = issued > NSLOT ? issued - NSLOT : 0;
        for (int i = first; i < issued; ++i)
          mbar_wait(kv_full(i % NSLOT), (i / NSLOT) & 1, &no_abort, nullptr, 0);
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer
      constexpr uint32_t idesc_qk = make_idesc_bf16(TQ, SUB, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(TQ, HD, 0, 1);
      const uint64_t q_desc0 = make_smem_desc_sw128(q_smem, 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(kv_smem, 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(kv_smem, HALF_BYTES, 1024);
      // scores of sub-block b (keys [64 b, 64 b + 64)) of tile t into sub-buffer b & 1
      auto issue_qk = [&](int t, int b) {
        const int slot = (2 * (b >> 1)) % NSLOT;
        const uint32_t d = tmem_base + t * 128 + (b & 1) * SUB;
        const uint64_t a0 = q_desc0 + uint64_t(t * (TILE_BYTES >> 4));
        const uint64_t b0 = k_desc0 + uint64_t(slot * (TILE_BYTES >> 4) + (b & 1) * ((SUB * 128) >> 4));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * (HALF_BYTES >> 4) + 2 * (kk & 3);
          mma_ss(d, a0 + off, b0 + off, idesc_qk, kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int t, int b) {
        const int slot = (2 * (b >> 1) + 1) % NSLOT;
        const uint32_t d = tmem_base + 256 + t * 128;
        const uint32_t a0 = tmem_base + t * 128 + (b & 1) * SUB;
        const uint64_t b0 = v_desc0 + uint64_t(slot * (TILE_BYTES >> 4) + (b & 1) * ((SUB * 128) >> 4));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_ts(d, a0 + kk * 8, b0 + uint64_t(kk * (2048 >> 4)), idesc_pv, (b > 0 || kk > 0) ? 1u : 0u);
      };
      auto kv_item_wait = [&](int item) {
        return mbar_wait(kv_full(item % NSLOT), (item / NSLOT) & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok) ok = kv_item_wait(0);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t) {
          issue_qk(t, 0);
          tc_commit(s_full(t, 0));
        }
        if (n_sub > 1) {
          for (int t = 0; t < 2; ++t) {
            issue_qk(t, 1);
            tc_commit(s_full(t, 1));
          }
        }
        tc_commit(kv_empty(0));  // K tile 0 is not needed again
      }
      for (int b = 0; b < n_sub && ok; ++b) {
        const int u = b & 1, j = b >> 1;
        const int nb = b + 2;  // sub-block whose scores go into the sub-buffer that PV(b) frees
        if (u == 0) ok = kv_item_wait(2 * j + 1);                       // V tile j
        if (ok && nb < n_sub && (nb & 1) == 0) ok = kv_item_wait(2 * (nb >> 1));  // K tile of sub-block nb
        if (!ok) break;
#pragma unroll 1
        for (int t = 0; t < 2; ++t) {
          ok = mbar_wait(p_full(t, u), (b >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_pv(t, b);
          tc_commit(pv_done(t));
          if (nb < n_sub) {
            issue_qk(t, nb);
            tc_commit(s_full(t, u));
          }
          if (b == n_sub - 1) tc_commit(o_final(t));
        }
        if (!ok) break;
        if (u == 1 || b == n_sub - 1) tc_commit(kv_empty((2 * j + 1) % NSLOT));                    // V tile j done
        if (nb < n_sub && ((nb & 1) == 1 || nb == n_sub - 1)) tc_commit(kv_empty((2 * (nb >> 1)) % NSLOT));  // K tile done
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ---------------- softmax + epilogue, one query row per thread
    const int t = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int qi = q0 + t * TQ + row;
    const int limit = kv_limit(min(qi, p.Sq - 1), p);
    const uint32_t lane_addr = tmem_base + (uint32_t(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + t * 128;
    const uint32_t o_addr = lane_addr + 256 + t * 128;
    const float sl2 = p.scale_log2;
    float m_used = -1e30f, l = 0.f;
    bool ok = true;
    for (int b = 0; b < n_sub; ++b) {
      const int u = b & 1;
      if (!mbar_wait(s_full(t, u), (b >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[64];
      tmem_ld32(s_addr + u * SUB, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld32(s_addr + u * SUB + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_wait_ld();
      const int kv0 = b * SUB;
      if (kv0 + SUB > limit) {
#pragma unroll
        for (int i = 0; i < SUB; ++i)
          if (kv0 + i >= limit) s[i] = 0xff800000u;  // -inf
      }
      float mx = __uint_as_float(s[0]);
#pragma unroll
      for (int i = 1; i < SUB; ++i) mx = fmaxf(mx, __uint_as_float(s[i]));
      const float m_new = fmaxf(m_used, mx * sl2);
      if (b == 0) {
        m_used = m_new;
      } else {
        const bool need = m_new > m_used + 8.f;
        if (__any_sync(0xffffffffu, need)) {
          // PV of the previous sub-block may still be accumulating into O: wait for it first
          if (!mbar_wait(pv_done(t), (b - 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const float sc = need ? ex2(m_used - m_new) : 1.f;
#pragma unroll 1
          for (int c = 0; c < 128; c += 32) {
            uint32_t o[32];
            tmem_ld32(o_addr + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * sc);
            tmem_st32(o_addr + c, o);
          }
          tmem_wait_st();
          l *= sc;
          if (need) m_used = m_new;
        }
      }
      uint32_t pk[32];
      float lsum = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0 = ex2(fmaf(__uint_as_float(s[2 * i]), sl2, -m_used));
        const float p1 = ex2(fmaf(__uint_as_float(s[2 * i + 1]), sl2, -m_used));
        lsum += p0 + p1;
        pk[i] = pack_bf16(p0, p1);
      }
      l += lsum;
      tmem_st32(s_addr + u * SUB, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full(t, u));
    }
    if (ok) ok = mbar_wait(o_final(t), 0, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qi < p.Sq;
      bf16* dst = nullptr;
      if (row_ok) {
        if (p.dest_ptr) {
          const int r = qi / p.rows_per_dest;
          dst = reinterpret_cast<bf16*>(p.dest_ptr[r]) + (long long)batch * p.o_stride_b +
                (long long)(qi - r * p.rows_per_dest) * p.o_stride_s + (long long)head * p.o_stride_h;
        } else {
          dst = p.O + (long long)batch * p.o_stride_b + (long long)qi * p.o_stride_s +
                (long long)head * p.o_stride_h;
        }
        if (p.lse)
          p.lse[((long long)batch * p.Hq + head) * p.Sq + qi] =
              l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t o[32];
        tmem_ld32(o_addr + c, o);
        tmem_wait_ld();
        if (row_ok) {
          uint4* d4 = reinterpret_cast<uint4*>(dst + c);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[q * 8 + 0]) * inv, __uint_as_float(o[q * 8 + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(o[q * 8 + 2]) * inv, __uint_as_float(o[q * 8 + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(o[q * 8 + 4]) * inv, __uint_as_float(o[q * 8 + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(o[q * 8 + 6]) * inv, __uint_as_float(o[q * 8 + 7]) * inv);
            d4[q] = v;
          }
        }
      }
    }
  }

  // ---------------- common tail
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

static CUtensorMap make_qkv_map(const void* base, int B, int S, int H, long long sb, long long ss,
                                long long sh) {
  const uint64_t dims[4] = {128, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)sh * 2, (uint64_t)ss * 2, (uint64_t)sb * 2};
  const uint32_t box[4] = {64, 1, 128, 1};
  return cbh::make_tmap_bf16(base, 4, dims, strides, box, true);
}

void flash_attn_fwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.Hkv <= 0 || a.Hq % a.Hkv != 0) throw std::runtime_error("flash_attn_fwd: Hq % Hkv != 0");
  if (a.Sq <= 0 || a.Skv <= 0 || a.B <= 0) return;
  if (a.mask == MASK_CAUSAL && a.Skv < a.Sq)
    throw std::runtime_error("flash_attn_fwd: causal mask needs Skv >= Sq");
  if (a.mask == MASK_MOT && a.Skv != a.Sq)
    throw std::runtime_error("flash_attn_fwd: MoT mask needs Skv == Sq");
  if ((a.o_stride_s % 8) || (a.o_stride_h % 8) || (a.o_stride_b % 8))
    throw std::runtime_error("flash_attn_fwd: output strides must be multiples of 8 elements");
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(cb::flash_attn_fwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, cb::ATT_SMEM);
    cudaFuncSetAttribute(cb::flash_attn_fwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, cb::ATT_SMEM);
    cudaFuncSetAttribute(cb::flash_attn_fwd_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, cb::ATT_SMEM);
    cudaFuncSetAttribute(cb::flash_attn_fwd_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, cb::ATT_SMEM);
    cudaFuncSetAttribute(cb::flash_attn_fwd_kernel_v2, cudaFuncAttributeMaxDynamicSharedMemorySize, cb::ATT_SMEM);
    configured = true;
  }
  // B == 1 tensors may carry a zero batch stride; TMA needs a non-zero multiple of 16 bytes.
  auto fix = [](long long sb, long long ss, int S) { return sb > 0 ? sb : ss * S; };
  CUtensorMap tq = make_qkv_map(a.Q, a.B, a.Sq, a.Hq, fix(a.q_stride_b, a.q_stride_s, a.Sq),
                                a.q_stride_s, a.q_stride_h);
  CUtensorMap tk = make_qkv_map(a.K, a.B, a.Skv, a.Hkv, fix(a.k_stride_b, a.k_stride_s, a.Skv),
                                a.k_stride_s, a.k_stride_h);
  CUtensorMap tv = make_qkv_map(a.V, a.B, a.Skv, a.Hkv, fix(a.v_stride_b, a.v_stride_s, a.Skv),
                                a.v_stride_s, a.v_stride_h);
  cb::AttnParams p{};
  p.Sq = a.Sq; p.Skv = a.Skv; p.Hq = a.Hq; p.Hkv = a.Hkv; p.group = a.Hq / a.Hkv;
  p.mask = a.mask; p.n_ar = a.n_ar;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.O = reinterpret_cast<bf16*>(a.O);
  p.o_stride_b = a.o_stride_b; p.o_stride_s = a.o_stride_s; p.o_stride_h = a.o_stride_h;
  p.lse = a.lse;
  p.dest_ptr = a.dest_ptr; p.rows_per_dest = a.rows_per_dest > 0 ? a.rows_per_dest : 1;
  p.status = a.status;
  dim3 grid((a.Sq + 2 * cb::TQ - 1) / (2 * cb::TQ), a.Hq, a.B);
  // a.exp_emulation: 0 = all exp2 on the MUFU pipe, k = every k-th element on the FMA pipe
  if (a.pipeline == 2) {
    cb::flash_attn_fwd_kernel_v2<<<grid, cb::ATT_THREADS, cb::ATT_SMEM, stream>>>(tq, tk, tv, p);
    return;
  }
  switch (a.exp_emulation) {
    case 2: cb::flash_attn_fwd_kernel<2><<<grid, cb::ATT_THREADS, cb::ATT_SMEM, stream>>>(tq, tk, tv, p); break;
    case 3: cb::flash_attn_fwd_kernel<3><<<grid, cb::ATT_THREADS, cb::ATT_SMEM, stream>>>(tq, tk, tv, p); break;
    case 4: cb::flash_attn_fwd_kernel<4><<<grid, cb::ATT_THREADS, cb::ATT_SMEM, stream>>>(tq, tk, tv, p); break;
    default: cb::flash_attn_fwd_kernel<0><<<grid, cb::ATT_THREADS, cb::ATT_SMEM, stream>>>(tq, tk, tv, p); break;
  }
}

}  // namespace cosmos
