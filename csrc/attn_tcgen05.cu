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
#include <cstdlib>

namespace cb {

constexpr int ATT_THREADS = 384;
constexpr int TQ = 128, TKV = 128, HD = 128;
constexpr int TILE_BYTES = TQ * HD * 2;        // 32 KB
constexpr int HALF_BYTES = TILE_BYTES / 2;     // one 64-column half, 16 KB
// NC = 1: one CTA streams whole 128-key K and V tiles (32 KB ring slots, 5 of them).
// NC = 2: a CTA pair (cluster of 2, tcgen05 cta_group::2, M = 256 = tile t of both CTAs) shares every K/V block:
// for S = Q K^T each CTA stages 64 of the block's 128 keys (the B operand's N rows are split over the pair), for
// O += P V each CTA stages all 128 keys of 64 of the 128 head-dim columns. A ring slot is 16 KB (8 of them), the
// K/V bytes copied into and read from each CTA's shared memory are halved, and so is the L2 -> SM traffic.
template <int NC> struct AttCfg {
  static constexpr int NSLOT = NC == 2 ? 8 : 5;
  static constexpr int SLOT_BYTES = TILE_BYTES / NC;
  static constexpr int SMEM = 2 * TILE_BYTES + NSLOT * SLOT_BYTES + 1024 + 256;
};

constexpr int MAX_KV_SRC = 9;  // K/V sources of one launch: e.g. a local prompt prefix + 8 ranks' sequence shards

// Tensor maps of the K/V sources. Source s covers src_len[s] keys; the kernel walks the sources in the given
// order, so the keys of the whole sequence never have to sit in one buffer. A source may be another GPU's
// symmetric buffer: the TMA loads then pull its tiles over NVLink straight into this SM's shared memory
// (plain loads of one CTA each, no multicast), which is the ring-KV schedule of context parallelism inside
// the attention main loop.
struct KVMaps {
  CUtensorMap k[MAX_KV_SRC];
  CUtensorMap v[MAX_KV_SRC];
};

struct AttnParams {
  int n_src;                    // number of K/V sources (1 = the ordinary single-buffer call)
  int src_len[MAX_KV_SRC];      // keys per source (MASK_FULL only when n_src > 1)
  int Sq, Skv, Hq, Hkv, group;  // group = Hq / Hkv; Skv = total number of keys
  int mask, n_ar;
  float scale_log2;  // softmax scale * log2(e)
  bf16* O;
  long long o_stride_b, o_stride_s, o_stride_h;
  float* lse;  // [B, Hq, Sq]
  const long long* dest_ptr;
  int rows_per_dest;
  int* status;
  int debug;  // timing experiments only: bit 0 skips the QK MMAs, bit 1 the PV MMAs, bit 2 the exponentials
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed / three-input fp32 instructions of sm_100: they halve the instruction count of the softmax
// inner loop, which (not the tensor or MUFU pipe) is what bounds this kernel.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// Two exponentials at once on the FMA pipe with packed fp32 instructions, for scores already turned into
// x = s * scale_log2 - m with x >= -126 (the caller clamps the raw score, one FMNMX each):
// round-to-nearest split x = n + f with f in [-0.5, 0.5] by the magic-number add (the integer n sits in the low
// mantissa bits of t = x + 1.5 * 2^23), degree-3 minimax polynomial for 2^f (max relative error 7.5e-5, far below
// the bf16 rounding of P), and 2^n applied by adding n << 23 to the exponent field. Per pair: 2 packed adds,
// 4 packed FMAs and 2 shift-adds, against 2 x 8 cycles of the 4-lane-per-scheduler MUFU pipe.
struct Ex2Consts {
  uint64_t magic, neg_magic, minus1, c3, c2, c1, c0;
};
__device__ __forceinline__ Ex2Consts ex2_consts() {
  Ex2Consts c;
  c.magic = pack2(12582912.f, 12582912.f);
  c.neg_magic = pack2(-12582912.f, -12582912.f);
  c.minus1 = pack2(-1.f, -1.f);
  c.c3 = pack2(0.0551716648f, 0.0551716648f);
  c.c2 = pack2(0.2426111251f, 0.2426111251f);
  c.c1 = pack2(0.6932609677f, 0.6932609677f);
  c.c0 = pack2(0.9999280572f, 0.9999280572f);
  return c;
}
__device__ __forceinline__ void ex2_poly2(uint64_t x2, const Ex2Consts& c, float& r0, float& r1) {
  const uint64_t t2 = add2(x2, c.magic);
  const uint64_t n2 = add2(t2, c.neg_magic);
  const uint64_t f2 = fma2(n2, c.minus1, x2);
  uint64_t p2 = fma2(c.c3, f2, c.c2);
  p2 = fma2(p2, f2, c.c1);
  p2 = fma2(p2, f2, c.c0);
  float pa, pb, ta, tb;
  unpack2(p2, pa, pb);
  unpack2(t2, ta, tb);
  r0 = __int_as_float(__float_as_int(pa) + (__float_as_int(ta) << 23));
  r1 = __int_as_float(__float_as_int(pb) + (__float_as_int(tb) << 23));
}

__device__ __forceinline__ int kv_limit(int qi, const AttnParams& p) {
  if (p.mask == MASK_CAUSAL) return min(p.Skv, qi + 1 + (p.Skv - p.Sq));
  if (p.mask == MASK_MOT) return qi < p.n_ar ? qi + 1 : p.Skv;
  return p.Skv;
}

// EMU: of every 8 pairs of scores, EMU pairs take their exp2 on the FMA pipe (ex2_poly2), the rest on the MUFU pipe.
// DBG: honour AttnParams::debug (timing experiments); the production instantiation ignores it so
// that the inner loops carry no tests of it.
// Measured and not kept: one "P ready" arrival per softmax warp instead of one per thread (slower); packed
// ex2.approx.f16x2 / bf16x2 (the MUFU pipe retires them at half the instruction rate, so no gain), and P in
// fp16 with V in bf16 is not possible at all: tcgen05.mma kind::f16 with an fp16 A and a bf16 B operand is an
// illegal instruction on sm_100a.
template <int EMU, bool DBG, int NC>
__global__ void __launch_bounds__(ATT_THREADS, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ KVMaps kv,
                      const AttnParams p) {
  constexpr int NSLOT = AttCfg<NC>::NSLOT;
  constexpr int SLOT_BYTES = AttCfg<NC>::SLOT_BYTES;
  constexpr int K_HALF = SLOT_BYTES / 2;   // one 64-column half of a K slot
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;
  const uint32_t kv_smem = smem_base + 2 * TILE_BYTES;
  const uint32_t bar_base = kv_smem + NSLOT * SLOT_BYTES;
  // CTA pair: rank 0 (the leader) issues the MMAs and owns the barriers that both CTAs signal (q_full, kv_full,
  // p_full); s_full, kv_empty and o_final exist in both CTAs and the leader's commits reach both.
  const uint32_t cta_rank = NC == 2 ? cluster_ctarank() : 0u;
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + NSLOT + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (1 + 2 * NSLOT + t); };
  auto p_full = [&](int t, int h) { return bar_base + 8u * (3 + 2 * NSLOT + 2 * t + h); };
  auto o_final = [&](int t) { return bar_base + 8u * (7 + 2 * NSLOT + t); };
  constexpr int NBAR = 9 + 2 * NSLOT;
  const uint32_t tmem_slot = bar_base + 8u * NBAR;
  constexpr int BAR_OFF = 2 * TILE_BYTES + NSLOT * SLOT_BYTES;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + BAR_OFF + 8 * NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + BAR_OFF + 8 * NBAR + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int dbg = DBG ? p.debug : 0;
  const int qt = (p.mask == MASK_FULL) ? blockIdx.x : (gridDim.x - 1 - blockIdx.x);
  // the other CTA of a pair holds the neighbouring query tile; both walk the K/V blocks that the later tile needs
  const int qt_peer = NC == 2 ? ((p.mask == MASK_FULL) ? int(blockIdx.x ^ 1u) : int(gridDim.x - 1 - (blockIdx.x ^ 1u))) : qt;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / p.group;
  const int q0 = qt * 2 * TQ;
  const int q0_hi = max(qt, qt_peer) * 2 * TQ;

  // Number of K/V blocks this CTA visits.
  int n_blocks;
  const bool multi = p.n_src > 1;
  if (multi) {
    n_blocks = 0;
    for (int s = 0; s < p.n_src; ++s) n_blocks += (p.src_len[s] + TKV - 1) / TKV;
  } else {
    const int last_row = min(p.Sq - 1, q0_hi + 2 * TQ - 1);
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
      mbar_init(p_full(t, 0), NC == 2 ? 8 : 128);   // pair: one arrival per softmax warp of both CTAs
      mbar_init(p_full(t, 1), NC == 2 ? 8 : 128);
      mbar_init(o_final(t), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    for (int s = 0; s < p.n_src; ++s) {
      prefetch_tmap(&kv.k[s]);
      prefetch_tmap(&kv.v[s]);
    }
  }
  if (warp == 1) {
    if constexpr (NC == 2) {
      tmem_alloc_pair(tmem_slot, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (NC == 2) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // Register re-partitioning: the CTA owns 384 x 168 registers; 128 x 56 + 256 x 224 uses
  // exactly that many. A split that needs more would block in setmaxnreg.inc forever.
  static_assert(128 * 56 + 256 * 224 <= ATT_THREADS * 168, "setmaxnreg split exceeds the CTA's registers");
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0 && lane == 0) {
      // ---------------- TMA producer
      const uint32_t qf = NC == 2 ? mapa(q_full, 0) : q_full;
      if (cta_rank == 0) mbar_arrive_expect_tx(q_full, NC * 2 * TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if constexpr (NC == 2)
            tma_load_4d_pair(q_smem + t * TILE_BYTES + h * HALF_BYTES, &tmQ, qf, h * 64, head, q0 + t * TQ, batch);
          else
            tma_load_4d(q_smem + t * TILE_BYTES + h * HALF_BYTES, &tmQ, qf, h * 64, head, q0 + t * TQ, batch);
        }
      int issued = 0;
      bool ok = true;
      int src = 0, jb = 0;  // current K/V source and block within it
      for (int i = 0; i < 2 * n_blocks; ++i) {
        const int s = i % NSLOT;
        const uint32_t ph = (i / NSLOT) & 1;
        if (!mbar_wait(kv_empty(s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMA)) {
          ok = false;
          break;
        }
        const CUtensorMap* tm = (i & 1) ? &kv.v[src] : &kv.k[src];
        const uint32_t dst = kv_smem + s * SLOT_BYTES;
        if constexpr (NC == 2) {
          // both CTAs' bytes are counted on the leader's barrier, which expects the pair's total
          const uint32_t fb = mapa(kv_full(s), 0);
          if (cta_rank == 0) mbar_arrive_expect_tx(kv_full(s), 2 * SLOT_BYTES);
          if (i & 1) {
            // V: all 128 keys of this CTA's 64 head-dim columns
            tma_load_4d_pair(dst, tm, fb, int(cta_rank) * 64, kv_head, jb * TKV, batch);
          } else {
            // K: this CTA's 64 keys of the block, both 64-column halves
            tma_load_4d_pair(dst, tm, fb, 0, kv_head, jb * TKV + int(cta_rank) * 64, batch);
            tma_load_4d_pair(dst + K_HALF, tm, fb, 64, kv_head, jb * TKV + int(cta_rank) * 64, batch);
          }
        } else {
          mbar_arrive_expect_tx(kv_full(s), SLOT_BYTES);
          tma_load_4d(dst, tm, kv_full(s), 0, kv_head, jb * TKV, batch);
          tma_load_4d(dst + HALF_BYTES, tm, kv_full(s), 64, kv_head, jb * TKV, batch);
        }
        issued = i + 1;
        if (i & 1) {  // K and V of this block are on their way: next block, possibly of the next source
          ++jb;
          if (multi && jb * TKV >= p.src_len[src]) {
            jb = 0;
            ++src;
          }
        }
      }
      if (!ok) {
        if (NC == 2 && cta_rank != 0) {
          // this CTA's copies are counted on the leader's barriers, which only the leader can wait on: give
          // them a fixed time (far beyond a copy's latency) to land instead
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000ll) {}
        } else {
          volatile int no_abort = 0;
          mbar_wait(q_full, 0, &no_abort, nullptr, 0);
          const int first = issued > NSLOT ? issued - NSLOT : 0;
          for (int i = first; i < issued; ++i)
            mbar_wait(kv_full(i % NSLOT), (i / NSLOT) & 1, &no_abort, nullptr, 0);
        }
      }
    } else if (warp == 1 && cta_rank == 0) {
      // ---------------- MMA issuer: the whole warp walks the schedule (barrier phases, descriptors and
      // addresses are warp-uniform values), one elected lane issues the tcgen05 instructions
      const bool issuer = elect_one();
      auto wait_all = [&](uint32_t bar, uint32_t phase) {
        return __all_sync(0xffffffffu, mbar_wait(bar, phase, abort_flag, p.status, ST_TIMEOUT_MMA)) != 0;
      };
      constexpr uint32_t idesc_qk = make_idesc_bf16(TQ * NC, TKV, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(TQ * NC, HD, 0, 1);
      // Descriptors differ only in their 14-bit start-address field, so they are built as
      // one 64-bit constant plus a small address offset (in 16-byte units).
      const uint64_t q_desc0 = make_smem_desc_sw128(q_smem, 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(kv_smem, 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(kv_smem, HALF_BYTES, 1024);
      auto issue_qk = [&](int t, int slot) {
        const uint32_t d = tmem_base + t * 128;
        const uint64_t a0 = q_desc0 + uint64_t(t * (TILE_BYTES >> 4));
        const uint64_t b0 = k_desc0 + uint64_t(slot * (SLOT_BYTES >> 4));
        if ((dbg & 1) || !issuer) return;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off_a = (kk >> 2) * (HALF_BYTES >> 4) + 2 * (kk & 3);
          const uint32_t off_b = (kk >> 2) * (K_HALF >> 4) + 2 * (kk & 3);
          if constexpr (NC == 2)
            mma_ss_pair(d, a0 + off_a, b0 + off_b, idesc_qk, kk > 0 ? 1u : 0u);
          else
            mma_ss(d, a0 + off_a, b0 + off_b, idesc_qk, kk > 0 ? 1u : 0u);
        }
      };
      // a commit releases / signals in this CTA and, for a pair, in the peer as well
      auto commit = [&](uint32_t bar) {
        if (!issuer) return;
        if constexpr (NC == 2) {
          tc_commit_pair(bar);
          tc_commit_pair(mapa(bar, 1));
        } else {
          tc_commit(bar);
        }
      };
      // P is handed over in two halves of 64 keys, so the first four k-steps of PV run while the
      // softmax warps still compute the exponentials of the second half.
      auto issue_pv = [&](int t, int slot, bool acc, int half) {
        const uint32_t d = tmem_base + 256 + t * 128;
        const uint32_t a0 = tmem_base + t * 128;
        const uint64_t b0 = v_desc0 + uint64_t(slot * (SLOT_BYTES >> 4));
        if ((dbg & 2) || !issuer) return;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const int kk = half * 4 + k4;
          if constexpr (NC == 2)
            mma_ts_pair(d, a0 + kk * 8, b0 + uint64_t(kk * (2048 >> 4)), idesc_pv, (acc || kk > 0) ? 1u : 0u);
          else
            mma_ts(d, a0 + kk * 8, b0 + uint64_t(kk * (2048 >> 4)), idesc_pv, (acc || kk > 0) ? 1u : 0u);
        }
      };
      bool ok = wait_all(q_full, 0);
      if (ok) ok = wait_all(kv_full(0), 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        commit(s_full(0));
        issue_qk(1, 0);
        commit(s_full(1));
        commit(kv_empty(0));
        __syncwarp();
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int iv = 2 * j + 1, ik = 2 * j + 2;
        const int sv = iv % NSLOT, sk = ik % NSLOT;
        const bool more = (j + 1 < n_blocks);
        ok = wait_all(kv_full(sv), (iv / NSLOT) & 1);
        if (ok && more) ok = wait_all(kv_full(sk), (ik / NSLOT) & 1);
        if (!ok) break;
#pragma unroll 1
        for (int t = 0; t < 2; ++t) {
          ok = wait_all(p_full(t, 0), j & 1);
          if (!ok) break;
          tc_fence_after();
          issue_pv(t, sv, j > 0, 0);
          ok = wait_all(p_full(t, 1), j & 1);
          if (!ok) break;
          tc_fence_after();
          issue_pv(t, sv, j > 0, 1);
          if (more) {
            issue_qk(t, sk);
            commit(s_full(t));
          } else {
            commit(o_final(t));
          }
          __syncwarp();
        }
        if (!ok) break;
        commit(kv_empty(sv));
        if (more) commit(kv_empty(sk));
        __syncwarp();
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
    const float inv_sl2 = 1.f / sl2;
    const Ex2Consts exc = ex2_consts();
    float m_used = -1e30f, l = 0.f;
    bool ok = true;
    int src = 0, jb = 0;  // K/V source and block within it (multi-source launches)
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
      if (multi) {
        // the last block of a source may be ragged: rows beyond the source's end were zero-filled by the copy
        const int valid = p.src_len[src] - jb * TKV;
        if (valid < TKV) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i >= valid) s[i] = 0xff800000u;  // -inf
        }
        ++jb;
        if (jb * TKV >= p.src_len[src]) {
          jb = 0;
          ++src;
        }
      } else {
        const int kv0 = j * TKV;
        if (kv0 + TKV > limit) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (kv0 + i >= limit) s[i] = 0xff800000u;  // -inf
        }
      }
      // eight independent chains of three-input max (60 instructions for 128 values)
      float mx8[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) mx8[e] = __uint_as_float(s[e]);
      if (!((dbg & 8) && j > 0)) {   // timing experiment: no row maximum after the first block
#pragma unroll
        for (int i = 8; i < 128; i += 16)
#pragma unroll
          for (int e = 0; e < 8; ++e) mx8[e] = max3(mx8[e], __uint_as_float(s[i + e]), __uint_as_float(s[i + 8 + e]));
      }
      const float mx = max3(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
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
      // x = s * scale_log2 - m with packed FMAs (two scores per instruction), exp2 on the MUFU
      // pipe, packed partial sums
      const uint64_t sl2_2 = pack2(sl2, sl2);
      const uint64_t negm_2 = pack2(-m_used, -m_used);
      // raw-score floor that keeps x >= -126 on the polynomial path (masked scores, -inf, land there too)
      const float s_floor = (m_used - 126.f) * inv_sl2;
      uint64_t ls2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int e = half * 64 + 2 * i;
          float p0, p1;
          if (EMU > 0 && (i & 7) < EMU) {
            const uint64_t x2 = fma2(pack2(fmaxf(__uint_as_float(s[e]), s_floor), fmaxf(__uint_as_float(s[e + 1]), s_floor)),
                                     sl2_2, negm_2);
            ex2_poly2(x2, exc, p0, p1);
          } else {
            const uint64_t x2 = fma2(pack2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), sl2_2, negm_2);
            unpack2(x2, p0, p1);
            if (!(dbg & 4)) {
              p0 = ex2(p0);
              p1 = ex2(p1);
            }
          }
          ls2[i & 3] = add2(ls2[i & 3], pack2(p0, p1));
          pk[i] = pack_bf16(p0, p1);
        }
        tmem_st32(s_addr + half * 32, pk);
        tmem_wait_st();
        tc_fence_before();
        if constexpr (NC == 2) {
          // one arrival per warp on the leader's barrier (a cluster-scope arrive from the peer CTA)
          __syncwarp();
          if (lane == 0) {
            if (cta_rank == 0)
              mbar_arrive(p_full(t, half));
            else
              mbar_arrive_cluster(mapa(p_full(t, half), 0));
          }
        } else {
          mbar_arrive(p_full(t, half));
        }
      }
      {
        float a0, a1, b0, b1;
        unpack2(add2(ls2[0], ls2[1]), a0, a1);
        unpack2(add2(ls2[2], ls2[3]), b0, b1);
        l += (a0 + a1) + (b0 + b1);
      }
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
  // neither CTA of a pair leaves (or frees tensor memory) while the other may still signal its barriers or have
  // MMAs in flight that read its shared memory
  if constexpr (NC == 2) cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if constexpr (NC == 2)
      tmem_dealloc_pair(tmem_base, 512);
    else
      tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace cb

namespace cosmos {

static CUtensorMap make_qkv_map(const void* base, int B, int S, int H, long long sb, long long ss,
                                long long sh, int box_rows = 128) {
  const uint64_t dims[4] = {128, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)sh * 2, (uint64_t)ss * 2, (uint64_t)sb * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return cbh::make_tmap_bf16(base, 4, dims, strides, box, true);
}

// A/B switch: query blocks of more than one 256-row tile run on CTA pairs when on (COSMOS_ATTN_CTA_PAIR=1 or
// attn_set_cta_pair). Off by default: the pair halves the K/V bytes through each CTA's shared memory, but every
// hand-over of the per-tile chain (scores ready -> softmax -> P ready -> MMA issue) then crosses to the other CTA,
// and the chain, not the operand traffic, bounds this kernel: measured 4.68 ms against 3.56 ms for single CTAs at
// 32768 x 32768, 8 / 2 heads, in seconds-long loops on a B200.
static int g_attn_pair = -1;
static bool attn_pair_enabled() {
  if (g_attn_pair < 0) {
    const char* e = std::getenv("COSMOS_ATTN_CTA_PAIR");
    g_attn_pair = (e && e[0] == '1') ? 1 : 0;
  }
  return g_attn_pair == 1;
}
void attn_set_cta_pair(bool on) { g_attn_pair = on ? 1 : 0; }

template <int EMU, bool DBG>
static void launch_attn(int nc, dim3 grid, const CUtensorMap& tq, const cb::KVMaps& kv, const cb::AttnParams& p,
                        cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(cb::ATT_THREADS, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = nc; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  if (nc == 2) {
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(cb::flash_attn_fwd_kernel<EMU, DBG, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           cb::AttCfg<2>::SMEM);
      configured = true;
    }
    grid.x = (grid.x + 1) & ~1u;   // whole pairs; a CTA beyond the last query row computes and stores nothing
    cfg.gridDim = grid;
    cfg.dynamicSmemBytes = cb::AttCfg<2>::SMEM;
    cudaLaunchKernelEx(&cfg, cb::flash_attn_fwd_kernel<EMU, DBG, 2>, tq, kv, p);
  } else {
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(cb::flash_attn_fwd_kernel<EMU, DBG, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           cb::AttCfg<1>::SMEM);
      configured = true;
    }
    cfg.gridDim = grid;
    cfg.dynamicSmemBytes = cb::AttCfg<1>::SMEM;
    cudaLaunchKernelEx(&cfg, cb::flash_attn_fwd_kernel<EMU, DBG, 1>, tq, kv, p);
  }
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
  const int n_src = a.n_src > 0 ? a.n_src : 1;
  if (n_src > cb::MAX_KV_SRC) throw std::runtime_error("flash_attn_fwd: too many K/V sources");
  if (n_src > 1 && a.mask != MASK_FULL) throw std::runtime_error("flash_attn_fwd: several K/V sources need the full mask");
  dim3 grid((a.Sq + 2 * cb::TQ - 1) / (2 * cb::TQ), a.Hq, a.B);
  // CTA pairs as soon as there is more than one 256-row query block
  const int nc = (attn_pair_enabled() && grid.x >= 2) ? 2 : 1;
  const int k_rows = nc == 2 ? 64 : 128;   // a pair's CTA copies 64 of a block's 128 keys for QK^T
  // B == 1 tensors may carry a zero batch stride; TMA needs a non-zero multiple of 16 bytes.
  auto fix = [](long long sb, long long ss, int S) { return sb > 0 ? sb : ss * S; };
  CUtensorMap tq = make_qkv_map(a.Q, a.B, a.Sq, a.Hq, fix(a.q_stride_b, a.q_stride_s, a.Sq),
                                a.q_stride_s, a.q_stride_h);
  cb::KVMaps kv{};
  cb::AttnParams p{};
  p.n_src = n_src;
  if (n_src == 1) {
    kv.k[0] = make_qkv_map(a.K, a.B, a.Skv, a.Hkv, fix(a.k_stride_b, a.k_stride_s, a.Skv), a.k_stride_s, a.k_stride_h,
                           k_rows);
    kv.v[0] = make_qkv_map(a.V, a.B, a.Skv, a.Hkv, fix(a.v_stride_b, a.v_stride_s, a.Skv), a.v_stride_s, a.v_stride_h);
    p.src_len[0] = a.Skv;
  } else {
    // every source is a contiguous [B, len, Hkv, 128] buffer (possibly on a peer GPU)
    for (int s = 0; s < n_src; ++s) {
      const int len = a.src_len[s];
      if (len <= 0) throw std::runtime_error("flash_attn_fwd: empty K/V source");
      const long long ss = (long long)a.Hkv * 128, sb = ss * len;
      kv.k[s] = make_qkv_map(a.src_k[s], a.B, len, a.Hkv, sb, ss, 128, k_rows);
      kv.v[s] = make_qkv_map(a.src_v[s], a.B, len, a.Hkv, sb, ss, 128);
      p.src_len[s] = len;
    }
  }
  p.Sq = a.Sq; p.Skv = a.Skv; p.Hq = a.Hq; p.Hkv = a.Hkv; p.group = a.Hq / a.Hkv;
  p.mask = a.mask; p.n_ar = a.n_ar;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.O = reinterpret_cast<bf16*>(a.O);
  p.o_stride_b = a.o_stride_b; p.o_stride_s = a.o_stride_s; p.o_stride_h = a.o_stride_h;
  p.lse = a.lse;
  p.dest_ptr = a.dest_ptr; p.rows_per_dest = a.rows_per_dest > 0 ? a.rows_per_dest : 1;
  p.status = a.status;
  p.debug = a.debug;
  // a.exp_emulation: of every 8 pairs of scores, this many take their exp2 on the FMA pipe (0, 2 or 3; measured
  // slower than 0 whenever the MMAs run); a.debug: timing experiments (wrong results)
  if (a.debug) {
    switch (a.exp_emulation) {
      case 2: launch_attn<2, true>(nc, grid, tq, kv, p, stream); break;
      case 3: launch_attn<3, true>(nc, grid, tq, kv, p, stream); break;
      default: launch_attn<0, true>(nc, grid, tq, kv, p, stream); break;
    }
  } else {
    switch (a.exp_emulation) {
      case 2: launch_attn<2, false>(nc, grid, tq, kv, p, stream); break;
      case 3: launch_attn<3, false>(nc, grid, tq, kv, p, stream); break;
      default: launch_attn<0, false>(nc, grid, tq, kv, p, stream); break;
    }
  }
}

}  // namespace cosmos
