// K1: persistent bf16 GEMM  C[M,N] = A[M,K] * B[N,K]^T  on tcgen05 tensor cores.
//
// Layout of one CTA (192 threads):
//   warp 0      TMA producer  (A 128x64 and B 256x64 tiles, 128-byte swizzle, 4-stage ring)
//   warp 1      MMA issuer    (tcgen05.mma M=128 N=256 K=16, fp32 accumulators in TMEM,
//                              two 256-column accumulator buffers so the epilogue of tile i
//                              overlaps the main loop of tile i+1)
//   warps 2..5  epilogue      (tcgen05.ld -> registers -> fused epilogue -> global / peer stores)
//
// Fused epilogues (template parameter EPI):
//   EPI_PLAIN        C = acc (+ bias)
//   EPI_SWIGLU       B holds [gate ; up] stacked along N; C[m, j] = silu(gate_j) * up_j  (N/2 wide)
//   EPI_GATED_RESID  C = R + gate[m / rows_per_batch, n] * (acc + bias)   (AdaLN gated residual)
//   EPI_QKV_ROPE     columns are heads of 128: per-head RMSNorm (q/k) + rotary embedding, and
//                    each 128-column chunk is written through a routing table, so a chunk
//                    can land in another GPU's buffer (sequence->head all-to-all of Ulysses
//                    context parallelism done by the epilogue's stores).
//
// All mbarrier waits are bounded; on expiry the kernel records a status code and exits
// through the common tail (TMEM is freed).
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"
#include <cstdlib>

namespace cb {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int A_BYTES = BM * BK * 2;      // 16 KB
constexpr int GEMM_THREADS = 192;
// NC = 1: one CTA per 128x256 tile, 4 stages of A 16 KB + B 32 KB.
// NC = 2: a CTA pair per 256x256 tile (tcgen05 cta_group::2, M = 256): each CTA stages its own 128 rows
// of A and its own 128 of the tile's 256 B rows, so a stage is 32 KB per CTA and the B operand crosses
// shared memory once per pair instead of once per CTA; 6 stages.
template <int NC> struct GemmCfg {
  static constexpr int STAGES = NC == 2 ? 6 : 4;
  static constexpr int B_BYTES = (BN / NC) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

struct GemmParams {
  int M, N, K;
  int b_row1;            // row offset in B of the second 128-row half of the tile
  int mma_n;             // N of the MMA instruction: BN, or 64 / 128 for a convolution with that few output channels
  int n_tiles, m_tiles;  // tile counts (n_tiles counts 256-wide (or 128-wide for SWIGLU) tiles)
  bf16* C;
  long long ldc;
  const bf16* bias;      // [N] or null
  const bf16* R;         // residual [M, ldr]
  long long ldr;
  const bf16* gate;      // [batches, N]
  int rows_per_batch;
  // EPI_QKV_ROPE
  const long long* route_ptr;  // per 128-col chunk: destination base address (bf16*)
  const long long* route_ld;   // per chunk: row stride in elements
  const float* cos_tab;        // [rope_rows, 64]
  const float* sin_tab;
  int rope_rows;
  const bf16* gamma_q;         // [128]
  const bf16* gamma_k;
  int n_q_heads, n_k_heads;
  float eps;
  int* status;
  // split-K (skinny problems, e.g. decode): the K range is divided among k_splits CTAs per output
  // tile; each writes its raw fp32 accumulators to partial[ks][M][N] and a second kernel reduces
  // them and applies the epilogue.
  int k_splits;
  float* partial;
  const float* rowvec;   // EPI_ATTN_P: lse[M]; EPI_ATTN_DS: D[M]
  float attn_scale;
  int attn_mask, attn_n_ar;
  // operand majors: 0 = K-major ([rows, K] storage), 1 = MN-major ([K, rows] storage, i.e. the
  // transposed operand is read in place; used by the backward GEMMs dX = dY W and dW = dY^T X)
  int a_mn, b_mn;
  // implicit-GEMM convolution (EPI_CONV)
  int conv_cblocks;      // input channels / 64
  int conv_hp, conv_wp, conv_tpad;
  int conv_shift[27];    // row offset of each filter tap in the flattened padded volume
  int debug;             // timing experiments (wrong results): 1 = every tile loads operand tile (0, 0); 2 = no loads at all
};

// Up to two independent problems served by one persistent launch (grouped GEMM): tiles
// [0, tiles0) belong to problem 0, the rest to problem 1. Used for the per-modality weight
// routing of the Mixture-of-Transformers layers (AR tokens x AR weights, DM tokens x DM weights).
struct GemmGroup {
  GemmParams p[2];
  int tiles0;
  int total;
};

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int& tm, int& tn) {
  // Rasterise in bands of 16 m-tiles so that CTAs running together share A and B tiles in L2.
  constexpr int GM = 16;
  const int band = t / (GM * n_tiles);
  const int first_m = band * GM;
  const int band_m = min(GM, m_tiles - first_m);
  const int r = t - band * GM * n_tiles;
  tm = first_m + r % band_m;
  tn = r / band_m;
}

template <int EPI, int NC>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                 const __grid_constant__ GemmGroup g) {
  constexpr int STAGES = GemmCfg<NC>::STAGES;
  constexpr int B_BYTES = GemmCfg<NC>::B_BYTES;
  constexpr int STAGE_BYTES = GemmCfg<NC>::STAGE_BYTES;
  constexpr int TILE_M = BM * NC;  // rows of one output tile (of the CTA pair when NC == 2)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  // CTA pair: rank 0 (the leader) issues the MMAs and owns the `full` and `tempty` barriers that
  // both CTAs signal; `empty` and `tfull` exist in both CTAs and the leader's commits reach both.
  const uint32_t cta_rank = NC == 2 ? cluster_ctarank() : 0u;
  const int first_tile = NC == 2 ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int tile_step = NC == 2 ? int(gridDim.x >> 1) : int(gridDim.x);
  // barriers: full[STAGES], empty[STAGES], tfull[2], tempty[2]; then tmem slot, abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(gen_base + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4) + 8);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(gen_base + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = g.total;

  int prefetched = 0;  // stages whose B half thread 0 has requested ahead of the producer loop
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4 * NC);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (g.total > g.tiles0) {
      prefetch_tmap(&tmA1);
      prefetch_tmap(&tmB1);
    }
    // Weight prefetch (single-CTA tiles, B in its [N, K] layout): the B halves of the first tile's first stages are
    // requested here, while warp 1 still allocates tensor memory and before the dependency wait of a programmatic
    // launch; their A halves follow in the producer loop. A stage's full barrier completes when both have landed.
    if (NC == 1 && EPI != EPI_CONV && first_tile < total_tiles && first_tile < g.tiles0 && !g.p[0].b_mn &&
        !g.p[0].debug) {
      const GemmParams& p = g.p[0];
      const int k_blocks = (p.K + BK - 1) / BK;
      const int ks = first_tile % p.k_splits;
      const int kb0 = ks * k_blocks / p.k_splits, kb1 = (ks + 1) * k_blocks / p.k_splits;
      int tm, tn;
      tile_coords(first_tile / p.k_splits, p.m_tiles, p.n_tiles, tm, tn);
      const int n0 = (EPI == EPI_SWIGLU) ? tn * 128 : tn * BN;
      for (int kb = kb0; kb < kb1 && prefetched < STAGES; ++kb, ++prefetched) {
        const uint32_t sa = smem_base + prefetched * STAGE_BYTES;
        mbar_arrive_expect_tx(full_bar(prefetched), STAGE_BYTES);
        tma_load_2d(sa + A_BYTES, &tmB, full_bar(prefetched), kb * BK, n0);
        tma_load_2d(sa + A_BYTES + B_BYTES / 2, &tmB, full_bar(prefetched), kb * BK, n0 + p.b_row1);
      }
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
  // The set-up above overlapped the previous kernel's tail when this one was launched as its programmatic
  // dependent; the successor may begin its own set-up now. Every thread but the producer waits here for the
  // previous kernel's results; the producer first starts the weight tiles of its first stages (below).
  pdl_launch_dependents();
  const bool is_producer = warp == 0 && lane == 0;
  if (!is_producer) pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      int it = 0;
      bool ok = true;
      pdl_wait();
      for (int t = first_tile; t < total_tiles && ok; t += tile_step) {
        const int second = t >= g.tiles0;
        const GemmParams& p = g.p[second];
        const CUtensorMap* mA = second ? &tmA1 : &tmA;
        const CUtensorMap* mB = second ? &tmB1 : &tmB;
        const int k_blocks = (p.K + BK - 1) / BK;
        const int tl = second ? t - g.tiles0 : t;
        const int ks = tl % p.k_splits;
        const int kb0 = ks * k_blocks / p.k_splits, kb1 = (ks + 1) * k_blocks / p.k_splits;
        int tm, tn;
        tile_coords(tl / p.k_splits, p.m_tiles, p.n_tiles, tm, tn);
        const int m0 = (p.debug & 1) ? 0 : tm * TILE_M + int(cta_rank) * BM;
        const int n0 = (p.debug & 1) ? 0 : ((EPI == EPI_SWIGLU) ? tn * 128 : tn * BN);
        if (p.debug & 2) continue;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          if (it < prefetched) {
            // stage already armed and its B half in flight: only the A half is left
            if (p.a_mn) {
              tma_load_2d(sa, mA, full_bar(s), m0, kb * BK);
              tma_load_2d(sa + A_BYTES / 2, mA, full_bar(s), m0 + 64, kb * BK);
            } else {
              tma_load_2d(sa, mA, full_bar(s), kb * BK, m0);
            }
            continue;
          }
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMA)) {
            ok = false;
            break;
          }
          if constexpr (NC == 2) {
            // both CTAs' bytes are counted on the leader's barrier, which expects the pair's total
            const uint32_t fb = mapa(full_bar(s), 0);
            if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * STAGE_BYTES);
            if constexpr (EPI == EPI_CONV) {
              const int tap = kb / p.conv_cblocks;
              tma_load_2d_pair(sa, mA, fb, (kb - tap * p.conv_cblocks) * BK, m0 + p.conv_shift[tap]);
            } else if (p.a_mn) {
              tma_load_2d_pair(sa, mA, fb, m0, kb * BK);
              tma_load_2d_pair(sa + A_BYTES / 2, mA, fb, m0 + 64, kb * BK);
            } else {
              tma_load_2d_pair(sa, mA, fb, kb * BK, m0);
            }
            const int nb = n0 + int(cta_rank) * p.b_row1;  // this CTA's 128 B rows (N columns of the tile)
            if (p.b_mn) {
              tma_load_2d_pair(sa + A_BYTES, mB, fb, nb, kb * BK);
              tma_load_2d_pair(sa + A_BYTES + B_BYTES / 2, mB, fb, nb + 64, kb * BK);
            } else {
              tma_load_2d_pair(sa + A_BYTES, mB, fb, kb * BK, nb);
            }
            continue;
          }
          mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
          if constexpr (EPI == EPI_CONV) {
            const int tap = kb / p.conv_cblocks;
            tma_load_2d(sa, mA, full_bar(s), (kb - tap * p.conv_cblocks) * BK, m0 + p.conv_shift[tap]);
          } else if (p.a_mn) {
            tma_load_2d(sa, mA, full_bar(s), m0, kb * BK);
            tma_load_2d(sa + A_BYTES / 2, mA, full_bar(s), m0 + 64, kb * BK);
          } else {
            tma_load_2d(sa, mA, full_bar(s), kb * BK, m0);
          }
          if (p.b_mn) {
#pragma unroll
            for (int h = 0; h < 4; ++h)
              tma_load_2d(sa + A_BYTES + h * (B_BYTES / 4), mB, full_bar(s),
                          n0 + (h & 1) * 64 + (h >> 1) * p.b_row1, kb * BK);
          } else {
            tma_load_2d(sa + A_BYTES, mB, full_bar(s), kb * BK, n0);
            tma_load_2d(sa + A_BYTES + B_BYTES / 2, mB, full_bar(s), kb * BK, n0 + p.b_row1);
          }
        }
      }
      if (!ok) {
        // Drain our own copies in flight (bounded) before the CTA leaves.
        if (NC == 2 && cta_rank != 0) {
          // this CTA's copies are counted on the leader's barrier, which only the leader can wait
          // on: give them a fixed time (far beyond a copy's latency) to land instead
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000ll) {}
        } else {
          volatile int no_abort = 0;
          const int first = it > STAGES ? it - STAGES : 0;
          for (int j = first; j < it; ++j)
            mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1, &no_abort, nullptr, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (cta_rank == 0) {
      // ---------------- MMA issuer. The whole warp walks the loop, so barrier phases, descriptors and
      // addresses are warp-uniform values; one elected lane issues the tcgen05 instructions.
      // (instruction descriptor is built per tile: the operand majors are per-problem)
      int it = 0, tcount = 0;
      bool ok = true;
      for (int t = first_tile; t < total_tiles && ok; t += tile_step, ++tcount) {
        const int second = t >= g.tiles0;
        const GemmParams& p = g.p[second];
        const int k_blocks = (p.K + BK - 1) / BK;
        const int ks = (second ? t - g.tiles0 : t) % p.k_splits;
        const int kb0 = ks * k_blocks / p.k_splits, kb1 = (ks + 1) * k_blocks / p.k_splits;
        const int b = tcount & 1;
        const uint32_t bph = (tcount >> 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(tempty_bar(b), bph ^ 1, abort_flag, p.status, ST_TIMEOUT_MMA))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * BN;
        const uint32_t a_step = p.a_mn ? 128u : 2u, b_step = p.b_mn ? 128u : 2u;
        const uint32_t idesc = make_idesc_bf16(TILE_M, p.mma_n, p.a_mn, p.b_mn);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!(p.debug & 2) &&
              !__all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, abort_flag, p.status, ST_TIMEOUT_MMA))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          // K-major: 128-byte rows along K, +32 B per k-step. MN-major: 64-element chunks along M/N
          // 8 KB apart (LBO), k advances by rows of 128 B, +2048 B per k-step of 16.
          const uint64_t adesc = p.a_mn ? make_smem_desc_sw128(sa, 8192, 1024) : make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = p.b_mn ? make_smem_desc_sw128(sa + A_BYTES, 8192, 1024)
                                        : make_smem_desc_sw128(sa + A_BYTES, 16, 1024);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              // advance 32 bytes (16 bf16) along K inside the 128-byte swizzle row: +2 in >>4 units
              if constexpr (NC == 2)
                mma_ss_pair(d_tmem, adesc + a_step * k, bdesc + b_step * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
              else
                mma_ss(d_tmem, adesc + a_step * k, bdesc + b_step * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            }
            if constexpr (NC == 2) {
              tc_commit_pair(empty_bar(s));            // frees the stage in this CTA ...
              tc_commit_pair(mapa(empty_bar(s), 1));   // ... and in the peer
            } else {
              tc_commit(empty_bar(s));
            }
          }
          __syncwarp();
        }
        if (ok) {
          if (elect_one()) {
            if constexpr (NC == 2) {
              tc_commit_pair(tfull_bar(b));
              tc_commit_pair(mapa(tfull_bar(b), 1));
            } else {
              tc_commit(tfull_bar(b));
            }
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ---------------- epilogue warps (2..5); TMEM lane quadrant = warp % 4
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int tcount = 0;
    for (int t = first_tile; t < total_tiles; t += tile_step, ++tcount) {
      const int b = tcount & 1;
      const uint32_t bph = (tcount >> 1) & 1;
      const int second = t >= g.tiles0;
      const GemmParams& p = g.p[second];
      const int tl = second ? t - g.tiles0 : t;
      int tm, tn;
      tile_coords(tl / p.k_splits, p.m_tiles, p.n_tiles, tm, tn);
      const int m = tm * TILE_M + int(cta_rank) * BM + row_in_tile;
      if (!mbar_wait(tfull_bar(b), bph, abort_flag, p.status, ST_TIMEOUT_EPI)) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t(quad * 32) << 16) + b * BN;
      const bool row_ok = m < p.M;

      if ((EPI == EPI_PLAIN || EPI == EPI_SWIGLU || EPI == EPI_GATED_RESID) && p.k_splits > 1) {
        // raw fp32 partial sums; accumulator column c maps to output column col(c)
        float* dst_row = p.partial + ((long long)(tl % p.k_splits) * p.M + m) * p.N;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          tmem_ld32(t_addr + c, v);
          tmem_wait_ld();
          const int col = (EPI == EPI_SWIGLU) ? (c < 128 ? tn * 128 + c : p.N / 2 + tn * 128 + (c - 128))
                                              : tn * BN + c;
          const int col_end = (EPI == EPI_SWIGLU) ? (c < 128 ? p.N / 2 : p.N) : p.N;
          if (row_ok && col < col_end) {
            if (col + 32 <= col_end) {
              float4* d4 = reinterpret_cast<float4*>(dst_row + col);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                d4[q] = make_float4(__uint_as_float(v[q * 4]), __uint_as_float(v[q * 4 + 1]),
                                    __uint_as_float(v[q * 4 + 2]), __uint_as_float(v[q * 4 + 3]));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col + i < col_end) dst_row[col + i] = __uint_as_float(v[i]);
            }
          }
        }
      } else if constexpr (EPI == EPI_PLAIN || EPI == EPI_GATED_RESID) {
        const int n0 = tn * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          tmem_ld32(t_addr + c, v);
          tmem_wait_ld();
          const int n = n0 + c;
          if (row_ok && n < p.N) {
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
            const bool full32 = (n + 32 <= p.N);
            if (p.bias) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (full32 || n + i < p.N) f[i] += __bfloat162float(p.bias[n + i]);
            }
            if constexpr (EPI == EPI_GATED_RESID) {
              const bf16* g = p.gate ? p.gate + (long long)(m / p.rows_per_batch) * p.N + n : nullptr;
              const bf16* r = p.R + (long long)m * p.ldr + n;
              if (full32) {
                const uint4* r4 = reinterpret_cast<const uint4*>(r);
                const uint4* g4 = reinterpret_cast<const uint4*>(g);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 rv = r4[q];
                  const uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
                  uint32_t gu[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
                  if (g) {
                    const uint4 gv = g4[q];
                    gu[0] = gv.x; gu[1] = gv.y; gu[2] = gv.z; gu[3] = gv.w;
                  }
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    f[q * 8 + e * 2] = bf16lo(ru[e]) + bf16lo(gu[e]) * f[q * 8 + e * 2];
                    f[q * 8 + e * 2 + 1] = bf16hi(ru[e]) + bf16hi(gu[e]) * f[q * 8 + e * 2 + 1];
                  }
                }
              } else {
                for (int i = 0; i < 32 && n + i < p.N; ++i) {
                  const float gg = g ? __bfloat162float(g[i]) : 1.f;
                  f[i] = __bfloat162float(r[i]) + gg * f[i];
                }
              }
            }
            bf16* dst = p.C + (long long)m * p.ldc + n;
            if (full32) {
              uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack_bf16(f[q * 8 + 0], f[q * 8 + 1]);
                o.y = pack_bf16(f[q * 8 + 2], f[q * 8 + 3]);
                o.z = pack_bf16(f[q * 8 + 4], f[q * 8 + 5]);
                o.w = pack_bf16(f[q * 8 + 6], f[q * 8 + 7]);
                d4[q] = o;
              }
            } else {
              for (int i = 0; i < 32 && n + i < p.N; ++i) dst[i] = __float2bfloat16(f[i]);
            }
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        // accumulator columns [0,128) = gate, [128,256) = up, for output columns tn*128 ...
        const int n0 = tn * 128;
        const int n_out = p.N / 2;
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld32(t_addr + c, g);
          tmem_ld32(t_addr + 128 + c, u);
          tmem_wait_ld();
          const int n = n0 + c;
          if (row_ok && n < n_out) {
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float gv = __uint_as_float(g[i]);
              const float uv = __uint_as_float(u[i]);
              f[i] = gv / (1.f + __expf(-gv)) * uv;
            }
            bf16* dst = p.C + (long long)m * p.ldc + n;
            if (n + 32 <= n_out) {
              uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack_bf16(f[q * 8 + 0], f[q * 8 + 1]);
                o.y = pack_bf16(f[q * 8 + 2], f[q * 8 + 3]);
                o.z = pack_bf16(f[q * 8 + 4], f[q * 8 + 5]);
                o.w = pack_bf16(f[q * 8 + 6], f[q * 8 + 7]);
                d4[q] = o;
              }
            } else {
              for (int i = 0; i < 32 && n + i < n_out; ++i) dst[i] = __float2bfloat16(f[i]);
            }
          }
        }
      } else if constexpr (EPI == EPI_ATTN_P || EPI == EPI_ATTN_DS) {
        const int n0 = tn * BN;
        const float rv = row_ok ? p.rowvec[m] : 0.f;
        int lim = p.N;
        if (p.attn_mask == MASK_CAUSAL) lim = min(p.N, m + 1 + (p.N - p.M));
        if (p.attn_mask == MASK_MOT) lim = m < p.attn_n_ar ? m + 1 : p.N;
        const float sl2 = p.attn_scale * 1.4426950408889634f;
        const float rv2 = rv * 1.4426950408889634f;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          const int n = n0 + c;
          if (n >= p.N) break;
          uint32_t v[32];
          tmem_ld32(t_addr + c, v);
          tmem_wait_ld();
          if (row_ok) {
            float f[32];
            const bool full32 = (n + 32 <= p.N);
            if constexpr (EPI == EPI_ATTN_P) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                f[i] = (n + i < lim) ? exp2f(fmaf(__uint_as_float(v[i]), sl2, -rv2)) : 0.f;
            } else {
              const bf16* pr = p.R + (long long)m * p.ldr + n;
              if (full32) {
                const uint4* r4 = reinterpret_cast<const uint4*>(pr);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 rr = r4[q];
                  const uint32_t ru[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    f[q * 8 + 2 * e] = bf16lo(ru[e]) * (__uint_as_float(v[q * 8 + 2 * e]) - rv) * p.attn_scale;
                    f[q * 8 + 2 * e + 1] = bf16hi(ru[e]) * (__uint_as_float(v[q * 8 + 2 * e + 1]) - rv) * p.attn_scale;
                  }
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  f[i] = (n + i < p.N) ? __bfloat162float(pr[i]) * (__uint_as_float(v[i]) - rv) * p.attn_scale : 0.f;
              }
            }
            bf16* dst = p.C + (long long)m * p.ldc + n;
            if (full32) {
              uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack_bf16(f[q * 8 + 0], f[q * 8 + 1]);
                o.y = pack_bf16(f[q * 8 + 2], f[q * 8 + 3]);
                o.z = pack_bf16(f[q * 8 + 4], f[q * 8 + 5]);
                o.w = pack_bf16(f[q * 8 + 6], f[q * 8 + 7]);
                d4[q] = o;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (n + i < p.N) dst[i] = __float2bfloat16(f[i]);
            }
          }
        }
      } else if constexpr (EPI == EPI_CONV) {
        const int plane = p.conv_hp * p.conv_wp;
        const int frame = m / plane;
        const int rem = m - frame * plane;
        const int hh = rem / p.conv_wp, ww = rem - hh * p.conv_wp;
        const bool interior = row_ok && frame >= p.conv_tpad && hh >= 1 && hh <= p.conv_hp - 2 && ww >= 1 &&
                              ww <= p.conv_wp - 2;
        const int n0 = tn * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          const int n = n0 + c;
          if (n >= p.N) break;  // uniform across the warp
          uint32_t v[32];
          tmem_ld32(t_addr + c, v);
          tmem_wait_ld();
          if (interior) {
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
            if (p.bias) {
#pragma unroll
              for (int i = 0; i < 32; ++i) f[i] += __bfloat162float(p.bias[n + i]);
            }
            if (p.R) {
              const uint4* r4 = reinterpret_cast<const uint4*>(p.R + (long long)m * p.ldr + n);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 rv = r4[q];
                const uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  f[q * 8 + e * 2] += bf16lo(ru[e]);
                  f[q * 8 + e * 2 + 1] += bf16hi(ru[e]);
                }
              }
            }
            uint4* d4 = reinterpret_cast<uint4*>(p.C + (long long)m * p.ldc + n);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16(f[q * 8 + 0], f[q * 8 + 1]);
              o.y = pack_bf16(f[q * 8 + 2], f[q * 8 + 3]);
              o.z = pack_bf16(f[q * 8 + 4], f[q * 8 + 5]);
              o.w = pack_bf16(f[q * 8 + 6], f[q * 8 + 7]);
              d4[q] = o;
            }
          }
        }
      } else {  // EPI_QKV_ROPE: two heads (128-column chunks) per tile
#pragma unroll 1
        for (int hc = 0; hc < 2; ++hc) {
          const int chunk = tn * 2 + hc;
          const int n = chunk * 128;
          float f[128];
#pragma unroll
          for (int c = 0; c < 128; c += 32) {
            uint32_t v[32];
            tmem_ld32(t_addr + hc * 128 + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) f[c + i] = __uint_as_float(v[i]);
          }
          if (row_ok && n < p.N) {
            if (p.bias) {
#pragma unroll
              for (int i = 0; i < 128; ++i) f[i] += __bfloat162float(p.bias[n + i]);
            }
            const int kind = chunk < p.n_q_heads ? 1 : (chunk < p.n_q_heads + p.n_k_heads ? 2 : 0);
            if (kind != 0) {
              const bf16* gam = kind == 1 ? p.gamma_q : p.gamma_k;
              if (gam) {
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < 128; ++i) ss += f[i] * f[i];
                const float rinv = rsqrtf(ss * (1.f / 128.f) + p.eps);
#pragma unroll
                for (int i = 0; i < 128; ++i) f[i] = f[i] * rinv * __bfloat162float(gam[i]);
              }
              if (p.cos_tab) {
                const float4* ct =
                    reinterpret_cast<const float4*>(p.cos_tab + (long long)(m % p.rope_rows) * 64);
                const float4* st =
                    reinterpret_cast<const float4*>(p.sin_tab + (long long)(m % p.rope_rows) * 64);
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                  const float4 c4 = ct[q], s4 = st[q];
                  const float cc[4] = {c4.x, c4.y, c4.z, c4.w};
                  const float sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const int i = q * 4 + e;
                    const float a = f[i], bb = f[i + 64];
                    f[i] = a * cc[e] - bb * sn[e];
                    f[i + 64] = bb * cc[e] + a * sn[e];
                  }
                }
              }
            }
            bf16* dst;
            if (p.route_ptr) {
              dst = reinterpret_cast<bf16*>(p.route_ptr[chunk]) + (long long)m * p.route_ld[chunk];
            } else {
              dst = p.C + (long long)m * p.ldc + n;
            }
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              uint4 o;
              o.x = pack_bf16(f[q * 8 + 0], f[q * 8 + 1]);
              o.y = pack_bf16(f[q * 8 + 2], f[q * 8 + 3]);
              o.z = pack_bf16(f[q * 8 + 4], f[q * 8 + 5]);
              o.w = pack_bf16(f[q * 8 + 6], f[q * 8 + 7]);
              d4[q] = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (NC == 2 && cta_rank != 0)
          mbar_arrive_cluster(mapa(tempty_bar(b), 0));  // the leader's MMA warp waits for both CTAs' epilogues
        else
          mbar_arrive(tempty_bar(b));
      }
    }
  }

  // ---------------- common tail
  tc_fence_before();
  __syncthreads();
  // neither CTA of a pair leaves (or frees tensor memory) while the other may still signal its
  // barriers or have MMAs in flight that read its shared memory
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

// Second pass of split-K fused with the residual add and the RMS-norm that follow an output projection in a
// decode step: x = R + sum_ks partial[ks]; X[m] = x; H[m] = x * rsqrt(mean(x^2) + eps) * gamma. One CTA per row.
constexpr int RN_THREADS = 1024;
// One CTA of 1024 threads per row: a row of 4096 columns is one float4 per thread and split, and the loads of four
// splits are in flight together (with 256 threads and one split at a time the kernel took 13 us for 147 KB).
__global__ void __launch_bounds__(RN_THREADS)
splitk_reduce_rmsnorm_kernel(const float* __restrict__ partial, int k_splits, int M, int N, const bf16* __restrict__ R,
                             long long ldr, const bf16* __restrict__ gamma, float eps, bf16* __restrict__ X,
                             bf16* __restrict__ H, long long ldc) {
  __shared__ float red[RN_THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int m = blockIdx.x, tid = threadIdx.x;
  const int nvec = N >> 2;
  constexpr int MAXJ = 2;  // N <= 8192
  float4 v[MAXJ];
  float ss = 0.f;
  const long long split_stride = (long long)M * N;
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    const int vi = tid + j * RN_THREADS;
    if (vi < nvec) {
      float4 a = make_float4(0, 0, 0, 0);
      const float* src = partial + (long long)m * N + vi * 4;
      int ks = 0;
      for (; ks + 4 <= k_splits; ks += 4) {
        const float4 x0 = *reinterpret_cast<const float4*>(src + (ks + 0) * split_stride);
        const float4 x1 = *reinterpret_cast<const float4*>(src + (ks + 1) * split_stride);
        const float4 x2 = *reinterpret_cast<const float4*>(src + (ks + 2) * split_stride);
        const float4 x3 = *reinterpret_cast<const float4*>(src + (ks + 3) * split_stride);
        a.x += (x0.x + x1.x) + (x2.x + x3.x); a.y += (x0.y + x1.y) + (x2.y + x3.y);
        a.z += (x0.z + x1.z) + (x2.z + x3.z); a.w += (x0.w + x1.w) + (x2.w + x3.w);
      }
      for (; ks < k_splits; ++ks) {
        const float4 x = *reinterpret_cast<const float4*>(src + ks * split_stride);
        a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
      }
      if (R) {
        const uint2 r = *reinterpret_cast<const uint2*>(R + (long long)m * ldr + vi * 4);
        a.x += bf16lo(r.x); a.y += bf16hi(r.x); a.z += bf16lo(r.y); a.w += bf16hi(r.y);
      }
      v[j] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < RN_THREADS / 32; ++w) tot += red[w];
  const float rinv = rsqrtf(tot / N + eps);
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    const int vi = tid + j * RN_THREADS;
    if (vi < nvec) {
      const float4 a = v[j];
      uint2 xo, ho;
      xo.x = pack_bf16(a.x, a.y); xo.y = pack_bf16(a.z, a.w);
      float g0 = 1.f, g1 = 1.f, g2 = 1.f, g3 = 1.f;
      if (gamma) {
        const uint2 g = *reinterpret_cast<const uint2*>(gamma + vi * 4);
        g0 = bf16lo(g.x); g1 = bf16hi(g.x); g2 = bf16lo(g.y); g3 = bf16hi(g.y);
      }
      ho.x = pack_bf16(a.x * rinv * g0, a.y * rinv * g1);
      ho.y = pack_bf16(a.z * rinv * g2, a.w * rinv * g3);
      *reinterpret_cast<uint2*>(X + (long long)m * ldc + vi * 4) = xo;
      *reinterpret_cast<uint2*>(H + (long long)m * ldc + vi * 4) = ho;
    }
  }
}

// Second pass of split-K: out = epilogue(sum_ks partial[ks]). One thread per 4 output columns.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, int k_splits, int M, int N, int epi, bf16* __restrict__ C,
                     long long ldc, const bf16* __restrict__ bias, const bf16* __restrict__ R, long long ldr,
                     const bf16* __restrict__ gate, int rows_per_batch) {
  pdl_launch_dependents();
  pdl_wait();
  const int n_out = epi == EPI_SWIGLU ? N / 2 : N;
  const int vec_per_row = n_out / 4;
  const long long total = (long long)M * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i / vec_per_row);
    const int n = (int)(i - (long long)m * vec_per_row) * 4;
    float4 a = make_float4(0, 0, 0, 0), u = make_float4(0, 0, 0, 0);
#pragma unroll 4
    for (int ks = 0; ks < k_splits; ++ks) {
      const float* row = partial + ((long long)ks * M + m) * N;
      const float4 x = *reinterpret_cast<const float4*>(row + n);
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
      if (epi == EPI_SWIGLU) {
        const float4 y = *reinterpret_cast<const float4*>(row + N / 2 + n);
        u.x += y.x; u.y += y.y; u.z += y.z; u.w += y.w;
      }
    }
    float f[4] = {a.x, a.y, a.z, a.w};
    if (epi == EPI_SWIGLU) {
      const float uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] = f[e] / (1.f + __expf(-f[e])) * uu[e];
    } else {
      if (bias) {
#pragma unroll
        for (int e = 0; e < 4; ++e) f[e] += __bfloat162float(bias[n + e]);
      }
      if (epi == EPI_GATED_RESID) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float gg = gate ? __bfloat162float(gate[(long long)(m / rows_per_batch) * N + n + e]) : 1.f;
          f[e] = __bfloat162float(R[(long long)m * ldr + n + e]) + gg * f[e];
        }
      }
    }
    uint2 o;
    o.x = pack_bf16(f[0], f[1]);
    o.y = pack_bf16(f[2], f[3]);
    *reinterpret_cast<uint2*>(C + (long long)m * ldc + n) = o;
  }
}

}  // namespace cb

// ====================================================================== host
namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !ptr)
      throw std::runtime_error("cuTensorMapEncodeTiled entry point not found");
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
}  // namespace

namespace cbh {
CUtensorMap make_tmap_bf16(const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  CUtensorMap m;
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  // The driver-API encode needs a current context in the calling thread; autograd's backward
  // threads may not have one bound yet, so bind the runtime's primary context once per thread.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaSetDevice(dev);
    cudaFree(nullptr);
    ctx_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    throw std::runtime_error("TMA base address must be 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i)
    if (gstr[i] % 16 != 0) throw std::runtime_error("TMA strides must be multiples of 16 bytes");
  CUresult r = get_encode()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base),
                            gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return m;
}
const char* status_str(int st) {
  switch (st & 0xff) {  // the upper bits say which wait gave up
    case cb::ST_OK: return "ok";
    case cb::ST_TIMEOUT_TMA: return "timeout: TMA producer waiting for a free stage";
    case cb::ST_TIMEOUT_MMA: return "timeout: MMA issuer waiting for data";
    case cb::ST_TIMEOUT_EPI: return "timeout: epilogue waiting for accumulators";
    case cb::ST_TIMEOUT_SOFTMAX: return "timeout: softmax waiting for scores";
    case cb::ST_TIMEOUT_PEER: return "timeout: waiting for a peer signal";
    case cb::ST_BAD_ARG: return "bad argument";
  }
  return "unknown";
}
}  // namespace cbh

namespace cosmos {

// Debug knob (gemm_set_grid_limit): caps the number of persistent CTAs, which changes which CTA computes
// which tile and how many tiles share one CTA's pipeline state. Results must not depend on it.
static int g_grid_limit = 0;

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 148;  // no device visible (host-side use of the heuristics): a B200's count
    }
  }
  return n;
}

// Whether problems with more than one 128-row tile run on CTA pairs (COSMOS_GEMM_CTA_PAIR=0 keeps
// every launch on single CTAs, for A/B timing).
static int g_debug = 0;
static int g_pair = -1;
static bool pair_enabled() {
  if (g_pair < 0) {
    const char* e = std::getenv("COSMOS_GEMM_CTA_PAIR");
    g_pair = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pair == 1;
}

template <int EPI, int NC>
static int max_grid() {
  // NC == 1: one CTA per SM. NC == 2: as many CTA pairs as the device can hold at once.
  static int n = 0;
  if (n) return n;
  cudaFuncSetAttribute(cb::gemm_bf16_kernel<EPI, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       cb::GemmCfg<NC>::SMEM);
  if (NC == 1) {
    n = sm_count();
    return n;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(sm_count() & ~1, 1, 1);
  cfg.blockDim = dim3(cb::GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = cb::GemmCfg<NC>::SMEM;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, cb::gemm_bf16_kernel<EPI, NC>, &cfg) != cudaSuccess || clusters < 1) {
    cudaGetLastError();
    clusters = sm_count() / 2;
  }
  if (clusters > sm_count() / 2) clusters = sm_count() / 2;
  n = 2 * clusters;
  return n;
}

// `units` = number of tiles (of CTA pairs when NC == 2); `limit` caps the number of CTAs (0 = none).
template <int EPI, int NC>
static void launch(const CUtensorMap* maps, const cb::GemmGroup& g, int units, int limit, cudaStream_t stream) {
  int grid = max_grid<EPI, NC>();
  if (limit > 0 && grid > limit) grid = limit;
  if (NC == 2) {
    grid &= ~1;
    if (grid < 2) grid = 2;
    if (grid > 2 * units) grid = 2 * units;
  } else if (grid > units) {
    grid = units;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(cb::GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = cb::GemmCfg<NC>::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = NC; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = (NC == 1 && pdl_on()) ? 2 : 1;
  cudaLaunchKernelEx(&cfg, cb::gemm_bf16_kernel<EPI, NC>, maps[0], maps[1], maps[2], maps[3], g);
}

template <int NC>
static void launch_epi(int epi, const CUtensorMap* maps, const cb::GemmGroup& g, int units, int limit,
                       cudaStream_t stream) {
  switch (epi) {
    case EPI_PLAIN: launch<EPI_PLAIN, NC>(maps, g, units, limit, stream); break;
    case EPI_SWIGLU: launch<EPI_SWIGLU, NC>(maps, g, units, limit, stream); break;
    case EPI_GATED_RESID: launch<EPI_GATED_RESID, NC>(maps, g, units, limit, stream); break;
    case EPI_QKV_ROPE: launch<EPI_QKV_ROPE, NC>(maps, g, units, limit, stream); break;
    case EPI_CONV: launch<EPI_CONV, NC>(maps, g, units, limit, stream); break;
    case EPI_ATTN_P: launch<EPI_ATTN_P, NC>(maps, g, units, limit, stream); break;
    case EPI_ATTN_DS: launch<EPI_ATTN_DS, NC>(maps, g, units, limit, stream); break;
    default: throw std::runtime_error("gemm_bf16: unknown epilogue");
  }
}

static void fill_problem(const GemmArgs& a, cb::GemmParams& p, CUtensorMap& ta, CUtensorMap& tb, int nc = 1) {
  // TMA needs 16-byte row strides; a ragged K is fine (out-of-range columns are zero-filled)
  if (a.lda % 8 != 0 || a.ldb % 8 != 0)
    throw std::runtime_error("gemm_bf16: leading dimensions must be multiples of 8");
  if (a.epi == EPI_SWIGLU && (a.N % 2 != 0 || (a.N / 2) % 8 != 0))
    throw std::runtime_error("gemm_bf16: SwiGLU epilogue needs N/2 to be a multiple of 8");
  if (a.epi == EPI_QKV_ROPE && a.N % 128 != 0)
    throw std::runtime_error("gemm_bf16: QKV epilogue needs N to be a multiple of 128");
  if ((a.epi == EPI_PLAIN || a.epi == EPI_GATED_RESID || a.epi == EPI_CONV) && (a.ldc % 8 != 0))
    throw std::runtime_error("gemm_bf16: ldc must be a multiple of 8");
  if (a.epi == EPI_CONV) {
    if (a.conv_c <= 0 || a.conv_c % 64 != 0 || a.K != 27 * a.conv_c || a.N % 32 != 0 || a.conv_hp < 3 ||
        a.conv_wp < 3 || a.ldc % 8 != 0)
      throw std::runtime_error("gemm_bf16: conv needs C % 64 == 0, K == 27 * C, Cout % 32 == 0 and a padded volume");
  }
  // for the convolution the A matrix is the [rows, C] volume; the K loop revisits it once per tap
  const uint64_t dimsA[2] = {(uint64_t)(a.epi == EPI_CONV ? a.conv_c : a.K), (uint64_t)a.M};
  const uint64_t strA[1] = {(uint64_t)a.lda * 2};
  const uint32_t boxA[2] = {cb::BK, cb::BM};
  const uint64_t dimsB[2] = {(uint64_t)a.K, (uint64_t)a.N};
  const uint64_t strB[1] = {(uint64_t)a.ldb * 2};
  const uint32_t boxB[2] = {cb::BK, 128};
  if (a.a_mn) {
    if (a.epi == EPI_CONV) throw std::runtime_error("gemm_bf16: the convolution needs a K-major A");
    const uint64_t d[2] = {(uint64_t)a.M, (uint64_t)a.K};
    const uint32_t bx[2] = {64, cb::BK};
    ta = cbh::make_tmap_bf16(a.A, 2, d, strA, bx, true);
  } else {
    ta = cbh::make_tmap_bf16(a.A, 2, dimsA, strA, boxA, true);
  }
  if (a.b_mn) {
    const uint64_t d[2] = {(uint64_t)a.N, (uint64_t)a.K};
    const uint32_t bx[2] = {64, cb::BK};
    tb = cbh::make_tmap_bf16(a.B, 2, d, strB, bx, true);
  } else {
    tb = cbh::make_tmap_bf16(a.B, 2, dimsB, strB, boxB, true);
  }
  p = cb::GemmParams{};
  p.rowvec = a.rowvec; p.attn_scale = a.attn_scale; p.attn_mask = a.attn_mask; p.attn_n_ar = a.attn_n_ar;
  if ((a.epi == EPI_ATTN_P || a.epi == EPI_ATTN_DS) && (!a.rowvec || a.ldc % 8 != 0))
    throw std::runtime_error("gemm_bf16: attention-backward epilogues need a row vector and ldc % 8 == 0");
  if (a.epi == EPI_ATTN_DS && (!a.R || a.ldr % 8 != 0))
    throw std::runtime_error("gemm_bf16: the dS epilogue needs P as the residual operand");
  p.a_mn = a.a_mn ? 1 : 0;
  p.b_mn = a.b_mn ? 1 : 0;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.m_tiles = (a.M + cb::BM * nc - 1) / (cb::BM * nc);
  if (a.epi == EPI_SWIGLU) {
    p.n_tiles = (a.N / 2 + 127) / 128;
    p.b_row1 = a.N / 2;
  } else {
    p.n_tiles = (a.N + cb::BN - 1) / cb::BN;
    p.b_row1 = 128;
  }
  p.mma_n = cb::BN;
  if (a.epi == EPI_CONV && a.N <= 128) {
    // a tokenizer layer with 64 or 128 output channels: a 256-column MMA would spend 3/4 or 1/2 of its cycles on
    // zero rows of B. The tile keeps its layout (one n tile, accumulator columns 0 .. N - 1); a CTA pair splits
    // the narrower B between its two CTAs.
    p.mma_n = a.N <= 64 ? 64 : 128;
    if (nc == 2) p.b_row1 = p.mma_n / 2;
  }
  p.C = reinterpret_cast<bf16*>(a.C); p.ldc = a.ldc;
  p.bias = reinterpret_cast<const bf16*>(a.bias);
  p.R = reinterpret_cast<const bf16*>(a.R); p.ldr = a.ldr;
  p.gate = reinterpret_cast<const bf16*>(a.gate);
  p.rows_per_batch = a.rows_per_batch > 0 ? a.rows_per_batch : (a.M > 0 ? a.M : 1);
  p.route_ptr = a.route_ptr; p.route_ld = a.route_ld;
  p.cos_tab = a.cos_tab; p.sin_tab = a.sin_tab; p.rope_rows = a.rope_rows > 0 ? a.rope_rows : 1;
  p.gamma_q = reinterpret_cast<const bf16*>(a.gamma_q);
  p.gamma_k = reinterpret_cast<const bf16*>(a.gamma_k);
  p.n_q_heads = a.n_q_heads; p.n_k_heads = a.n_k_heads; p.eps = a.eps;
  p.status = a.status;
  p.k_splits = 1;
  p.partial = nullptr;
  p.debug = g_debug;
  if (a.epi == EPI_CONV) {
    p.conv_cblocks = a.conv_c / 64;
    p.conv_hp = a.conv_hp; p.conv_wp = a.conv_wp; p.conv_tpad = a.conv_tpad;
    int tap = 0;
    for (int dt = 0; dt < 3; ++dt)
      for (int dh = 0; dh < 3; ++dh)
        for (int dw = 0; dw < 3; ++dw)
          p.conv_shift[tap++] = (dt - 2) * a.conv_hp * a.conv_wp + (dh - 1) * a.conv_wp + (dw - 1);
  }
}

void gemm_set_grid_limit(int max_ctas) { g_grid_limit = max_ctas > 0 ? max_ctas : 0; }
void gemm_set_cta_pair(bool on) { g_pair = on ? 1 : 0; }
void gemm_set_debug(int bits) { g_debug = bits; }

int gemm_pick_k_splits(int M, int N, int K, int epi) {
  if (epi != EPI_PLAIN && epi != EPI_SWIGLU && epi != EPI_GATED_RESID) return 1;
  const int m_tiles = (M + cb::BM - 1) / cb::BM;
  const int n_tiles = epi == EPI_SWIGLU ? (N / 2 + 127) / 128 : (N + cb::BN - 1) / cb::BN;
  const int tiles = m_tiles * n_tiles;
  const int k_blocks = (K + cb::BK - 1) / cb::BK;
  const int sms = sm_count();
  if (tiles >= sms || k_blocks < 8 || N % 8 != 0) return 1;
  if (tiles * 2 <= sms) {
    int ks = sms / tiles;                      // one wave: tiles * ks <= number of SMs
    if (ks > k_blocks / 4) ks = k_blocks / 4;  // at least 4 k-blocks (256 columns of K) per split
    if (ks > 32) ks = 32;
    return ks < 2 ? 1 : ks;
  }
  // Between half a wave and a full one (the 96 tiles of a 24576-wide SwiGLU projection leave 52 SMs idle and took
  // 59 us for 201 MB of weights): split so that the work items fill whole rounds of the persistent CTAs. Cost of a
  // choice = rounds x k-blocks per item; the smallest split count within 3 % of the best wins. Only for skinny
  // problems (at most two 128-row tiles), where the weights dominate the traffic; taller ones would pay more for
  // the fp32 partial sums than they gain.
  if (m_tiles > 2) return 1;
  int best = 1;
  double best_cost = (double)k_blocks;
  for (int ks = 2; ks <= 8 && ks <= k_blocks / 4; ++ks) {
    const int rounds = (tiles * ks + sms - 1) / sms;
    const double cost = rounds * (double)((k_blocks + ks - 1) / ks);
    if (cost < 0.97 * best_cost) {
      best = ks;
      best_cost = cost;
    }
  }
  return best;
}

// One launch for one or two problems that share the epilogue kind.
void gemm_bf16_grouped(const GemmArgs* args, int n, cudaStream_t stream) {
  if (n < 1 || n > 2) throw std::runtime_error("gemm_bf16_grouped: 1 or 2 problems per launch");
  if (n == 2 && args[0].epi != args[1].epi)
    throw std::runtime_error("gemm_bf16_grouped: both problems must use the same epilogue");
  // CTA pairs (256-row tiles) as soon as a problem has more than one 128-row tile
  const bool two = n == 2 && args[1].M > 0;
  // (not for the SwiGLU epilogue: measured 3 - 10 % slower on pairs at 16384 x 24576 x 4096)
  const int nc = (pair_enabled() && args[0].epi != EPI_SWIGLU && (args[0].M > cb::BM || (two && args[1].M > cb::BM)))
                     ? 2 : 1;
  cb::GemmGroup g{};
  CUtensorMap maps[4];
  fill_problem(args[0], g.p[0], maps[0], maps[1], nc);
  g.tiles0 = g.p[0].m_tiles * g.p[0].n_tiles;
  g.total = g.tiles0;
  if (two) {
    fill_problem(args[1], g.p[1], maps[2], maps[3], nc);
    g.total += g.p[1].m_tiles * g.p[1].n_tiles;
  } else {
    maps[2] = maps[0];
    maps[3] = maps[1];
  }
  if (g.total == 0) return;
  int limit = args[0].max_ctas > 0 ? args[0].max_ctas : 0;
  if (g_grid_limit > 0 && (limit == 0 || limit > g_grid_limit)) limit = g_grid_limit;
  if (nc == 2)
    launch_epi<2>(args[0].epi, maps, g, g.total, limit, stream);
  else
    launch_epi<1>(args[0].epi, maps, g, g.total, limit, stream);
}

void gemm_bf16(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return;
  if (a.k_splits <= 1) {
    gemm_bf16_grouped(&a, 1, stream);
    return;
  }
  // split-K: pass 1 writes fp32 partials, pass 2 reduces and applies the epilogue
  if (a.epi == EPI_QKV_ROPE) throw std::runtime_error("gemm_bf16: split-K does not support the QKV epilogue");
  if (!a.partial || a.N % 8 != 0) throw std::runtime_error("gemm_bf16: split-K needs a partial buffer and N % 8 == 0");
  cb::GemmGroup g{};
  CUtensorMap maps[4];
  // more than one 128-row tile (a serving batch of 256): CTA pairs, so that each CTA stages half of the weight tile
  // (the skinny GEMMs of such a batch are bound by operand delivery into shared memory, not by HBM)
  const int nc = (pair_enabled() && a.epi != EPI_SWIGLU && a.M > cb::BM) ? 2 : 1;
  fill_problem(a, g.p[0], maps[0], maps[1], nc);
  const int k_blocks = (a.K + cb::BK - 1) / cb::BK;
  const int ks = a.k_splits < k_blocks ? a.k_splits : k_blocks;
  g.p[0].k_splits = ks;
  g.p[0].partial = a.partial;
  g.tiles0 = g.total = g.p[0].m_tiles * g.p[0].n_tiles * ks;
  maps[2] = maps[0];
  maps[3] = maps[1];
  if (nc == 2) {
    switch (a.epi) {
      case EPI_PLAIN: launch<EPI_PLAIN, 2>(maps, g, g.total, 0, stream); break;
      case EPI_GATED_RESID: launch<EPI_GATED_RESID, 2>(maps, g, g.total, 0, stream); break;
      default: throw std::runtime_error("gemm_bf16: unknown epilogue");
    }
  } else {
    switch (a.epi) {
      case EPI_PLAIN: launch<EPI_PLAIN, 1>(maps, g, g.total, 0, stream); break;
      case EPI_SWIGLU: launch<EPI_SWIGLU, 1>(maps, g, g.total, 0, stream); break;
      case EPI_GATED_RESID: launch<EPI_GATED_RESID, 1>(maps, g, g.total, 0, stream); break;
      default: throw std::runtime_error("gemm_bf16: unknown epilogue");
    }
  }
  if (a.partial_only) return;
  if (a.norm_out) {
    if (a.epi != EPI_PLAIN || a.N > 8192 || a.N % 4 != 0 || a.ldc % 4 != 0 || (a.R && a.ldr % 4 != 0))
      throw std::runtime_error("gemm_bf16: the fused reduce + RMS-norm pass needs a plain epilogue and N <= 8192");
    launch_pdl(cb::splitk_reduce_rmsnorm_kernel, dim3(a.M), dim3(cb::RN_THREADS), 0, stream,
        a.partial, ks, a.M, a.N, reinterpret_cast<const bf16*>(a.R), a.ldr, reinterpret_cast<const bf16*>(a.norm_gamma),
        a.norm_eps, reinterpret_cast<bf16*>(a.C), reinterpret_cast<bf16*>(a.norm_out), a.ldc);
    return;
  }
  const int n_out = a.epi == EPI_SWIGLU ? a.N / 2 : a.N;
  const long long vecs = (long long)a.M * (n_out / 4);
  const int blocks = (int)std::min<long long>((vecs + 255) / 256, 148 * 8);
  launch_pdl(cb::splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream,
      a.partial, ks, a.M, a.N, a.epi, reinterpret_cast<bf16*>(a.C), a.ldc,
      reinterpret_cast<const bf16*>(a.bias), reinterpret_cast<const bf16*>(a.R), a.ldr,
      reinterpret_cast<const bf16*>(a.gate), a.rows_per_batch > 0 ? a.rows_per_batch : (a.M > 0 ? a.M : 1));
}

}  // namespace cosmos
