// K14: decode-time attention over a paged KV cache (one new query token per sequence).
//
//   q        [B, Hq, 128] bf16
//   k_cache  [num_pages, Hkv, page_size, 128] bf16   (v_cache alike; the page_size rows of one
//            (page, kv head) are contiguous, so a CTA streams whole 256 * page_size byte blocks)
//   table    [B, max_pages] int32 page ids, seq_lens [B] int32
//   out      [B, Hq, 128] bf16
//
// Decode attention is bandwidth bound (every cached K/V byte is read once per step), so the
// kernel is organised around loads: a CTA owns one (sequence, kv head, kv split) and all
// Hq/Hkv query heads that share the kv head, so K/V are read once for the whole GQA group.
// Phase 1 (thread = token): 128-dim dot products against the group's queries (held in shared
// memory, broadcast reads). Phase 2 (thread = pair of output dims): P.V with coalesced V loads.
// Long sequences are split along kv across CTAs; each split writes an unnormalised partial
// (acc, running max, running sum) to a scratch buffer and a second kernel merges the splits.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace cb {

constexpr int PD_THREADS = 128;
constexpr int PD_TILE = 128;   // tokens per tile

// 16-byte read-only load; NO_L1 skips L1 allocation for fully coalesced rows that are used once
template <bool NO_L1>
__device__ __forceinline__ uint4 ld_nc_u4(const uint4* p) {
  uint4 v;
  if (NO_L1)
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  else
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int GROUP>
__global__ void __launch_bounds__(PD_THREADS, 3)
paged_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                    const int* __restrict__ table, const int* __restrict__ seq_lens, int max_pages,
                    int page_size, int Hq, int Hkv, int n_splits, float scale_log2,
                    float* __restrict__ part_acc,   // [B, Hq, n_splits, 128]
                    float* __restrict__ part_ml,    // [B, Hq, n_splits, 2]
                    bf16* __restrict__ out          // used directly when n_splits == 1
                    COSMOS_BC_PARAMS) {
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int len = seq_lens[b];
  const int chunk = ((len + n_splits - 1) / n_splits + PD_TILE - 1) / PD_TILE * PD_TILE;
  const int kv_begin = split * chunk;
  const int kv_end = min(len, kv_begin + chunk);

  __shared__ float q_s[GROUP][128];
  __shared__ float p_s[GROUP][PD_TILE];
  __shared__ long long row_s[PD_TILE];
  __shared__ float red_s[GROUP][4];
  __shared__ float acc_s[4][GROUP][128];

  for (int i = tid; i < GROUP * 128; i += PD_THREADS) {
    const int g = i >> 7, d = i & 127;
    q_s[g][d] = __bfloat162float(q[((long long)b * Hq + kvh * GROUP + g) * 128 + d]) * scale_log2;
  }
  __syncthreads();

  float m_run[GROUP], l_run[GROUP];
  float acc[GROUP][8];
#pragma unroll
  for (int g = 0; g < GROUP; ++g) {
    m_run[g] = -1e30f; l_run[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  }
  // phase-2 mapping: 16 threads cover one 256-byte V row with 16-byte loads; 8 token groups
  const int c16 = tid & 15, tg = tid >> 4;

  for (int t0 = kv_begin; t0 < kv_end; t0 += PD_TILE) {
    // ---- phase 1: scores of this thread's token against the GROUP queries
    const int pos = t0 + tid;
    const bool valid = pos < kv_end;
    float s[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) s[g] = 0.f;
    long long row = 0;
    if (valid) {
      int page = table[(long long)b * max_pages + pos / page_size];
      if (!COSMOS_INDEX_OK(page, SITE_PAGED_DECODE_PAGE)) page = 0;  // reported; reads a valid page instead
      row = (((long long)page * Hkv + kvh) * page_size + pos % page_size) * 128;
    }
    row_s[tid] = row;
    __syncthreads();
    // All of this tile's K and V bytes are requested here, before the first use: the 256-byte K
    // row of this thread's token and, for phase 2, 16 bytes of each of 16 V rows. With three
    // CTAs per SM that keeps ~190 KB in flight per SM, which covers the DRAM latency; the
    // softmax between the two phases then runs under the V loads.
    const int n_tok = min(PD_TILE, kv_end - t0);
    uint4 kbuf[16];
    uint4 vbuf[PD_TILE / 8];
    {
      const uint4* kp = reinterpret_cast<const uint4*>(kc + row);
#pragma unroll
      for (int c = 0; c < 16; ++c) kbuf[c] = valid ? ld_nc_u4<false>(kp + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < PD_TILE / 8; ++i) {
        const int t = tg + 8 * i;
        vbuf[i] = t < n_tok ? ld_nc_u4<true>(reinterpret_cast<const uint4*>(vc + row_s[t] + 8 * c16))
                            : make_uint4(0, 0, 0, 0);
      }
    }
    if (valid) {
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint4 kk = kbuf[c];
        const float f[8] = {bf16lo(kk.x), bf16hi(kk.x), bf16lo(kk.y), bf16hi(kk.y),
                            bf16lo(kk.z), bf16hi(kk.z), bf16lo(kk.w), bf16hi(kk.w)};
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
          const float* qq = &q_s[g][c * 8];
#pragma unroll
          for (int e = 0; e < 8; ++e) s[g] = fmaf(f[e], qq[e], s[g]);
        }
      }
    }
    // tile max per head
    float mx[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      float v = valid ? s[g] : -1e30f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      mx[g] = v;
    }
    if ((tid & 31) == 0) {
#pragma unroll
      for (int g = 0; g < GROUP; ++g) red_s[g][tid >> 5] = mx[g];
    }
    __syncthreads();
    float corr[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const float tm = fmaxf(fmaxf(red_s[g][0], red_s[g][1]), fmaxf(red_s[g][2], red_s[g][3]));
      const float m_new = fmaxf(m_run[g], tm);
      corr[g] = exp2f(m_run[g] - m_new);
      m_run[g] = m_new;
      const float p = valid ? exp2f(s[g] - m_new) : 0.f;
      p_s[g][tid] = p;
      float ps = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      mx[g] = ps;  // reuse as the warp's partial sum
    }
    __syncthreads();  // p_s, row_s visible; red_s reads done
    if ((tid & 31) == 0) {
#pragma unroll
      for (int g = 0; g < GROUP; ++g) red_s[g][tid >> 5] = mx[g];
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      l_run[g] = l_run[g] * corr[g] + (red_s[g][0] + red_s[g][1] + red_s[g][2] + red_s[g][3]);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= corr[g];
    }
    // ---- phase 2: acc[g][dims 8*c16 .. +7] += sum_t p[g][t] * V[t][dims] over this thread's tokens
#pragma unroll
    for (int i = 0; i < PD_TILE / 8; ++i) {
      const int t = tg + 8 * i;
      const uint4 vv = vbuf[i];
      const float f[8] = {bf16lo(vv.x), bf16hi(vv.x), bf16lo(vv.y), bf16hi(vv.y),
                          bf16lo(vv.z), bf16hi(vv.z), bf16lo(vv.w), bf16hi(vv.w)};
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
        const float pp = p_s[g][t];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pp, f[e], acc[g][e]);
      }
    }
    __syncthreads();  // before p_s / row_s / red_s are overwritten
  }

  // combine the 8 token groups: lanes l and l^16 of a warp, then the 4 warps through shared memory
#pragma unroll
  for (int g = 0; g < GROUP; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], 16);
  if ((tid & 31) < 16) {
#pragma unroll
    for (int g = 0; g < GROUP; ++g)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc_s[tid >> 5][g][8 * c16 + e] = acc[g][e];
  }
  __syncthreads();
  if (tid < 16) {
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      float a[8];
#pragma unroll
      for (int e = 0; e < 8; ++e)
        a[e] = acc_s[0][g][8 * c16 + e] + acc_s[1][g][8 * c16 + e] + acc_s[2][g][8 * c16 + e] + acc_s[3][g][8 * c16 + e];
      const int h = kvh * GROUP + g;
      if (n_splits == 1) {
        const float inv = l_run[g] > 0.f ? 1.f / l_run[g] : 0.f;
        uint4 o;
        o.x = pack_bf16(a[0] * inv, a[1] * inv); o.y = pack_bf16(a[2] * inv, a[3] * inv);
        o.z = pack_bf16(a[4] * inv, a[5] * inv); o.w = pack_bf16(a[6] * inv, a[7] * inv);
        *reinterpret_cast<uint4*>(out + ((long long)b * Hq + h) * 128 + 8 * c16) = o;
      } else {
        const long long base = ((long long)b * Hq + h) * n_splits + split;
        float4* dst = reinterpret_cast<float4*>(part_acc + base * 128 + 8 * c16);
        dst[0] = make_float4(a[0], a[1], a[2], a[3]);
        dst[1] = make_float4(a[4], a[5], a[6], a[7]);
        if (c16 == 0) {
          part_ml[base * 2] = m_run[g];
          part_ml[base * 2 + 1] = l_run[g];
        }
      }
    }
  }
}

// out[b, h, :] = sum_s w_s acc_s / sum_s w_s l_s,  w_s = 2^(m_s - max m)
__global__ void __launch_bounds__(128)
paged_decode_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                          int n_splits, bf16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long bh = blockIdx.x;
  const int d = threadIdx.x;
  float m = -1e30f;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(bh * n_splits + s) * 2]);
  float num = 0.f, den = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float w = exp2f(part_ml[(bh * n_splits + s) * 2] - m);
    num += w * part_acc[(bh * n_splits + s) * 128 + d];
    den += w * part_ml[(bh * n_splits + s) * 2 + 1];
  }
  out[bh * 128 + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

}  // namespace cb

namespace cosmos {

int paged_decode_pick_splits(int B, int Hkv, int max_len) {
  // Several waves of CTAs (about 5 CTAs fit per SM) so that the last, partly filled wave costs
  // little, but no split shorter than 256 tokens.
  const int want = (148 * 24 + B * Hkv - 1) / (B * Hkv);
  const int cap = (max_len + 255) / 256;
  int s = want < cap ? want : cap;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return s;
}

size_t paged_decode_scratch_bytes(int B, int Hq, int n_splits) {
  return n_splits <= 1 ? 0 : (size_t)B * Hq * n_splits * (128 + 2) * sizeof(float);
}

template <int GROUP>
static void launch_pd(const PagedDecodeArgs& a, float* pa, float* pm, cudaStream_t s) {
  dim3 grid(a.n_splits, a.Hkv, a.B);
  cb::paged_decode_kernel<GROUP><<<grid, cb::PD_THREADS, 0, s>>>(
      (const bf16*)a.q, (const bf16*)a.k_cache, (const bf16*)a.v_cache, a.block_table, a.seq_lens,
      a.max_pages, a.page_size, a.Hq, a.Hkv, a.n_splits, a.scale * 1.4426950408889634f, pa, pm,
      (bf16*)a.out COSMOS_BC_ARGS(a.num_pages, a.status));
}

// Loads the CUDA-core decode kernels (every GQA group size) and the split merge kernel into the current context:
// cudaFuncGetAttributes forces the load that lazy module loading would otherwise do at a kernel's first launch.
void paged_decode_preload() {
  cudaFuncAttributes fa;
  cudaFuncGetAttributes(&fa, cb::paged_decode_kernel<1>);
  cudaFuncGetAttributes(&fa, cb::paged_decode_kernel<2>);
  cudaFuncGetAttributes(&fa, cb::paged_decode_kernel<4>);
  cudaFuncGetAttributes(&fa, cb::paged_decode_kernel<8>);
  cudaFuncGetAttributes(&fa, cb::paged_decode_merge_kernel);
}

void paged_decode(const PagedDecodeArgs& a, cudaStream_t s) {
  if (a.B <= 0) return;
  if (a.Hkv <= 0 || a.Hq % a.Hkv != 0) throw std::runtime_error("paged_decode: Hq % Hkv != 0");
  const int group = a.Hq / a.Hkv;
  if (a.n_splits < 1 || a.n_splits > 64) throw std::runtime_error("paged_decode: n_splits must be in [1, 64]");
  float* pa = nullptr;
  float* pm = nullptr;
  if (a.n_splits > 1) {
    if (!a.scratch || a.scratch_bytes < paged_decode_scratch_bytes(a.B, a.Hq, a.n_splits))
      throw std::runtime_error("paged_decode: scratch buffer missing or too small");
    pa = reinterpret_cast<float*>(a.scratch);
    pm = pa + (size_t)a.B * a.Hq * a.n_splits * 128;
  }
  if (a.impl == 0 && paged_decode_tc_supported(a)) {
    paged_decode_tc_launch(a, pa, pm, s);
  } else {
    switch (group) {
      case 1: launch_pd<1>(a, pa, pm, s); break;
      case 2: launch_pd<2>(a, pa, pm, s); break;
      case 4: launch_pd<4>(a, pa, pm, s); break;
      case 8: launch_pd<8>(a, pa, pm, s); break;
      default: throw std::runtime_error("paged_decode: GQA group size must be 1, 2, 4 or 8");
    }
  }
  if (a.n_splits > 1)
    launch_pdl(cb::paged_decode_merge_kernel, dim3(a.B * a.Hq), dim3(128), 0, s, pa, pm, a.n_splits, (bf16*)a.out);
}

}  // namespace cosmos

namespace cb {
// k, v [n_rows, Hkv, 128] -> cache rows: slot = page * page_size + offset selects the token row,
// head h of it lives at ((page * Hkv + h) * page_size + offset) * 128.
__global__ void __launch_bounds__(256)
kv_cache_write_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v, const long long* __restrict__ slots,
                      uint4* __restrict__ kc, uint4* __restrict__ vc, long long n_rows, int Hkv, int page_size
                      COSMOS_BC_PARAMS) {
  const int vec_per_row = Hkv * 16;
  const long long total = n_rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row);
    const int h = c >> 4;
    const long long slot = slots[r];
    if (!COSMOS_INDEX_OK(slot, SITE_KV_WRITE_SLOT)) continue;
    const long long page = slot / page_size;
    const int off = (int)(slot - page * page_size);
    const long long dst = (((page * Hkv + h) * page_size + off) << 4) + (c & 15);
    kc[dst] = k[i];
    vc[dst] = v[i];
  }
}
}  // namespace cb

namespace cosmos {
void kv_cache_write(const void* k, const void* v, const long long* slots, void* k_cache, void* v_cache,
                    long long n_rows, int Hkv, int page_size, long long n_slots, int* status, cudaStream_t s) {
  (void)n_slots; (void)status;  // used by the bounds-checked build
  if (n_rows <= 0) return;
  const long long total = n_rows * Hkv * 16;
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 8);
  cb::kv_cache_write_kernel<<<blocks, 256, 0, s>>>((const uint4*)k, (const uint4*)v, slots, (uint4*)k_cache,
                                                  (uint4*)v_cache, n_rows, Hkv, page_size
                                                  COSMOS_BC_ARGS(n_slots, status));
}
}  // namespace cosmos

// ====================================================================== fused decode-step glue
// One launch between the QKV GEMM and the decode attention of a decode step: q heads get the q
// RMS-norm and the rotary rotation and go to a contiguous q buffer; k heads get the k RMS-norm and
// the rotation and go straight into their cache row; v heads are copied into theirs.
// One warp per (sequence, head); a lane holds elements [2l, 2l+1] of both 64-channel halves.
namespace cb {
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256)
decode_qkv_post_kernel(const bf16* __restrict__ qkv, int B, int Hq, int Hkv, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, const bf16* __restrict__ gamma_q,
                       const bf16* __restrict__ gamma_k, float eps, const long long* __restrict__ slots,
                       bf16* __restrict__ q_out, bf16* __restrict__ kc, bf16* __restrict__ vc, int page_size,
                       const float* __restrict__ partial, int k_splits COSMOS_BC_PARAMS) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hkv;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)B * heads) return;
  const int b = (int)(w / heads), h = (int)(w % heads);
  uint32_t lo, hi;
  if (partial) {
    // the projection's split-K partial sums [k_splits, B, heads * 128] (fp32) are reduced here
    float2 a = make_float2(0.f, 0.f), c = make_float2(0.f, 0.f);
    const long long split_stride = (long long)B * heads * 128;
    const float* pp = partial + ((long long)b * heads + h) * 128;
    for (int ks = 0; ks < k_splits; ++ks, pp += split_stride) {
      const float2 x = reinterpret_cast<const float2*>(pp)[lane];
      const float2 y = reinterpret_cast<const float2*>(pp + 64)[lane];
      a.x += x.x; a.y += x.y; c.x += y.x; c.y += y.y;
    }
    lo = pack_bf16(a.x, a.y);
    hi = pack_bf16(c.x, c.y);
  } else {
    const bf16* p = qkv + ((long long)b * heads + h) * 128;
    lo = reinterpret_cast<const uint32_t*>(p)[lane];
    hi = reinterpret_cast<const uint32_t*>(p + 64)[lane];
  }
  bf16* dst;
  if (h < Hq) {
    dst = q_out + ((long long)b * Hq + h) * 128;
  } else {
    const long long slot = slots[b];
    if (!COSMOS_INDEX_OK(slot, SITE_DECODE_POST_SLOT)) return;  // whole warp: b and h are warp-uniform
    const long long page = slot / page_size;
    const int off = (int)(slot - page * page_size);
    const int hk = (h - Hq) % Hkv;
    dst = (h < Hq + Hkv ? kc : vc) + (((page * Hkv + hk) * page_size + off) << 7);
  }
  uint32_t out_lo = lo, out_hi = hi;
  if (h < Hq + Hkv) {
    const bf16* gamma = h < Hq ? gamma_q : gamma_k;
    float a0 = bf16lo(lo), a1 = bf16hi(lo), b0 = bf16lo(hi), b1 = bf16hi(hi);
    const float ss = warp_sum_f(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1);
    const float rinv = rsqrtf(ss * (1.f / 128.f) + eps);
    a0 *= rinv * __bfloat162float(gamma[2 * lane]);
    a1 *= rinv * __bfloat162float(gamma[2 * lane + 1]);
    b0 *= rinv * __bfloat162float(gamma[64 + 2 * lane]);
    b1 *= rinv * __bfloat162float(gamma[64 + 2 * lane + 1]);
    const float2 c = reinterpret_cast<const float2*>(cos_t + (long long)b * 64)[lane];
    const float2 sn = reinterpret_cast<const float2*>(sin_t + (long long)b * 64)[lane];
    out_lo = pack_bf16(a0 * c.x - b0 * sn.x, a1 * c.y - b1 * sn.y);
    out_hi = pack_bf16(b0 * c.x + a0 * sn.x, b1 * c.y + a1 * sn.y);
  }
  reinterpret_cast<uint32_t*>(dst)[lane] = out_lo;
  reinterpret_cast<uint32_t*>(dst + 64)[lane] = out_hi;
}
}  // namespace cb

namespace cosmos {
void decode_qkv_post(const void* qkv, int B, int Hq, int Hkv, const float* cos_t, const float* sin_t,
                     const void* gamma_q, const void* gamma_k, float eps, const long long* slots, void* q_out,
                     void* k_cache, void* v_cache, int page_size, long long n_slots, int* status, cudaStream_t s,
                     const float* partial, int k_splits) {
  (void)n_slots; (void)status;  // used by the bounds-checked build
  const long long warps = (long long)B * (Hq + 2 * Hkv);
  if (warps <= 0) return;
  launch_pdl(cb::decode_qkv_post_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, s,
      (const bf16*)qkv, B, Hq, Hkv, cos_t, sin_t, (const bf16*)gamma_q, (const bf16*)gamma_k, eps, slots,
      (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, page_size, partial, k_splits COSMOS_BC_ARGS(n_slots, status));
}
}  // namespace cosmos

// ====================================================================== bounds-check self-test
namespace cb {
__global__ void bounds_check_selftest_kernel(const long long* __restrict__ idx, const long long* __restrict__ limit,
                                             int* __restrict__ ok, int n, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
#ifdef COSMOS_BOUNDS_CHECK
  ok[i] = index_ok(idx[i], limit[i], status, SITE_SELFTEST) ? 1 : 0;
#else
  (void)idx; (void)limit; (void)status;
  ok[i] = 1;
#endif
}
}  // namespace cb

namespace cosmos {
bool bounds_check_enabled() {
#ifdef COSMOS_BOUNDS_CHECK
  return true;
#else
  return false;
#endif
}
void bounds_check_selftest(const long long* idx, const long long* limit, int* ok, int n, int* status, cudaStream_t s) {
  if (n <= 0) return;
  cb::bounds_check_selftest_kernel<<<(n + 127) / 128, 128, 0, s>>>(idx, limit, ok, n, status);
}
}  // namespace cosmos

// ====================================================================== allocation-free entry point
// Declared and documented in paged_decode_noalloc.h (no counterpart in the reference).
#include <cstdio>
#include <cstring>
#include <mutex>

#include "paged_decode_noalloc.h"

namespace {

constexpr size_t kNoAllocFloats = (size_t)COSMOS_PAGED_DECODE_NOALLOC_MAX_ROWS * (128 + 2);

// Split-KV partials of the allocation-free entry point. In host code this name is only a
// stand-in for the symbol; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocFloats];

constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mu;

int fail(int code, char* errbuf, int errbuf_len, const char* msg) {
  if (errbuf && errbuf_len > 0) {
    std::strncpy(errbuf, msg, (size_t)errbuf_len - 1);
    errbuf[errbuf_len - 1] = '\0';
  }
  return code;
}

// Once per device, with that device current: resolve the scratch array's device address.
int noalloc_scratch(float** out, char* errbuf, int errbuf_len) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(COSMOS_NOALLOC_CUDA_ERROR, errbuf, errbuf_len, "cudaGetDevice failed or device index out of range");
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      char msg[160];
      std::snprintf(msg, sizeof(msg), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return fail(COSMOS_NOALLOC_CUDA_ERROR, errbuf, errbuf_len, msg);
    }
    // Load every kernel this entry point can launch now (lazy module loading would otherwise do it,
    // and possibly allocate, at a variant's first launch).
    cosmos::paged_decode_preload();
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return COSMOS_NOALLOC_OK;
}

}  // namespace

extern "C" int cosmos_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                           const int* block_table, const int* seq_lens, void* out, int B,
                                           int Hq, int Hkv, int page_size, int max_pages, float scale,
                                           int n_splits, void* stream, char* errbuf, int errbuf_len) {
  if (!q || !k_cache || !v_cache || !block_table || !seq_lens || !out)
    return fail(COSMOS_NOALLOC_BAD_ARGUMENT, errbuf, errbuf_len, "null pointer argument");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || page_size <= 0 || max_pages <= 0 || Hq % Hkv != 0)
    return fail(COSMOS_NOALLOC_BAD_ARGUMENT, errbuf, errbuf_len, "bad shape (need B, Hq, Hkv, page_size, max_pages > 0 and Hq % Hkv == 0)");
  const int group = Hq / Hkv;
  if (group != 1 && group != 2 && group != 4 && group != 8)
    return fail(COSMOS_NOALLOC_BAD_ARGUMENT, errbuf, errbuf_len, "Hq / Hkv must be 1, 2, 4 or 8");
  if (n_splits < 1 || n_splits > 64)
    return fail(COSMOS_NOALLOC_BAD_ARGUMENT, errbuf, errbuf_len, "n_splits must be in [1, 64]");
  const long long rows = (long long)B * Hq * n_splits;
  if (rows > COSMOS_PAGED_DECODE_NOALLOC_MAX_ROWS) {
    char msg[200];
    std::snprintf(msg, sizeof(msg),
                  "problem too large for the built-in scratch: B*Hq*n_splits = %lld > %d rows; lower n_splits "
                  "or use the allocating entry point", rows, COSMOS_PAGED_DECODE_NOALLOC_MAX_ROWS);
    return fail(COSMOS_NOALLOC_TOO_LARGE, errbuf, errbuf_len, msg);
  }
  // an error left pending by somebody else's earlier call is theirs: report it, do not consume it
  const cudaError_t pending = cudaPeekAtLastError();
  if (pending != cudaSuccess) {
    char msg[200];
    std::snprintf(msg, sizeof(msg), "pending CUDA error from an earlier call: %s", cudaGetErrorString(pending));
    return fail(COSMOS_NOALLOC_CUDA_ERROR, errbuf, errbuf_len, msg);
  }
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch, errbuf, errbuf_len);
  if (rc != COSMOS_NOALLOC_OK) return rc;
  cosmos::PagedDecodeArgs a;
  a.q = q; a.k_cache = k_cache; a.v_cache = v_cache; a.block_table = block_table; a.seq_lens = seq_lens;
  a.out = out; a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.page_size = page_size; a.max_pages = max_pages;
  a.scale = scale; a.n_splits = n_splits;
  a.scratch = scratch; a.scratch_bytes = kNoAllocFloats * sizeof(float);
  try {
    cosmos::paged_decode(a, reinterpret_cast<cudaStream_t>(stream));
  } catch (const std::exception& ex) {
    return fail(COSMOS_NOALLOC_BAD_ARGUMENT, errbuf, errbuf_len, ex.what());
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(COSMOS_NOALLOC_CUDA_ERROR, errbuf, errbuf_len, cudaGetErrorString(e));
  return COSMOS_NOALLOC_OK;
}
