// Communication kernels over NVLink peer mappings (symmetric memory):
//   * group barrier on signal pads (st.release.sys / ld.acquire.sys, epoch-tagged, bounded wait)
//   * one-shot all-reduce for small decode activations: every rank reads all peers' buffers
//     with plain P2P loads after a barrier and reduces locally in rank order (deterministic)
//   * fused reduce-scatter + AdamW: the owner of a parameter shard pulls the matching gradient
//     slices from every peer, reduces in fp32, and applies the optimizer update in one pass
//   * reduce-scatter by pull (16-byte peer loads, or one multimem.ld_reduce per vector when the buffer
//     has an NVLink multicast mapping: the switch adds the ranks' values), fp32 shard out + sum of squares
//   * decode all-reduce fused with what surrounds it: (split-K partial sums ->) symmetric buffer ->
//     device barrier -> sum over ranks (peer loads or multimem.ld_reduce) -> + residual -> RMS-norm
// Peers never run on the same GPU as the waiting kernel (one process per GPU).
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace cb {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// pads[r] = address of rank r's signal pad (int32 words). Slot layout: pad[slot * 64 + src_rank].
// Rank `rank` writes `epoch` into every peer's pad[slot][rank], then waits until its own
// pad[slot][p] >= epoch for every p. Epochs only grow, so no reset is needed.
__device__ __forceinline__ bool barrier_device(const long long* pads, int rank, int world, int slot,
                                               int epoch, int* status) {
  const int p = threadIdx.x;
  bool ok = true;
  if (p < world) {
    __threadfence_system();
    int* remote = reinterpret_cast<int*>(pads[p]) + slot * 64 + rank;
    st_release_sys(remote, epoch);
    const int* mine = reinterpret_cast<const int*>(pads[rank]) + slot * 64 + p;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) < epoch) {
      if (clock64() - t0 > COSMOS_WAIT_LIMIT_CYCLES) {
        if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER);
        ok = false;
        break;
      }
    }
  }
  return ok;
}

__global__ void barrier_kernel(const long long* pads, int rank, int world, int slot, int epoch,
                               int* status) {
  barrier_device(pads, rank, world, slot, epoch, status);
}

// The same barrier with the epoch kept on the device (counters[slot], advanced by the kernel), so the
// launch arguments never change and the call can sit in a CUDA graph.
__global__ void barrier_counted_kernel(const long long* pads, int rank, int world, int slot, int* counters,
                                       int* status) {
  __shared__ int e_s;
  if (threadIdx.x == 0) e_s = counters[slot] + 1;
  __syncthreads();
  const int epoch = e_s;
  barrier_device(pads, rank, world, slot, epoch, status);
  __syncthreads();
  if (threadIdx.x == 0) counters[slot] = epoch;
}

// out[i] = sum_r peer_r[i] (bf16, fp32 accumulate); bufs[r] = rank r's input buffer.
// Launched on every rank after all inputs are written; the leading barrier makes the peers'
// writes visible, the trailing one keeps a fast rank from overwriting its input early.
// With `counters` (a local device array, one int per signal slot) the kernel keeps the barrier
// epoch itself: it reads counters[slot] + 1, uses that and the next value, and stores the result
// back. No launch argument changes from call to call then, so the call can sit in a CUDA graph.
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(const long long* bufs, const long long* pads, bf16* out, long long n_vec,
                         int rank, int world, int slot, int epoch, int* counters, int* status) {
  // every block runs the barrier on its own slot row, so blocks do not depend on each other
  const int myslot = slot + blockIdx.x;
  if (counters) {
    __shared__ int e_s;
    if (threadIdx.x == 0) e_s = counters[myslot] + 1;
    __syncthreads();
    epoch = e_s;
  }
  const bool ok = barrier_device(pads, rank, world, myslot, epoch, status);
  if (!__syncthreads_and(ok ? 1 : 0)) return;
  // All peers' vectors of one index are requested before the first add (eight NVLink round trips
  // in flight per thread instead of one after the other); ranks beyond eight go in further rounds.
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r0 = 0; r0 < world; r0 += 8) {
      uint4 v[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        v[r] = (r0 + r < world) ? reinterpret_cast<const uint4*>(bufs[r0 + r])[i] : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        acc[0] += bf16lo(v[r].x); acc[1] += bf16hi(v[r].x); acc[2] += bf16lo(v[r].y); acc[3] += bf16hi(v[r].y);
        acc[4] += bf16lo(v[r].z); acc[5] += bf16hi(v[r].z); acc[6] += bf16lo(v[r].w); acc[7] += bf16hi(v[r].w);
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
  __syncthreads();
  barrier_device(pads, rank, world, myslot, epoch + 1, status);
  if (counters && threadIdx.x == 0) counters[myslot] = epoch + 1;
}

// Fused reduce-scatter + AdamW on this rank's shard [shard_off, shard_off + n) of a flat
// gradient: g = (sum_r grad_r[shard_off + i]) * grad_scale, then
//   m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 ; w32 -= lr (m_hat / (sqrt(v_hat) + eps) + wd w32)
// and the bf16 parameter shard is rewritten from the fp32 master. grads[r] are peer pointers
// (plain P2P loads). With sq_out != null the kernel only accumulates sum(g^2) (pre-pass for
// global-norm clipping) and performs no update.
struct AdamW {
  float grad_scale, lr, b1, b2, eps, wd, bc1, bc2;
  __device__ __forceinline__ void step(float g, float& m, float& v, float& w) const {
    g *= grad_scale;
    m = b1 * m + (1.f - b1) * g;
    v = b2 * v + (1.f - b2) * g * g;
    w -= lr * ((m / bc1) / (sqrtf(v / bc2) + eps) + wd * w);
  }
};

// Four elements per thread and trip (8-byte gradient loads from every peer, 16-byte loads and stores of the fp32
// state) when the shard allows it; `vec` says so (offset, length and base addresses checked by the host).
__global__ void __launch_bounds__(256)
rs_adamw_kernel(const long long* grads, int world, long long shard_off, long long n,
                float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                bf16* __restrict__ param_shard, AdamW opt, float* sq_out, float* reduced_out, int vec) {
  float local_sq = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  // the gradient sources are only known here: 8-byte loads need every source 8-byte aligned at the shard's offset
  bool g_aligned = true;
  if (!(reduced_out && !sq_out))
    for (int r = 0; r < world; ++r) g_aligned = g_aligned && ((grads[r] + 2 * shard_off) & 7ll) == 0;
  const long long n4 = (vec && g_aligned) ? n >> 2 : 0;
  for (long long i4 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i4 < n4; i4 += stride) {
    const long long i = i4 << 2;
    float g[4] = {0.f, 0.f, 0.f, 0.f};
    if (reduced_out && !sq_out) {
      const float4 r = *reinterpret_cast<const float4*>(reduced_out + i);
      g[0] = r.x; g[1] = r.y; g[2] = r.z; g[3] = r.w;
    } else {
      // all peers' values are requested before the first add (one NVLink round trip, not `world`)
      for (int r0 = 0; r0 < world; r0 += 8) {
        uint2 pv[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          pv[r] = (r0 + r < world) ? *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(grads[r0 + r]) + shard_off + i)
                                   : make_uint2(0u, 0u);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          g[0] += bf16lo(pv[r].x); g[1] += bf16hi(pv[r].x); g[2] += bf16lo(pv[r].y); g[3] += bf16hi(pv[r].y);
        }
      }
    }
    if (sq_out) {
      if (reduced_out) *reinterpret_cast<float4*>(reduced_out + i) = make_float4(g[0], g[1], g[2], g[3]);
      local_sq += g[0] * g[0] + g[1] * g[1] + g[2] * g[2] + g[3] * g[3];
      continue;
    }
    float4 mm = *reinterpret_cast<const float4*>(m + i), vv = *reinterpret_cast<const float4*>(v + i);
    float4 ww = *reinterpret_cast<const float4*>(master + i);
    opt.step(g[0], mm.x, vv.x, ww.x); opt.step(g[1], mm.y, vv.y, ww.y);
    opt.step(g[2], mm.z, vv.z, ww.z); opt.step(g[3], mm.w, vv.w, ww.w);
    *reinterpret_cast<float4*>(m + i) = mm;
    *reinterpret_cast<float4*>(v + i) = vv;
    *reinterpret_cast<float4*>(master + i) = ww;
    *reinterpret_cast<uint2*>(param_shard + i) = make_uint2(pack_bf16(ww.x, ww.y), pack_bf16(ww.z, ww.w));
  }
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = 0.f;
    if (reduced_out && !sq_out) {
      g = reduced_out[i];
    } else {
      for (int r = 0; r < world; ++r) g += __bfloat162float(reinterpret_cast<const bf16*>(grads[r])[shard_off + i]);
    }
    if (sq_out) {
      if (reduced_out) reduced_out[i] = g;
      local_sq += g * g;
      continue;
    }
    float mi = m[i], vi = v[i], w = master[i];
    opt.step(g, mi, vi, w);
    m[i] = mi;
    v[i] = vi;
    master[i] = w;
    param_shard[i] = __float2bfloat16(w);
  }
  if (sq_out) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local_sq += __shfl_xor_sync(0xffffffffu, local_sq, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(sq_out, local_sq);
  }
}

// All-gather by pull: dst[r * n_vec + i] = peer_r[i]; used to materialise FSDP parameters
// from the peers' shards (one kernel, all peers in flight at once over NVSwitch).
// Each thread keeps four 16-byte peer loads in flight per trip (NVLink latency is microseconds, so the copy rate
// is bytes in flight / latency).
__global__ void __launch_bounds__(256)
allgather_pull_kernel(const long long* srcs, int world, uint4* __restrict__ dst, long long n_vec) {
  // The sources are visited round-robin in chunks of 64 vectors (1 KB), so at any moment a GPU reads from all of
  // its peers at once. Walking through the sources one after the other made every rank read the same source at the
  // same time: 366 GB/s per rank on 4 GPUs against 574 on 2.
  constexpr int CH = 64;
  const long long nch = (n_vec + CH - 1) / CH;  // chunks per source
  const long long total = nch * world * CH;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
    uint4 v[4];
    long long at[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      at[u] = -1;
      if (i < total) {
        const long long c = i / CH;
        const int r = (int)(c % world);
        const long long pos = (c / world) * CH + (i % CH);
        if (pos < n_vec) {
          v[u] = reinterpret_cast<const uint4*>(srcs[r])[pos];
          at[u] = (long long)r * n_vec + pos;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (at[u] >= 0) dst[at[u]] = v[u];
  }
}

// ------------------------------------------------------------------ NVLink multicast (NVLS)
// `mc` is the multicast address of a symmetric buffer: a load-reduce through it returns the sum over
// all ranks' copies, added inside the switch (fp32 accumulation, bf16 result); a store through it
// writes every rank's copy.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_bf16x8(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Sum over ranks of one 8-element bf16 vector at element offset `e` of the ranks' buffers, in fp32.
template <bool MC>
__device__ __forceinline__ void gather_sum8(const long long* bufs, const bf16* mc, int world, long long e,
                                            float (&acc)[8]) {
  if constexpr (MC) {
    const uint4 v = multimem_ld_reduce_bf16x8(mc + e);
    acc[0] = bf16lo(v.x); acc[1] = bf16hi(v.x); acc[2] = bf16lo(v.y); acc[3] = bf16hi(v.y);
    acc[4] = bf16lo(v.z); acc[5] = bf16hi(v.z); acc[6] = bf16lo(v.w); acc[7] = bf16hi(v.w);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int r0 = 0; r0 < world; r0 += 8) {
      uint4 v[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        v[r] = (r0 + r < world) ? *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(bufs[r0 + r]) + e)
                                : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        acc[0] += bf16lo(v[r].x); acc[1] += bf16hi(v[r].x); acc[2] += bf16lo(v[r].y); acc[3] += bf16hi(v[r].y);
        acc[4] += bf16lo(v[r].z); acc[5] += bf16hi(v[r].z); acc[6] += bf16lo(v[r].w); acc[7] += bf16hi(v[r].w);
      }
    }
  }
}

// Reduce-scatter by pull: out[i] (+)= sum_r grad_r[shard_off + i] for this rank's shard, plus the sum of
// squares of the reduced values (global-norm clipping). The caller has run a group barrier on the stream,
// so every rank's gradients are in place. n and shard_off are multiples of 8.
template <bool MC>
__global__ void __launch_bounds__(256)
reduce_scatter_pull_kernel(const long long* grads, const bf16* mc, int world, long long shard_off, long long n,
                           float* __restrict__ out, int accumulate, float scale, float* sq_out) {
  float local_sq = 0.f;
  const long long n_vec = n >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
    gather_sum8<MC>(grads, mc, world, shard_off + i * 8, acc);
    float4* o = reinterpret_cast<float4*>(out + i * 8);
    float4 a = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
    float4 b = make_float4(acc[4] * scale, acc[5] * scale, acc[6] * scale, acc[7] * scale);
    if (accumulate) {
      const float4 pa = o[0], pb = o[1];
      a.x += pa.x; a.y += pa.y; a.z += pa.z; a.w += pa.w;
      b.x += pb.x; b.y += pb.y; b.z += pb.z; b.w += pb.w;
    }
    o[0] = a;
    o[1] = b;
    local_sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
  }
  if (sq_out) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local_sq += __shfl_xor_sync(0xffffffffu, local_sq, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(sq_out, local_sq);
  }
}

// AdamW on a local fp32 gradient shard: g = grad[i] * grad_scale; moments, fp32 master and the bf16
// parameter shard are updated in one pass.
__global__ void __launch_bounds__(256)
adamw_shard_kernel(const float* __restrict__ grad, long long n, float* __restrict__ master, float* __restrict__ m,
                   float* __restrict__ v, bf16* __restrict__ param_shard, AdamW opt, int vec) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long n4 = vec ? n >> 2 : 0;
  for (long long i4 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i4 < n4; i4 += stride) {
    const long long i = i4 << 2;
    const float4 g = *reinterpret_cast<const float4*>(grad + i);
    float4 mm = *reinterpret_cast<const float4*>(m + i), vv = *reinterpret_cast<const float4*>(v + i);
    float4 ww = *reinterpret_cast<const float4*>(master + i);
    opt.step(g.x, mm.x, vv.x, ww.x); opt.step(g.y, mm.y, vv.y, ww.y);
    opt.step(g.z, mm.z, vv.z, ww.z); opt.step(g.w, mm.w, vv.w, ww.w);
    *reinterpret_cast<float4*>(m + i) = mm;
    *reinterpret_cast<float4*>(v + i) = vv;
    *reinterpret_cast<float4*>(master + i) = ww;
    *reinterpret_cast<uint2*>(param_shard + i) = make_uint2(pack_bf16(ww.x, ww.y), pack_bf16(ww.z, ww.w));
  }
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float mi = m[i], vi = v[i], w = master[i];
    opt.step(grad[i], mi, vi, w);
    m[i] = mi;
    v[i] = vi;
    master[i] = w;
    param_shard[i] = __float2bfloat16(w);
  }
}

// Decode all-reduce fused with the operations around it. Per block (one signal-slot row each, so
// blocks never wait for each other) and for the rows m = blockIdx.x, blockIdx.x + gridDim.x, ...:
//   1. (partial != null) own[m] = sum_ks partial[ks][m]   the split-K pass of the preceding GEMM, written
//      as bf16 into this rank's symmetric buffer `own`
//   2. group barrier (leading only: callers alternate two buffers, so a rank that has passed the
//      barrier of call c knows every peer has finished reading the buffer of call c - 1)
//   3. x[m] = sum_r buf_r[m] (+ R[m]);  X[m] = x;  H[m] = x * rsqrt(mean(x^2) + eps) * gamma
// MC: the sum over ranks is one multimem.ld_reduce per vector instead of `world` peer loads.
// N <= 8192, N % 8 == 0. Epochs come from `counters` (device ints, one per slot), so the launch
// arguments never change and the call can sit in a CUDA graph.
template <bool MC>
__global__ void __launch_bounds__(256)
allreduce_norm_kernel(const long long* bufs, const bf16* mc, bf16* own, const long long* pads, int rank, int world,
                      int slot, int* counters, const float* __restrict__ partial, int k_splits, int M, int N,
                      const bf16* __restrict__ R, const bf16* __restrict__ gamma, float eps, bf16* __restrict__ X,
                      bf16* __restrict__ H, int* status) {
  __shared__ float red[8];
  __shared__ int e_s;
  const int tid = threadIdx.x;
  const int nvec = N >> 3;
  constexpr int MAXJ = 4;  // 256 threads x 4 vectors x 8 = 8192 columns
  pdl_launch_dependents();
  pdl_wait();
  if (partial) {
    for (int m = blockIdx.x; m < M; m += gridDim.x) {
      for (int vi = tid; vi < nvec; vi += 256) {
        float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
        for (int ks = 0; ks < k_splits; ++ks) {
          const float4* src = reinterpret_cast<const float4*>(partial + ((long long)ks * M + m) * N + vi * 8);
          const float4 x = src[0], y = src[1];
          a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w;
          a[4] += y.x; a[5] += y.y; a[6] += y.z; a[7] += y.w;
        }
        uint4 o;
        o.x = pack_bf16(a[0], a[1]); o.y = pack_bf16(a[2], a[3]);
        o.z = pack_bf16(a[4], a[5]); o.w = pack_bf16(a[6], a[7]);
        *reinterpret_cast<uint4*>(own + (long long)m * N + vi * 8) = o;
      }
    }
  }
  const int myslot = slot + blockIdx.x;
  if (tid == 0) e_s = counters[myslot] + 1;
  __syncthreads();  // also orders this block's writes of `own` before the barrier's release stores
  const int epoch = e_s;
  const bool ok = barrier_device(pads, rank, world, myslot, epoch, status);
  const int all_ok = __syncthreads_and(ok ? 1 : 0);
  // the epoch advances even when a peer never showed up, so that the ranks stay in step afterwards
  if (tid == 0) counters[myslot] = epoch;
  if (!all_ok) return;
  for (int m = blockIdx.x; m < M; m += gridDim.x) {
    float x[MAXJ][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int vi = tid + j * 256;
      if (vi < nvec) {
        const long long e = (long long)m * N + vi * 8;
        gather_sum8<MC>(bufs, mc, world, e, x[j]);
        if (R) {
          const uint4 r = *reinterpret_cast<const uint4*>(R + e);
          x[j][0] += bf16lo(r.x); x[j][1] += bf16hi(r.x); x[j][2] += bf16lo(r.y); x[j][3] += bf16hi(r.y);
          x[j][4] += bf16lo(r.z); x[j][5] += bf16hi(r.z); x[j][6] += bf16lo(r.w); x[j][7] += bf16hi(r.w);
        }
        uint4 o;
        o.x = pack_bf16(x[j][0], x[j][1]); o.y = pack_bf16(x[j][2], x[j][3]);
        o.z = pack_bf16(x[j][4], x[j][5]); o.w = pack_bf16(x[j][6], x[j][7]);
        if (X) *reinterpret_cast<uint4*>(X + e) = o;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x[j][i] * x[j][i];
      }
    }
    if (!H) continue;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();  // `red` of the previous row has been read
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float rinv = rsqrtf(tot / N + eps);
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int vi = tid + j * 256;
      if (vi < nvec) {
        float g[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
        if (gamma) {
          const uint4 gv = *reinterpret_cast<const uint4*>(gamma + vi * 8);
          g[0] = bf16lo(gv.x); g[1] = bf16hi(gv.x); g[2] = bf16lo(gv.y); g[3] = bf16hi(gv.y);
          g[4] = bf16lo(gv.z); g[5] = bf16hi(gv.z); g[6] = bf16lo(gv.w); g[7] = bf16hi(gv.w);
        }
        uint4 o;
        o.x = pack_bf16(x[j][0] * rinv * g[0], x[j][1] * rinv * g[1]);
        o.y = pack_bf16(x[j][2] * rinv * g[2], x[j][3] * rinv * g[3]);
        o.z = pack_bf16(x[j][4] * rinv * g[4], x[j][5] * rinv * g[5]);
        o.w = pack_bf16(x[j][6] * rinv * g[6], x[j][7] * rinv * g[7]);
        *reinterpret_cast<uint4*>(H + (long long)m * N + vi * 8) = o;
      }
    }
  }
}

// out = R + gate[m / rows_per_batch] * sum_p part[p]  (tensor-parallel row-parallel GEMMs: the tp partial
// products of this rank's rows were stored by the peers' GEMM epilogues; gate may be null = 1).
__global__ void __launch_bounds__(256)
sum_partials_gated_residual_kernel(const bf16* __restrict__ part, int n_part, long long rows, int d,
                                   const bf16* __restrict__ R, const bf16* __restrict__ gate, int rows_per_batch,
                                   bf16* __restrict__ out) {
  const long long n_vec = rows * (d >> 3);
  const long long stride = rows * d;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 8;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < n_part; ++p) {
      const uint4 v = *reinterpret_cast<const uint4*>(part + p * stride + e);
      a[0] += bf16lo(v.x); a[1] += bf16hi(v.x); a[2] += bf16lo(v.y); a[3] += bf16hi(v.y);
      a[4] += bf16lo(v.z); a[5] += bf16hi(v.z); a[6] += bf16lo(v.w); a[7] += bf16hi(v.w);
    }
    if (gate) {
      const long long m = e / d;
      const int n = (int)(e - m * d);
      const uint4 g = *reinterpret_cast<const uint4*>(gate + (m / rows_per_batch) * d + n);
      a[0] *= bf16lo(g.x); a[1] *= bf16hi(g.x); a[2] *= bf16lo(g.y); a[3] *= bf16hi(g.y);
      a[4] *= bf16lo(g.z); a[5] *= bf16hi(g.z); a[6] *= bf16lo(g.w); a[7] *= bf16hi(g.w);
    }
    if (R) {
      const uint4 r = *reinterpret_cast<const uint4*>(R + e);
      a[0] += bf16lo(r.x); a[1] += bf16hi(r.x); a[2] += bf16lo(r.y); a[3] += bf16hi(r.y);
      a[4] += bf16lo(r.z); a[5] += bf16hi(r.z); a[6] += bf16lo(r.w); a[7] += bf16hi(r.w);
    }
    uint4 o;
    o.x = pack_bf16(a[0], a[1]); o.y = pack_bf16(a[2], a[3]);
    o.z = pack_bf16(a[4], a[5]); o.w = pack_bf16(a[6], a[7]);
    *reinterpret_cast<uint4*>(out + e) = o;
  }
}

}  // namespace cb

namespace cosmos {

void comm_barrier(const long long* pads_dev, int rank, int world, int slot, int epoch, int* status,
                  cudaStream_t s) {
  if (world > 64) throw std::runtime_error("comm_barrier: at most 64 ranks per group");
  cb::barrier_kernel<<<1, 64, 0, s>>>(pads_dev, rank, world, slot, epoch, status);
}

void comm_barrier_counted(const long long* pads_dev, int rank, int world, int slot, int* counters, int* status,
                          cudaStream_t s) {
  if (world > 64) throw std::runtime_error("comm_barrier: at most 64 ranks per group");
  cb::barrier_counted_kernel<<<1, 64, 0, s>>>(pads_dev, rank, world, slot, counters, status);
}

void allreduce_oneshot(const long long* bufs_dev, const long long* pads_dev, void* out,
                       long long n_elems, int rank, int world, int slot, int epoch, int* counters,
                       int* status, cudaStream_t s) {
  if (n_elems % 8 != 0) throw std::runtime_error("allreduce_oneshot: element count must be % 8");
  if (world > 64) throw std::runtime_error("allreduce_oneshot: at most 64 ranks per group");
  const long long n_vec = n_elems / 8;
  // one signal-slot row per block: slots [slot, slot + blocks) must be reserved for this call site
  int blocks = (int)std::min<long long>((n_vec + 511) / 512, 32);
  if (blocks < 1) blocks = 1;
  if (slot + blocks > 64) throw std::runtime_error("allreduce_oneshot: signal slots out of range");
  cb::allreduce_oneshot_kernel<<<blocks, 512, 0, s>>>(bufs_dev, pads_dev, (bf16*)out, n_vec, rank,
                                                     world, slot, epoch, counters, status);
}

void rs_adamw(const long long* grads_dev, int world, long long shard_off, long long n, float* master,
              float* m, float* v, void* param_shard, float grad_scale, float lr, float b1, float b2,
              float eps, float wd, int step, float* sq_out, float* reduced_out, cudaStream_t s) {
  if (n == 0) return;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  auto al = [](const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; };
  // peers' gradient buffers are symmetric allocations (page aligned), so the offset decides their alignment
  const int vec = (shard_off % 4 == 0) && al(master, 16) && al(m, 16) && al(v, 16) && al(param_shard, 8) &&
                  (!reduced_out || al(reduced_out, 16));
  const int blocks = (int)std::min<long long>(((vec ? n / 4 : n) + 255) / 256 + 1, 148 * 8);
  const cb::AdamW opt{grad_scale, lr, b1, b2, eps, wd, bc1, bc2};
  cb::rs_adamw_kernel<<<blocks, 256, 0, s>>>(grads_dev, world, shard_off, n, master, m, v, (bf16*)param_shard, opt,
                                             sq_out, reduced_out, vec);
}

void allgather_pull(const long long* srcs_dev, int world, void* dst, long long bytes_per_rank,
                    cudaStream_t s) {
  if (bytes_per_rank % 16 != 0) throw std::runtime_error("allgather_pull: shard bytes must be % 16");
  const long long n_vec = bytes_per_rank / 16;
  if (n_vec == 0) return;
  const int blocks = (int)std::min<long long>((n_vec * world + 1023) / 1024 + 1, 148 * 8);
  cb::allgather_pull_kernel<<<blocks, 256, 0, s>>>(srcs_dev, world, (uint4*)dst, n_vec);
}

void reduce_scatter_pull(const long long* grads_dev, const void* mc, int world, long long shard_off, long long n,
                         float* out, bool accumulate, float scale, float* sq_out, cudaStream_t s) {
  if (n == 0) return;
  if (n % 8 != 0 || shard_off % 8 != 0)
    throw std::runtime_error("reduce_scatter_pull: shard length and offset must be multiples of 8");
  const int blocks = (int)std::min<long long>((n / 8 + 255) / 256, 148 * 8);
  if (mc)
    cb::reduce_scatter_pull_kernel<true><<<blocks, 256, 0, s>>>(grads_dev, (const bf16*)mc, world, shard_off, n, out,
                                                                accumulate ? 1 : 0, scale, sq_out);
  else
    cb::reduce_scatter_pull_kernel<false><<<blocks, 256, 0, s>>>(grads_dev, nullptr, world, shard_off, n, out,
                                                                 accumulate ? 1 : 0, scale, sq_out);
}

void adamw_shard(const float* grad, long long n, float* master, float* m, float* v, void* param_shard,
                 float grad_scale, float lr, float b1, float b2, float eps, float wd, int step, cudaStream_t s) {
  if (n == 0) return;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  auto al = [](const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; };
  const int vec = al(grad, 16) && al(master, 16) && al(m, 16) && al(v, 16) && al(param_shard, 8);
  const int blocks = (int)std::min<long long>(((vec ? n / 4 : n) + 255) / 256 + 1, 148 * 8);
  const cb::AdamW opt{grad_scale, lr, b1, b2, eps, wd, bc1, bc2};
  cb::adamw_shard_kernel<<<blocks, 256, 0, s>>>(grad, n, master, m, v, (bf16*)param_shard, opt, vec);
}

int allreduce_norm_blocks(int M) { return M < 32 ? (M < 1 ? 1 : M) : 32; }

void allreduce_norm(const long long* bufs_dev, const void* mc, void* own, const long long* pads_dev, int rank,
                    int world, int slot, int* counters, const float* partial, int k_splits, int M, int N,
                    const void* R, const void* gamma, float eps, void* X, void* H, int* status, cudaStream_t s) {
  if (N % 8 != 0 || N > 8192) throw std::runtime_error("allreduce_norm: N must be a multiple of 8 and <= 8192");
  if (world > 64) throw std::runtime_error("allreduce_norm: at most 64 ranks per group");
  if (!counters) throw std::runtime_error("allreduce_norm: needs the group's epoch counters");
  const int blocks = allreduce_norm_blocks(M);
  if (slot + blocks > 64) throw std::runtime_error("allreduce_norm: signal slots out of range");
  if (mc)
    launch_pdl(cb::allreduce_norm_kernel<true>, dim3(blocks), dim3(256), 0, s, bufs_dev, (const bf16*)mc, (bf16*)own,
               pads_dev, rank, world, slot, counters, partial, k_splits, M, N, (const bf16*)R, (const bf16*)gamma, eps,
               (bf16*)X, (bf16*)H, status);
  else
    launch_pdl(cb::allreduce_norm_kernel<false>, dim3(blocks), dim3(256), 0, s, bufs_dev, (const bf16*)nullptr,
               (bf16*)own, pads_dev, rank, world, slot, counters, partial, k_splits, M, N, (const bf16*)R,
               (const bf16*)gamma, eps, (bf16*)X, (bf16*)H, status);
}

void sum_partials_gated_residual(const void* part, int n_part, long long rows, int d, const void* R, const void* gate,
                                 int rows_per_batch, void* out, cudaStream_t s) {
  if (rows == 0) return;
  if (d % 8 != 0) throw std::runtime_error("sum_partials_gated_residual: d must be a multiple of 8");
  const long long n_vec = rows * (d / 8);
  const int blocks = (int)std::min<long long>((n_vec + 255) / 256, 148 * 16);
  cb::sum_partials_gated_residual_kernel<<<blocks, 256, 0, s>>>((const bf16*)part, n_part, rows, d, (const bf16*)R,
                                                                (const bf16*)gate, rows_per_batch > 0 ? rows_per_batch : 1,
                                                                (bf16*)out);
}

}  // namespace cosmos
