// Communication kernels over NVLink peer mappings (symmetric memory):
//   * group barrier on signal pads (st.release.sys / ld.acquire.sys, epoch-tagged, bounded wait)
//   * one-shot all-reduce for small decode activations: every rank reads all peers' buffers
//     with plain P2P loads after a barrier and reduces locally in rank order (deterministic)
//   * fused reduce-scatter + AdamW: the owner of a parameter shard pulls the matching gradient
//     slices from every peer, reduces in fp32, and applies the optimizer update in one pass
// Peers never run on the same GPU as the waiting kernel (one process per GPU).
#include "common.cuh"
#include "kernels.h"

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
__global__ void __launch_bounds__(256)
rs_adamw_kernel(const long long* grads, int world, long long shard_off, long long n,
                float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                bf16* __restrict__ param_shard, float grad_scale, float lr, float b1, float b2,
                float eps, float wd, float bc1, float bc2, float* sq_out, float* reduced_out) {
  float local_sq = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float g = 0.f;
    if (reduced_out && !sq_out) {
      g = reduced_out[i];
    } else {
      for (int r = 0; r < world; ++r)
        g += __bfloat162float(reinterpret_cast<const bf16*>(grads[r])[shard_off + i]);
    }
    if (sq_out) {
      if (reduced_out) reduced_out[i] = g;
      local_sq += g * g;
      continue;
    }
    g *= grad_scale;
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    float w = master[i];
    w -= lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * w);
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
__global__ void __launch_bounds__(256)
allgather_pull_kernel(const long long* srcs, int world, uint4* __restrict__ dst, long long n_vec) {
  const long long total = n_vec * world;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n_vec);
    dst[i] = reinterpret_cast<const uint4*>(srcs[r])[i - (long long)r * n_vec];
  }
}

}  // namespace cb

namespace cosmos {

void comm_barrier(const long long* pads_dev, int rank, int world, int slot, int epoch, int* status,
                  cudaStream_t s) {
  if (world > 64) throw std::runtime_error("comm_barrier: at most 64 ranks per group");
  cb::barrier_kernel<<<1, 64, 0, s>>>(pads_dev, rank, world, slot, epoch, status);
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
  const int blocks = (int)std::min<long long>((n + 255) / 256, 148 * 8);
  cb::rs_adamw_kernel<<<blocks, 256, 0, s>>>(grads_dev, world, shard_off, n, master, m, v,
                                             (bf16*)param_shard, grad_scale, lr, b1, b2, eps, wd, bc1,
                                             bc2, sq_out, reduced_out);
}

void allgather_pull(const long long* srcs_dev, int world, void* dst, long long bytes_per_rank,
                    cudaStream_t s) {
  if (bytes_per_rank % 16 != 0) throw std::runtime_error("allgather_pull: shard bytes must be % 16");
  const long long n_vec = bytes_per_rank / 16;
  if (n_vec == 0) return;
  const int blocks = (int)std::min<long long>((n_vec * world + 255) / 256, 148 * 16);
  cb::allgather_pull_kernel<<<blocks, 256, 0, s>>>(srcs_dev, world, (uint4*)dst, n_vec);
}

}  // namespace cosmos
