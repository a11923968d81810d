// Backward kernels of the bandwidth-bound layer pieces (training path): RMSNorm / AdaLN-RMSNorm,
// q/k RMSNorm + rotary (with the q / k / v split), SwiGLU, gated residual. bf16 storage, fp32 math,
// 16-byte accesses. Reductions over rows (gradients of gamma, shift, scale, gate) are written as
// per-block partial sums [blocks, ..., d] in fp32 and summed by the caller, which keeps the result
// independent of the launch order.
#include "common.cuh"
#include "kernels.h"

namespace cb {

__device__ __forceinline__ float bw_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void bw_unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16lo(u.x); f[1] = bf16hi(u.x); f[2] = bf16lo(u.y); f[3] = bf16hi(u.y);
  f[4] = bf16lo(u.z); f[5] = bf16hi(u.z); f[6] = bf16lo(u.w); f[7] = bf16hi(u.w);
}
__device__ __forceinline__ uint4 bw_pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
  o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
  return o;
}

// ---------------------------------------------------------------------- RMSNorm / AdaLN rows
// y = n * w + shift,  n = x * rinv,  rinv = rsqrt(mean(x^2) + eps),  w = gamma * (1 + scale)
// dx = rinv * (dy * w) - x * rinv^3 * mean(dy * w * x);  rinv is saved for the column sums.
// One CTA (256 threads) per row, grid-strided; a thread holds up to MAXJ 8-element vectors.
constexpr int NB_THREADS = 256;
constexpr int NB_MAXJ = 4;  // d <= 8192

__global__ void __launch_bounds__(NB_THREADS)
rmsnorm_bwd_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, const bf16* __restrict__ gamma,
                        const bf16* __restrict__ scale, long long rows, int d, int rows_per_batch,
                        long long mod_stride, float eps, bf16* __restrict__ dx, float* __restrict__ rinv_out) {
  __shared__ float red[2][NB_THREADS / 32][2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nvec = d >> 3;
  float gv[NB_MAXJ][8];
#pragma unroll
  for (int j = 0; j < NB_MAXJ; ++j) {
    const int vi = tid + j * NB_THREADS;
#pragma unroll
    for (int e = 0; e < 8; ++e) gv[j][e] = 1.f;
    if (gamma && vi < nvec) bw_unpack8(reinterpret_cast<const uint4*>(gamma)[vi], gv[j]);
  }
  int it = 0;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * d);
    const uint4* sr = scale ? reinterpret_cast<const uint4*>(scale + (row / rows_per_batch) * mod_stride) : nullptr;
    float xv[NB_MAXJ][8], gw[NB_MAXJ][8];
    float a = 0.f, c = 0.f;
#pragma unroll
    for (int j = 0; j < NB_MAXJ; ++j) {
      const int vi = tid + j * NB_THREADS;
      if (vi < nvec) {
        bw_unpack8(xr[vi], xv[j]);
        bw_unpack8(gr[vi], gw[j]);
        float sc[8];
        if (sr) bw_unpack8(sr[vi], sc);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float w = sr ? gv[j][e] * (1.f + sc[e]) : gv[j][e];
          gw[j][e] *= w;
          a += xv[j][e] * xv[j][e];
          c += gw[j][e] * xv[j][e];
        }
      }
    }
    a = bw_warp_sum(a);
    c = bw_warp_sum(c);
    const int buf = it & 1;  // two buffers: the next row's writes cannot overtake this row's reads
    if (lane == 0) {
      red[buf][warp][0] = a;
      red[buf][warp][1] = c;
    }
    __syncthreads();
    float A = 0.f, C = 0.f;
#pragma unroll
    for (int w = 0; w < NB_THREADS / 32; ++w) {
      A += red[buf][w][0];
      C += red[buf][w][1];
    }
    const float rinv = rsqrtf(A / d + eps);
    const float k = rinv * rinv * rinv * (C / d);
    if (tid == 0 && rinv_out) rinv_out[row] = rinv;
    uint4* dr = reinterpret_cast<uint4*>(dx + row * d);
#pragma unroll
    for (int j = 0; j < NB_MAXJ; ++j) {
      const int vi = tid + j * NB_THREADS;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rinv * gw[j][e] - xv[j][e] * k;
        dr[vi] = bw_pack8(o);
      }
    }
  }
}

// Column sums of one block of rows (all in batch `b`), one 8-column vector per thread:
//   part[b][blk][0][col] = sum dy                    (d shift)
//   part[b][blk][1][col] = sum dy * n * gamma        (d scale)
//   part[b][blk][2][col] = sum dy * n * (1 + scale)  (d gamma)          n = x * rinv[row]
constexpr int CS_ROWS = 64;
__global__ void __launch_bounds__(128)
rmsnorm_bwd_cols_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, const float* __restrict__ rinv,
                        const bf16* __restrict__ gamma, const bf16* __restrict__ scale, int d, int rows_per_batch,
                        long long mod_stride, float* __restrict__ part) {
  const int nvec = d >> 3;
  const int vi = blockIdx.x * 128 + threadIdx.x;
  if (vi >= nvec) return;
  const int blk = blockIdx.y, b = blockIdx.z, nblk = gridDim.y;
  const long long r0 = (long long)b * rows_per_batch + (long long)blk * CS_ROWS;
  const int n = min(CS_ROWS, rows_per_batch - blk * CS_ROWS);
  float g[8], sc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { g[e] = 1.f; sc[e] = 0.f; }
  if (gamma) bw_unpack8(reinterpret_cast<const uint4*>(gamma)[vi], g);
  if (scale) bw_unpack8(reinterpret_cast<const uint4*>(scale + (long long)b * mod_stride)[vi], sc);
  float s0[8] = {0, 0, 0, 0, 0, 0, 0, 0}, s1[8] = {0, 0, 0, 0, 0, 0, 0, 0}, s2[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
  for (int i = 0; i < n; ++i) {
    const long long row = r0 + i;
    float xv[8], gy[8];
    bw_unpack8(reinterpret_cast<const uint4*>(x + row * d)[vi], xv);
    bw_unpack8(reinterpret_cast<const uint4*>(dy + row * d)[vi], gy);
    const float ri = rinv[row];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float t = gy[e] * xv[e] * ri;
      s0[e] += gy[e];
      s1[e] += t * g[e];
      s2[e] += t * (1.f + sc[e]);
    }
  }
  float* dst = part + (((long long)b * nblk + blk) * 3) * d + (long long)vi * 8;
  reinterpret_cast<float4*>(dst)[0] = make_float4(s0[0], s0[1], s0[2], s0[3]);
  reinterpret_cast<float4*>(dst)[1] = make_float4(s0[4], s0[5], s0[6], s0[7]);
  reinterpret_cast<float4*>(dst + d)[0] = make_float4(s1[0], s1[1], s1[2], s1[3]);
  reinterpret_cast<float4*>(dst + d)[1] = make_float4(s1[4], s1[5], s1[6], s1[7]);
  reinterpret_cast<float4*>(dst + 2 * d)[0] = make_float4(s2[0], s2[1], s2[2], s2[3]);
  reinterpret_cast<float4*>(dst + 2 * d)[1] = make_float4(s2[4], s2[5], s2[6], s2[7]);
}

// ---------------------------------------------------------------------- gated residual
// y = resid + gate[b] * f:  df = dy * gate[b]; part[b][blk][col] = sum_rows dy * f  (d gate)
__global__ void __launch_bounds__(128)
gated_residual_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ f, const bf16* __restrict__ gate,
                          int d, int rows_per_batch, long long gate_stride, bf16* __restrict__ df,
                          float* __restrict__ part) {
  const int nvec = d >> 3;
  const int vi = blockIdx.x * 128 + threadIdx.x;
  if (vi >= nvec) return;
  const int blk = blockIdx.y, b = blockIdx.z, nblk = gridDim.y;
  const long long r0 = (long long)b * rows_per_batch + (long long)blk * CS_ROWS;
  const int n = min(CS_ROWS, rows_per_batch - blk * CS_ROWS);
  float g[8];
  bw_unpack8(reinterpret_cast<const uint4*>(gate + (long long)b * gate_stride)[vi], g);
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
  for (int i = 0; i < n; ++i) {
    const long long row = r0 + i;
    float gy[8], fv[8], o[8];
    bw_unpack8(reinterpret_cast<const uint4*>(dy + row * d)[vi], gy);
    bw_unpack8(reinterpret_cast<const uint4*>(f + row * d)[vi], fv);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      o[e] = gy[e] * g[e];
      s[e] += gy[e] * fv[e];
    }
    reinterpret_cast<uint4*>(df + row * d)[vi] = bw_pack8(o);
  }
  float* dst = part + ((long long)b * nblk + blk) * d + (long long)vi * 8;
  reinterpret_cast<float4*>(dst)[0] = make_float4(s[0], s[1], s[2], s[3]);
  reinterpret_cast<float4*>(dst)[1] = make_float4(s[4], s[5], s[6], s[7]);
}

// ---------------------------------------------------------------------- SwiGLU
// y = silu(g) * u with gate_up = [g | u]:  dg = dy * u * sig * (1 + g * (1 - sig)),  du = dy * silu(g)
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const bf16* __restrict__ gate_up, const bf16* __restrict__ dy, bf16* __restrict__ d_gate_up,
                  long long rows, int dff) {
  const int vec_per_row = dff >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vec_per_row;
    const int vi = (int)(i - row * vec_per_row);
    const uint4* src = reinterpret_cast<const uint4*>(gate_up + row * 2 * dff);
    float g[8], u[8], gy[8], dg[8], du[8];
    bw_unpack8(src[vi], g);
    bw_unpack8(src[vec_per_row + vi], u);
    bw_unpack8(reinterpret_cast<const uint4*>(dy)[i], gy);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sig = 1.f / (1.f + __expf(-g[e]));
      dg[e] = gy[e] * u[e] * sig * (1.f + g[e] * (1.f - sig));
      du[e] = gy[e] * g[e] * sig;
    }
    uint4* dst = reinterpret_cast<uint4*>(d_gate_up + row * 2 * dff);
    dst[vi] = bw_pack8(dg);
    dst[vec_per_row + vi] = bw_pack8(du);
  }
}

// ---------------------------------------------------------------------- q/k norm + rotary, q/k/v split
// Forward: qkv [rows, Hq + 2 Hkv, 128] -> q [rows, Hq, 128], k, v [rows, Hkv, 128]; q and k heads get
// RMS-norm (gamma_q / gamma_k, may be null) and the rotary rotation (cos/sin [rope_rows, 64], row
// r uses table row r % rope_rows; may be null). One warp per (row, head); a lane holds elements
// [2l, 2l+1] of both 64-channel halves.
__global__ void __launch_bounds__(256)
qkv_post_fwd_kernel(const bf16* __restrict__ qkv, long long rows, int Hq, int Hkv, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, int rope_rows, const bf16* __restrict__ gamma_q,
                    const bf16* __restrict__ gamma_k, float eps, bf16* __restrict__ q, bf16* __restrict__ k,
                    bf16* __restrict__ v) {
  const int lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hkv;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= rows * heads) return;
  const long long row = w / heads;
  const int h = (int)(w % heads);
  const bf16* p = qkv + w * 128;
  const uint32_t lo = reinterpret_cast<const uint32_t*>(p)[lane];
  const uint32_t hi = reinterpret_cast<const uint32_t*>(p + 64)[lane];
  bf16* dst;
  if (h < Hq) dst = q + (row * Hq + h) * 128;
  else if (h < Hq + Hkv) dst = k + (row * Hkv + (h - Hq)) * 128;
  else dst = v + (row * Hkv + (h - Hq - Hkv)) * 128;
  uint32_t out_lo = lo, out_hi = hi;
  if (h < Hq + Hkv) {
    const bf16* gamma = h < Hq ? gamma_q : gamma_k;
    float a0 = bf16lo(lo), a1 = bf16hi(lo), b0 = bf16lo(hi), b1 = bf16hi(hi);
    if (gamma) {
      const float ss = bw_warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1);
      const float rinv = rsqrtf(ss * (1.f / 128.f) + eps);
      a0 *= rinv * __bfloat162float(gamma[2 * lane]);
      a1 *= rinv * __bfloat162float(gamma[2 * lane + 1]);
      b0 *= rinv * __bfloat162float(gamma[64 + 2 * lane]);
      b1 *= rinv * __bfloat162float(gamma[64 + 2 * lane + 1]);
    }
    if (cos_t) {
      const long long tr = (row % rope_rows) * 64;
      const float2 c = reinterpret_cast<const float2*>(cos_t + tr)[lane];
      const float2 s = reinterpret_cast<const float2*>(sin_t + tr)[lane];
      const float r0 = a0 * c.x - b0 * s.x, r1 = a1 * c.y - b1 * s.y;
      const float q0 = b0 * c.x + a0 * s.x, q1 = b1 * c.y + a1 * s.y;
      a0 = r0; a1 = r1; b0 = q0; b1 = q1;
    }
    out_lo = pack_bf16(a0, a1);
    out_hi = pack_bf16(b0, b1);
  }
  reinterpret_cast<uint32_t*>(dst)[lane] = out_lo;
  reinterpret_cast<uint32_t*>(dst + 64)[lane] = out_hi;
}

// Backward of the above: d_qkv from (dq, dk, dv) and the raw qkv; per-CTA partial sums of d gamma_q /
// d gamma_k in part[block][2][128].
__global__ void __launch_bounds__(256)
qkv_post_bwd_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ dq, const bf16* __restrict__ dk,
                    const bf16* __restrict__ dv, long long rows, int Hq, int Hkv, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, int rope_rows, const bf16* __restrict__ gamma_q,
                    const bf16* __restrict__ gamma_k, float eps, bf16* __restrict__ d_qkv,
                    float* __restrict__ part) {
  __shared__ float acc[2][128];
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 256) acc[threadIdx.x >> 7][threadIdx.x & 127] = 0.f;
  __syncthreads();
  const int heads = Hq + 2 * Hkv;
  const long long total = rows * heads;
  for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total;
       w += (long long)gridDim.x * (blockDim.x >> 5)) {
    const long long row = w / heads;
    const int h = (int)(w % heads);
    const bf16* src;
    if (h < Hq) src = dq + (row * Hq + h) * 128;
    else if (h < Hq + Hkv) src = dk + (row * Hkv + (h - Hq)) * 128;
    else src = dv + (row * Hkv + (h - Hq - Hkv)) * 128;
    const uint32_t glo = reinterpret_cast<const uint32_t*>(src)[lane];
    const uint32_t ghi = reinterpret_cast<const uint32_t*>(src + 64)[lane];
    uint32_t out_lo = glo, out_hi = ghi;
    if (h < Hq + Hkv) {
      const int which = h < Hq ? 0 : 1;
      const bf16* gamma = which == 0 ? gamma_q : gamma_k;
      float ga0 = bf16lo(glo), ga1 = bf16hi(glo), gb0 = bf16lo(ghi), gb1 = bf16hi(ghi);
      if (cos_t) {  // transpose of the rotation
        const long long tr = (row % rope_rows) * 64;
        const float2 c = reinterpret_cast<const float2*>(cos_t + tr)[lane];
        const float2 s = reinterpret_cast<const float2*>(sin_t + tr)[lane];
        const float t0 = ga0 * c.x + gb0 * s.x, t1 = ga1 * c.y + gb1 * s.y;
        const float u0 = gb0 * c.x - ga0 * s.x, u1 = gb1 * c.y - ga1 * s.y;
        ga0 = t0; ga1 = t1; gb0 = u0; gb1 = u1;
      }
      if (gamma) {
        const bf16* p = qkv + w * 128;
        const uint32_t lo = reinterpret_cast<const uint32_t*>(p)[lane];
        const uint32_t hi = reinterpret_cast<const uint32_t*>(p + 64)[lane];
        const float x0 = bf16lo(lo), x1 = bf16hi(lo), x2 = bf16lo(hi), x3 = bf16hi(hi);
        const float ss = bw_warp_sum(x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3);
        const float rinv = rsqrtf(ss * (1.f / 128.f) + eps);
        const float n0 = x0 * rinv, n1 = x1 * rinv, n2 = x2 * rinv, n3 = x3 * rinv;
        atomicAdd(&acc[which][2 * lane], ga0 * n0);
        atomicAdd(&acc[which][2 * lane + 1], ga1 * n1);
        atomicAdd(&acc[which][64 + 2 * lane], gb0 * n2);
        atomicAdd(&acc[which][64 + 2 * lane + 1], gb1 * n3);
        const float w0 = ga0 * __bfloat162float(gamma[2 * lane]), w1 = ga1 * __bfloat162float(gamma[2 * lane + 1]);
        const float w2 = gb0 * __bfloat162float(gamma[64 + 2 * lane]);
        const float w3 = gb1 * __bfloat162float(gamma[64 + 2 * lane + 1]);
        const float m = bw_warp_sum(w0 * n0 + w1 * n1 + w2 * n2 + w3 * n3) * (1.f / 128.f);
        ga0 = rinv * (w0 - n0 * m); ga1 = rinv * (w1 - n1 * m);
        gb0 = rinv * (w2 - n2 * m); gb1 = rinv * (w3 - n3 * m);
      }
      out_lo = pack_bf16(ga0, ga1);
      out_hi = pack_bf16(gb0, gb1);
    }
    bf16* dst = d_qkv + w * 128;
    reinterpret_cast<uint32_t*>(dst)[lane] = out_lo;
    reinterpret_cast<uint32_t*>(dst + 64)[lane] = out_hi;
  }
  __syncthreads();
  if (part && threadIdx.x < 256)
    part[(long long)blockIdx.x * 256 + threadIdx.x] = acc[threadIdx.x >> 7][threadIdx.x & 127];
}

}  // namespace cb

namespace cosmos {

static void check_d8(int d, const char* what) {
  if (d <= 0 || d % 8 != 0) throw std::runtime_error(std::string(what) + ": row length must be a positive multiple of 8");
}

void rmsnorm_bwd(const void* x, const void* dy, const void* gamma, const void* scale, long long rows, int d,
                 int rows_per_batch, long long mod_stride, float eps, void* dx, float* rinv, float* part,
                 cudaStream_t s) {
  check_d8(d, "rmsnorm_bwd");
  if (d > 8 * cb::NB_THREADS * cb::NB_MAXJ) throw std::runtime_error("rmsnorm_bwd: row length above 8192 is not supported");
  if (rows <= 0) return;
  if (rows_per_batch <= 0 || rows % rows_per_batch != 0) throw std::runtime_error("rmsnorm_bwd: rows must be a multiple of rows_per_batch");
  const int grid = (int)std::min<long long>(rows, 148 * 8);
  cb::rmsnorm_bwd_rows_kernel<<<grid, cb::NB_THREADS, 0, s>>>((const bf16*)x, (const bf16*)dy, (const bf16*)gamma,
                                                             (const bf16*)scale, rows, d, rows_per_batch, mod_stride,
                                                             eps, (bf16*)dx, rinv);
  if (part) {
    const int nvec = d / 8;
    dim3 g((nvec + 127) / 128, rmsnorm_bwd_blocks(rows_per_batch), (unsigned)(rows / rows_per_batch));
    cb::rmsnorm_bwd_cols_kernel<<<g, 128, 0, s>>>((const bf16*)x, (const bf16*)dy, rinv, (const bf16*)gamma,
                                                 (const bf16*)scale, d, rows_per_batch, mod_stride, part);
  }
}

int rmsnorm_bwd_blocks(int rows_per_batch) { return (rows_per_batch + cb::CS_ROWS - 1) / cb::CS_ROWS; }

void gated_residual_bwd(const void* dy, const void* f, const void* gate, long long rows, int d, int rows_per_batch,
                        long long gate_stride, void* df, float* part, cudaStream_t s) {
  check_d8(d, "gated_residual_bwd");
  if (rows <= 0) return;
  if (rows_per_batch <= 0 || rows % rows_per_batch != 0) throw std::runtime_error("gated_residual_bwd: rows must be a multiple of rows_per_batch");
  const int nvec = d / 8;
  dim3 g((nvec + 127) / 128, rmsnorm_bwd_blocks(rows_per_batch), (unsigned)(rows / rows_per_batch));
  cb::gated_residual_bwd_kernel<<<g, 128, 0, s>>>((const bf16*)dy, (const bf16*)f, (const bf16*)gate, d, rows_per_batch,
                                                 gate_stride, (bf16*)df, part);
}

void swiglu_bwd(const void* gate_up, const void* dy, void* d_gate_up, long long rows, int dff, cudaStream_t s) {
  check_d8(dff, "swiglu_bwd");
  const long long nvec = rows * (dff / 8);
  if (nvec <= 0) return;
  const unsigned grid = (unsigned)std::min<long long>((nvec + 255) / 256, 148 * 16);
  cb::swiglu_bwd_kernel<<<grid, 256, 0, s>>>((const bf16*)gate_up, (const bf16*)dy, (bf16*)d_gate_up, rows, dff);
}

void qkv_post_fwd(const void* qkv, long long rows, int Hq, int Hkv, const float* cos_t, const float* sin_t,
                  int rope_rows, const void* gamma_q, const void* gamma_k, float eps, void* q, void* k, void* v,
                  cudaStream_t s) {
  const long long warps = rows * (Hq + 2 * Hkv);
  if (warps <= 0) return;
  cb::qkv_post_fwd_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>(
      (const bf16*)qkv, rows, Hq, Hkv, cos_t, sin_t, rope_rows > 0 ? rope_rows : 1, (const bf16*)gamma_q,
      (const bf16*)gamma_k, eps, (bf16*)q, (bf16*)k, (bf16*)v);
}

int qkv_post_bwd_blocks(long long rows, int Hq, int Hkv) {
  const long long warps = rows * (Hq + 2 * Hkv);
  return (int)std::max<long long>(1, std::min<long long>((warps + 7) / 8, 148 * 8));
}

void qkv_post_bwd(const void* qkv, const void* dq, const void* dk, const void* dv, long long rows, int Hq, int Hkv,
                  const float* cos_t, const float* sin_t, int rope_rows, const void* gamma_q, const void* gamma_k,
                  float eps, void* d_qkv, float* part, cudaStream_t s) {
  if (rows <= 0) return;
  cb::qkv_post_bwd_kernel<<<qkv_post_bwd_blocks(rows, Hq, Hkv), 256, 0, s>>>(
      (const bf16*)qkv, (const bf16*)dq, (const bf16*)dk, (const bf16*)dv, rows, Hq, Hkv, cos_t, sin_t,
      rope_rows > 0 ? rope_rows : 1, (const bf16*)gamma_q, (const bf16*)gamma_k, eps, (bf16*)d_qkv, part);
}

}  // namespace cosmos
