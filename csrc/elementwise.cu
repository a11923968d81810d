// Bandwidth-bound kernels: RMSNorm (+residual), AdaLN-modulated RMSNorm, 3D mRoPE apply
// (+ per-head q/k RMSNorm), gated residual, SwiGLU, and the CFG-combine + Euler sampler step.
// One warp per row, 16-byte vector accesses, fp32 math, bf16 storage.
#include "common.cuh"
#include "kernels.h"

namespace cb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16lo(u.x); f[1] = bf16hi(u.x); f[2] = bf16lo(u.y); f[3] = bf16hi(u.y);
  f[4] = bf16lo(u.z); f[5] = bf16hi(u.z); f[6] = bf16lo(u.w); f[7] = bf16hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
  o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
  return o;
}

// MAXV = max number of 8-element vectors a lane holds (d <= 32 * 8 * MAXV).
// MODE 0: y = norm(x [+ res]) * gamma            (res_out = x + res when given)
// MODE 1: y = norm(x) * gamma * (1 + scale) + shift
// MODE 2: y = silu(norm(x) * gamma)
template <int MAXV, int MODE>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gamma, bf16* __restrict__ y,
               long long rows, int d, float eps, const bf16* __restrict__ res_in,
               bf16* __restrict__ res_out, const bf16* __restrict__ shift,
               const bf16* __restrict__ scale, int rows_per_batch, long long mod_stride) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
  const uint4* rr = res_in ? reinterpret_cast<const uint4*>(res_in + row * d) : nullptr;
  float v[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      unpack8(xr[vi], v[i]);
      if (rr) {
        float r[8];
        unpack8(rr[vi], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += r[e];
        if (res_out) reinterpret_cast<uint4*>(res_out + row * d)[vi] = pack8(v[i]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = warp_sum(ss);
  const float rinv = rsqrtf(ss / (float)d + eps);
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  const long long b = MODE == 1 ? row / rows_per_batch : 0;
  const uint4* shr = MODE == 1 ? reinterpret_cast<const uint4*>(shift + b * mod_stride) : nullptr;
  const uint4* scr = MODE == 1 ? reinterpret_cast<const uint4*>(scale + b * mod_stride) : nullptr;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float g[8], o[8];
      if (gamma) unpack8(gr[vi], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rinv * (gamma ? g[e] : 1.f);
      if (MODE == 1) {
        float sh[8], sc[8];
        unpack8(shr[vi], sh);
        unpack8(scr[vi], sc);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = o[e] * (1.f + sc[e]) + sh[e];
      }
      if (MODE == 2) {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = o[e] / (1.f + __expf(-o[e]));
      }
      reinterpret_cast<uint4*>(y + row * d)[vi] = pack8(o);
    }
  }
}

// Wide rows (d >= 1024): one CTA per row, VPT 16-byte vectors per thread, so a thread holds few
// registers and many rows are in flight per SM (the warp-per-row kernel above keeps a whole
// 8 KB row in one warp's registers, which limits occupancy and reaches under half of HBM speed).
template <int VPT, int MODE>
__global__ void __launch_bounds__(256)
rmsnorm_row_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gamma, bf16* __restrict__ y, int d,
                   float eps, const bf16* __restrict__ res_in, bf16* __restrict__ res_out,
                   const bf16* __restrict__ shift, const bf16* __restrict__ scale, int rows_per_batch,
                   long long mod_stride) {
  __shared__ float red[8];
  const long long row = blockIdx.x;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
  const uint4* rr = res_in ? reinterpret_cast<const uint4*>(res_in + row * d) : nullptr;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (vi < nvec) {
      unpack8(xr[vi], v[i]);
      if (rr) {
        float r[8];
        unpack8(rr[vi], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += r[e];
        if (res_out) reinterpret_cast<uint4*>(res_out + row * d)[vi] = pack8(v[i]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
  const float rinv = rsqrtf(tot / (float)d + eps);
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  const long long b = MODE == 1 ? row / rows_per_batch : 0;
  const uint4* shr = MODE == 1 ? reinterpret_cast<const uint4*>(shift + b * mod_stride) : nullptr;
  const uint4* scr = MODE == 1 ? reinterpret_cast<const uint4*>(scale + b * mod_stride) : nullptr;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (vi < nvec) {
      float g[8], o[8];
      if (gamma) unpack8(gr[vi], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rinv * (gamma ? g[e] : 1.f);
      if (MODE == 1) {
        float sh[8], sc[8];
        unpack8(shr[vi], sh);
        unpack8(scr[vi], sc);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = o[e] * (1.f + sc[e]) + sh[e];
      }
      if (MODE == 2) {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = o[e] / (1.f + __expf(-o[e]));
      }
      reinterpret_cast<uint4*>(y + row * d)[vi] = pack8(o);
    }
  }
}

// One warp per (row, head): lane handles 4 of the 128 channels in both halves (i, i+64).
__global__ void __launch_bounds__(256)
mrope_kernel(bf16* __restrict__ x, long long rows, int heads, long long row_stride,
             const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rope_rows,
             const bf16* __restrict__ gamma, float eps) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= rows * heads) return;
  const long long row = w / heads;
  const int h = (int)(w % heads);
  bf16* p = x + row * row_stride + (long long)h * 128;
  // lane l: elements [2l, 2l+1] of the low half and the same of the high half
  uint32_t lo = reinterpret_cast<uint32_t*>(p)[lane];
  uint32_t hi = reinterpret_cast<uint32_t*>(p + 64)[lane];
  float a0 = bf16lo(lo), a1 = bf16hi(lo), b0 = bf16lo(hi), b1 = bf16hi(hi);
  if (gamma) {
    float ss = warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1);
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
  reinterpret_cast<uint32_t*>(p)[lane] = pack_bf16(a0, a1);
  reinterpret_cast<uint32_t*>(p + 64)[lane] = pack_bf16(b0, b1);
}

__global__ void __launch_bounds__(256)
gated_residual_kernel(const uint4* __restrict__ x, const uint4* __restrict__ f,
                      const bf16* __restrict__ gate, uint4* __restrict__ y, long long nvec_total,
                      int vec_per_row, int rows_per_batch, long long gate_stride) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec_total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vec_per_row;
    const int vi = (int)(i - row * vec_per_row);
    float a[8], b[8], g[8];
    unpack8(x[i], a);
    unpack8(f[i], b);
    if (gate) {
      unpack8(reinterpret_cast<const uint4*>(gate + (row / rows_per_batch) * gate_stride)[vi], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] += g[e] * b[e];
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] += b[e];
    }
    y[i] = pack8(a);
  }
}

__global__ void __launch_bounds__(256)
swiglu_kernel(const bf16* __restrict__ gu, bf16* __restrict__ y, long long rows, int dff) {
  const int vec_per_row = dff >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vec_per_row;
    const int vi = (int)(i - row * vec_per_row);
    const uint4* g4 = reinterpret_cast<const uint4*>(gu + row * 2 * dff);
    float g[8], u[8], o[8];
    unpack8(g4[vi], g);
    unpack8(g4[vec_per_row + vi], u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    reinterpret_cast<uint4*>(y + row * dff)[vi] = pack8(o);
  }
}

// One warp per row of the latent (d channels, d % 8 == 0, d <= 1024).
__global__ void __launch_bounds__(256)
cfg_euler_kernel(float* __restrict__ x, const bf16* __restrict__ vc, const bf16* __restrict__ vu,
                 float guidance, float dt, int normalize, long long rows, int d) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = d >> 3;
  float v[4][8];
  float nc = 0.f, nv = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float c[8];
      unpack8(reinterpret_cast<const uint4*>(vc + row * d)[vi], c);
      if (vu) {
        float u[8];
        unpack8(reinterpret_cast<const uint4*>(vu + row * d)[vi], u);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = u[e] + guidance * (c[e] - u[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = c[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        nc += c[e] * c[e];
        nv += v[i][e] * v[i][e];
      }
    }
  }
  float rs = 1.f;
  if (normalize) {
    nc = warp_sum(nc);
    nv = warp_sum(nv);
    rs = nv > 0.f ? fminf(1.f, sqrtf(nc / nv)) : 1.f;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float4* xp = reinterpret_cast<float4*>(x + row * d + vi * 8);
      float4 a = xp[0], b = xp[1];
      a.x += dt * rs * v[i][0]; a.y += dt * rs * v[i][1];
      a.z += dt * rs * v[i][2]; a.w += dt * rs * v[i][3];
      b.x += dt * rs * v[i][4]; b.y += dt * rs * v[i][5];
      b.z += dt * rs * v[i][6]; b.w += dt * rs * v[i][7];
      xp[0] = a; xp[1] = b;
    }
  }
}

// CFG combine + one UniPC step (predictor and, from the second step on, the corrector of the previous step) in one
// pass over the latent. One warp per row; d % 8 == 0, d <= 1024. With v = cfg(vc, vu):
//   x0 = x - s_cur v;   if correct: xf = cL L + cP P + cP2 P2 + cX0 x0, x0 = xf - s_cur v   else xf = x
//   out = final ? x0 : dX xf + dX0 x0 + dP P
// and then  x <- out,  L <- xf,  P2's buffer <- x0  (the caller swaps the roles of P and P2 afterwards).
// vu may be a peer GPU's buffer (CFG-parallel): it is only read.
struct UniPCCoef {
  float s_cur, cL, cP, cP2, cX0, dX, dX0, dP;
  int correct, final_step, has_p, has_p2;
};
__global__ void __launch_bounds__(256)
cfg_unipc_kernel(float* __restrict__ x, const bf16* __restrict__ vc, const bf16* __restrict__ vu,
                 float* __restrict__ L, const float* __restrict__ P, float* __restrict__ P2, float guidance,
                 int normalize, UniPCCoef k, long long rows, int d) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = d >> 3;
  float v[4][8];
  float nc = 0.f, nv = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float c[8];
      unpack8(reinterpret_cast<const uint4*>(vc + row * d)[vi], c);
      if (vu) {
        float u[8];
        unpack8(reinterpret_cast<const uint4*>(vu + row * d)[vi], u);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = u[e] + guidance * (c[e] - u[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = c[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        nc += c[e] * c[e];
        nv += v[i][e] * v[i][e];
      }
    }
  }
  float rs = 1.f;
  if (normalize) {
    nc = warp_sum(nc);
    nv = warp_sum(nv);
    rs = nv > 0.f ? fminf(1.f, sqrtf(nc / nv)) : 1.f;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      const long long off = row * d + vi * 8;
      float xv[8], lv[8], pv[8], p2v[8];
      const float4* xp = reinterpret_cast<const float4*>(x + off);
      *reinterpret_cast<float4*>(&xv[0]) = xp[0];
      *reinterpret_cast<float4*>(&xv[4]) = xp[1];
#pragma unroll
      for (int e = 0; e < 8; ++e) lv[e] = pv[e] = p2v[e] = 0.f;
      if (k.correct) {
        *reinterpret_cast<float4*>(&lv[0]) = reinterpret_cast<const float4*>(L + off)[0];
        *reinterpret_cast<float4*>(&lv[4]) = reinterpret_cast<const float4*>(L + off)[1];
      }
      if (k.has_p) {
        *reinterpret_cast<float4*>(&pv[0]) = reinterpret_cast<const float4*>(P + off)[0];
        *reinterpret_cast<float4*>(&pv[4]) = reinterpret_cast<const float4*>(P + off)[1];
      }
      if (k.has_p2 && k.correct) {
        *reinterpret_cast<float4*>(&p2v[0]) = reinterpret_cast<const float4*>(P2 + off)[0];
        *reinterpret_cast<float4*>(&p2v[4]) = reinterpret_cast<const float4*>(P2 + off)[1];
      }
      float xf[8], x0[8], out[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float ve = rs * v[i][e];
        x0[e] = xv[e] - k.s_cur * ve;
        xf[e] = xv[e];
        if (k.correct) {
          xf[e] = k.cL * lv[e] + k.cP * pv[e] + k.cP2 * p2v[e] + k.cX0 * x0[e];
          x0[e] = xf[e] - k.s_cur * ve;
        }
        out[e] = k.final_step ? x0[e] : k.dX * xf[e] + k.dX0 * x0[e] + k.dP * pv[e];
      }
      float4* xo = reinterpret_cast<float4*>(x + off);
      xo[0] = *reinterpret_cast<float4*>(&out[0]);
      xo[1] = *reinterpret_cast<float4*>(&out[4]);
      float4* lo = reinterpret_cast<float4*>(L + off);
      lo[0] = *reinterpret_cast<float4*>(&xf[0]);
      lo[1] = *reinterpret_cast<float4*>(&xf[4]);
      float4* po = reinterpret_cast<float4*>(P2 + off);
      po[0] = *reinterpret_cast<float4*>(&x0[0]);
      po[1] = *reinterpret_cast<float4*>(&x0[4]);
    }
  }
}

__global__ void l2_flush_kernel(uint4* buf, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    buf[i] = make_uint4(0, 0, 0, 0);
}

}  // namespace cb

namespace cosmos {

static bool g_pdl = false;
void set_pdl(bool on) { g_pdl = on; }
bool pdl_on() { return g_pdl; }

static void check_d(int d, const char* who) {
  if (d % 8 != 0 || d <= 0)
    throw std::runtime_error(std::string(who) + ": feature size must be a positive multiple of 8");
}

template <int MODE>
static void launch_norm(const void* x, const void* gamma, void* y, long long rows, int d, float eps,
                        const void* rin, void* rout, const void* shift, const void* scale,
                        int rows_per_batch, long long mod_stride, cudaStream_t s) {
  if (rows == 0) return;
  if (d >= 1024) {
    // one CTA per row, 4 vectors per thread (d = 4096 -> 128 threads)
    const int nvec = d / 8;
    int threads = ((nvec + 3) / 4 + 31) / 32 * 32;
    if (threads > 256) {
      if (nvec > 256 * 8) throw std::runtime_error("rmsnorm: feature size above 16384 is not supported");
      cb::rmsnorm_row_kernel<8, MODE><<<(unsigned)rows, 256, 0, s>>>(
          (const bf16*)x, (const bf16*)gamma, (bf16*)y, d, eps, (const bf16*)rin, (bf16*)rout,
          (const bf16*)shift, (const bf16*)scale, rows_per_batch, mod_stride);
    } else {
      cb::rmsnorm_row_kernel<4, MODE><<<(unsigned)rows, threads, 0, s>>>(
          (const bf16*)x, (const bf16*)gamma, (bf16*)y, d, eps, (const bf16*)rin, (bf16*)rout,
          (const bf16*)shift, (const bf16*)scale, rows_per_batch, mod_stride);
    }
    return;
  }
  const int wpb = 8;
  const unsigned grid = (unsigned)((rows + wpb - 1) / wpb);
#define COSMOS_NORM(MAXV)                                                                        \
  cb::rmsnorm_kernel<MAXV, MODE><<<grid, wpb * 32, 0, s>>>(                                      \
      (const bf16*)x, (const bf16*)gamma, (bf16*)y, rows, d, eps, (const bf16*)rin, (bf16*)rout, \
      (const bf16*)shift, (const bf16*)scale, rows_per_batch, mod_stride)
  if (d <= 256) COSMOS_NORM(1);   // one warp per row; rows of 1024 elements and more took the row kernel above
  else COSMOS_NORM(4);
#undef COSMOS_NORM
}

void rmsnorm(const void* x, const void* gamma, void* y, long long rows, int d, float eps,
             const void* residual_in, void* residual_out, cudaStream_t s) {
  check_d(d, "rmsnorm");
  launch_norm<0>(x, gamma, y, rows, d, eps, residual_in, residual_out, nullptr, nullptr, 1, 0, s);
}

void adaln_rmsnorm(const void* x, const void* gamma, const void* shift, const void* scale, void* y,
                   long long rows, int d, int rows_per_batch, long long mod_stride, float eps,
                   cudaStream_t s) {
  check_d(d, "adaln_rmsnorm");
  if (mod_stride % 8 != 0) throw std::runtime_error("adaln_rmsnorm: modulation stride % 8 != 0");
  launch_norm<1>(x, gamma, y, rows, d, eps, nullptr, nullptr, shift, scale,
                 rows_per_batch > 0 ? rows_per_batch : 1, mod_stride, s);
}

void rmsnorm_silu(const void* x, const void* gamma, void* y, long long rows, int d, float eps, cudaStream_t s) {
  check_d(d, "rmsnorm_silu");
  launch_norm<2>(x, gamma, y, rows, d, eps, nullptr, nullptr, nullptr, nullptr, 1, 0, s);
}

void mrope_apply(void* x, long long rows, int heads, long long row_stride, const float* cos_t,
                 const float* sin_t, int rope_rows, const void* gamma, float eps, cudaStream_t s) {
  const long long warps = rows * heads;
  if (warps == 0) return;
  if (row_stride % 2 != 0) throw std::runtime_error("mrope_apply: row stride must be even");
  const unsigned grid = (unsigned)((warps + 7) / 8);
  cb::mrope_kernel<<<grid, 256, 0, s>>>((bf16*)x, rows, heads, row_stride, cos_t, sin_t,
                                        rope_rows > 0 ? rope_rows : 1, (const bf16*)gamma, eps);
}

void gated_residual(const void* x, const void* f, const void* gate, void* y, long long rows, int d,
                    int rows_per_batch, long long gate_stride, cudaStream_t s) {
  check_d(d, "gated_residual");
  const long long nvec = rows * (d / 8);
  if (nvec == 0) return;
  const unsigned grid = (unsigned)std::min<long long>((nvec + 255) / 256, 148 * 16);
  cb::gated_residual_kernel<<<grid, 256, 0, s>>>((const uint4*)x, (const uint4*)f,
                                                 (const bf16*)gate, (uint4*)y, nvec, d / 8,
                                                 rows_per_batch > 0 ? rows_per_batch : 1,
                                                 gate_stride);
}

void swiglu(const void* gate_up, void* y, long long rows, int dff, cudaStream_t s) {
  check_d(dff, "swiglu");
  const long long nvec = rows * (dff / 8);
  if (nvec == 0) return;
  const unsigned grid = (unsigned)std::min<long long>((nvec + 255) / 256, 148 * 16);
  cb::swiglu_kernel<<<grid, 256, 0, s>>>((const bf16*)gate_up, (bf16*)y, rows, dff);
}

void cfg_euler_step(float* x, const void* vc, const void* vu, float guidance, float dt,
                    int normalize, long long rows, int d, cudaStream_t s) {
  check_d(d, "cfg_euler_step");
  if (d > 1024) throw std::runtime_error("cfg_euler_step: row length above 1024 is not supported");
  if (rows == 0) return;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  cb::cfg_euler_kernel<<<grid, 256, 0, s>>>(x, (const bf16*)vc, (const bf16*)vu, guidance, dt,
                                            normalize, rows, d);
}

void cfg_unipc_step(float* x, const void* vc, const void* vu, float* L, const float* P, float* P2, float guidance,
                    int normalize, const float* coef8, int correct, int final_step, int has_p, int has_p2,
                    long long rows, int d, cudaStream_t s) {
  check_d(d, "cfg_unipc_step");
  if (d > 1024) throw std::runtime_error("cfg_unipc_step: row length above 1024 is not supported");
  if (rows == 0) return;
  cb::UniPCCoef k{coef8[0], coef8[1], coef8[2], coef8[3], coef8[4], coef8[5], coef8[6], coef8[7],
                  correct, final_step, has_p, has_p2};
  const unsigned grid = (unsigned)((rows + 7) / 8);
  cb::cfg_unipc_kernel<<<grid, 256, 0, s>>>(x, (const bf16*)vc, (const bf16*)vu, L, P, P2, guidance, normalize, k,
                                            rows, d);
}

void l2_flush(void* buf, size_t bytes, cudaStream_t s) {
  cb::l2_flush_kernel<<<148 * 8, 256, 0, s>>>((uint4*)buf, bytes / 16);
}

}  // namespace cosmos
