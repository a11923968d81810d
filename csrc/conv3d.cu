// K13 support kernels for the video tokenizer's decoder on zero-padded channels-last volumes
// [frames, H + 2, W + 2, C] (bf16). The 3x3x3 causal convolutions themselves run as an implicit
// GEMM on the tensor cores (EPI_CONV in gemm_tcgen05.cu: every filter tap is a row-shifted view
// of the same flattened volume, fetched by TMA with zero fill outside). Here:
//   * nearest-neighbour upsampling (x2 in space, optionally x2 in time with the "first frame is
//     not duplicated" rule of the causal tokenizer) from one padded volume into another
//   * the final 64 -> 3 convolution fused with the [-1, 1] -> uint8 conversion (3 output channels
//     would waste a 256-wide tensor-core tile, so this one runs on the CUDA cores with the
//     weights in shared memory)
#include "common.cuh"
#include "kernels.h"

namespace cb {

// dst interior (t, h, w) <- src interior (ts, h / 2, w / 2); both volumes have `tpad` context
// frames in front that this kernel does not touch.
__global__ void __launch_bounds__(256)
upsample_cl_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int t_dst, int hs, int ws, int vec_c,
                   int tpad, int temporal, int first_chunk) {
  const int hd = 2 * hs, wd = 2 * ws;
  const long long total = (long long)t_dst * hd * wd * vec_c;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % vec_c);
    long long r = i / vec_c;
    const int w = (int)(r % wd); r /= wd;
    const int h = (int)(r % hd);
    const int t = (int)(r / hd);
    const int ts = temporal ? (first_chunk ? (t + 1) / 2 : t / 2) : t;
    const long long s_idx = (((long long)(ts + tpad) * (hs + 2) + (h / 2 + 1)) * (ws + 2) + (w / 2 + 1)) * vec_c + c;
    const long long d_idx = (((long long)(t + tpad) * (hd + 2) + (h + 1)) * (wd + 2) + (w + 1)) * vec_c + c;
    dst[d_idx] = src[s_idx];
  }
}

// out[t, h, w, 0..2] (uint8) = clamp((conv(x)[c] + bias[c] + 1) * 127.5); x: padded CL volume with
// C = 64 channels and `tpad` = 2 context frames; weights [3][27][64] fp32 in shared memory.
__global__ void __launch_bounds__(256)
conv_out_rgb_kernel(const bf16* __restrict__ x, const float* __restrict__ wgt, const float* __restrict__ bias,
                    uint8_t* __restrict__ out, int t_out, int h, int w) {
  __shared__ float w_s[3 * 27 * 64];
  for (int i = threadIdx.x; i < 3 * 27 * 64; i += blockDim.x) w_s[i] = wgt[i];
  __syncthreads();
  const int hp = h + 2, wp = w + 2;
  const long long total = (long long)t_out * h * w;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ww = (int)(i % w);
    const int hh = (int)((i / w) % h);
    const int tt = (int)(i / ((long long)w * h));
    float acc[3] = {bias[0], bias[1], bias[2]};
#pragma unroll 1
    for (int tap = 0; tap < 27; ++tap) {
      const int dt = tap / 9, dh = (tap / 3) % 3, dw = tap % 3;
      const uint4* px = reinterpret_cast<const uint4*>(
          x + ((((long long)(tt + dt) * hp + (hh + dh)) * wp + (ww + dw)) * 64));
      const float* w0 = w_s + tap * 64;
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const uint4 u = px[v];
        const float f[8] = {bf16lo(u.x), bf16hi(u.x), bf16lo(u.y), bf16hi(u.y),
                            bf16lo(u.z), bf16hi(u.z), bf16lo(u.w), bf16hi(u.w)};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          acc[0] = fmaf(f[e], w0[v * 8 + e], acc[0]);
          acc[1] = fmaf(f[e], w0[27 * 64 + v * 8 + e], acc[1]);
          acc[2] = fmaf(f[e], w0[2 * 27 * 64 + v * 8 + e], acc[2]);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      const float v = fminf(fmaxf(acc[c], -1.f), 1.f);
      out[i * 3 + c] = (uint8_t)__float2int_rn((v + 1.f) * 127.5f);
    }
  }
}

}  // namespace cb

namespace cosmos {

void upsample_cl(const void* src, void* dst, int t_dst, int hs, int ws, int c, int tpad, int temporal,
                 int first_chunk, cudaStream_t s) {
  if (c % 8 != 0) throw std::runtime_error("upsample_cl: channels must be a multiple of 8");
  const long long total = (long long)t_dst * 2 * hs * 2 * ws * (c / 8);
  if (total == 0) return;
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 16);
  cb::upsample_cl_kernel<<<blocks, 256, 0, s>>>((const uint4*)src, (uint4*)dst, t_dst, hs, ws, c / 8, tpad,
                                               temporal, first_chunk);
}

void conv_out_rgb(const void* x, const float* wgt, const float* bias, void* out, int t_out, int h, int w,
                  cudaStream_t s) {
  const long long total = (long long)t_out * h * w;
  if (total == 0) return;
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 8);
  cb::conv_out_rgb_kernel<<<blocks, 256, 0, s>>>((const bf16*)x, wgt, bias, (uint8_t*)out, t_out, h, w);
}

}  // namespace cosmos
