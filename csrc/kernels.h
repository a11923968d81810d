// Host-callable launchers of the sm_100a kernel library. Plain C++ (no torch types) so the
// .cu files compile in seconds; the torch glue lives in bindings.cpp.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

enum GemmEpilogue : int {
  EPI_PLAIN = 0,
  EPI_SWIGLU = 1,
  EPI_GATED_RESID = 2,
  EPI_QKV_ROPE = 3,
  EPI_CONV = 4,  // implicit-GEMM causal 3x3x3 convolution on a zero-padded channels-last volume
  // attention backward (scores are materialised per head): C = exp(acc * scale - lse[m]) under the mask
  EPI_ATTN_P = 5,
  // C = P[m, n] * (acc - D[m]) * scale, with P passed as the residual operand
  EPI_ATTN_DS = 6,
};

enum AttnMask : int {
  MASK_FULL = 0,    // every query sees every key
  MASK_CAUSAL = 1,  // query i sees keys j <= i + (Skv - Sq)
  MASK_MOT = 2,     // rows < n_ar: causal over the first n_ar keys; rows >= n_ar: all keys
};

namespace cosmos {

// Programmatic dependent launch for the decode-step kernels (GEMM, split-K reductions, QKV post-processing, paged
// attention and its merge, all-reduce + norm): while on, those kernels are launched so that their set-up and their
// weight prefetch overlap the tail of the kernel before them. Only kernels whose early part reads nothing that
// another kernel of the stream writes honour it; the caller turns it on around a decode step (where the GEMMs'
// B operands are weights) and off afterwards. The switch is process-wide: launches from other host threads see it.
void set_pdl(bool on);
bool pdl_on();

struct GemmArgs {
  const void* A = nullptr;  // [M, K] bf16, row stride lda
  const void* B = nullptr;  // [N, K] bf16, row stride ldb  (nn.Linear weight layout)
  void* C = nullptr;        // [M, N] (or [M, N/2] for SwiGLU), row stride ldc
  int M = 0, N = 0, K = 0;
  long long lda = 0, ldb = 0, ldc = 0;
  int epi = EPI_PLAIN;
  const void* bias = nullptr;  // [N] bf16
  const void* R = nullptr;     // residual, row stride ldr
  long long ldr = 0;
  const void* gate = nullptr;  // [M / rows_per_batch, N] bf16 (null = 1)
  int rows_per_batch = 0;
  const long long* route_ptr = nullptr;  // device arrays, one entry per 128-column chunk
  const long long* route_ld = nullptr;
  const float* cos_tab = nullptr;  // [rope_rows, 64]
  const float* sin_tab = nullptr;
  int rope_rows = 0;
  const void* gamma_q = nullptr;  // [128] bf16
  const void* gamma_k = nullptr;
  int n_q_heads = 0, n_k_heads = 0;
  float eps = 1e-6f;
  int* status = nullptr;  // device status word (0 = ok)
  int max_ctas = 0;       // 0 = one CTA per SM
  // EPI_ATTN_P / EPI_ATTN_DS: per-row fp32 vector (lse or D), softmax scale, and the mask of the
  // forward pass (AttnMask, n_ar); rows are queries, columns keys.
  const float* rowvec = nullptr;
  float attn_scale = 1.f;
  int attn_mask = 0, attn_n_ar = 0;
  // Operand majors. a_mn: A is stored as [K, M] (row stride lda) and read transposed in place;
  // b_mn: B is stored as [K, N] (row stride ldb). M (resp. N) and the strides must be % 8 == 0.
  bool a_mn = false, b_mn = false;
  int k_splits = 1;       // > 1: split-K with fp32 partials in `partial` ([k_splits, M, N] floats)
  float* partial = nullptr;
  bool partial_only = false;  // split-K: stop after the partial sums (the caller's next kernel reduces them)
  // split-K only (EPI_PLAIN): the reduction pass also adds the residual R (ldr) and applies an RMS-norm, writing
  // x_new = R + A B^T to `C` and rmsnorm(x_new) * norm_gamma to `norm_out` (both [M, N] bf16, row stride ldc)
  const void* norm_gamma = nullptr;
  void* norm_out = nullptr;
  float norm_eps = 1e-6f;
  // EPI_CONV: A is the padded input volume flattened to [frames * hp * wp, C] (C % 64 == 0), B the
  // weights as [Cout, 27 * C] (tap-major: kt, kh, kw, then channel), K = 27 * C. Output rows are
  // the same padded positions; only interior rows (frame >= conv_tpad, 1 <= h <= hp-2,
  // 1 <= w <= wp-2) are written, so a zero border stays zero.
  int conv_c = 0, conv_hp = 0, conv_wp = 0, conv_tpad = 0;
};
// Split count that fills the machine for a skinny problem (1 = do not split).
int gemm_pick_k_splits(int M, int N, int K, int epi);
// Debug knob for race hunting: at most `max_ctas` persistent CTAs per GEMM launch (0 = one per SM).
void gemm_set_grid_limit(int max_ctas);
// A/B switch: problems taller than one 128-row tile run on CTA pairs (256-row tiles, tcgen05 cta_group::2)
// when on (the default; COSMOS_GEMM_CTA_PAIR=0 starts with it off).
void gemm_set_cta_pair(bool on);
// Timing experiments (results are wrong): bit 0 = every tile loads the operand tiles at (0, 0) (all loads hit L2),
// bit 1 = no operand loads at all (the MMA issue rate alone).
void gemm_set_debug(int bits);
void gemm_bf16(const GemmArgs& a, cudaStream_t stream);
// K12: one persistent launch over one or two problems with the same epilogue kind (per-modality
// weight routing: tokens are already grouped into an AR segment and a DM segment).
void gemm_bf16_grouped(const GemmArgs* args, int n, cudaStream_t stream);

// Decode-step sampling (csrc/sampling.cu). sample_topk: bf16 logits [B, V] (row stride ld) of one vocabulary shard
// -> cand [B, 64] (penalised logit, global token id as int bits), best first; seen_any / seen_out are [B, V] byte
// flags (null = no penalties), updated for tokens[b]. sample_pick: cand [n_src, B, 64] -> tokens_out [B] (int64).
void sample_topk(const void* logits, long long ld, int B, int V, void* seen_any, void* seen_out,
                 const long long* tokens, const float* presence, const float* repetition, int vocab_offset,
                 void* cand, cudaStream_t s);
void sample_pick(const void* cand, int n_src, int B, const float* temperature, const long long* top_k,
                 const float* top_p, const float* noise, long long noise_ld, int vocab_size, long long* tokens_out,
                 cudaStream_t s);

struct AttnArgs {
  // Q [B, Sq, Hq, 128], K/V [B, Skv, Hkv, 128], O [B, Sq, Hq, 128]; element strides given.
  const void* Q = nullptr;
  const void* K = nullptr;
  const void* V = nullptr;
  void* O = nullptr;
  float* lse = nullptr;  // optional [B, Hq, Sq] natural-log sum-exp of scaled scores
  int B = 1, Sq = 0, Skv = 0, Hq = 0, Hkv = 0;
  long long q_stride_b = 0, q_stride_s = 0, q_stride_h = 0;
  long long k_stride_b = 0, k_stride_s = 0, k_stride_h = 0;
  long long v_stride_b = 0, v_stride_s = 0, v_stride_h = 0;
  long long o_stride_b = 0, o_stride_s = 0, o_stride_h = 0;
  float scale = 0.f;  // softmax scale (1/sqrt(d))
  int mask = MASK_FULL;
  int n_ar = 0;  // MASK_MOT only
  // Optional routing of output rows to other buffers (head->sequence all-to-all of Ulysses
  // context parallelism done by the epilogue): rows [r*rows_per_dest, (r+1)*rows_per_dest)
  // go to dest_ptr[r] with row index local to that block.
  const long long* dest_ptr = nullptr;
  int rows_per_dest = 0;
  int* status = nullptr;
  // Several K/V sources in one launch (ring-KV context parallelism: this rank's shard, the peers' shards in their
  // symmetric buffers, a local prompt prefix): n_src > 1, src_k / src_v [n_src] device addresses of contiguous
  // [B, src_len[s], Hkv, 128] bf16 buffers, walked in this order; K, V and Skv (= sum of src_len) then only describe
  // the total. Full mask only.
  int n_src = 0;
  const void* src_k[9] = {};
  const void* src_v[9] = {};
  int src_len[9] = {};
  // Of every 8 pairs of scores, this many compute exp2 with a polynomial on the FMA pipe (2, 3; 0 = none).
  // Measured on B200: faster than 0 with the MMAs switched off, slower with them on, so 0 is the default.
  int exp_emulation = 0;
  int debug = 0;  // timing experiments (results are wrong): 1 = no QK MMAs, 2 = no PV MMAs, 4 = no exponentials
};
void flash_attn_fwd(const AttnArgs& a, cudaStream_t stream);
// A/B switch: CTA-pair (cta_group::2) attention tiles on / off (off by default: measured slower, see attn_tcgen05.cu).
void attn_set_cta_pair(bool on);

// Flash attention backward (attn_bwd_tcgen05.cu): dQ, dK, dV from Q, K, V, dO, the forward's
// log-sum-exp and delta = rowsum(dO * O). Inputs [B, S, H, 128] bf16 with element strides; outputs
// contiguous [B, Sq, Hq, 128] / [B, Skv, Hkv, 128] bf16; lse, delta [B, Hq, Sq] fp32.
struct AttnBwdArgs {
  const void* Q = nullptr;
  const void* K = nullptr;
  const void* V = nullptr;
  const void* dO = nullptr;
  const float* lse = nullptr;
  const float* delta = nullptr;
  void* dQ = nullptr;
  void* dK = nullptr;
  void* dV = nullptr;
  int B = 1, Sq = 0, Skv = 0, Hq = 0, Hkv = 0;
  long long q_stride_b = 0, q_stride_s = 0, q_stride_h = 0;
  long long k_stride_b = 0, k_stride_s = 0, k_stride_h = 0;
  long long v_stride_b = 0, v_stride_s = 0, v_stride_h = 0;
  long long do_stride_b = 0, do_stride_s = 0, do_stride_h = 0;
  float scale = 0.f;
  int mask = MASK_FULL;
  int n_ar = 0;
  int* status = nullptr;
};
void flash_attn_bwd(const AttnBwdArgs& a, cudaStream_t stream);

// ---- bandwidth kernels (elementwise.cu) ----
void rmsnorm(const void* x, const void* gamma, void* y, long long rows, int d, float eps,
             const void* residual_in, void* residual_out, cudaStream_t s);
// y = rmsnorm(x) * gamma * (1 + scale[b]) + shift[b]; scale/shift rows of length d, one per batch.
void adaln_rmsnorm(const void* x, const void* gamma, const void* shift, const void* scale, void* y,
                   long long rows, int d, int rows_per_batch, long long mod_stride, float eps,
                   cudaStream_t s);
// x: [rows, heads, 128] in place; cos/sin [rope_rows, 64] fp32; optional per-head rmsnorm gamma.
void mrope_apply(void* x, long long rows, int heads, long long row_stride, const float* cos_t,
                 const float* sin_t, int rope_rows, const void* gamma, float eps, cudaStream_t s);
// y = x + gate[b] * f
void gated_residual(const void* x, const void* f, const void* gate, void* y, long long rows, int d,
                    int rows_per_batch, long long gate_stride, cudaStream_t s);
void swiglu(const void* gate_up, void* y, long long rows, int dff, cudaStream_t s);
// Flow-matching Euler step with classifier-free guidance, fp32 latents:
//   v = vu + g * (vc - vu) [optionally renormalised to |vc| per row]; x += dt * v
// vc/vu may point into another GPU's memory (CFG-parallel exchange by peer loads).
void cfg_euler_step(float* x, const void* vc, const void* vu, float guidance, float dt,
                    int normalize, long long rows, int d, cudaStream_t s);
// CFG combine + one UniPC step (order 2, with the previous step's corrector) on the fp32 latent x [rows, d]:
// coef8 = {s_cur, cL, cP, cP2, cX0, dX, dX0, dP} (models/sampler.py::UniPCSampler.plan). L (latent of the previous
// step), P (latest stored prediction) are read; on return x holds the new latent, L the corrected latent of this
// step and P2's buffer the new prediction (the caller then swaps P and P2).
void cfg_unipc_step(float* x, const void* vc, const void* vu, float* L, const float* P, float* P2, float guidance,
                    int normalize, const float* coef8, int correct, int final_step, int has_p, int has_p2,
                    long long rows, int d, cudaStream_t s);
void l2_flush(void* buf, size_t bytes, cudaStream_t s);
// y = silu(rmsnorm(x) * gamma) over rows of d channels (channels-last tokenizer activations)
void rmsnorm_silu(const void* x, const void* gamma, void* y, long long rows, int d, float eps, cudaStream_t s);

// ---- tokenizer decoder helpers on padded channels-last volumes (conv3d.cu) ----
void upsample_cl(const void* src, void* dst, int t_dst, int hs, int ws, int c, int tpad, int temporal,
                 int first_chunk, cudaStream_t s);
void conv_out_rgb(const void* x, const float* wgt, const float* bias, void* out, int t_out, int h, int w,
                  cudaStream_t s);

// ---- paged-KV decode attention (paged_decode.cu) ----
struct PagedDecodeArgs {
  const void* q = nullptr;        // [B, Hq, 128] bf16
  const void* k_cache = nullptr;  // [num_pages, Hkv, page_size, 128] bf16
  const void* v_cache = nullptr;
  const int* block_table = nullptr;  // [B, max_pages]
  const int* seq_lens = nullptr;     // [B]
  void* out = nullptr;               // [B, Hq, 128] bf16
  int B = 0, Hq = 0, Hkv = 0, page_size = 0, max_pages = 0;
  float scale = 0.f;
  int n_splits = 1;
  void* scratch = nullptr;  // >= paged_decode_scratch_bytes(B, Hq, n_splits) when n_splits > 1
  size_t scratch_bytes = 0;
  int num_pages = 0;        // pages in the cache tensors; needed by the tensor-core kernel (TMA bounds)
  int* status = nullptr;    // status word for bounded waits (tensor-core kernel)
  int impl = 0;             // 0 = tensor-core kernel when the shape allows it, 1 = CUDA-core kernel
};
// kv splits for the CUDA-core kernel (several CTAs per SM) and for the tensor-core kernel (one per SM)
int paged_decode_pick_splits(int B, int Hkv, int max_len);
int paged_decode_tc_pick_splits(int B, int Hkv, int max_len);
bool paged_decode_tc_supported(const PagedDecodeArgs& a);
void paged_decode_tc_launch(const PagedDecodeArgs& a, float* pa, float* pm, cudaStream_t s);
size_t paged_decode_scratch_bytes(int B, int Hq, int n_splits);
void paged_decode(const PagedDecodeArgs& a, cudaStream_t s);
// Loads every CUDA-core decode kernel variant and the merge kernel into the current context (no launch).
void paged_decode_preload();
// Scatters new K/V rows [N, Hkv, 128] into the paged caches at flat slots (page * page_size + offset).
// `n_slots` (token rows of the cache) and `status` serve the bounds-checked build, which reports a slot
// outside the cache instead of writing there.
void kv_cache_write(const void* k, const void* v, const long long* slots, void* k_cache, void* v_cache,
                    long long n_rows, int Hkv, int page_size, long long n_slots, int* status, cudaStream_t s);

// Decode-step glue after the QKV GEMM: q/k RMS-norm + rotary, q to a contiguous buffer, k and v into
// their paged-cache rows (slot = page * page_size + offset, one per sequence). cos/sin [B, 64] fp32.
void decode_qkv_post(const void* qkv, int B, int Hq, int Hkv, const float* cos_t, const float* sin_t,
                     const void* gamma_q, const void* gamma_k, float eps, const long long* slots, void* q_out,
                     void* k_cache, void* v_cache, int page_size, long long n_slots, int* status, cudaStream_t s,
                     const float* partial = nullptr, int k_splits = 0);  // partial: split-K sums [k_splits, B, heads * 128] instead of qkv

// True in a build with -DCOSMOS_BOUNDS_CHECK. The self-test runs the index check on (idx[i], limit[i])
// pairs and writes 1 / 0 to ok[i]; it touches no memory through the tested indices.
bool bounds_check_enabled();
void bounds_check_selftest(const long long* idx, const long long* limit, int* ok, int n, int* status, cudaStream_t s);

// ---- backward of the bandwidth kernels (elementwise_bwd.cu) ----
// RMSNorm / AdaLN-RMSNorm: dx [rows, d]; with `part` != null also per-block column sums
// part[B][rmsnorm_bwd_blocks(rows_per_batch)][3][d] (d shift, d scale, d gamma), B = rows / rows_per_batch.
// gamma / scale may be null (treated as 1 / 0); scale rows are mod_stride elements apart.
int rmsnorm_bwd_blocks(int rows_per_batch);
void rmsnorm_bwd(const void* x, const void* dy, const void* gamma, const void* scale, long long rows, int d,
                 int rows_per_batch, long long mod_stride, float eps, void* dx, float* rinv, float* part,
                 cudaStream_t s);
// y = resid + gate[b] * f: df = dy * gate[b], part[B][blocks][d] = per-block sums of dy * f.
void gated_residual_bwd(const void* dy, const void* f, const void* gate, long long rows, int d, int rows_per_batch,
                        long long gate_stride, void* df, float* part, cudaStream_t s);
void swiglu_bwd(const void* gate_up, const void* dy, void* d_gate_up, long long rows, int dff, cudaStream_t s);
// qkv [rows, Hq + 2 Hkv, 128] -> q, k, v with q/k RMS-norm and rotary; and its backward
// (part[qkv_post_bwd_blocks][2][128] = per-block sums of d gamma_q, d gamma_k).
void qkv_post_fwd(const void* qkv, long long rows, int Hq, int Hkv, const float* cos_t, const float* sin_t,
                  int rope_rows, const void* gamma_q, const void* gamma_k, float eps, void* q, void* k, void* v,
                  cudaStream_t s);
int qkv_post_bwd_blocks(long long rows, int Hq, int Hkv);
void qkv_post_bwd(const void* qkv, const void* dq, const void* dk, const void* dv, long long rows, int Hq, int Hkv,
                  const float* cos_t, const float* sin_t, int rope_rows, const void* gamma_q, const void* gamma_k,
                  float eps, void* d_qkv, float* part, cudaStream_t s);

// ---- communication kernels over peer mappings (comm.cu) ----
// pads_dev / bufs_dev / grads_dev / srcs_dev: device arrays with one address per rank of the group.
// Signal pads are int32 arrays laid out as [slot][64]; epochs must grow monotonically per slot.
void comm_barrier(const long long* pads_dev, int rank, int world, int slot, int epoch, int* status,
                  cudaStream_t s);
// Epoch read from and advanced in counters[slot] on the device (CUDA-graph friendly).
void comm_barrier_counted(const long long* pads_dev, int rank, int world, int slot, int* counters, int* status,
                          cudaStream_t s);
// Uses slots [slot, slot + 8) and epochs (epoch, epoch + 1); with `counters` (device ints, one per
// slot) the kernel tracks the epochs itself and `epoch` is ignored (CUDA-graph friendly).
void allreduce_oneshot(const long long* bufs_dev, const long long* pads_dev, void* out,
                       long long n_elems, int rank, int world, int slot, int epoch, int* counters,
                       int* status, cudaStream_t s);
void rs_adamw(const long long* grads_dev, int world, long long shard_off, long long n, float* master,
              float* m, float* v, void* param_shard, float grad_scale, float lr, float b1, float b2,
              float eps, float wd, int step, float* sq_out, float* reduced_out, cudaStream_t s);
// Reduce-scatter by pull into an fp32 shard (out[i] (+)= scale * sum_r grad_r[shard_off + i]) with the sum of squares
// of the results added to *sq_out (may be null). `mc` != null: the buffers' NVLink multicast address; the sum over
// ranks is then one multimem.ld_reduce per 16-byte vector (added inside the switch) instead of `world` peer loads.
void reduce_scatter_pull(const long long* grads_dev, const void* mc, int world, long long shard_off, long long n,
                         float* out, bool accumulate, float scale, float* sq_out, cudaStream_t s);
// AdamW on a local fp32 gradient shard (fp32 master + moments, bf16 parameter shard rewritten).
void adamw_shard(const float* grad, long long n, float* master, float* m, float* v, void* param_shard,
                 float grad_scale, float lr, float b1, float b2, float eps, float wd, int step, cudaStream_t s);
// Decode all-reduce fused with its neighbours: (sum of the GEMM's split-K partials -> `own`, this rank's symmetric
// buffer) -> group barrier -> sum over ranks (+ residual R) -> X, and H = rmsnorm(X) * gamma. One launch; epochs in
// `counters` (one device int per signal slot; slots [slot, slot + allreduce_norm_blocks(M)) belong to the call).
// Callers alternate two symmetric buffers between consecutive calls (there is no trailing barrier).
int allreduce_norm_blocks(int M);
void allreduce_norm(const long long* bufs_dev, const void* mc, void* own, const long long* pads_dev, int rank,
                    int world, int slot, int* counters, const float* partial, int k_splits, int M, int N,
                    const void* R, const void* gamma, float eps, void* X, void* H, int* status, cudaStream_t s);
// out = R + gate[m / rows_per_batch] * sum_p part[p] over n_part stacked [rows, d] bf16 partial products.
void sum_partials_gated_residual(const void* part, int n_part, long long rows, int d, const void* R, const void* gate,
                                 int rows_per_batch, void* out, cudaStream_t s);
void allgather_pull(const long long* srcs_dev, int world, void* dst, long long bytes_per_rank,
                    cudaStream_t s);

}  // namespace cosmos
