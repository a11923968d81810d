"""Micro-benchmarks of the hot kernels: CUDA-event timing after warm-up, L2 flushed between
iterations, achieved TFLOP/s (or GB/s) and fraction of the measured peaks.

    python -m cosmos_b200.ops.bench_kernels [--what gemm,qkvroute,attn,attnbwd,norm,paged,vae] [--iters 5] [--small]

`--sustained SECONDS` times every GEMM / attention case in a back-to-back loop of that length instead (no L2 flush;
the inputs are larger than L2) and reports the median SM clock and power sampled with nvidia-smi during the loop:
on a power-capped part this, not the burst figure, is what a long-running step sees. A/B switches:
`--gemm-pair 0|1` (CTA-pair tiles), `--attn-pair 0|1`, `--gemm-debug BITS` and COSMOS_ATTN_DEBUG=BITS (timing
experiments that switch parts of a kernel off; results are wrong with them).
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch

from cosmos_b200 import ops


def _peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["bf16_tflops"], d["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


def timeit(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        ops.l2_flush(flush)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


class _Smi:
    """Samples SM clock and power every 100 ms while a loop runs."""

    def __init__(self):
        import subprocess
        import threading
        self.rows = []
        try:
            self.p = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits",
                                       "-lms", "100", "-i", str(torch.cuda.current_device())], stdout=subprocess.PIPE,
                                      text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:  # noqa: BLE001 - no nvidia-smi: no clocks
            self.p = None

    def _read(self):
        import time
        for line in self.p.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def window(self, t0, t1):
        import statistics
        r = [x for t, x in self.rows if t0 + 0.5 <= t <= t1]
        if not r:
            return {}
        return {"sm_mhz": statistics.median(float(x[0]) for x in r), "power_w": statistics.median(float(x[1]) for x in r)}


_SMI = None


def sustained(fn, secs):
    """Back-to-back calls for `secs` seconds -> (ms per call, clocks during the loop)."""
    import time
    global _SMI
    if _SMI is None:
        _SMI = _Smi()
        time.sleep(1.0)
    fn()
    torch.cuda.synchronize()
    t0 = time.time()
    n = 0
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    while time.time() - t0 < secs:
        for _ in range(20):
            fn()
        n += 20
        torch.cuda.synchronize()
    e.record()
    torch.cuda.synchronize()
    t1 = time.time()
    time.sleep(0.5)
    return s.elapsed_time(e) / n, _SMI.window(t0, t1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,attn,norm")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--small", action="store_true", help="sizes for a profiler capture")
    ap.add_argument("--cublas", action="store_true", help="also time torch.matmul / SDPA for comparison")
    ap.add_argument("--attn-shape", default=None, help="sq,skv,hq,hkv for a single attention case")
    ap.add_argument("--sustained", type=float, default=0.0, help="seconds of back-to-back calls per case (0 = burst timing)")
    ap.add_argument("--gemm-pair", type=int, default=None, help="0 / 1: single-CTA or CTA-pair GEMM tiles")
    ap.add_argument("--attn-pair", type=int, default=None, help="0 / 1: single-CTA or CTA-pair attention tiles")
    ap.add_argument("--page", type=int, default=16, help="tokens per KV-cache page in the paged decode case")
    ap.add_argument("--gemm-debug", type=int, default=0, help="timing experiment bits of the GEMM (1: all tiles load tile (0,0); 2: no loads)")
    args = ap.parse_args()
    ops.load_extension()
    if args.gemm_pair is not None:
        torch.ops.cosmos_b200.gemm_set_cta_pair(bool(args.gemm_pair))
    if args.attn_pair is not None:
        torch.ops.cosmos_b200.attn_set_cta_pair(bool(args.attn_pair))
    if args.gemm_debug:
        torch.ops.cosmos_b200.gemm_set_debug(args.gemm_debug)

    def measure(fn):
        """(ms, extra record fields) by the selected method."""
        if args.sustained > 0:
            ms, clk = sustained(fn, args.sustained)
            return ms, {"method": f"sustained {args.sustained:g} s", **clk}
        return timeit(fn, args.iters, flush), {"method": "burst, L2 flushed"}

    tf_peak, bw_peak, src = _peaks()
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = []
    what = args.what.split(",")
    if "gemm" in what:
        shapes = [(8192, 4096, 4096)] if args.small else [
            (16384, 4096, 4096), (16384, 6144, 4096), (16384, 24576, 4096), (16384, 4096, 12288)]
        for m, n, k in shapes:
            a = torch.randn(m, k, device=dev).bfloat16()
            w = torch.randn(n, k, device=dev).bfloat16()
            epi = ops.EPI_SWIGLU if n == 24576 else ops.EPI_PLAIN
            ms, how = measure(lambda: ops.gemm(a, w, epi=epi))
            tf = 2.0 * m * n * k / ms / 1e9
            rec = {"kernel": "gemm_bf16_tcgen05", "shape": [m, n, k], "epi": epi, "ms": round(ms, 4),
                   "tflops": round(tf, 1), f"frac_of_{src}_bf16": round(tf / tf_peak, 3), **how}
            if args.cublas:
                ms2, how2 = measure(lambda: torch.matmul(a, w.t()))
                rec["cublas_ms"] = round(ms2, 4)
                rec["cublas_clocks"] = {k_: v_ for k_, v_ in how2.items() if k_ != "method"}
            out.append(rec)
            print(json.dumps(rec), flush=True)
    if "qkvroute" in what:
        # the QKV projection whose epilogue applies q/k RMS-norm + rotary and scatters every 128-column head chunk
        # through a routing table: the seq -> head all-to-all of Ulysses context parallelism as epilogue stores.
        # On one GPU the table points at local buffers (the kernel issues the same stores; with peers they are
        # peer mappings), which is what a single-GPU profiler capture can see of the fused kernel.
        m, d, hq, hk = (8192, 4096, 32, 8) if args.small else (27904, 4096, 32, 8)   # 111,616 tokens / cp 4
        n = (hq + 2 * hk) * 128
        a = torch.randn(m, d, device=dev).bfloat16()
        w = (torch.randn(n, d, device=dev) / math.sqrt(d)).bfloat16()
        ang = torch.rand(m, 64, device=dev) * 6.0
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        gq = torch.ones(128, device=dev).bfloat16()
        gk = torch.ones(128, device=dev).bfloat16()
        bufs = [torch.empty(m, 128, device=dev, dtype=torch.bfloat16) for _ in range(n // 128)]
        ptr = torch.tensor([b.data_ptr() for b in bufs], device=dev, dtype=torch.int64)
        ld = torch.full((n // 128,), 128, device=dev, dtype=torch.int64)
        ms = timeit(lambda: ops.gemm_qkv_rope(a, w, None, cos, sin, gq, gk, hq, hk, 1e-6, ptr, ld), args.iters, flush)
        tf = 2.0 * m * n * d / ms / 1e9
        ms0 = timeit(lambda: ops.gemm(a, w), args.iters, flush)
        rec = {"kernel": "gemm_bf16_tcgen05 + q/k norm + rotary + routed head stores", "shape": [m, n, d],
               "ms": round(ms, 4), "tflops": round(tf, 1), f"frac_of_{src}_bf16": round(tf / tf_peak, 3),
               "plain_epilogue_ms": round(ms0, 4)}
        out.append(rec)
        print(json.dumps(rec), flush=True)
    if "attn" in what:
        cfgs = [(4096, 4096, 8, 2)] if args.small else [(16384, 16384, 8, 2), (32768, 32768, 8, 2)]
        if args.attn_shape:
            cfgs = [tuple(int(v) for v in args.attn_shape.split(","))]
        for sq, skv, hq, hkv in cfgs:
            q = torch.randn(1, sq, hq, 128, device=dev).bfloat16()
            k = torch.randn(1, skv, hkv, 128, device=dev).bfloat16()
            v = torch.randn(1, skv, hkv, 128, device=dev).bfloat16()
            ms, how = measure(lambda: ops.attention(q, k, v))
            tf = 4.0 * sq * skv * hq * 128 / ms / 1e9
            rec = {"kernel": "flash_attn_fwd_tcgen05", "shape": [sq, skv, hq, hkv], "ms": round(ms, 4),
                   "tflops": round(tf, 1), f"frac_of_{src}_bf16": round(tf / tf_peak, 3), **how}
            if args.cublas:
                qt, kt, vt = (t.permute(0, 2, 1, 3) for t in (q, k, v))
                ms2, how2 = measure(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, enable_gqa=True))
                rec["sdpa_ms"] = round(ms2, 4)
                rec["sdpa_clocks"] = {k_: v_ for k_, v_ in how2.items() if k_ != "method"}
            out.append(rec)
            print(json.dumps(rec), flush=True)
    if "norm" in what:
        rows, d = (16384, 4096) if args.small else (111600, 4096)
        x = torch.randn(rows, d, device=dev).bfloat16()
        g = torch.ones(d, device=dev).bfloat16()
        mod = torch.randn(1, 2 * d, device=dev).bfloat16()
        ms = timeit(lambda: ops.adaln_rmsnorm(x, g, mod[:, :d], mod[:, d:], rows), args.iters, flush)
        gbs = 2.0 * rows * d * 2 / ms / 1e6
        rec = {"kernel": "adaln_rmsnorm", "shape": [rows, d], "ms": round(ms, 4), "gbs": round(gbs, 1),
               f"frac_of_{src}_hbm": round(gbs / bw_peak, 3)}
        out.append(rec)
        print(json.dumps(rec), flush=True)
    if "attnbwd" in what:
        # flash attention backward (dK/dV kernel + dQ kernel) at the per-rank training shape
        sq, hq, hkv = (4096, 8, 2) if args.small else (14336, 32, 8)
        q = torch.randn(1, sq, hq, 128, device=dev).bfloat16()
        k = torch.randn(1, sq, hkv, 128, device=dev).bfloat16()
        v = torch.randn(1, sq, hkv, 128, device=dev).bfloat16()
        do = torch.randn(1, sq, hq, 128, device=dev).bfloat16()
        o, lse = torch.ops.cosmos_b200.attn_fwd(q, k, v, 128 ** -0.5, ops.MASK_FULL, 0, True, None, 0, None)
        delta = (do.float() * o.float()).sum(-1).permute(0, 2, 1).contiguous()
        ms = timeit(lambda: torch.ops.cosmos_b200.attn_bwd(q, k, v, do, lse, delta, 128 ** -0.5, ops.MASK_FULL, 0),
                    args.iters, flush)
        fl = 7 * 2.0 * sq * sq * 128 * hq  # 4 MMAs in the dK/dV kernel + 3 in the dQ kernel
        rec = {"kernel": "flash_attn_bwd_tcgen05", "shape": [sq, sq, hq, hkv], "ms": round(ms, 4),
               "tflops_executed": round(fl / ms / 1e9, 1), "tflops_algorithmic": round(fl * 5 / 7 / ms / 1e9, 1),
               f"frac_of_{src}_bf16": round(fl / ms / 1e9 / tf_peak, 3)}
        out.append(rec)
        print(json.dumps(rec), flush=True)
    if "paged" in what:
        # decode attention over a paged cache: batch 32, 32 q heads / 8 kv heads, 8448 cached tokens
        b, hq, hkv, ctx, page = (8, 32, 8, 2048, args.page) if args.small else (32, 32, 8, 8448, args.page)
        n_pages = b * ((ctx + page - 1) // page)
        kc = torch.randn(n_pages, hkv, page, 128, device=dev).bfloat16()
        vc = torch.randn(n_pages, hkv, page, 128, device=dev).bfloat16()
        table = torch.randperm(n_pages, device=dev).int().view(b, -1)
        lens = torch.full((b,), ctx, dtype=torch.int32, device=dev)
        q = torch.randn(b, hq, 128, device=dev).bfloat16()
        for impl, name in ((0, "paged_decode_tc (TMA + tcgen05)"), (1, "paged_decode (CUDA cores)")):
            ms = timeit(lambda: ops.paged_decode(q, kc, vc, table, lens, 128 ** -0.5, max_len=ctx, impl=impl),
                        args.iters, flush)
            gbs = 2.0 * b * ctx * hkv * 128 * 2 / ms / 1e6
            rec = {"kernel": name, "shape": [b, hq, hkv, ctx], "page": page, "ms": round(ms, 4), "gbs": round(gbs, 1),
                   f"frac_of_{src}_hbm": round(gbs / bw_peak, 3)}
            out.append(rec)
            print(json.dumps(rec), flush=True)
    if "sample" in what:
        # decode-step sampler over one vocabulary shard: penalties + top-64 selection, then the draw
        b, v = (32, 151936) if args.small else (256, 151936)
        g = torch.Generator(device=dev).manual_seed(0)
        logits = (torch.randn(b, v, device=dev, generator=g) * 3).bfloat16()
        seen_any = torch.rand(b, v, device=dev, generator=g) < 0.01
        seen_out = seen_any & (torch.rand(b, v, device=dev, generator=g) < 0.5)
        tokens = torch.randint(0, v, (b,), device=dev, generator=g)
        pres, rep = torch.full((b,), 1.5, device=dev), torch.full((b,), 1.1, device=dev)
        temp, top_p = torch.full((b,), 0.7, device=dev), torch.full((b,), 0.8, device=dev)
        top_k = torch.full((b,), 20, device=dev, dtype=torch.long)
        noise = torch.rand(b, 64, device=dev, generator=g).clamp_min(1e-7)
        out_tok = torch.empty(b, dtype=torch.long, device=dev)

        def run_sample():
            cand = ops.sample_topk(logits, seen_any, seen_out, tokens, pres, rep, 0)
            ops.sample_pick(cand, 1, temp, top_k, top_p, noise, v, out_tok)

        ms = timeit(run_sample, args.iters, flush)
        traffic = b * v * (2 + 1 + 1)
        rec = {"kernel": "sample_topk + sample_pick", "shape": [b, v], "ms": round(ms, 4),
               "one_pass_gbs": round(traffic / ms / 1e6, 1)}
        if args.cublas:
            lf = logits.float()

            def run_ref():
                cand = ops.sample_topk(lf, seen_any, seen_out, tokens, pres, rep, 0)   # fp32 logits: PyTorch definition
                ops.sample_pick(cand, 1, temp, top_k, top_p, noise, v, out_tok)
            rec["pytorch_ms"] = round(timeit(run_ref, args.iters, flush), 4)
        out.append(rec)
        print(json.dumps(rec), flush=True)
    if "vae" in what:
        # tokenizer decode of one clip through the channels-last implicit-GEMM decoder
        from cosmos_b200.models.vae import CausalVideoVAE
        from cosmos_b200.models.vae_cuda import CLDecoder

        t_lat, h_lat, w_lat = (3, 30, 40) if args.small else (31, 90, 160)
        torch.manual_seed(0)
        vae = CausalVideoVAE(16, (64, 128, 256, 256)).to(device=dev, dtype=torch.bfloat16).eval()
        dec = CLDecoder(vae)
        z = torch.randn(1, 16, t_lat, h_lat, w_lat, device=dev).bfloat16()
        frames = None

        def run():
            nonlocal frames
            frames = dec.decode(z)

        ms = timeit(run, max(1, min(args.iters, 3)), flush)
        rec = {"kernel": "vae_decode_cl", "latent": [t_lat, h_lat, w_lat], "frames": list(frames.shape[1:4]),
               "ms": round(ms, 2)}
        out.append(rec)
        print(json.dumps(rec), flush=True)
        # tokenizer encode of the same clip: implicit-GEMM encoder, and the PyTorch modules (cuDNN) with --cublas
        from cosmos_b200.models.vae_cuda import CLEncoder
        enc = CLEncoder(vae)
        video = torch.rand(1, 3, 1 + 4 * (t_lat - 1), 8 * h_lat, 8 * w_lat, device=dev).bfloat16() * 2 - 1
        lat = None

        def run_enc():
            nonlocal lat
            lat = enc.encode(video)

        ms = timeit(run_enc, max(1, min(args.iters, 3)), flush)
        rec = {"kernel": "vae_encode_cl", "frames": list(video.shape[2:]), "latent": list(lat.shape[2:]), "ms": round(ms, 2)}
        if args.cublas:
            def run_ref():
                with torch.no_grad():
                    vae.encode(video, chunk_frames=4)
            rec["pytorch_cudnn_ms"] = round(timeit(run_ref, 1, flush), 2)
        out.append(rec)
        print(json.dumps(rec), flush=True)
    torch.cuda.synchronize()
    ops.check_status()
    return out


if __name__ == "__main__":
    main()
