"""Batched Reasoner decoding with tensor parallelism, a paged KV cache and CUDA graphs.

One decode step for B sequences on each of `tp` ranks (heads and FFN units split by rank):
  RMSNorm -> QKV split-K GEMM -> q/k RMSNorm + rotary -> KV-cache write -> paged-KV decode
  attention -> out-proj split-K GEMM -> one-shot all-reduce over NVLink -> (residual + RMSNorm
  fused) -> SwiGLU FC1 -> FC2 -> all-reduce -> ... -> final norm -> vocab-parallel LM head ->
  greedy arg-max across the vocab shards.
Every kernel is this package's own; the whole step is captured in a CUDA graph (all step state —
sequence lengths, cache slots, rotary tables — lives in device tensors updated inside the graph,
and the all-reduce tracks its barrier epochs on the device), so a step costs one graph launch.

Benchmark (Cosmos3-Nano Reasoner, batch 32, prompt = 8192 vision embeddings + 256 text ids,
256 greedy tokens):
    torchrun --nproc-per-node 8 -m cosmos_b200.serve.decoder --batch 32 --prompt-vision 8192 \
        --prompt-text 256 --new-tokens 256
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import ops
from ..config import MoTConfig, get_model_config
from ..models import rope
from .paged import PagedKVCache


class TPDecoder:
    def __init__(self, cfg: MoTConfig, tp: int, rank: int, group, device, page_size: int = 32,
                 max_batch: int = 32, max_len: int = 9000, seed: int = 0, fused: bool = True, dtype=torch.bfloat16):
        assert cfg.n_heads % tp == 0 and cfg.n_kv_heads % tp == 0 and cfg.ffn_dim % tp == 0
        # page_size 32: the decode-attention kernel fetches one TMA box per page, tensor and 64-column half; measured
        # 0.73 of the copy bandwidth with 16-token pages (2 KB boxes), 0.86 with 32, 0.89 with 128
        self.cfg, self.tp, self.rank, self.group = cfg, tp, rank, group
        self.device = torch.device(device)
        self.hq, self.hk, self.hd = cfg.n_heads // tp, cfg.n_kv_heads // tp, cfg.head_dim
        self.ffn = cfg.ffn_dim // tp
        d = cfg.d_model
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)  # same seed on every rank: replicated tensors agree, shards are cut from them

        def rnd(*shape):
            return (torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * cfg.init_std).to(dtype)

        # local shards are drawn directly (no rank ever holds the full weights)
        g.manual_seed(seed * 1000 + rank + 1)
        self.layers: List[Dict[str, torch.Tensor]] = []
        for _ in range(cfg.n_layers):
            self.layers.append({
                "norm1": torch.ones(d, device=self.device, dtype=dtype),
                "norm2": torch.ones(d, device=self.device, dtype=dtype),
                "wqkv": rnd((self.hq + 2 * self.hk) * self.hd, d),
                "q_norm": torch.ones(self.hd, device=self.device, dtype=dtype),
                "k_norm": torch.ones(self.hd, device=self.device, dtype=dtype),
                "wo": rnd(d, self.hq * self.hd),
                "w_gate_up": rnd(2 * self.ffn, d),
                "w_down": rnd(d, self.ffn),
            })
        self.v_loc = (cfg.vocab_size + tp - 1) // tp
        self.lm_head = rnd(self.v_loc, d)
        g.manual_seed(seed)
        self.embed = rnd(cfg.vocab_size, d)
        self.final_norm = torch.ones(d, device=self.device, dtype=dtype)
        pages_per_seq = (max_len + page_size - 1) // page_size
        self.cache = PagedKVCache(cfg.n_layers, self.hk, self.hd, max_batch * pages_per_seq + 1, page_size,
                                  pages_per_seq, dtype, self.device)
        self.page_size = page_size
        half = self.hd // 2
        self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, half, device=self.device, dtype=torch.float32)
                                                   * 2.0 / self.hd)))
        self.fused = fused and tp > 1 and self.device.type == "cuda"
        self._tpctx = None
        if tp > 1:
            from ..parallel.tp import TPContext
            ranks = list(range(tp)) if group is None else dist.get_process_group_ranks(group)
            self._tpctx = TPContext(cfg, group, ranks, self.device, fused=self.fused, sequence_parallel=False)
        self.graph = None
        self.step_inc: Optional[torch.Tensor] = None  # int32 [B] of 0/1 set by the serving engine; None = all ones
        self.sampling: Optional[Dict[str, torch.Tensor]] = None  # see enable_sampling
        self.pos_delta: Optional[torch.Tensor] = None  # int64 [B]: rotary position minus cache position

    # ------------------------------------------------------------------ helpers
    def _allreduce(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.tp == 1 else self._tpctx._all_reduce(x)

    def _layer(self, li: int, x: torch.Tensor, resid_delta: Optional[torch.Tensor], cos, sin, slots, table, lens,
               max_len: int):
        """x: residual stream [B, d]; resid_delta: pending update to add before the first norm."""
        p = self.layers[li]
        cfg = self.cfg
        b = x.shape[0]
        if resid_delta is None:
            h, _ = ops.rmsnorm(x, p["norm1"], cfg.rms_eps)
        else:
            h, x = ops.rmsnorm(resid_delta, p["norm1"], cfg.rms_eps, residual=x)
        q = ops.gemm_decode_qkv_post(h, p["wqkv"], self.hq, cos, sin, p["q_norm"], p["k_norm"], cfg.rms_eps, slots,
                                self.cache.k[li], self.cache.v[li])
        o = ops.paged_decode(q, self.cache.k[li], self.cache.v[li], table, lens, max_len=max_len)
        y = self._allreduce(ops.gemm(o.view(b, -1), p["wo"]))
        h, x = ops.rmsnorm(y, p["norm2"], cfg.rms_eps, residual=x)
        a = ops.gemm(h, p["w_gate_up"], epi=ops.EPI_SWIGLU)
        y = self._allreduce(ops.gemm(a, p["w_down"]))
        return x, y

    def _layer_single(self, li: int, h: torch.Tensor, x: torch.Tensor, next_gamma: torch.Tensor, cos, sin, slots,
                      table, lens, max_len: int):
        """One layer on one rank (no all-reduce): `h` is the normalised input, `x` the residual stream. Both output
        projections go through `gemm_reduce_rmsnorm`, whose reduction pass adds the residual and applies the next
        norm (this layer's norm2, then the NEXT layer's norm1 / the final norm), so the layer is nine launches."""
        p = self.layers[li]
        cfg = self.cfg
        b = x.shape[0]
        q = ops.gemm_decode_qkv_post(h, p["wqkv"], self.hq, cos, sin, p["q_norm"], p["k_norm"], cfg.rms_eps, slots,
                                self.cache.k[li], self.cache.v[li])
        o = ops.paged_decode(q, self.cache.k[li], self.cache.v[li], table, lens, max_len=max_len)
        h, x = ops.gemm_reduce_rmsnorm(o.view(b, -1), p["wo"], x, p["norm2"], cfg.rms_eps)
        a = ops.gemm(h, p["w_gate_up"], epi=ops.EPI_SWIGLU)
        return ops.gemm_reduce_rmsnorm(a, p["w_down"], x, next_gamma, cfg.rms_eps)

    def _layer_tp(self, li: int, h: torch.Tensor, x: torch.Tensor, next_gamma: torch.Tensor, cos, sin, slots,
                  table, lens, max_len: int):
        """One layer on a tensor-parallel rank with the fused collectives: each row-parallel projection is a GEMM
        that leaves its split-K partial sums plus ONE kernel that reduces them, meets the peers, sums over the ranks
        (through the NVLink switch when a multicast mapping exists), adds the residual and applies the next norm."""
        p = self.layers[li]
        cfg = self.cfg
        b = x.shape[0]
        tpc = self._tpctx
        q = ops.gemm_decode_qkv_post(h, p["wqkv"], self.hq, cos, sin, p["q_norm"], p["k_norm"], cfg.rms_eps, slots,
                                self.cache.k[li], self.cache.v[li])
        o = ops.paged_decode(q, self.cache.k[li], self.cache.v[li], table, lens, max_len=max_len)
        h, x = tpc.gemm_allreduce_norm(o.view(b, -1), p["wo"], x, p["norm2"], cfg.rms_eps)
        a = ops.gemm(h, p["w_gate_up"], epi=ops.EPI_SWIGLU)
        return tpc.gemm_allreduce_norm(a, p["w_down"], x, next_gamma, cfg.rms_eps)

    def _step_impl(self) -> None:
        """Consumes self.tokens / self.lens (device), writes self.next_tokens and advances lens."""
        b = self.tokens.shape[0]
        pos = self.lens.long()                       # cache position of the new token = current length
        # rotary position: the same for text; prompts with vision grids advance slower than one per token
        # (3-D ids), so the serving engine keeps a per-slot offset
        rpos = pos if self.pos_delta is None else pos + self.pos_delta
        ang = rpos.float()[:, None] * self.inv_freq[None]
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        slots = PagedKVCache.slots(self.table, pos[:, None], self.page_size)[:, 0].contiguous()
        # attention sees the token being written; idle slots of a serving batch do not advance
        if self.step_inc is None:
            self.lens.add_(1)
        else:
            self.lens.add_(self.step_inc)
        x = self.embed[self.tokens]
        # Programmatic dependent launch for the layer kernels: each one's set-up, and the GEMMs' first weight tiles,
        # may overlap the tail of the kernel before it. Measured per step: 5.80 -> 5.45 ms at TP 4 and 8.96 -> 8.77 ms
        # at TP 2, but 12.45 -> 12.6 ms on one GPU at batch 32 and 5.30 -> 5.50 ms at batch 1 (a GEMM CTA needs most
        # of an SM's shared memory, so the next GEMM cannot become resident before the current one leaves, and the
        # programmatic edges cost about 0.5 us per launch in the replayed graph). Hence on from TP 4, where the step
        # is latency-bound; COSMOS_DECODE_PDL=0 / 1 overrides.
        pdl = self.device.type == "cuda" and ops.get_backend() != "library" and \
            os.environ.get("COSMOS_DECODE_PDL", "1" if self.tp >= 4 else "0") == "1"
        if pdl:
            torch.ops.cosmos_b200.set_pdl(True)
        try:
            logits = self._forward_layers(x, cos, sin, slots)
        finally:
            if pdl:
                torch.ops.cosmos_b200.set_pdl(False)
        self._finish_step(logits, b)

    def _forward_layers(self, x, cos, sin, slots) -> torch.Tensor:
        if self.tp == 1:
            h, _ = ops.rmsnorm(x, self.layers[0]["norm1"], self.cfg.rms_eps)
            n = self.cfg.n_layers
            for li in range(n):
                nxt = self.layers[li + 1]["norm1"] if li + 1 < n else self.final_norm
                h, x = self._layer_single(li, h, x, nxt, cos, sin, slots, self.table, self.lens, self.max_len)
        elif self.fused and os.environ.get("COSMOS_DECODE_FUSED_AR", "1") != "0":
            self._tpctx.begin_step()
            h, _ = ops.rmsnorm(x, self.layers[0]["norm1"], self.cfg.rms_eps)
            n = self.cfg.n_layers
            for li in range(n):
                nxt = self.layers[li + 1]["norm1"] if li + 1 < n else self.final_norm
                h, x = self._layer_tp(li, h, x, nxt, cos, sin, slots, self.table, self.lens, self.max_len)
        else:
            delta = None
            for li in range(self.cfg.n_layers):
                x, delta = self._layer(li, x, delta, cos, sin, slots, self.table, self.lens, self.max_len)
            h, _ = ops.rmsnorm(delta, self.final_norm, self.cfg.rms_eps, residual=x)
        return ops.gemm(h, self.lm_head)             # [B, V/tp]

    def _finish_step(self, logits: torch.Tensor, b: int) -> None:
        self.last_logits = logits                    # this rank's vocab shard, kept for inspection
        if self.sampling is not None:
            self._sample(logits)                     # global ids across the vocab shards, into self.next_tokens
            return
        val, idx = logits.float().max(dim=-1)
        idx = idx + self.rank * self.v_loc
        if self.tp > 1:
            packed = torch.stack([val, idx.float()], dim=-1)      # [B, 2]
            allp = torch.empty(self.tp * b, 2, device=self.device)            # rank-major concatenation
            dist.all_gather_into_tensor(allp, packed, group=self.group)
            allp = allp.view(self.tp, b, 2)
            best = allp[..., 0].argmax(dim=0)
            idx = allp[best, torch.arange(b, device=self.device), 1].long()
        self.next_tokens.copy_(idx.clamp(max=self.cfg.vocab_size - 1))

    # ------------------------------------------------------------------ sampling (tp = 1)
    SAMPLE_K = ops.SAMPLE_K  # candidates kept per slot; a request's top_k is clamped to it

    def enable_sampling(self, batch: int) -> None:
        """Per-slot sampling state, all on the device so that the step stays one CUDA graph:
        temperature (0 = greedy), top_k, top_p, presence / repetition penalty, `seen_out` / `seen_any`
        ([B, V] flags of tokens generated / seen in prompt or output) and a buffer of uniform noise that
        the host refills before every step (the Gumbel-max draw inside the graph then needs no generator)."""
        dev, v = self.device, self.v_loc  # `seen_*` cover this rank's vocabulary shard
        self.sampling = {
            "temperature": torch.zeros(batch, device=dev), "top_k": torch.ones(batch, dtype=torch.long, device=dev),
            "top_p": torch.ones(batch, device=dev), "presence": torch.zeros(batch, device=dev),
            "repetition": torch.ones(batch, device=dev),
            "seen_out": torch.zeros(batch, v, dtype=torch.bool, device=dev),
            "seen_any": torch.zeros(batch, v, dtype=torch.bool, device=dev),
            "noise": torch.full((batch, self.SAMPLE_K), 0.5, device=dev),
        }

    def refill_noise(self, generator: Optional[torch.Generator] = None) -> None:
        if self.sampling is not None:
            self.sampling["noise"].uniform_(1e-7, 1.0, generator=generator)

    def _sample(self, logits: torch.Tensor) -> torch.Tensor:
        """Penalties, top-k / top-p and the Gumbel-max draw for every slot (`ops.sample_topk`, `ops.sample_pick`):
        the 64 best penalised logits of this rank's vocabulary shard, the candidates of all shards gathered, then
        the draw. Every rank ends up with the same choice (same candidates, same noise). The token consumed by
        this step (self.tokens) counts as generated. Writes self.next_tokens."""
        sp = self.sampling
        cand = ops.sample_topk(logits, sp["seen_any"], sp["seen_out"], self.tokens, sp["presence"], sp["repetition"],
                               self.rank * self.v_loc)
        if self.tp > 1:
            allc = torch.empty(self.tp * cand.shape[0], ops.SAMPLE_K, 2, device=cand.device)  # rank-major
            dist.all_gather_into_tensor(allc, cand, group=self.group)
            cand = allc
        return ops.sample_pick(cand, self.tp, sp["temperature"], sp["top_k"], sp["top_p"], sp["noise"],
                               self.cfg.vocab_size, self.next_tokens)

    # ------------------------------------------------------------------ public
    @torch.no_grad()
    def prefill_synthetic(self, batch: int, prompt_len: int, new_tokens: int, seed: int = 1) -> None:
        """Fills the cache with `prompt_len` tokens of synthetic K/V per sequence (N(0,1) keys and
        values, as produced by random patch embeddings through random-init layers) and reserves the
        pages for the whole generation."""
        g = torch.Generator(device=self.device)
        g.manual_seed(seed + self.rank)
        self.seq_ids = list(range(batch))
        for s in self.seq_ids:
            self.cache.release(s)
            assert self.cache.reserve(s, prompt_len + new_tokens), "KV pool exhausted"
        self.table, _ = self.cache.tables(self.seq_ids)
        self.max_len = prompt_len + new_tokens
        pos = torch.arange(prompt_len, device=self.device)[None].expand(batch, -1)
        slots = PagedKVCache.slots(self.table, pos, self.page_size).reshape(-1)
        for li in range(self.cfg.n_layers):
            k = torch.randn(batch * prompt_len, self.hk, self.hd, generator=g, device=self.device).bfloat16()
            v = torch.randn(batch * prompt_len, self.hk, self.hd, generator=g, device=self.device).bfloat16()
            self.cache.write(li, k, v, slots)
        self.lens = torch.full((batch,), prompt_len, dtype=torch.int32, device=self.device)
        self.tokens = torch.randint(0, self.cfg.vocab_size, (batch,), generator=g, device=self.device)
        if self.tp > 1:
            dist.broadcast(self.tokens, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                           group=self.group)
        self.next_tokens = torch.zeros_like(self.tokens)

    @torch.no_grad()
    def prefill(self, model, ids: torch.Tensor, embeds: Optional[torch.Tensor], new_tokens: int, ctx=None) -> None:
        """Real prefill through the AR tower (`model` holds full weights; used by tests and the
        single-GPU server): runs the causal forward per sequence and writes K/V into the pages.
        The decoder's own layer weights must have been loaded from the same model (`load_from`)."""
        batch, n = ids.shape
        self.seq_ids = list(range(batch))
        for s in self.seq_ids:
            self.cache.release(s)
            assert self.cache.reserve(s, n + new_tokens), "KV pool exhausted"
        self.table, _ = self.cache.tables(self.seq_ids)
        self.max_len = n + new_tokens
        pos_ids = rope.text_positions(n, 0, self.device)
        last = []
        for b in range(batch):
            x = model.embed_tokens(ids[b:b + 1]) if embeds is None else embeds[b:b + 1]
            h, kvs = model.ar_forward(x, pos_ids) if ctx is None else model.ar_forward(x, pos_ids, None, ctx)
            slots = PagedKVCache.slots(self.table[b:b + 1], torch.arange(n, device=self.device)[None], self.page_size)[0]
            for li, (k, v) in enumerate(kvs):
                sl = slice(self.rank * self.hk, (self.rank + 1) * self.hk) if k.shape[2] != self.hk else slice(None)
                self.cache.write(li, k[0, :, sl].contiguous(), v[0, :, sl].contiguous(), slots)
            last.append(model.lm_logits(h[:, -1:]).float()[0, 0].argmax())
        self.lens = torch.full((batch,), n, dtype=torch.int32, device=self.device)
        self.tokens = torch.stack(last).to(self.device)
        self.next_tokens = torch.zeros_like(self.tokens)

    def load_from(self, model) -> None:
        """Cuts this rank's shards out of a full MoTModel's AR tower."""
        cfg, r = self.cfg, self.rank
        hd = self.hd
        for li, layer in enumerate(model.ar.layers):
            v = layer.views()
            q0, k0, v0 = 0, cfg.q_dim, cfg.q_dim + cfg.kv_dim
            w = v["wqkv"]
            self.layers[li]["wqkv"] = torch.cat([w[q0 + r * self.hq * hd:q0 + (r + 1) * self.hq * hd],
                                                 w[k0 + r * self.hk * hd:k0 + (r + 1) * self.hk * hd],
                                                 w[v0 + r * self.hk * hd:v0 + (r + 1) * self.hk * hd]]).contiguous()
            self.layers[li]["wo"] = v["wo"][:, r * self.hq * hd:(r + 1) * self.hq * hd].contiguous()
            self.layers[li]["w_gate_up"] = torch.cat([v["w_gate_up"][r * self.ffn:(r + 1) * self.ffn],
                                                      v["w_gate_up"][cfg.ffn_dim + r * self.ffn:
                                                                     cfg.ffn_dim + (r + 1) * self.ffn]]).contiguous()
            self.layers[li]["w_down"] = v["w_down"][:, r * self.ffn:(r + 1) * self.ffn].contiguous()
            for k in ("norm1", "norm2", "q_norm", "k_norm"):
                self.layers[li][k] = v[k].clone()
        lo, hi = r * self.v_loc, min((r + 1) * self.v_loc, cfg.vocab_size)
        self.lm_head = torch.zeros(self.v_loc, cfg.d_model, dtype=model.lm_head.dtype, device=self.device)
        self.lm_head[:hi - lo] = model.lm_head[lo:hi]
        if hi - lo < self.v_loc:  # padded vocab rows must never win the arg-max
            self.lm_head[hi - lo:] = 0
        self.embed = model.embed.data
        self.final_norm = model.ar_norm.data

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """One decode step for the whole batch; returns the new tokens [B] (device tensor)."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step_impl()
        self.tokens.copy_(self.next_tokens)
        return self.next_tokens

    @torch.no_grad()
    def capture(self, warmup: int = 2) -> None:
        """Captures `_step_impl` into a CUDA graph. Warm-up steps run first (workspace and
        symmetric-memory set-up must not happen during capture); they advance the sequences."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._step_impl()
                self.tokens.copy_(self.next_tokens)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if self.tp > 1:
            dist.barrier(group=self.group)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._step_impl()
        self.graph = g
        self.tokens.copy_(self.next_tokens)  # the capture ran one real step as well


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="Cosmos3-Nano")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt-vision", type=int, default=8192)
    ap.add_argument("--prompt-text", type=int, default=256)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-fused", action="store_true", help="NCCL all-reduce instead of the one-shot kernel")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--page-size", type=int, default=32, help="tokens per KV-cache page (8, 16, 32, 64 or 128)")
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = get_model_config(args.model, **({"n_layers": args.layers} if args.layers else {}))
    prompt = args.prompt_vision + args.prompt_text
    dec = TPDecoder(cfg, world, rank, dist.group.WORLD if world > 1 else None, dev, max_batch=args.batch,
                    max_len=prompt + args.new_tokens + args.warmup + 8, fused=not args.no_fused,
                    page_size=args.page_size)
    dec.prefill_synthetic(args.batch, prompt, args.new_tokens + args.warmup + 8)
    if args.no_graph:
        for _ in range(args.warmup):
            dec.step()
    else:
        dec.capture(warmup=max(2, args.warmup - 1))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.new_tokens):
        dec.step()
    e1.record()
    torch.cuda.synchronize()
    ops.check_status()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    if rank == 0:
        toks = args.batch * args.new_tokens
        kv_bytes = 2 * cfg.n_layers * args.batch * (prompt + args.new_tokens / 2) * (cfg.n_kv_heads // world) * cfg.head_dim * 2
        w_bytes = (cfg.tower_params() // world + (cfg.vocab_size // world) * cfg.d_model) * 2
        floor_ms = (kv_bytes + w_bytes) / 6551.4e9 * 1e3
        print(json.dumps({"metric": "reasoner_decode_tokens_per_s", "value": round(toks / ms * 1e3, 1),
                          "ms_per_step": round(ms / args.new_tokens, 4), "n_gpus": world, "batch": args.batch,
                          "prompt_tokens": prompt, "new_tokens": args.new_tokens, "model": cfg.name,
                          "layers": cfg.n_layers, "cuda_graph": not args.no_graph, "fused_allreduce": not args.no_fused,
                          "hbm_floor_ms_per_step": round(floor_ms, 4),
                          "fraction_of_hbm_floor": round(floor_ms / (ms / args.new_tokens), 3),
                          "data": "synthetic KV (N(0,1)), random-init weights"}), flush=True)
    if world > 1:
        from ..parallel.runtime import finish
        finish(hard=(__name__ == "__main__"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
