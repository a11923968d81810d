"""Continuous batching for the Reasoner: requests join and leave a fixed set of decode slots while
the batch keeps stepping (the serving pattern behind the reference's published Reasoner numbers,
which are measured through vLLM at client concurrency 1..256, reference
inference_benchmarks.md:239-241,501-535).

`BatchEngine` owns a `TPDecoder` whose batch is `max_batch` slots. A slot is either idle (length 0,
block table pointing at a scratch page, its lane of the step ignored) or bound to a request. Each
engine step (1) admits waiting requests into idle slots while KV pages last — the prompts of the
admitted group run through the AR tower in one padded forward and their K/V go into the requests' pages, (2) runs ONE decode step for all
slots (the same CUDA graph whatever the mix of requests, because the per-slot state lives in device
tensors that the host edits in place), (3) reads the new tokens back, appends them to their
requests and retires the ones that hit an end token or their token limit, freeing pages and slot.
Sampling (temperature, top-k, top-p, presence and repetition penalties, per request) runs on the device
inside the same graph; temperature 0 is greedy.

`EngineWorker` runs the loop in a thread and hands out futures, so concurrent HTTP requests of
`serve/server.py` share decode steps.
"""
from __future__ import annotations

import threading
import time
from collections import deque
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

import torch

from .. import ops
from ..config import MoTConfig
from ..models import rope
from .decoder import TPDecoder
from .paged import PagedKVCache


@dataclass
class Request:
    rid: int
    ids: List[int]
    max_new_tokens: int
    eos_ids: Sequence[int] = ()
    temperature: float = 0.0       # 0 = greedy
    top_k: int = 20
    top_p: float = 1.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    # prompts with media: embeddings [n, d] with the vision rows spliced in, 3-D rotary ids [3, n], the vision
    # mask [n] and DeepStack features; such a request is prefilled on its own
    embeds: Optional[torch.Tensor] = None
    positions: Optional[torch.Tensor] = None
    vision_mask: Optional[torch.Tensor] = None
    deepstack: Optional[Sequence[torch.Tensor]] = None
    on_token: Optional[object] = None   # callable(token id), called from the engine thread for every new token
    out: List[int] = field(default_factory=list)
    slot: int = -1
    t_submit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    finish_reason: str = ""
    future: Optional[Future] = None


class BatchEngine:
    def __init__(self, model, max_batch: int = 8, max_len: int = 4096, page_size: int = 32, device=None,
                 dtype=None, use_graph: Optional[bool] = None, group=None):
        """`group`: tensor-parallel process group (None = one rank). Every rank of the group builds the engine on
        the same model weights; rank 0 of the group takes the requests (`submit`), the others call `follow()`."""
        import torch.distributed as dist

        self.model = model
        self.cfg: MoTConfig = model.cfg
        p = next(model.parameters())
        self.device = torch.device(device) if device is not None else p.device
        dtype = dtype or p.dtype
        self.max_batch, self.max_len = max_batch, max_len
        self.group = group
        self.tp = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self._new: List[dict] = []      # requests submitted on rank 0 since the last step (sent to the followers)
        self._stop = False
        self.dec = TPDecoder(self.cfg, self.tp, self.rank, group, self.device, page_size=page_size, max_batch=max_batch,
                             max_len=max_len, dtype=dtype)
        self.dec.load_from(model)
        cache = self.dec.cache
        # one page is set aside for idle slots: their (ignored) K/V writes land there
        self.scratch_seq = -1
        assert cache.reserve(self.scratch_seq, 1), "KV pool too small"
        self.scratch_page = int(cache.alloc.blocks(self.scratch_seq)[0])
        self.max_pages = cache.max_pages
        dev = self.device
        self.dec.table = torch.full((max_batch, self.max_pages), self.scratch_page, dtype=torch.int32, device=dev)
        self.dec.lens = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.dec.tokens = torch.zeros(max_batch, dtype=torch.long, device=dev)
        self.dec.next_tokens = torch.zeros(max_batch, dtype=torch.long, device=dev)
        self.dec.step_inc = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.dec.max_len = max_len
        self.dec.enable_sampling(max_batch)
        self.dec.pos_delta = torch.zeros(max_batch, dtype=torch.long, device=dev)
        self.noise_gen = torch.Generator(device=dev)
        self.noise_gen.manual_seed(0)
        self.slots: List[Optional[Request]] = [None] * max_batch
        self.waiting: Deque[Request] = deque()
        self.finished: Dict[int, Request] = {}
        self._next_rid = 0
        self.steps = 0
        self.max_prefill_tokens = 16384  # padded prompt tokens per prefill forward
        self.use_graph = (self.device.type == "cuda") if use_graph is None else use_graph
        self._graph_ready = False

    # ------------------------------------------------------------------ requests
    def submit(self, ids: Sequence[int], max_new_tokens: int = 256, eos_ids: Sequence[int] = (),
               temperature: float = 0.0, top_k: int = 20, top_p: float = 1.0, presence_penalty: float = 0.0,
               repetition_penalty: float = 1.0, embeds: Optional[torch.Tensor] = None,
               positions: Optional[torch.Tensor] = None, vision_mask: Optional[torch.Tensor] = None,
               deepstack: Optional[Sequence[torch.Tensor]] = None, on_token=None) -> Request:
        if len(ids) < 1:
            raise ValueError("empty prompt")
        if len(ids) + max_new_tokens > self.max_len:
            raise ValueError(f"prompt ({len(ids)}) + max_new_tokens ({max_new_tokens}) exceeds max_len {self.max_len}")
        params = dict(ids=[min(int(t), self.cfg.vocab_size - 1) for t in ids], max_new_tokens=int(max_new_tokens),
                      eos_ids=tuple(eos_ids), temperature=float(temperature),
                      top_k=int(top_k) if top_k and top_k > 0 else ops.SAMPLE_K, top_p=float(top_p),
                      presence_penalty=float(presence_penalty), repetition_penalty=float(repetition_penalty))
        r = self._enqueue(params, embeds, positions, vision_mask, deepstack, on_token)
        if embeds is not None and (positions is None or embeds.shape[0] != len(r.ids)):
            self.waiting.pop()
            raise ValueError("a request with embeddings needs positions [3, n] and one embedding row per prompt token")
        if self.tp > 1:
            if embeds is not None:
                # the vision encoder ran once, on this rank; its outputs travel to the followers with the request
                cpu = lambda t: None if t is None else t.detach().to("cpu")  # noqa: E731
                params = dict(params, media=dict(embeds=cpu(embeds), positions=cpu(positions), vision_mask=cpu(vision_mask),
                                                 deepstack=None if deepstack is None else [cpu(t) for t in deepstack]))
            self._new.append(params)
        return r

    def _enqueue(self, params: dict, embeds=None, positions=None, vision_mask=None, deepstack=None, on_token=None
                 ) -> Request:
        r = Request(self._next_rid, params["ids"], params["max_new_tokens"], params["eos_ids"], params["temperature"],
                    params["top_k"], params["top_p"], params["presence_penalty"], params["repetition_penalty"],
                    embeds, positions, vision_mask, deepstack, on_token, t_submit=time.time())
        self._next_rid += 1
        self.waiting.append(r)
        return r

    def _sync_requests(self) -> None:
        """Tensor-parallel engines: rank 0 sends what was submitted since the last step (and the stop flag); the
        followers queue identical requests, so that admission, decoding and retirement run in lock-step."""
        import torch.distributed as dist

        payload = [(self._new, self._stop)] if self.rank == 0 else [None]
        dist.broadcast_object_list(payload, src=dist.get_global_rank(self.group, 0), group=self.group)
        new, stop = payload[0]
        if self.rank == 0:
            self._new = []
        else:
            self._stop = stop
            for params in new:
                self._enqueue(params, **(params.get("media") or {}))

    def follow(self) -> None:
        """Loop of the ranks other than 0: mirror every step of rank 0 until it calls `shutdown()`."""
        assert self.tp > 1 and self.rank != 0
        while True:
            self.step()
            if self._stop and not self.has_work():
                return

    def shutdown(self) -> None:
        """Rank 0: lets the followers leave `follow()` (after the work in flight is done)."""
        if self.tp > 1 and self.rank == 0:
            self.run_until_done()
            self._stop = True
            self.step()

    def has_work(self) -> bool:
        return bool(self.waiting) or any(s is not None for s in self.slots)

    def n_active(self) -> int:
        return sum(s is not None for s in self.slots)

    # ------------------------------------------------------------------ admission (prefill)
    @torch.no_grad()
    def _admit_group(self, group: List[Request], slots: List[int]) -> None:
        """Prefills several requests in ONE forward of the AR tower: prompts are right-padded to the longest
        of the group (causal attention keeps the padding from reaching real tokens), the K/V rows of the real
        tokens of all requests go into their pages with one cache write per layer, and each request's first
        token is the arg-max at its own last position."""
        dec, cache, dev = self.dec, self.dec.cache, self.device
        lens = [len(r.ids) for r in group]
        n_max, bsz = max(lens), len(group)
        ids = torch.zeros(bsz, n_max, dtype=torch.long)
        for i, r in enumerate(group):
            ids[i, :lens[i]] = torch.tensor(r.ids, dtype=torch.long)
        ids = ids.to(dev)
        media = group[0].embeds is not None
        if media:  # admitted alone (its rotary ids are its own)
            r0 = group[0]
            x = r0.embeds.to(device=dev, dtype=self.model.embed.dtype)[None]
            vm = None if r0.vision_mask is None else r0.vision_mask.to(dev).reshape(1, -1)
            deep = None if r0.deepstack is None else [d.to(device=dev, dtype=x.dtype) for d in r0.deepstack]
            h, kvs = self.model.ar_forward(x, r0.positions.to(dev), deepstack=deep, vision_mask=vm)
            delta = [int(rope.next_start(r0.positions)) - lens[0]]
        else:
            h, kvs = self.model.ar_forward(self.model.embed_tokens(ids), rope.text_positions(n_max, 0, dev))
            delta = [0] * bsz
        table, _ = cache.tables([r.rid for r in group])
        slot_idx = torch.tensor(slots, dtype=torch.long, device=dev)
        dec.table[slot_idx] = table
        len_t = torch.tensor(lens, device=dev)
        pos = torch.arange(n_max, device=dev)[None].expand(bsz, -1)
        real = pos < len_t[:, None]                                          # [B, n_max]
        rows = PagedKVCache.slots(table, pos.clamp(max=cache.max_pages * dec.page_size - 1), dec.page_size)[real]
        # every rank ran the full prefill; it keeps the K/V heads of its tensor-parallel shard
        hs = slice(self.rank * dec.hk, (self.rank + 1) * dec.hk)
        for li, (k, v) in enumerate(kvs):
            cache.write(li, k[real][:, hs].contiguous(), v[real][:, hs].contiguous(), rows)
        last = h[torch.arange(bsz, device=dev), len_t - 1][:, None]          # [B, 1, d]
        logits = self.model.lm_logits(last).float()[:, 0]                    # [B, V]
        # per-slot sampling state; the prompt tokens count as "seen" for the repetition penalty
        sp = dec.sampling
        for name, vals in (("temperature", [r.temperature for r in group]), ("top_p", [r.top_p for r in group]),
                           ("presence", [r.presence_penalty for r in group]),
                           ("repetition", [r.repetition_penalty for r in group])):
            sp[name][slot_idx] = torch.tensor(vals, dtype=torch.float32, device=dev)
        sp["top_k"][slot_idx] = torch.tensor([r.top_k for r in group], dtype=torch.long, device=dev)
        seen = torch.zeros(bsz, dec.v_loc * self.tp, dtype=torch.bool, device=dev)   # whole (padded) vocabulary
        seen.scatter_(1, ids, real)
        sp["seen_any"][slot_idx] = seen[:, self.rank * dec.v_loc:(self.rank + 1) * dec.v_loc]
        sp["seen_out"][slot_idx] = False
        first = self._first_tokens(logits, slot_idx, seen[:, :logits.shape[1]])
        dec.lens[slot_idx] = len_t.to(dec.lens.dtype)
        dec.pos_delta[slot_idx] = torch.tensor(delta, dtype=torch.long, device=dev)
        dec.tokens[slot_idx] = first
        dec.step_inc[slot_idx] = 1
        now = time.time()
        for r, slot, tok in zip(group, slots, first.tolist()):
            r.slot, r.t_first = slot, now
            self.slots[slot] = r
            self._accept(r, int(tok))

    def _first_tokens(self, logits: torch.Tensor, slot_idx: torch.Tensor, seen: torch.Tensor) -> torch.Tensor:
        """First token of every request of a prefill group with the decoder's own sampler (same rules as the
        decode steps: repetition penalty over the prompt, top-k / top-p / temperature per request)."""
        dec, sp = self.dec, self.dec.sampling
        rep = sp["repetition"][slot_idx][:, None]
        pen = torch.where(logits > 0, logits / rep, logits * rep)
        logits = torch.where(seen, pen, logits)
        noise = torch.rand(len(slot_idx), ops.SAMPLE_K, device=logits.device, generator=self.noise_gen).clamp_min(1e-7)
        cand = ops.sample_topk(logits, None, None, None, None, None, 0)
        out = torch.empty(len(slot_idx), dtype=torch.long, device=logits.device)
        return ops.sample_pick(cand, 1, sp["temperature"][slot_idx].contiguous(), sp["top_k"][slot_idx].contiguous(),
                               sp["top_p"][slot_idx].contiguous(), noise, dec.cfg.vocab_size, out)

    def _accept(self, r: Request, tok: int) -> None:
        """Books a generated token; retires the request when it ends."""
        r.out.append(tok)
        halt = False
        if r.on_token is not None:
            # a callback that returns False ends the request here (e.g. a stop string completed); only honoured on a
            # single rank, because followers of a tensor-parallel engine do not run the callback
            halt = r.on_token(tok) is False and self.tp == 1
        if halt:
            self._retire(r, "stop")
        elif tok in r.eos_ids:
            self._retire(r, "stop")
        elif len(r.out) >= r.max_new_tokens:
            self._retire(r, "length")

    def _retire(self, r: Request, reason: str) -> None:
        s = r.slot
        r.finish_reason, r.t_done = reason, time.time()
        self.dec.cache.release(r.rid)
        self.dec.table[s].fill_(self.scratch_page)
        self.dec.lens[s] = 0
        self.dec.step_inc[s] = 0
        self.dec.tokens[s] = 0
        self.slots[s] = None
        self.finished[r.rid] = r
        if r.future is not None and not r.future.done():
            r.future.set_result(r)

    # ------------------------------------------------------------------ one engine step
    @torch.no_grad()
    def step(self) -> List[Request]:
        """Admits what fits, runs one decode step for the batch, returns the requests that finished."""
        done_before = set(self.finished)
        if self.tp > 1:
            self._sync_requests()
        cache = self.dec.cache
        free = [i for i in range(self.max_batch) if self.slots[i] is None]
        while self.waiting and free:
            # a group of waiting requests whose padded prompts fit the prefill token limit
            group: List[Request] = []
            slots: List[int] = []
            n_max = 0
            while self.waiting and free:
                r = self.waiting[0]
                new_max = max(n_max, len(r.ids))
                if group and (new_max * (len(group) + 1) > self.max_prefill_tokens or r.embeds is not None
                              or group[0].embeds is not None):
                    break
                if not cache.reserve(r.rid, len(r.ids) + r.max_new_tokens):
                    break  # pages are short: the request stays first in line until others retire
                self.waiting.popleft()
                group.append(r)
                slots.append(free.pop(0))
                n_max = new_max
            if not group:
                break
            self._admit_group(group, slots)
            free = [i for i in range(self.max_batch) if self.slots[i] is None]
            if self.waiting and not cache.alloc.can_allocate(len(self.waiting[0].ids) + self.waiting[0].max_new_tokens):
                break
        if any(s is not None for s in self.slots):
            if self.use_graph and not self._graph_ready:
                self._capture()
            self.dec.refill_noise(self.noise_gen)
            new = self.dec.step().tolist()  # one device-to-host read per step (end-token detection)
            self.steps += 1
            for slot, r in enumerate(self.slots):
                if r is not None:
                    self._accept(r, int(new[slot]))
        return [self.finished[k] for k in self.finished if k not in done_before]

    def _capture(self) -> None:
        """Graph capture without side effects on the requests: the warm-up and capture steps run with every
        slot parked on the scratch page (length 0, no advance), then the live state is put back."""
        dec = self.dec
        keep = (dec.table.clone(), dec.lens.clone(), dec.tokens.clone(), dec.step_inc.clone())
        dec.table.fill_(self.scratch_page)
        dec.lens.zero_()
        dec.step_inc.zero_()
        dec.capture(warmup=2)
        for dst, src in zip((dec.table, dec.lens, dec.tokens, dec.step_inc), keep):
            dst.copy_(src)
        self._graph_ready = True

    def run_until_done(self, max_steps: int = 1 << 20) -> None:
        n = 0
        while self.has_work() and n < max_steps:
            self.step()
            n += 1


class EngineWorker:
    """Runs a BatchEngine in a background thread; `submit` returns a Future that resolves to the Request."""

    def __init__(self, engine: BatchEngine):
        self.engine = engine
        self._cv = threading.Condition()
        self._pending: Deque = deque()
        self._stop = False
        self._thread = threading.Thread(target=self._loop, name="cosmos-batch-engine", daemon=True)
        self._thread.start()

    def submit(self, ids: Sequence[int], max_new_tokens: int = 256, eos_ids: Sequence[int] = (), **sampling) -> Future:
        """`sampling`: temperature, top_k, top_p, presence_penalty, repetition_penalty (see BatchEngine.submit)."""
        fut: Future = Future()
        with self._cv:
            self._pending.append((list(ids), max_new_tokens, tuple(eos_ids), sampling, fut))
            self._cv.notify()
        return fut

    def close(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify()
        self._thread.join(timeout=30)

    def _loop(self) -> None:
        eng = self.engine
        while True:
            with self._cv:
                while not self._pending and not eng.has_work() and not self._stop:
                    self._cv.wait()
                if self._stop:
                    return
                new = list(self._pending)
                self._pending.clear()
            for ids, n, eos, sampling, fut in new:
                try:
                    eng.submit(ids, n, eos, **sampling).future = fut
                except Exception as e:  # noqa: BLE001 - delivered to the caller through the future
                    fut.set_exception(e)
            try:
                eng.step()
            except Exception as e:  # noqa: BLE001 - fail every request in flight rather than hang the callers
                for r in list(eng.waiting) + [s for s in eng.slots if s is not None]:
                    if r.future is not None and not r.future.done():
                        r.future.set_exception(e)
                eng.waiting.clear()
                for s, r in enumerate(eng.slots):
                    if r is not None:
                        eng.slots[s] = None
                raise


def main(argv=None) -> int:
    """Serving benchmark: `--requests` prompts of `--prompt-len` random tokens arrive at once and are served
    with at most `--max-num-seqs` in the decode batch; prints output tokens per second, time to first token
    and request latency (the metrics of the reference's Reasoner tables, inference_benchmarks.md:501-535)."""
    import argparse
    import json

    from ..config import get_model_config
    from ..models.mot import MoTModel

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--model", default="Cosmos3-Nano")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=306, help="50 text tokens + a short clip's vision tokens")
    ap.add_argument("--new-tokens", type=int, default=100)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--page-size", type=int, default=32, help="tokens per KV-cache page (8, 16, 32, 64 or 128)")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy; else top-k 20 / top-p 0.8 sampling")
    args = ap.parse_args(argv)
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", 0) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    cfg = get_model_config(args.model, **({"n_layers": args.layers} if args.layers else {}))
    model = MoTModel(cfg, dtype=dtype, device=dev, towers=("ar",))  # the Reasoner needs the AR tower only
    model.init_weights(seed=0)
    eng = BatchEngine(model, max_batch=args.max_num_seqs, max_len=args.prompt_len + args.new_tokens + 16,
                      page_size=args.page_size)
    g = torch.Generator().manual_seed(0)
    warm = eng.submit(torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist(), 4)
    eng.run_until_done()  # graph capture and workspace set-up happen here
    assert len(warm.out) == 4
    steps0 = eng.steps
    if cuda:
        torch.cuda.synchronize()
    t0 = time.time()
    reqs = [eng.submit(torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist(), args.new_tokens,
                       temperature=args.temperature, top_k=20, top_p=0.8 if args.temperature > 0 else 1.0,
                       presence_penalty=1.5 if args.temperature > 0 else 0.0)
            for _ in range(args.requests)]
    eng.run_until_done()
    if cuda:
        torch.cuda.synchronize()
    dt = time.time() - t0
    toks = sum(len(r.out) for r in reqs)
    ttft = sorted((r.t_first - r.t_submit) * 1e3 for r in reqs)
    lat = sorted((r.t_done - r.t_submit) * 1e3 for r in reqs)
    print(json.dumps({"metric": "reasoner_serving_output_tokens_per_s", "value": round(toks / dt, 1),
                      "requests": args.requests, "max_num_seqs": args.max_num_seqs, "prompt_len": args.prompt_len,
                      "new_tokens": args.new_tokens, "wall_s": round(dt, 3), "decode_steps": eng.steps - steps0,
                      "ttft_ms_avg": round(sum(ttft) / len(ttft), 1), "ttft_ms_p50": round(ttft[len(ttft) // 2], 1),
                      "request_latency_ms_avg": round(sum(lat) / len(lat), 1), "model": cfg.name,
                      "layers": cfg.n_layers, "n_gpus": 1, "cuda_graph": eng.use_graph,
                      "temperature": args.temperature,
                      "data": "random prompt token ids, random-init weights"}), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
