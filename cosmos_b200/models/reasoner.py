"""Reasoner engine: causal prefill of the AR tower (text + ViT vision tokens) and token-by-token
decode with a KV cache, with the reference's sampling controls (temperature, top-p, top-k,
repetition and presence penalties; reference README.md:159-167 and
cookbooks/cosmos3/reasoner/reasoner_prompt_guide.md:19-33).

Two cache layouts: a contiguous per-sequence cache (simple, used by the CLI for single requests)
and the paged cache of `cosmos_b200.serve.paged` used by the batched server and the TP decode
benchmark, whose attention runs in the paged-KV decode kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..config import DecodingConfig, MoTConfig
from . import rope
from .mot import KV, LOCAL_ATTN, AttnContext, MoTModel


def apply_penalties(logits: torch.Tensor, generated: Sequence[int], prompt_ids: Sequence[int],
                    repetition_penalty: float, presence_penalty: float) -> torch.Tensor:
    """logits [V] fp32. Repetition penalty (CTRL-style) divides positive / multiplies negative
    logits of tokens seen in prompt or output; presence penalty subtracts a constant from tokens
    already generated."""
    if repetition_penalty != 1.0:
        seen = torch.tensor(sorted(set(prompt_ids) | set(generated)), dtype=torch.long, device=logits.device)
        if seen.numel():
            vals = logits[seen]
            logits[seen] = torch.where(vals > 0, vals / repetition_penalty, vals * repetition_penalty)
    if presence_penalty != 0.0 and generated:
        gen = torch.tensor(sorted(set(generated)), dtype=torch.long, device=logits.device)
        logits[gen] -= presence_penalty
    return logits


def sample_token(logits: torch.Tensor, dc: DecodingConfig, generator: Optional[torch.Generator] = None) -> int:
    """logits [V] fp32 -> token id; greedy when do_sample is false or temperature is 0."""
    if not dc.do_sample or dc.temperature <= 0:
        return int(torch.argmax(logits))
    logits = logits / dc.temperature
    if dc.top_k and dc.top_k > 0:
        k = min(dc.top_k, logits.numel())
        kth = torch.topk(logits, k).values[-1]
        logits = torch.where(logits < kth, torch.full_like(logits, float("-inf")), logits)
    probs = torch.softmax(logits, dim=-1)
    if dc.top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        cum = torch.cumsum(sp, dim=-1)
        keep = cum - sp < dc.top_p  # always keeps the most likely token
        sp = torch.where(keep, sp, torch.zeros_like(sp))
        probs = torch.zeros_like(probs).scatter_(0, si, sp)
        probs = probs / probs.sum()
    return int(torch.multinomial(probs, 1, generator=generator))


class ReasonerEngine:
    def __init__(self, model: MoTModel, vit=None, ctx: AttnContext = LOCAL_ATTN):
        self.model, self.vit, self.ctx = model, vit, ctx
        self.cfg: MoTConfig = model.cfg

    @torch.no_grad()
    def embed(self, ids: torch.Tensor, vision_embeds: Optional[torch.Tensor] = None,
              vision_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """ids [B, S]; positions flagged by vision_mask [B, S] are replaced by vision_embeds rows."""
        x = self.model.embed_tokens(ids)
        if vision_embeds is not None and vision_mask is not None and vision_mask.any():
            x = x.clone()
            x[vision_mask] = vision_embeds.to(x.dtype).reshape(-1, x.shape[-1])[:int(vision_mask.sum())]
        return x

    def positions(self, ids: torch.Tensor, vision_mask: Optional[torch.Tensor], grids: Sequence[Tuple[int, int, int]]
                  ) -> torch.Tensor:
        """3-D mRoPE ids of a prompt: text tokens advance all axes together; each run of vision tokens
        is a (t, h, w) grid anchored at the running index."""
        s = ids.shape[1]
        if vision_mask is None or not vision_mask.any() or not grids:
            return rope.text_positions(s, 0, ids.device)
        mask = vision_mask[0].tolist()
        parts, cur, i, gi = [], 0, 0, 0
        while i < s:
            if mask[i] and gi < len(grids):
                t, h, w = grids[gi]
                n = t * h * w
                p = rope.grid_positions(t, h, w, cur, ids.device)
                parts.append(p)
                cur = rope.next_start(p)
                i += n
                gi += 1
            else:
                j = i
                while j < s and not (mask[j] and gi < len(grids)):
                    j += 1
                parts.append(rope.text_positions(j - i, cur, ids.device))
                cur += j - i
                i = j
        return torch.cat(parts, dim=1)[:, :s]

    @torch.no_grad()
    def prefill(self, x: torch.Tensor, pos: torch.Tensor, deepstack=None, vision_mask=None
                ) -> Tuple[torch.Tensor, List[KV]]:
        """x [B, S, d] -> (logits of the last position [B, V] fp32, per-layer KV)."""
        h, kvs = self.model.ar_forward(x, pos, None, self.ctx, deepstack=deepstack, vision_mask=vision_mask)
        return self.model.lm_logits(h[:, -1:]).float()[:, 0], kvs

    @torch.no_grad()
    def decode_one(self, token: torch.Tensor, pos_index: int, kvs: List[KV]) -> Tuple[torch.Tensor, List[KV]]:
        """token [B] -> (logits [B, V] fp32, grown KV)."""
        x = self.model.embed_tokens(token[:, None])
        pos = rope.text_positions(1, pos_index, token.device)
        h, kvs = self.model.ar_forward(x, pos, kvs, self.ctx)
        return self.model.lm_logits(h).float()[:, 0], kvs

    @torch.no_grad()
    def generate(self, ids: Sequence[int], dc: DecodingConfig, eos_ids: Sequence[int] = (),
                 vision_embeds: Optional[torch.Tensor] = None, vision_token_id: Optional[int] = None,
                 grids: Sequence[Tuple[int, int, int]] = (), on_token: Optional[Callable[[int], None]] = None,
                 deepstack: Optional[Sequence[torch.Tensor]] = None) -> Tuple[List[int], dict]:
        dev = next(self.model.parameters()).device
        ids_t = torch.tensor([list(ids)], dtype=torch.long, device=dev)
        vmask = (ids_t == vision_token_id) if vision_token_id is not None and vision_embeds is not None else None
        x = self.embed(ids_t.clamp(max=self.cfg.vocab_size - 1), vision_embeds, vmask)
        pos = self.positions(ids_t, vmask, grids)
        gen = None
        if dc.seed is not None:
            gen = torch.Generator(device=dev)
            gen.manual_seed(dc.seed)
        logits, kvs = self.prefill(x, pos, deepstack if vmask is not None else None, vmask)
        next_pos = rope.next_start(pos)
        out: List[int] = []
        for _ in range(dc.max_new_tokens):
            lg = apply_penalties(logits[0].clone(), out, ids, dc.repetition_penalty, dc.presence_penalty)
            tok = sample_token(lg, dc, gen)
            out.append(tok)
            if on_token is not None:
                on_token(tok)
            if tok in eos_ids:
                break
            logits, kvs = self.decode_one(torch.tensor([tok], device=dev), next_pos, kvs)
            next_pos += 1
        return out, {"prompt_tokens": len(ids), "completion_tokens": len(out)}
