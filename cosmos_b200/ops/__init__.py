"""Fused ops of the framework.

Every function takes torch tensors. CUDA bf16 tensors run the hand-written sm_100a kernels
of ``cosmos_b200/_C.so`` (``torch.ops.cosmos_b200.*``); CPU tensors (and fp32 CUDA tensors
in tests of the oracle itself) run the plain-PyTorch definitions in ``reference.py``.
There is no silent fallback on a GPU: if the extension cannot be loaded, calling an op with
a CUDA bf16 tensor raises.
"""
from __future__ import annotations

import math
import os
from pathlib import Path
from typing import Optional, Tuple

import torch

from . import reference as ref
from .reference import (EPI_GATED_RESID, EPI_PLAIN, EPI_QKV_ROPE, EPI_SWIGLU, MASK_CAUSAL, MASK_FULL,
                        MASK_MOT)

# COSMOS_BOUNDS_CHECK=1 selects the debug build of the library (device-side checks of every index that a
# kernel reads from a tensor; a bad one is reported through the status word and its access skipped).
_BOUNDS_CHECK = os.environ.get("COSMOS_BOUNDS_CHECK") == "1"
_SO = Path(__file__).resolve().parents[1] / ("_C_check.so" if _BOUNDS_CHECK else "_C.so")
_loaded = False
_load_error: Optional[str] = None


def load_extension(build_if_missing: bool = True) -> bool:
    """Loads (building in-tree first if needed) the kernel library. Returns True on success."""
    global _loaded, _load_error
    if _loaded:
        return True
    try:
        if not _SO.exists() and build_if_missing and os.environ.get("COSMOS_B200_NO_BUILD") != "1":
            from ._build import build
            build(bounds_check=_BOUNDS_CHECK)
        torch.ops.load_library(str(_SO))
        _loaded = True
    except Exception as e:  # noqa: BLE001 - reported to the caller on first GPU use
        _load_error = f"{type(e).__name__}: {e}"
    return _loaded


def extension_loaded() -> bool:
    return _loaded


# "own" = the hand-written sm_100a kernels for CUDA bf16 tensors (the product); "library" = the same ops on
# PyTorch's library kernels (ops/library.py), the comparison arm of the benchmarks.
_backend = os.environ.get("COSMOS_OPS_BACKEND", "own")


def set_backend(name: str) -> None:
    global _backend
    if name not in ("own", "library"):
        raise ValueError("backend must be 'own' or 'library'")
    _backend = name


def get_backend() -> str:
    return _backend


def _library(t: torch.Tensor) -> bool:
    return _backend == "library" and t.is_cuda


def _grad_needed(*tensors) -> bool:
    return torch.is_grad_enabled() and any(isinstance(t, torch.Tensor) and t.requires_grad for t in tensors)


def _use_cuda(t: torch.Tensor, *others) -> bool:
    """True when the call should run the forward sm_100a kernel directly: CUDA bf16 input and no autograd
    graph to build. Calls that need gradients go through `_train_cuda` (autograd functions over the forward
    and backward kernels). A CUDA bf16 call without the kernel library raises: there is no silent fallback."""
    if not (t.is_cuda and t.dtype == torch.bfloat16) or _backend == "library":
        return False
    if _grad_needed(t, *others):
        return False
    if not load_extension():
        raise RuntimeError(
            "cosmos_b200 kernel library is not available on this GPU host "
            f"({_load_error}); run `python -m cosmos_b200.ops._build`")
    return True


def _train_cuda(t: torch.Tensor, *others) -> bool:
    """True when a call that needs gradients should run the autograd functions built on the sm_100a
    kernels (ops/autograd.py): CUDA bf16 input, gradients required, kernel library present.
    COSMOS_TRAIN_LIBRARY_BACKWARD=1 selects the PyTorch / library baseline instead."""
    import os
    if not (t.is_cuda and t.dtype == torch.bfloat16 and _grad_needed(t, *others)) or _backend == "library":
        return False
    if os.environ.get("COSMOS_TRAIN_LIBRARY_BACKWARD") == "1":
        return False
    if not load_extension():
        raise RuntimeError(
            "cosmos_b200 kernel library is not available on this GPU host "
            f"({_load_error}); run `python -m cosmos_b200.ops._build`")
    return True


class _Counted:
    """Proxy over torch.ops.cosmos_b200 that counts kernel launches (one per op call)."""

    def __init__(self):
        self.launches = 0

    def __getattr__(self, name):
        fn = getattr(torch.ops.cosmos_b200, name)

        def call(*a, **kw):
            self.launches += 1
            return fn(*a, **kw)

        return call


_counted = _Counted()


def _k():
    return _counted


def launch_count() -> int:
    """Number of sm_100a kernel launches issued through this module so far."""
    return _counted.launches


STATUS_MESSAGES = {
    0: "ok",
    1: "timeout: TMA producer waiting for a free stage",
    2: "timeout: MMA issuer waiting for data",
    3: "timeout: epilogue waiting for accumulators",
    4: "timeout: softmax waiting for scores",
    5: "timeout: waiting for a peer signal",
    6: "bad argument",
    7: "index out of range (bounds-checked build)",
}
STATUS_SITES = {1: "kv_cache_write slot", 2: "decode_qkv_post slot", 3: "paged_decode page id",
                4: "paged_decode (tensor-core) page id", 15: "self-test"}


def check_status(reset: bool = True) -> None:
    """Synchronises and raises if any kernel recorded a failure (bounded wait expired)."""
    if not _loaded or not torch.cuda.is_available():
        return
    w = torch.ops.cosmos_b200.status_word()
    code = int(w.item())
    if code != 0:
        if reset:
            w.zero_()
        what = STATUS_MESSAGES.get(code & 0xFF, "?")
        if 1 <= (code & 0xFF) <= 4 and code >> 8:
            d = code >> 8   # the wait that gave up (csrc/common.cuh, mbar_wait)
            what += (f" (barrier slot {d & 0x7F}, parity {(d >> 7) & 1}, grid size {(d >> 8) & 0xFF} mod 256, "
                     f"{2 * ((d >> 16) & 0x7F)} KB of dynamic shared memory)")
        elif code >> 8:
            what += f" at {STATUS_SITES.get(code >> 8, f'site {code >> 8}')}"
        raise RuntimeError(f"cosmos_b200 kernel reported status {code}: {what}")


def bounds_check_enabled() -> bool:
    """True when the loaded library is the bounds-checked debug build."""
    return bool(load_extension(build_if_missing=False) and _k().bounds_check_enabled())


# --------------------------------------------------------------------------- ops
def gemm(a, w, bias=None, epi: int = EPI_PLAIN, resid=None, gate=None, rows_per_batch: int = 0, out=None):
    """a [.., K] @ w[N, K]^T with a fused epilogue (see csrc/gemm_tcgen05.cu)."""
    if _use_cuda(a, w, bias, resid, gate):
        return _k().gemm(a, w, bias, epi, resid, gate, rows_per_batch, out)
    if _library(a):
        from . import library as lib
        r = lib.gemm(a, w, bias, epi, resid, gate, rows_per_batch)
        if out is not None:
            out.copy_(r.reshape(out.shape))
            return out
        return r
    if a.is_cuda and a.dtype != torch.float32:
        from . import diff
        r = diff.gemm(a, w, bias, epi, resid, gate, rows_per_batch)
    else:
        r = ref.gemm(a, w, bias, epi, resid, gate, rows_per_batch)
    if out is not None:
        out.copy_(r.reshape(out.shape))
        return out
    return r


def gemm_grouped2(a0, w0, a1, w1, epi: int = EPI_PLAIN, resid0=None, resid1=None, gate0=None, gate1=None,
                  rows_per_batch0: int = 0, rows_per_batch1: int = 0):
    """Two GEMMs with their own weights in ONE persistent launch (MoT per-modality routing: AR
    tokens x AR weights, DM tokens x DM weights). Returns (c0, c1)."""
    if (_use_cuda(a0, w0, a1, w1, resid0, resid1, gate0, gate1) and a1.is_cuda and a1.dtype == torch.bfloat16):
        return _k().gemm_grouped2(a0, w0, a1, w1, epi, resid0, resid1, gate0, gate1, rows_per_batch0, rows_per_batch1)
    return (gemm(a0, w0, None, epi, resid0, gate0, rows_per_batch0),
            gemm(a1, w1, None, epi, resid1, gate1, rows_per_batch1))


def linear(x, w, bias=None):
    return gemm(x, w, bias)


def gemm_qkv_rope(a, w, bias, cos, sin, gamma_q, gamma_k, n_q_heads: int, n_k_heads: int,
                  eps: float = 1e-6, route_ptr=None, route_ld=None, out=None):
    if _use_cuda(a, w, bias, gamma_q, gamma_k):
        return _k().gemm_qkv_rope(a, w, bias, cos, sin, gamma_q, gamma_k, n_q_heads, n_k_heads, eps,
                                  route_ptr, route_ld, out)
    assert route_ptr is None, "routed epilogue is CUDA-only"
    if _library(a):
        from . import library as lib
        r = lib.gemm_qkv_rope(a, w, bias, cos, sin, gamma_q, gamma_k, n_q_heads, n_k_heads, eps)
    else:
        r = ref.gemm_qkv_rope(a, w, bias, cos, sin, gamma_q, gamma_k, n_q_heads, n_k_heads, eps)
    if out is not None:
        out.copy_(r.reshape(out.shape))
        return out
    return r


def attention(q, k, v, scale: Optional[float] = None, mask: int = MASK_FULL, n_ar: int = 0,
              return_lse: bool = False, dest_ptr=None, rows_per_dest: int = 0, out=None
              ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Flash attention, q [B, Sq, Hq, D], k/v [B, Skv, Hkv, D] -> (o [B, Sq, Hq, D], lse|None)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if _use_cuda(q, k, v) and q.shape[-1] == 128:
        o, lse = _k().attn_fwd(q, k, v, scale, mask, n_ar, return_lse, dest_ptr, rows_per_dest, out)
        return o, (lse if return_lse else None)
    assert dest_ptr is None, "routed epilogue is CUDA-only"
    if _library(q) and not _grad_needed(q, k, v):
        from . import library as lib
        o, lse = lib.attention(q, k, v, scale, mask, n_ar, return_lse)
        if out is not None:
            out.copy_(o)
            o = out
        return o, lse
    if q.is_cuda and q.dtype != torch.float32 and _grad_needed(q, k, v):
        from . import diff
        o, lse = diff.attention(q, k, v, scale, mask, n_ar, return_lse)
    else:
        o, lse = ref.attention(q, k, v, scale, mask, n_ar, return_lse)
    if out is not None:
        out.copy_(o)
        o = out
    return o, lse


def rmsnorm(x, gamma=None, eps: float = 1e-6, residual=None):
    """Returns (y, x + residual | None)."""
    if _use_cuda(x, gamma, residual):
        y, r = _k().rmsnorm(x.contiguous(), gamma, eps, None if residual is None else residual.contiguous())
        return y, (r if residual is not None else None)
    if residual is None and _train_cuda(x, gamma) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        from . import autograd as own
        return own.rmsnorm(x, gamma, eps), None
    if _library(x):
        from . import library as lib
        return lib.rmsnorm(x, gamma, eps, residual)
    return ref.rmsnorm(x, gamma, eps, residual)


def adaln_rmsnorm(x, gamma, shift, scale, rows_per_batch: int, eps: float = 1e-6):
    if _use_cuda(x, gamma, shift, scale):
        return _k().adaln_rmsnorm(x.contiguous(), gamma, shift, scale, rows_per_batch, eps)
    d = x.shape[-1]
    if (_train_cuda(x, gamma, shift, scale) and d % 8 == 0 and d <= 8192 and shift.dtype == torch.bfloat16
            and (x.numel() // d) % rows_per_batch == 0 and shift.numel() // d in (1, (x.numel() // d) // rows_per_batch)):
        from . import autograd as own
        return own.adaln_rmsnorm(x, gamma, shift, scale, rows_per_batch, eps)
    if _library(x):
        from . import library as lib
        return lib.adaln_rmsnorm(x, gamma, shift, scale, rows_per_batch, eps)
    return ref.adaln_rmsnorm(x, gamma, shift, scale, rows_per_batch, eps)


def mrope(x, cos=None, sin=None, gamma=None, eps: float = 1e-6):
    """Per-head RMSNorm + rotary embedding on x [.., rows, H, 128]; returns a new tensor on CPU,
    works in place on CUDA (and returns x)."""
    if _use_cuda(x, gamma) and x.shape[-1] == 128:
        _k().mrope_(x, cos, sin, gamma, eps)
        return x
    if _library(x):
        from . import library as lib
        return lib.mrope(x, cos, sin, gamma, eps)
    return ref.mrope(x, cos, sin, gamma, eps)


def gated_residual(x, f, gate=None, rows_per_batch: int = 1):
    if _use_cuda(x, f, gate):
        return _k().gated_residual(x.contiguous(), f.contiguous(), gate, rows_per_batch)
    if _train_cuda(x, f, gate) and _gate_ok(x, gate, rows_per_batch):
        from . import autograd as own
        return own.gated_residual(x, f, gate, rows_per_batch)
    if _library(x):
        from . import library as lib
        return lib.gated_residual(x, f, gate, rows_per_batch)
    return ref.gated_residual(x, f, gate, rows_per_batch)


def _gate_ok(x, gate, rows_per_batch: int) -> bool:
    d = x.shape[-1]
    if d % 8 != 0 or x.dtype != torch.bfloat16:
        return False
    if gate is None:
        return True
    rows = x.numel() // d
    return (gate.dtype == torch.bfloat16 and rows_per_batch > 0 and rows % rows_per_batch == 0
            and gate.numel() // d in (1, rows // rows_per_batch))


def swiglu(gate_up):
    if _use_cuda(gate_up, gate_up):
        return _k().swiglu(gate_up.contiguous())
    if _train_cuda(gate_up) and gate_up.shape[-1] % 16 == 0:
        from . import autograd as own
        return own.swiglu(gate_up)
    if _library(gate_up):
        from . import library as lib
        return lib.swiglu(gate_up)
    return ref.swiglu(gate_up)


def cfg_euler_step(x, vc, vu, guidance: float, dt: float, normalize: bool = False):
    """x fp32 latent [rows, d]; CUDA path updates x in place and returns it."""
    if (_backend != "library" and x.is_cuda and vc.dtype == torch.bfloat16 and load_extension() and x.shape[-1] % 8 == 0
            and x.shape[-1] <= 1024):
        _k().cfg_euler_step_(x, vc.contiguous(), None if vu is None else vu.contiguous(), guidance, dt, normalize)
        return x
    return ref.cfg_euler_step(x, vc, vu, guidance, dt, normalize)


def cfg_unipc_step(x, vc, vu, guidance: float, smp, normalize: bool = False):
    """CFG combine + one UniPC step of `smp` (models/sampler.py::UniPCSampler) on the fp32 latent x [rows, d]. On CUDA
    one kernel reads x, both velocities and the sampler's stored tensors and writes the new latent and the sampler
    state (x is updated in place and returned); elsewhere the sampler's own `step` runs on the combined velocity."""
    if (_backend != "library" and x.is_cuda and vc.dtype == torch.bfloat16 and load_extension()
            and x.shape[-1] % 8 == 0 and x.shape[-1] <= 1024 and x.dtype == torch.float32):
        pl = smp.plan()
        st = smp.device_state(x)
        coef = [pl["s_cur"], pl["cL"], pl["cP"], pl["cP2"], pl["cX0"], pl["dX"], pl["dX0"], pl["dP"]]
        _k().cfg_unipc_step_(x, vc.contiguous(), None if vu is None else vu.contiguous(), st["L"], st["P"], st["P2"],
                             guidance, normalize, coef, pl["correct"], pl["final"], st["n"] >= 1, st["n"] >= 2)
        st["P"], st["P2"] = st["P2"], st["P"]      # the kernel wrote the new prediction into P2's buffer
        st["n"] += 1
        smp.advance()
        return x
    v = ref.cfg_combine(vc.reshape(x.shape), None if vu is None else vu.reshape(x.shape), guidance, normalize)
    return smp.step(x, v.to(x.dtype))


def l2_flush(buf: torch.Tensor) -> None:
    """Overwrites `buf` (larger than L2) so that the next kernel starts with a cold cache."""
    if buf.is_cuda and load_extension():
        _k().l2_flush_(buf)
    else:
        buf.zero_()


# --------------------------------------------------------------------------- paged KV decode
def paged_decode_ref(q, k_cache, v_cache, block_table, seq_lens, scale: Optional[float] = None):
    """fp32 definition: gather each sequence's pages, then softmax(q k^T) v per head (GQA)."""
    b, hq, d = q.shape
    hkv, page = k_cache.shape[1], k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    out = torch.zeros(b, hq, d, dtype=torch.float32, device=q.device)
    for i in range(b):
        n = int(seq_lens[i])
        if n == 0:
            continue
        pages = block_table[i, :(n + page - 1) // page].long()
        k = k_cache[pages].transpose(1, 2).reshape(-1, hkv, d)[:n].float()   # [tokens, Hkv, d]
        v = v_cache[pages].transpose(1, 2).reshape(-1, hkv, d)[:n].float()
        k = k.repeat_interleave(hq // hkv, dim=1)
        v = v.repeat_interleave(hq // hkv, dim=1)
        s = torch.einsum("hd,nhd->hn", q[i].float(), k) * scale
        out[i] = torch.einsum("hn,nhd->hd", torch.softmax(s, dim=-1), v)
    return out.to(q.dtype)


def gemm_reduce_rmsnorm(a, w, residual, gamma, eps: float = 1e-6):
    """x_new = residual + a @ w^T and h = rmsnorm(x_new) * gamma -> (h, x_new). On CUDA with a skinny problem
    (decode: a few rows) the split-K reduction pass does the add and the norm as well, so an output projection
    costs two launches instead of four."""
    if _use_cuda(a, w, residual, gamma):
        return _k().gemm_reduce_rmsnorm(a, w, residual.contiguous(), gamma, eps)
    y = gemm(a, w)
    h, x_new = rmsnorm(y, gamma, eps, residual=residual)
    return h, x_new


def decode_qkv_post(qkv, n_q_heads: int, cos, sin, q_gamma, k_gamma, eps: float, slots, k_cache, v_cache):
    """Decode-step glue after the QKV projection. qkv [B, Hq + 2 Hkv, 128]; q and k heads get their
    RMS-norm and the rotary rotation (cos/sin [B, 64]); k and v of sequence b are written into the
    paged caches [pages, Hkv, page_size, 128] at slot slots[b]; returns q [B, Hq, 128].
    One kernel on CUDA; on CPU the same steps with the reference ops."""
    hkv = (qkv.shape[1] - n_q_heads) // 2
    if _use_cuda(qkv, q_gamma) and qkv.shape[-1] == 128:
        return _k().decode_qkv_post(qkv.contiguous(), n_q_heads, cos.contiguous(), sin.contiguous(), q_gamma, k_gamma,
                                    eps, slots.contiguous(), k_cache, v_cache)
    q = ref.mrope(qkv[:, :n_q_heads], cos, sin, q_gamma, eps)
    k = ref.mrope(qkv[:, n_q_heads:n_q_heads + hkv], cos, sin, k_gamma, eps)
    v = qkv[:, n_q_heads + hkv:]
    page_size = k_cache.shape[2]
    page, off = slots // page_size, slots % page_size
    k_cache[page, :, off] = k.to(k_cache.dtype)
    v_cache[page, :, off] = v.to(v_cache.dtype)
    return q


def gemm_decode_qkv_post(h, w, n_q_heads: int, cos, sin, q_gamma, k_gamma, eps: float, slots, k_cache, v_cache):
    """QKV projection of a decode step followed by `decode_qkv_post`. h [B, d]; w [(Hq + 2 Hkv) * 128, d]. On CUDA the
    skinny GEMM leaves its split-K partial sums and the post-processing kernel reduces them as it reads: one launch
    and one bf16 round trip fewer per layer."""
    if _use_cuda(h, w) and k_cache.shape[-1] == 128 and w.shape[0] % 128 == 0:
        return _k().gemm_decode_qkv_post(h, w, n_q_heads, cos.contiguous(), sin.contiguous(), q_gamma, k_gamma, eps,
                                         slots.contiguous(), k_cache, v_cache)
    qkv = gemm(h, w).view(h.shape[0], -1, k_cache.shape[-1])
    return decode_qkv_post(qkv, n_q_heads, cos, sin, q_gamma, k_gamma, eps, slots, k_cache, v_cache)


SAMPLE_K = 64  # candidates kept per sequence and vocabulary shard by the sampling ops


def sample_topk(logits, seen_any, seen_out, tokens, presence, repetition, vocab_offset: int = 0):
    """First half of the decode-step sampler. `logits` [B, V]: this rank's vocabulary shard. Marks tokens[b] (the
    token consumed by this step) in the [B, V] flag tensors `seen_any` / `seen_out` when it lies in the shard, applies
    the repetition penalty (CTRL style, on tokens seen in prompt or output) and the presence penalty (on generated
    tokens), and returns cand [B, 64, 2] float: the 64 largest penalised logits, best first, each with its global
    token id stored as int32 bits. Flags may be None (no penalties). One kernel on CUDA (bf16 logits): radix select
    over the row, no [B, V] intermediate."""
    b, v = logits.shape
    if _use_cuda(logits) and logits.dtype == torch.bfloat16:
        return _k().sample_topk(logits, seen_any, seen_out, tokens, presence, repetition, int(vocab_offset))
    l = logits.float()
    if seen_any is not None:
        loc = tokens - vocab_offset
        mine = ((loc >= 0) & (loc < v))[:, None]
        idx = loc.clamp(0, v - 1)[:, None]
        # tokens of other shards write back what was there
        seen_out.scatter_(1, idx, seen_out.gather(1, idx) | mine)
        seen_any.scatter_(1, idx, seen_any.gather(1, idx) | mine)
        rep = repetition[:, None]
        l = torch.where(seen_any.bool(), torch.where(l > 0, l / rep, l * rep), l)
        l = l - presence[:, None] * seen_out.float()
    k = min(SAMPLE_K, v)
    vals, idx = torch.topk(l, k, dim=-1)
    if k < SAMPLE_K:
        vals = torch.cat([vals, vals.new_full((b, SAMPLE_K - k), float("-inf"))], dim=1)
        idx = torch.cat([idx, idx.new_zeros((b, SAMPLE_K - k))], dim=1)
    ids = (idx + vocab_offset).to(torch.int32).view(torch.float32)
    return torch.stack([vals, ids], dim=-1).contiguous()


def sample_pick(cand, n_src: int, temperature, top_k, top_p, noise, vocab_size: int, out):
    """Second half: cand [n_src * B, 64, 2] (the candidates of every vocabulary shard, shard-major) -> out [B]
    (int64 token ids). Merges the shards' candidates, keeps the top_k[b] best, softmax at temperature[b], nucleus
    cut at top_p[b] (the most likely token always stays) and the Gumbel-max draw with noise[b, :64] (uniform in
    (0, 1)); temperature 0 takes the best candidate. Ids are clamped to vocab_size - 1 (padded LM-head rows)."""
    if cand.is_cuda and _backend != "library" and load_extension():
        _k().sample_pick_(cand.contiguous(), int(n_src), temperature, top_k, top_p, noise, int(vocab_size), out)
        return out
    b = cand.shape[0] // n_src
    c = cand.view(n_src, b, SAMPLE_K, 2).permute(1, 0, 2, 3).reshape(b, n_src * SAMPLE_K, 2)
    vals, ids = c[..., 0], c[..., 1].contiguous().view(torch.int32).long()
    if n_src > 1:
        # best value first; equal values: the smaller token id first
        o = torch.argsort(ids, dim=1, stable=True)
        vals, ids = vals.gather(1, o), ids.gather(1, o)
        o = torch.argsort(vals, dim=1, descending=True, stable=True)[:, :SAMPLE_K]
        vals, ids = vals.gather(1, o), ids.gather(1, o)
    k = SAMPLE_K
    t = temperature[:, None]
    z = vals / torch.where(t > 0, t, torch.ones_like(t))
    rank = torch.arange(k, device=cand.device)[None]
    z = torch.where(rank < top_k[:, None].clamp(1, k), z, torch.full_like(z, float("-inf")))
    p = torch.softmax(z, dim=-1)
    keep = (torch.cumsum(p, dim=-1) - p) < top_p[:, None]
    z = torch.where(keep, z, torch.full_like(z, float("-inf")))
    g = -torch.log(-torch.log(noise[:, :k]))
    pick = torch.argmax(z + g, dim=-1)
    sampled = ids.gather(1, pick[:, None])[:, 0]
    out.copy_(torch.where(temperature > 0, sampled, ids[:, 0]).clamp(0, vocab_size - 1))
    return out


def paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale: Optional[float] = None,
                 n_splits: Optional[int] = None, scratch=None, max_len: Optional[int] = None, impl: int = 0):
    """q [B, Hq, 128] against a paged cache [pages, Hkv, page_size, 128] -> [B, Hq, 128].
    `max_len` (an upper bound of seq_lens known on the host) picks the kv split count without
    a device synchronisation. impl 0 = tensor-core kernel (TMA page copies + tcgen05) when the page
    size is 8..128 and the GQA group is 1, 2, 4 or 8, else the CUDA-core kernel; impl 1 forces the latter."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if _use_cuda(q) and q.shape[-1] == 128:
        page = k_cache.shape[2]
        group = q.shape[1] // k_cache.shape[1]
        if not (page in (8, 16, 32, 64, 128) and group in (1, 2, 4, 8)):
            impl = 1
        if n_splits is None:
            ml = max_len if max_len is not None else block_table.shape[1] * page
            n_splits = int(torch.ops.cosmos_b200.paged_decode_pick_splits(q.shape[0], k_cache.shape[1], ml, impl))
        return _k().paged_decode(q.contiguous(), k_cache, v_cache, block_table, seq_lens, scale, n_splits, scratch,
                                 impl)
    return paged_decode_ref(q, k_cache, v_cache, block_table, seq_lens, scale)
