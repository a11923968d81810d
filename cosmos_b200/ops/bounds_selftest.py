"""Self-test of the bounds-checked debug build of the kernel library.

    COSMOS_BOUNDS_CHECK=1 python -m cosmos_b200.ops.bounds_selftest

The debug build (`python -m cosmos_b200.ops._build --bounds-check`, cosmos_b200/_C_check.so) compares every
index that a kernel reads from a tensor - cache slots of `kv_cache_write` / `decode_qkv_post`, page ids
of both paged-decode kernels - with its limit before the index becomes an address; a bad one is reported
through the status word (code 7, site in bits 8..15) and its access is skipped. It stands in for a memory
checker on hosts where none can be run.

The self-test (1) runs the device-side check itself on good and bad (index, limit) pairs through a
kernel that addresses nothing with them and reads back the verdicts and the status word, and (2) runs
the checked kernels on valid inputs against their fp32 definitions with a clean status word. It never
hands a bad index to a kernel that would use it. Prints one JSON line; exit code 0 on success."""
from __future__ import annotations

import json
import sys

import torch


def run() -> dict:
    from cosmos_b200 import ops
    from cosmos_b200.ops import reference as ref

    assert torch.cuda.is_available(), "needs a GPU"
    assert ops.load_extension(build_if_missing=False), "kernel library not built"
    dev = torch.device("cuda", 0)
    k = torch.ops.cosmos_b200
    enabled = bool(k.bounds_check_enabled())
    out = {"bounds_check_build": enabled}
    ops.check_status()

    # (1) the check itself
    idx = torch.tensor([0, 5, 9, -1, 10, 2 ** 40, 3], dtype=torch.long, device=dev)
    lim = torch.tensor([1, 10, 10, 10, 10, 2 ** 20, 0], dtype=torch.long, device=dev)   # limit 0 = "not given"
    ok = k.bounds_check_selftest(idx, lim).cpu().tolist()
    want = [1, 1, 1, 0, 0, 0, 1] if enabled else [1] * 7
    assert ok == want, (ok, want)
    word = int(k.status_word().item())
    assert word == ((7 | (15 << 8)) if enabled else 0), word
    if enabled:
        try:
            ops.check_status()
            raise AssertionError("check_status did not raise")
        except RuntimeError as e:
            assert "index out of range" in str(e) and "self-test" in str(e), str(e)
    out["selftest_verdicts"], out["selftest_status_word"] = ok, word

    # (2) checked kernels on valid inputs
    torch.manual_seed(0)
    b, hq, hkv, page = 6, 8, 2, 16
    lens = [1, 17, 200, 64, 333, 16]
    max_pages = (max(lens) + page - 1) // page + 1
    n_pages = b * max_pages + 3
    rnd = lambda *s: torch.randn(*s, device=dev).bfloat16()  # noqa: E731
    kc, vc = rnd(n_pages, hkv, page, 128), rnd(n_pages, hkv, page, 128)
    table = torch.randperm(n_pages, device=dev)[:b * max_pages].view(b, max_pages).int()
    sl = torch.tensor(lens, device=dev, dtype=torch.int32)
    # append one token per sequence through the fused decode glue, then through the plain cache write
    qkv = rnd(b, hq + 2 * hkv, 128)
    ang = torch.rand(b, 64, device=dev) * 6.0
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    gq = (1 + 0.1 * torch.randn(128, device=dev)).bfloat16()
    gk = (1 + 0.1 * torch.randn(128, device=dev)).bfloat16()
    pos = sl.long()
    slots = table.long()[torch.arange(b, device=dev), pos // page] * page + pos % page
    q = ops.decode_qkv_post(qkv, hq, cos, sin, gq, gk, 1e-6, slots, kc, vc)
    k_want = ref.mrope(qkv.float()[:, hq:hq + hkv], cos, sin, gk.float(), 1e-6)
    pg, off = slots // page, slots % page
    err_k = (kc[pg, :, off].float() - k_want).abs().max().item()
    assert err_k < 5e-2, err_k
    assert torch.equal(vc[pg, :, off], qkv[:, hq + hkv:])
    k2, v2 = rnd(b, hkv, 128), rnd(b, hkv, 128)
    k.kv_cache_write(k2, v2, slots, kc, vc)
    assert torch.equal(kc[pg, :, off], k2) and torch.equal(vc[pg, :, off], v2)
    sl1 = sl + 1
    want_o = ops.paged_decode_ref(q.float(), kc.float(), vc.float(), table, sl1)
    errs = {}
    for impl in (0, 1):
        got = ops.paged_decode(q, kc, vc, table, sl1, n_splits=2, max_len=max(lens) + 1, impl=impl)
        errs[f"paged_decode_impl{impl}_max_err"] = (got.float() - want_o).abs().max().item()
        assert errs[f"paged_decode_impl{impl}_max_err"] < 5e-2, errs
    torch.cuda.synchronize()
    ops.check_status()   # valid inputs leave the status word clean
    out.update(errs)
    out["k_rows_max_err"] = err_k
    out["ok"] = True
    return out


if __name__ == "__main__":
    res = run()
    print(json.dumps(res))
    sys.exit(0 if res.get("ok") else 1)
