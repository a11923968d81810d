"""The allocation-free C entry point for paged-KV decode attention.

Some callers of the kernel library cannot allocate GPU memory when they need attention (engines
with a fixed, pre-planned memory budget, real-time policy loops, threads that must not touch the
CUDA allocator, C hosts without PyTorch). This test plays such a caller: it resolves the exported
C symbol with ctypes, hands it raw device pointers, and compares the result with the regular
(allocating) entry point, on two consecutive calls that share the library's built-in scratch.
The file name sorts last so that a `pytest -x` run has already run every other test before it.
"""
import ctypes
from pathlib import Path

import pytest
import torch

from cosmos_b200 import ops

pytestmark = pytest.mark.gpu
MAX_ROWS = 8192


def _lib():
    assert ops.load_extension()
    lib = ctypes.CDLL(str(Path(ops.__file__).resolve().parents[1] / "_C.so"))
    fn = lib.cosmos_paged_decode_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p,
                                                                ctypes.c_char_p, ctypes.c_int]
    return fn


def _case(seed, b, hq, hkv, page, lens):
    g = torch.Generator(device="cuda").manual_seed(seed)
    max_pages = (max(lens) + page - 1) // page + 1
    n_pages = b * max_pages + 2
    kc = torch.randn(n_pages, hkv, page, 128, device="cuda", generator=g).bfloat16()
    vc = torch.randn(n_pages, hkv, page, 128, device="cuda", generator=g).bfloat16()
    table = torch.randperm(n_pages, device="cuda", generator=g)[:b * max_pages].view(b, max_pages).int().contiguous()
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    q = torch.randn(b, hq, 128, device="cuda", generator=g).bfloat16()
    return q, kc, vc, table, sl


def _call(fn, q, kc, vc, table, sl, n_splits):
    out = torch.empty_like(q)
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), sl.data_ptr(), out.data_ptr(),
            q.shape[0], q.shape[1], kc.shape[1], kc.shape[2], table.shape[1], 1.0 / 128 ** 0.5, n_splits,
            ctypes.c_void_p(stream), err, 256)
    return rc, out, err.value.decode()


def test_noalloc_matches_allocating_entry_point_twice():
    fn = _lib()
    torch.cuda.synchronize()
    for seed, (b, hq, hkv, page, lens, splits) in enumerate([(3, 8, 2, 16, [900, 17, 400], 5),
                                                              (2, 4, 1, 32, [1500, 1200], 8)]):
        q, kc, vc, table, sl = _case(100 + seed, b, hq, hkv, page, lens)
        want = ops.paged_decode(q, kc, vc, table, sl, n_splits=splits, impl=1)  # the same CUDA-core kernel
        before = torch.cuda.memory_allocated()
        rc, got, msg = _call(fn, q, kc, vc, table, sl, splits)
        torch.cuda.synchronize()
        assert rc == 0, msg
        grown = torch.cuda.memory_allocated() - before
        assert grown <= (got.numel() * 2 + 511) // 512 * 512, grown  # only the output tensor this test made
        err = (got.float() - want.float()).abs()
        tol = 2e-2 + 2e-2 * want.float().abs()
        assert (err <= tol).all(), f"call {seed}: max err {err.max().item()}"
    ops.check_status()


def test_noalloc_rejects_oversize_and_bad_arguments():
    fn = _lib()
    q, kc, vc, table, sl = _case(7, 2, 8, 2, 16, [64, 64])
    big_b = MAX_ROWS // (8 * 64) + 1
    qb = q[:1].expand(big_b, -1, -1).contiguous()
    tb = table[:1].expand(big_b, -1).contiguous()
    slb = sl[:1].expand(big_b).contiguous()
    rc, _, msg = _call(fn, qb, kc, vc, tb, slb, 64)
    assert rc == 1 and "too large" in msg and str(MAX_ROWS) in msg
    rc, _, msg = _call(fn, q, kc, vc, table, sl, 0)
    assert rc == 2 and "n_splits" in msg
