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
    lib = ctypes.CDLL(str(ops._SO))   # the library file that `ops` loaded (regular or bounds-checked build)
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
        ref = ops.paged_decode_ref(q, kc, vc, table, sl)                         # and the fp32 definition
        rc, got, msg = _call(fn, q, kc, vc, table, sl, splits)                   # first call: set-up happens here
        torch.cuda.synchronize()
        assert rc == 0, msg
        # The second call must not take device memory from anybody: neither from PyTorch's caching allocator
        # (memory_allocated) nor from the driver behind its back (free device memory, which a raw cudaMalloc
        # would lower). Its output tensor is made before the measurement.
        out2 = torch.empty_like(q)
        err2 = ctypes.create_string_buffer(256)
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        alloc0 = torch.cuda.memory_allocated()
        rc2 = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), sl.data_ptr(), out2.data_ptr(),
                 q.shape[0], q.shape[1], kc.shape[1], kc.shape[2], table.shape[1], 1.0 / 128 ** 0.5, splits,
                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), err2, 256)
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        assert rc2 == 0, err2.value.decode()
        assert torch.cuda.memory_allocated() == alloc0
        assert free1 >= free0, f"free device memory fell by {free0 - free1} bytes during the call"
        assert torch.equal(out2, got)
        for name, target in (("allocating entry point", want), ("fp32 definition", ref)):
            err = (got.float() - target.float()).abs()
            tol = 2e-2 + 2e-2 * target.float().abs()
            assert (err <= tol).all(), f"call {seed} vs {name}: max err {err.max().item()}"
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
