"""Numerics of the sm_100a kernels against the plain-PyTorch fp32 definitions."""
import math

import pytest
import torch

from cosmos_b200 import ops
from cosmos_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(dtype)


def _close(got, want, atol, rtol, what=""):
    got = got.float()
    want = want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{what}: {bad}/{err.numel()} elements off, max err {err.max().item():.4g}"


@pytest.fixture(autouse=True)
def _status_clean():
    ops.load_extension()
    yield
    torch.cuda.synchronize()
    ops.check_status()


def test_extension_is_loaded():
    assert ops.load_extension(), "kernel library must load on a GPU host"
    assert hasattr(torch.ops.cosmos_b200, "gemm")


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (1000, 768, 320), (77, 136, 72),
                                    (4096, 4096, 1024), (300, 6144, 4096)])
def test_gemm_plain(m, n, k):
    torch.manual_seed(0)
    a = _rand(m, k)
    w = _rand(n, k, scale=1 / math.sqrt(k))
    got = ops.gemm(a, w)
    want = a.float() @ w.float().t()
    _close(got, want, 2e-2, 2e-2, f"gemm {m}x{n}x{k}")


def test_gemm_bias_and_strided_a():
    torch.manual_seed(1)
    m, n, k = 513, 384, 256
    big = _rand(m, k + 64)
    a = big[:, :k]
    w = _rand(n, k, scale=1 / math.sqrt(k))
    bias = _rand(n)
    got = ops.gemm(a, w, bias)
    want = a.float() @ w.float().t() + bias.float()
    _close(got, want, 2e-2, 2e-2, "gemm+bias")


@pytest.mark.parametrize("m,dff,k", [(256, 512, 128), (700, 1536, 512), (130, 200, 64)])
def test_gemm_swiglu(m, dff, k):
    torch.manual_seed(2)
    a = _rand(m, k)
    w = _rand(2 * dff, k, scale=1 / math.sqrt(k))
    got = ops.gemm(a, w, epi=ops.EPI_SWIGLU)
    want = ref.gemm(a.float(), w.float(), epi=ops.EPI_SWIGLU)
    assert got.shape == (m, dff)
    _close(got, want, 2e-2, 2e-2, "gemm swiglu")


@pytest.mark.parametrize("m,n,k,rpb", [(512, 256, 128, 256), (600, 520, 192, 300), (384, 1024, 512, 384)])
def test_gemm_gated_residual(m, n, k, rpb):
    torch.manual_seed(3)
    a = _rand(m, k)
    w = _rand(n, k, scale=1 / math.sqrt(k))
    r = _rand(m, n)
    gate = _rand(m // rpb, n)
    got = ops.gemm(a, w, None, ops.EPI_GATED_RESID, r, gate, rpb)
    want = ref.gemm(a.float(), w.float(), None, ops.EPI_GATED_RESID, r.float(), gate.float(), rpb)
    _close(got, want, 3e-2, 2e-2, "gemm gated residual")
    got2 = ops.gemm(a, w, None, ops.EPI_GATED_RESID, r, None, rpb)
    want2 = r.float() + a.float() @ w.float().t()
    _close(got2, want2, 3e-2, 2e-2, "gemm residual without gate")


@pytest.mark.parametrize("m,hq,hk", [(256, 4, 2), (333, 8, 2)])
def test_gemm_qkv_rope(m, hq, hk):
    torch.manual_seed(4)
    k = 256
    n = (hq + 2 * hk) * 128
    a = _rand(m, k)
    w = _rand(n, k, scale=1 / math.sqrt(k))
    ang = torch.rand(m, 64, device=DEV) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    gq = (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16()
    gk = (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16()
    got = ops.gemm_qkv_rope(a, w, None, cos, sin, gq, gk, hq, hk, 1e-6)
    want = ref.gemm_qkv_rope(a.float(), w.float(), None, cos, sin, gq.float(), gk.float(), hq, hk, 1e-6)
    _close(got, want, 3e-2, 2e-2, "qkv rope epilogue")


def test_gemm_qkv_rope_routed():
    """Head chunks written through the routing table land where the table says."""
    torch.manual_seed(5)
    m, k, hq, hk = 256, 128, 2, 1
    n = (hq + 2 * hk) * 128
    a = _rand(m, k)
    w = _rand(n, k, scale=1 / math.sqrt(k))
    bufs = [torch.zeros(m, 128, device=DEV, dtype=torch.bfloat16) for _ in range(n // 128)]
    ptr = torch.tensor([b.data_ptr() for b in bufs], device=DEV, dtype=torch.int64)
    ld = torch.full((n // 128,), 128, device=DEV, dtype=torch.int64)
    ops.gemm_qkv_rope(a, w, None, None, None, None, None, hq, hk, 1e-6, ptr, ld)
    want = (a.float() @ w.float().t())
    for i, b in enumerate(bufs):
        _close(b, want[:, i * 128:(i + 1) * 128], 2e-2, 2e-2, f"routed chunk {i}")


@pytest.mark.parametrize("b,sq,skv,hq,hkv,mask", [
    (1, 256, 256, 1, 1, ops.MASK_FULL),
    (1, 512, 1024, 4, 1, ops.MASK_FULL),
    (2, 300, 777, 4, 2, ops.MASK_FULL),
    (1, 1024, 1024, 2, 1, ops.MASK_CAUSAL),
    (1, 500, 500, 4, 2, ops.MASK_CAUSAL),
    (1, 200, 456, 2, 2, ops.MASK_CAUSAL),
    (1, 2048, 2304, 8, 2, ops.MASK_FULL),
])
def test_attention(b, sq, skv, hq, hkv, mask):
    torch.manual_seed(6)
    q = _rand(b, sq, hq, 128)
    k = _rand(b, skv, hkv, 128)
    v = _rand(b, skv, hkv, 128)
    got, lse = ops.attention(q, k, v, mask=mask, return_lse=True)
    want, lse_ref = ref.attention(q.float(), k.float(), v.float(), None, mask, 0, True)
    _close(got, want, 2e-2, 2e-2, "attention out")
    _close(lse, lse_ref, 2e-2, 1e-3, "attention lse")


def test_attention_mot_mask():
    torch.manual_seed(7)
    s, n_ar = 640, 200
    q = _rand(1, s, 4, 128)
    k = _rand(1, s, 2, 128)
    v = _rand(1, s, 2, 128)
    got, _ = ops.attention(q, k, v, mask=ops.MASK_MOT, n_ar=n_ar)
    want, _ = ref.attention(q.float(), k.float(), v.float(), None, ops.MASK_MOT, n_ar)
    _close(got, want, 2e-2, 2e-2, "attention MoT mask")


def test_attention_large_scores_rescale():
    """Scores whose running max grows block after block exercise the lazy O rescale."""
    torch.manual_seed(8)
    sq, skv = 256, 1024
    q = _rand(1, sq, 1, 128)
    k = _rand(1, skv, 1, 128)
    ramp = torch.linspace(0.2, 3.0, skv, device=DEV)[None, :, None, None]
    k = (k.float() * ramp).bfloat16()
    v = _rand(1, skv, 1, 128)
    got, _ = ops.attention(q, k, v, scale=1.0)
    want, _ = ref.attention(q.float(), k.float(), v.float(), 1.0)
    _close(got, want, 3e-2, 3e-2, "attention with growing max")


def test_attention_strided_qkv_views():
    """q/k/v as views into one fused [S, (Hq+2Hkv)*128] projection buffer."""
    torch.manual_seed(9)
    s, hq, hkv = 384, 4, 1
    qkv = _rand(1, s, (hq + 2 * hkv) * 128)
    q = qkv[..., :hq * 128].view(1, s, hq, 128)
    k = qkv[..., hq * 128:(hq + hkv) * 128].view(1, s, hkv, 128)
    v = qkv[..., (hq + hkv) * 128:].view(1, s, hkv, 128)
    got, _ = ops.attention(q, k, v)
    want, _ = ref.attention(q.float(), k.float(), v.float())
    _close(got, want, 2e-2, 2e-2, "attention on strided views")


def test_attention_routed_output():
    torch.manual_seed(10)
    s, h, parts = 512, 2, 4
    q, k, v = _rand(1, s, h, 128), _rand(1, s, h, 128), _rand(1, s, h, 128)
    rows = s // parts
    bufs = [torch.zeros(1, rows, h, 128, device=DEV, dtype=torch.bfloat16) for _ in range(parts)]
    ptr = torch.tensor([b.data_ptr() for b in bufs], device=DEV, dtype=torch.int64)
    ops.attention(q, k, v, dest_ptr=ptr, rows_per_dest=rows, out=bufs[0])
    want, _ = ref.attention(q.float(), k.float(), v.float())
    for i, bfr in enumerate(bufs):
        _close(bfr, want[:, i * rows:(i + 1) * rows], 2e-2, 2e-2, f"routed rows {i}")


@pytest.mark.parametrize("rows,d", [(64, 128), (1000, 512), (333, 4096), (50, 5120)])
def test_rmsnorm(rows, d):
    torch.manual_seed(11)
    x, g, r = _rand(rows, d), _rand(d), _rand(rows, d)
    y, _ = ops.rmsnorm(x, g, 1e-6)
    want, _ = ref.rmsnorm(x.float(), g.float(), 1e-6)
    _close(y, want, 2e-2, 1e-2, "rmsnorm")
    y2, res = ops.rmsnorm(x, g, 1e-6, r)
    w2, wres = ref.rmsnorm(x.float(), g.float(), 1e-6, r.float())
    _close(y2, w2, 2e-2, 1e-2, "rmsnorm+res")
    _close(res, wres, 2e-2, 1e-2, "residual out")


def test_adaln_rmsnorm():
    torch.manual_seed(12)
    b, s, d = 2, 300, 512
    x = _rand(b * s, d)
    mod = _rand(b, 6 * d, scale=0.3)
    shift, scale = mod[:, :d], mod[:, d:2 * d]
    y = ops.adaln_rmsnorm(x, None, shift, scale, s, 1e-6)
    want = ref.adaln_rmsnorm(x.float(), None, shift.float(), scale.float(), s, 1e-6)
    _close(y, want, 2e-2, 1e-2, "adaln")


def test_mrope_and_qknorm():
    torch.manual_seed(13)
    s, h = 500, 6
    x = _rand(s, h, 128)
    ang = torch.rand(s, 64, device=DEV) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    g = (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16()
    want = ref.mrope(x.float(), cos, sin, g.float(), 1e-6)
    got = ops.mrope(x.clone(), cos, sin, g, 1e-6)
    _close(got, want, 2e-2, 1e-2, "mrope")


def test_gated_residual_and_swiglu():
    torch.manual_seed(14)
    b, s, d = 2, 200, 256
    x, f, gate = _rand(b * s, d), _rand(b * s, d), _rand(b, d)
    _close(ops.gated_residual(x, f, gate, s), ref.gated_residual(x.float(), f.float(), gate.float(), s),
           2e-2, 1e-2, "gated residual")
    gu = _rand(b * s, 2 * d)
    _close(ops.swiglu(gu), ref.swiglu(gu.float()), 2e-2, 1e-2, "swiglu")


@pytest.mark.parametrize("normalize", [False, True])
def test_cfg_euler_step(normalize):
    torch.manual_seed(15)
    rows, d = 1000, 64
    x = torch.randn(rows, d, device=DEV)
    vc, vu = _rand(rows, d), _rand(rows, d)
    want = ref.cfg_euler_step(x.clone(), vc, vu, 7.0, -0.03, normalize)
    got = ops.cfg_euler_step(x.clone(), vc, vu, 7.0, -0.03, normalize)
    _close(got, want, 1e-5, 1e-5, "cfg euler step")


@pytest.mark.parametrize("b,hq,hkv,page,lens,splits", [
    (2, 4, 1, 16, [100, 37], 1),
    (3, 8, 2, 32, [700, 1, 333], 4),
    (4, 4, 4, 16, [513, 512, 511, 64], 3),
    (2, 8, 1, 16, [2000, 1500], None),
    (3, 4, 2, 8, [1000, 129, 128], 2),
    (2, 32, 8, 128, [3000, 4097], None),
])
@pytest.mark.parametrize("impl", [0, 1])
def test_paged_decode(b, hq, hkv, page, lens, splits, impl):
    """impl 0: TMA + tcgen05 kernel, impl 1: CUDA-core kernel; both against the fp32 definition."""
    torch.manual_seed(16)
    max_pages = (max(lens) + page - 1) // page + 1
    n_pages = b * max_pages + 3
    kc = _rand(n_pages, hkv, page, 128)
    vc = _rand(n_pages, hkv, page, 128)
    perm = torch.randperm(n_pages, device=DEV)[:b * max_pages].view(b, max_pages).int()
    sl = torch.tensor(lens, device=DEV, dtype=torch.int32)
    q = _rand(b, hq, 128)
    got = ops.paged_decode(q, kc, vc, perm, sl, n_splits=splits, max_len=max(lens), impl=impl)
    torch.cuda.synchronize()
    ops.check_status()
    want = ops.paged_decode_ref(q.float(), kc.float(), vc.float(), perm, sl)
    _close(got, want, 2e-2, 2e-2, "paged decode")


@pytest.mark.parametrize("b,hq,hkv,page", [(5, 4, 1, 16), (32, 32, 8, 16), (3, 8, 2, 4)])
def test_decode_qkv_post(b, hq, hkv, page):
    """The fused decode glue (q/k norm + rotary + cache write) against the fp32 definition of each step."""
    torch.manual_seed(18)
    n_pages = 2 * b + 1
    qkv = _rand(b, hq + 2 * hkv, 128)
    ang = torch.rand(b, 64, device=DEV) * 6.0
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    gq, gk = (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16(), (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16()
    slots = (torch.randperm(n_pages * page, device=DEV)[:b]).long()
    kc, vc = _rand(n_pages, hkv, page, 128), _rand(n_pages, hkv, page, 128)
    kc0, vc0 = kc.clone(), vc.clone()
    q = ops.decode_qkv_post(qkv, hq, cos, sin, gq, gk, 1e-6, slots, kc, vc)
    torch.cuda.synchronize()
    ops.check_status()
    f = qkv.float()
    q_want = ref.mrope(f[:, :hq], cos, sin, gq.float(), 1e-6)
    k_want = ref.mrope(f[:, hq:hq + hkv], cos, sin, gk.float(), 1e-6)
    _close(q, q_want, 2e-2, 2e-2, "q")
    pg, off = slots // page, slots % page
    _close(kc[pg, :, off], k_want, 2e-2, 2e-2, "k rows")
    assert torch.equal(vc[pg, :, off], qkv[:, hq + hkv:])
    # every other cache row is untouched
    mask = torch.ones(n_pages, page, dtype=torch.bool, device=DEV)
    mask[pg, off] = False
    assert torch.equal(kc.transpose(1, 2)[mask], kc0.transpose(1, 2)[mask])
    assert torch.equal(vc.transpose(1, 2)[mask], vc0.transpose(1, 2)[mask])


@pytest.mark.parametrize("epi", [ops.EPI_PLAIN, ops.EPI_SWIGLU, ops.EPI_GATED_RESID])
def test_gemm_grouped_two_segments(epi):
    """MoT routing: an AR segment and a DM segment with their own weights in one launch."""
    torch.manual_seed(17)
    k, n = 256, 512
    m0, m1 = 200, 1100
    a0, a1 = _rand(m0, k), _rand(2, m1 // 2, k)
    w0, w1 = _rand(n, k, scale=1 / 16), _rand(n, k, scale=1 / 16)
    n_out = n // 2 if epi == ops.EPI_SWIGLU else n
    r0 = r1 = g1 = None
    if epi == ops.EPI_GATED_RESID:
        r0, r1, g1 = _rand(m0, n_out), _rand(2, m1 // 2, n_out), _rand(2, n_out)
    c0, c1 = ops.gemm_grouped2(a0, w0, a1, w1, epi, r0, r1, None, g1, m0, m1 // 2)
    f = lambda t: None if t is None else t.float()  # noqa: E731
    want0 = ref.gemm(a0.float(), w0.float(), None, epi, f(r0), None, m0)
    want1 = ref.gemm(a1.float(), w1.float(), None, epi, f(r1), f(g1), m1 // 2)
    assert c0.shape == want0.shape and c1.shape == want1.shape
    _close(c0, want0, 3e-2, 2e-2, "grouped segment 0")
    _close(c1, want1, 3e-2, 2e-2, "grouped segment 1")


@pytest.mark.parametrize("m,n,k,epi", [(32, 768, 4096, ops.EPI_PLAIN), (32, 3072, 4096, ops.EPI_SWIGLU),
                                        (32, 4096, 1536, ops.EPI_GATED_RESID), (7, 512, 1024, ops.EPI_PLAIN),
                                        (64, 1000, 2048, ops.EPI_PLAIN),
                                        # more than one 128-row tile: split-K on CTA pairs
                                        (256, 6144, 4096, ops.EPI_PLAIN), (200, 4096, 12288, ops.EPI_GATED_RESID),
                                        (384, 1024, 4096, ops.EPI_PLAIN), (256, 24576, 4096, ops.EPI_SWIGLU)])
def test_gemm_skinny_split_k(m, n, k, epi):
    """Decode-sized problems take the split-K path (fp32 partials + reduce/epilogue kernel)."""
    torch.manual_seed(18)
    a = _rand(m, k)
    w = _rand(n, k, scale=1 / math.sqrt(k))
    r = _rand(m, n) if epi == ops.EPI_GATED_RESID else None
    got = ops.gemm(a, w, None, epi, r, None, m)
    want = ref.gemm(a.float(), w.float(), None, epi, None if r is None else r.float(), None, m)
    _close(got, want, 3e-2, 2e-2, f"skinny gemm {m}x{n}x{k} epi {epi}")


@pytest.mark.parametrize("cin,cout", [(64, 128), (64, 64), (128, 32), (64, 256), (128, 384)])
def test_conv3d_implicit_gemm_matches_conv3d(cin, cout):
    """One causal 3x3x3 convolution on a padded channels-last volume vs F.conv3d (64 / 128 output channels and fewer
    run narrower MMAs; 384 takes two n tiles)."""
    import torch.nn.functional as F
    torch.manual_seed(19)
    t, h, w = 5, 12, 20
    x = _rand(1, cin, t, h, w)
    wt = _rand(cout, cin, 3, 3, 3, scale=1 / math.sqrt(27 * cin))
    b = _rand(cout)
    r = _rand(1, cout, t, h, w)
    want = F.conv3d(F.pad(x.float(), (1, 1, 1, 1, 2, 0)), wt.float(), b.float()) + r.float()
    vol = torch.zeros(t + 2, h + 2, w + 2, cin, device=DEV, dtype=torch.bfloat16)
    vol[2:, 1:-1, 1:-1] = x[0].permute(1, 2, 3, 0)
    rv = torch.zeros(t + 2, h + 2, w + 2, cout, device=DEV, dtype=torch.bfloat16)
    rv[2:, 1:-1, 1:-1] = r[0].permute(1, 2, 3, 0)
    wp = wt.permute(0, 2, 3, 4, 1).reshape(cout, 27 * cin).contiguous()
    out = torch.zeros(t + 2, h + 2, w + 2, cout, device=DEV, dtype=torch.bfloat16)
    torch.ops.cosmos_b200.conv3d_cl(vol, wp, b, rv, out, 2)
    got = out[2:, 1:-1, 1:-1].permute(3, 0, 1, 2)[None]
    _close(got, want, 3e-2, 2e-2, "implicit-GEMM conv3d")
    assert out[:2].abs().max() == 0 and out[:, 0].abs().max() == 0 and out[:, :, -1].abs().max() == 0


def test_vae_channels_last_decoder_matches_pytorch():
    from cosmos_b200.models.vae import CausalVideoVAE
    from cosmos_b200.models.vae_cuda import CLDecoder
    torch.manual_seed(20)
    vae = CausalVideoVAE(16, (64, 128, 256, 256)).to(DEV).float().eval()
    z = torch.randn(1, 16, 3, 6, 8, device=DEV)
    with torch.no_grad():
        want = CausalVideoVAE.to_uint8(vae.decode(z))
    dec = CLDecoder(vae)
    got = dec.decode(z, chunk_latents=2)
    assert got.shape == want.shape == (1, 9, 48, 64, 3)
    diff = (got.int() - want.int()).abs()
    assert diff.float().mean() < 1.5 and (diff > 8).float().mean() < 0.01, (diff.float().mean(), diff.max())
    one = dec.decode(z, chunk_latents=3)
    assert (one.int() - got.int()).abs().max() <= 1  # chunking does not change the result


@pytest.mark.parametrize("m,n,k", [(256, 512, 384), (300, 264, 1000), (1024, 4096, 2048)])
def test_gemm_operand_majors(m, n, k):
    """Backward-pass GEMMs read transposed operands in place (MN-major shared-memory tiles)."""
    torch.manual_seed(21)
    dy = _rand(m, n)                       # [tokens, out]
    w = _rand(n, k, scale=1 / math.sqrt(n))  # [out, in]
    x = _rand(m, k)                        # [tokens, in]
    dx = torch.ops.cosmos_b200.gemm_ex(dy, w, False, True, None)       # dY @ W
    _close(dx, dy.float() @ w.float(), 3e-2, 2e-2, "dX = dY W")
    dw = torch.ops.cosmos_b200.gemm_ex(dy, x, True, True, None)        # dY^T @ X
    _close(dw, (dy.float().t() @ x.float()) / 1.0, 6e-2, 3e-2, "dW = dY^T X")


def test_linear_autograd_on_own_kernels():
    from cosmos_b200.ops import autograd as own
    torch.manual_seed(22)
    x = _rand(2, 300, 256).requires_grad_(True)
    w = _rand(512, 256, scale=1 / 16).requires_grad_(True)
    y = own.linear(x, w)
    g = _rand(2, 300, 512)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    (xf @ wf.t()).backward(g.float())
    _close(y, xf @ wf.t(), 3e-2, 2e-2, "linear fwd")
    _close(x.grad, xf.grad, 3e-2, 2e-2, "linear dX")
    _close(w.grad, wf.grad, 8e-2, 3e-2, "linear dW")


@pytest.mark.parametrize("materialized", [False, True])
@pytest.mark.parametrize("b,sq,skv,hq,hkv,mask,n_ar", [
    (1, 384, 384, 4, 2, ops.MASK_FULL, 0), (1, 300, 300, 2, 1, ops.MASK_CAUSAL, 0),
    (1, 256, 520, 2, 2, ops.MASK_FULL, 0), (2, 640, 640, 8, 2, ops.MASK_MOT, 200),
    (1, 130, 700, 4, 1, ops.MASK_CAUSAL, 0), (2, 1024, 1024, 4, 4, ops.MASK_FULL, 0)])
def test_attention_autograd_on_own_kernels(b, sq, skv, hq, hkv, mask, n_ar, materialized, monkeypatch):
    from cosmos_b200.ops import autograd as own
    monkeypatch.setattr(own, "_MATERIALIZED", materialized)
    if materialized and b * hq > 8:
        pytest.skip("the per-head variant is covered by the smaller cases")
    torch.manual_seed(23)
    q = _rand(b, sq, hq, 128).requires_grad_(True)
    k = _rand(b, skv, hkv, 128).requires_grad_(True)
    v = _rand(b, skv, hkv, 128).requires_grad_(True)
    g = _rand(b, sq, hq, 128)
    o = own.attention(q, k, v, None, mask, n_ar)
    o.backward(g)
    torch.cuda.synchronize()
    ops.check_status()
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    of, _ = ref.attention(qf, kf, vf, None, mask, n_ar)
    of.backward(g.float())
    _close(o, of, 2e-2, 2e-2, "attention fwd")
    _close(q.grad, qf.grad, 3e-2, 3e-2, "dQ")
    _close(k.grad, kf.grad, 3e-2, 3e-2, "dK")
    _close(v.grad, vf.grad, 3e-2, 3e-2, "dV")


def _grads_close(own_in, ref_in, names, atol=4e-2, rtol=4e-2):
    for a, b, n in zip(own_in, ref_in, names):
        assert a.grad is not None, f"no gradient for {n}"
        _close(a.grad, b.grad, atol, rtol, f"d{n}")


@pytest.mark.parametrize("b,s,d", [(2, 300, 512), (1, 200, 4096), (3, 64, 1024)])
def test_norm_autograd_on_own_kernels(b, s, d):
    """AdaLN-RMSNorm and plain RMSNorm: forward and backward kernels against fp32 autograd."""
    from cosmos_b200.ops import autograd as own
    torch.manual_seed(31)
    x = _rand(b, s, d).requires_grad_(True)
    gamma = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16().requires_grad_(True)
    mod = (0.3 * torch.randn(b, 2, d, device=DEV)).bfloat16().requires_grad_(True)
    g = _rand(b, s, d)
    y = own.adaln_rmsnorm(x, gamma, mod[:, 0], mod[:, 1], s, 1e-6)
    y.backward(g)
    xf, gf, mf = (t.detach().float().requires_grad_(True) for t in (x, gamma, mod))
    yf = ref.adaln_rmsnorm(xf, gf, mf[:, 0], mf[:, 1], s, 1e-6)
    yf.backward(g.float())
    _close(y, yf, 3e-2, 3e-2, "adaln fwd")
    _grads_close((x, mod), (xf, mf), ("x", "mod"))
    _close(gamma.grad, gf.grad, 0.5, 5e-2, "dgamma")  # sums over b*s rows of bf16-rounded terms
    x2 = _rand(b * s, d).requires_grad_(True)
    gamma2 = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16().requires_grad_(True)
    y2 = own.rmsnorm(x2, gamma2, 1e-6)
    y2.backward(g.reshape(b * s, d))
    x2f, g2f = x2.detach().float().requires_grad_(True), gamma2.detach().float().requires_grad_(True)
    y2f, _ = ref.rmsnorm(x2f, g2f, 1e-6)
    y2f.backward(g.reshape(b * s, d).float())
    _close(y2, y2f, 3e-2, 3e-2, "rmsnorm fwd")
    _close(x2.grad, x2f.grad, 4e-2, 4e-2, "rmsnorm dx")
    _close(gamma2.grad, g2f.grad, 0.5, 5e-2, "rmsnorm dgamma")
    ops.check_status()


def test_qkv_post_autograd_on_own_kernels():
    from cosmos_b200.ops import autograd as own
    torch.manual_seed(32)
    rows, hq, hk, rr = 70, 4, 2, 35
    qkv = _rand(rows, hq + 2 * hk, 128).requires_grad_(True)
    ang = torch.rand(rr, 64, device=DEV) * 6.0
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    gq = (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16().requires_grad_(True)
    gk = (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16().requires_grad_(True)
    go = [_rand(rows, h, 128) for h in (hq, hk, hk)]
    q, k, v = own.qkv_post(qkv, hq, cos, sin, gq, gk, 1e-6)
    torch.autograd.backward([q, k, v], go)
    f, gqf, gkf = (t.detach().float().requires_grad_(True) for t in (qkv, gq, gk))
    qf = ref.mrope(f[:, :hq], cos, sin, gqf, 1e-6)
    kf = ref.mrope(f[:, hq:hq + hk], cos, sin, gkf, 1e-6)
    vf = f[:, hq + hk:]
    torch.autograd.backward([qf, kf, vf], [t.float() for t in go])
    _close(q, qf, 3e-2, 3e-2, "q")
    _close(k, kf, 3e-2, 3e-2, "k")
    assert torch.equal(v, qkv.detach()[:, hq + hk:])
    _close(qkv.grad, f.grad, 4e-2, 4e-2, "dqkv")
    _close(gq.grad, gqf.grad, 0.3, 5e-2, "dgamma_q")
    _close(gk.grad, gkf.grad, 0.3, 5e-2, "dgamma_k")
    ops.check_status()


def test_swiglu_and_gated_residual_autograd_on_own_kernels():
    from cosmos_b200.ops import autograd as own
    torch.manual_seed(33)
    gu = _rand(100, 512).requires_grad_(True)
    g = _rand(100, 256)
    y = own.swiglu(gu)
    y.backward(g)
    guf = gu.detach().float().requires_grad_(True)
    yf = ref.swiglu(guf)
    yf.backward(g.float())
    _close(y, yf, 3e-2, 3e-2, "swiglu fwd")
    _close(gu.grad, guf.grad, 4e-2, 4e-2, "swiglu bwd")
    b, s, d = 2, 150, 1024
    x, f = _rand(b * s, d).requires_grad_(True), _rand(b * s, d).requires_grad_(True)
    gate = (0.5 * torch.randn(b, d, device=DEV)).bfloat16().requires_grad_(True)
    go = _rand(b * s, d)
    y = own.gated_residual(x, f, gate, s)
    y.backward(go)
    xf, ff, gf = (t.detach().float().requires_grad_(True) for t in (x, f, gate))
    yf = ref.gated_residual(xf, ff, gf, s)
    yf.backward(go.float())
    _close(y, yf, 3e-2, 3e-2, "gated residual fwd")
    _grads_close((x, f), (xf, ff), ("x", "f"))
    _close(gate.grad, gf.grad, 0.5, 5e-2, "dgate")
    ops.check_status()


def test_training_step_own_kernels_match_library_baseline(monkeypatch):
    """One optimizer step of a small head_dim-128 model: the autograd path on this package's kernels
    against the PyTorch / library path (same seeds), compared on loss, gradient norm and parameters."""
    from cosmos_b200.config import ParallelConfig, tiny128_config
    from cosmos_b200.models.mot import MoTModel
    from cosmos_b200.parallel.mesh import Mesh
    from cosmos_b200.train import TrainConfig, Trainer

    def run(library):
        if library:
            monkeypatch.setenv("COSMOS_TRAIN_LIBRARY_BACKWARD", "1")
        else:
            monkeypatch.delenv("COSMOS_TRAIN_LIBRARY_BACKWARD", raising=False)
        cfg = tiny128_config(max_text_len=32, n_layers=2)
        model = MoTModel(cfg, dtype=torch.bfloat16, device=DEV, pad_to=128)
        model.init_weights(seed=3)
        tr = Trainer(model, Mesh(ParallelConfig(), 1, 0), TrainConfig(lr=1e-3, max_grad_norm=0.5))
        g = torch.Generator(device=DEV).manual_seed(100)
        lat = torch.randn(1, 16, 3, 16, 16, generator=g, device=DEV, dtype=torch.bfloat16)
        ids = torch.randint(0, cfg.vocab_size, (1, 32), generator=g, device=DEV)
        t = torch.rand(1, generator=g, device=DEV)
        eps = torch.randn(lat.shape, generator=g, device=DEV, dtype=torch.bfloat16)
        log = tr.train_step(lat, ids, t=t, eps=eps)
        torch.cuda.synchronize()
        ops.check_status()
        return log, tr.fsdp.full_state()

    log_o, st_o = run(False)
    log_l, st_l = run(True)
    assert abs(log_o["loss"] - log_l["loss"]) < 2e-2 * max(1.0, abs(log_l["loss"]))
    assert abs(log_o["grad_norm"] - log_l["grad_norm"]) < 5e-2 * max(1.0, log_l["grad_norm"])
    worst = max((st_o[k].float() - st_l[k].float()).abs().max().item() for k in st_l)
    assert worst < 2e-2, f"parameters differ by {worst}"


@pytest.mark.parametrize("m,n,k", [(32, 4096, 4096), (1, 4096, 12288), (7, 1024, 2048), (300, 512, 256),
                                   (256, 4096, 12288), (130, 4096, 4096)])
def test_gemm_reduce_rmsnorm(m, n, k):
    """Output projection + residual + RMS-norm (the split-K reduction pass does all three for skinny problems;
    the last shape takes the unfused fallback) against the fp32 definition."""
    torch.manual_seed(41)
    a = _rand(m, k)
    w = _rand(n, k, scale=1 / math.sqrt(k))
    resid = _rand(m, n)
    gamma = (1 + 0.1 * torch.randn(n, device=DEV)).bfloat16()
    h, x_new = ops.gemm_reduce_rmsnorm(a, w, resid, gamma, 1e-6)
    torch.cuda.synchronize()
    ops.check_status()
    xf = resid.float() + a.float() @ w.float().t()
    hf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float()
    _close(x_new, xf, 3e-2, 2e-2, "x_new")
    _close(h, hf, 3e-2, 2e-2, "h")



def test_kernels_do_not_write_outside_their_outputs():
    """Canary check: outputs are views into larger buffers whose guard regions hold a bit pattern; after ragged
    GEMM, QKV-epilogue and attention launches the guards must be untouched."""
    torch.manual_seed(43)
    guard = 4096  # elements before and after

    def guarded(rows, cols):
        buf = torch.full((2 * guard + rows * cols,), -7.0, device=DEV, dtype=torch.bfloat16)
        return buf, buf[guard:guard + rows * cols].view(rows, cols)

    def intact(buf, what):
        assert bool((buf[:guard] == -7.0).all()) and bool((buf[-guard:] == -7.0).all()), f"{what}: guard region overwritten"

    for m, n, k in [(300, 264, 1000), (1, 512, 256), (129, 136, 72)]:
        a, w = _rand(m, k), _rand(n, k, scale=1 / math.sqrt(k))
        buf, out = guarded(m, n)
        ops.gemm(a, w, out=out)
        torch.cuda.synchronize()
        intact(buf, f"gemm {m}x{n}x{k}")
        _close(out, a.float() @ w.float().t(), 3e-2, 3e-2, "gemm into a guarded view")
    # SwiGLU epilogue writes N / 2 columns
    a, w = _rand(77, 512), _rand(1024, 512, scale=1 / math.sqrt(512))
    buf, out = guarded(77, 512)
    ops.gemm(a, w, epi=ops.EPI_SWIGLU, out=out)
    torch.cuda.synchronize()
    intact(buf, "gemm swiglu")
    # attention with ragged lengths writes exactly [B, Sq, Hq, 128]
    b, sq, skv, hq, hkv = 2, 300, 517, 4, 2
    q, kk, v = _rand(b, sq, hq, 128), _rand(b, skv, hkv, 128), _rand(b, skv, hkv, 128)
    buf, out = guarded(b * sq, hq * 128)
    o, _ = ops.attention(q, kk, v, out=out.view(b, sq, hq, 128))
    torch.cuda.synchronize()
    intact(buf, "attention")
    want, _ = ref.attention(q.float(), kk.float(), v.float())
    _close(o, want, 2e-2, 2e-2, "attention into a guarded view")
    ops.check_status()


@pytest.mark.parametrize("checked", [False, True])
def test_bounds_checked_build_selftest(checked):
    """The debug build with device-side index checks (cosmos_b200/_C_check.so): its check classifies good and
    bad indices and reports through the status word, and the checked kernels still match their definitions
    on valid inputs. Runs in a child process because the build is chosen when the library is loaded."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    if checked and not (root / "cosmos_b200" / "_C_check.so").exists():
        pytest.skip("bounds-checked build not present (python -m cosmos_b200.ops._build --bounds-check)")
    env = dict(os.environ, COSMOS_BOUNDS_CHECK="1" if checked else "0", COSMOS_B200_NO_BUILD="1")
    r = subprocess.run([sys.executable, "-m", "cosmos_b200.ops.bounds_selftest"], cwd=root, env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["ok"] and res["bounds_check_build"] == checked
    assert res["selftest_verdicts"] == ([1, 1, 1, 0, 0, 0, 1] if checked else [1] * 7)



def test_gemm_result_does_not_depend_on_the_tile_to_cta_assignment():
    """Race check by schedule: the persistent GEMM is run with one CTA per SM, with 37 and with 3 CTAs, so
    that tiles land on other CTAs, in another order, and many tiles share one CTA's smem ring and TMEM
    double buffer. Accumulation order inside a tile and across split-K partials is fixed, so all runs
    must agree bit for bit."""
    torch.manual_seed(31)
    k = torch.ops.cosmos_b200
    cases = [
        (lambda: (_rand(1500, 512), _rand(1024, 512, scale=1 / 16)), dict(epi=ops.EPI_PLAIN)),
        (lambda: (_rand(700, 1024), _rand(2048, 1024, scale=1 / 16)), dict(epi=ops.EPI_SWIGLU)),
        (lambda: (_rand(8, 4096), _rand(512, 4096, scale=1 / 32)), dict(epi=ops.EPI_PLAIN)),   # split-K path
    ]
    try:
        for make, kw in cases:
            a, w = make()
            outs = []
            for limit in (0, 37, 3):
                k.gemm_set_grid_limit(limit)
                outs.append(ops.gemm(a, w, **kw).clone())
            torch.cuda.synchronize()
            ops.check_status()
            assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), kw
            want = ref.gemm(a.float(), w.float(), None, kw["epi"])
            _close(outs[0], want, 3e-2, 2e-2, "gemm")
    finally:
        k.gemm_set_grid_limit(0)


def test_attention_over_several_kv_sources_in_one_launch():
    """Ring-KV in the kernel: K/V given as separate buffers of different (ragged) lengths, visited in order by one
    launch, equals attention over their concatenation."""
    torch.manual_seed(5)
    b, sq, hq, hkv = 1, 700, 8, 2
    lens = [512, 300, 129, 77]
    q = torch.randn(b, sq, hq, 128, device="cuda").bfloat16()
    ks = [torch.randn(b, n, hkv, 128, device="cuda").bfloat16() for n in lens]
    vs = [torch.randn(b, n, hkv, 128, device="cuda").bfloat16() for n in lens]
    o = torch.ops.cosmos_b200.attn_fwd_sources(q, [t.data_ptr() for t in ks], [t.data_ptr() for t in vs], lens, hkv,
                                               128 ** -0.5, None)
    ref, _ = ops.ref.attention(q.float(), torch.cat(ks, 1).float(), torch.cat(vs, 1).float())
    assert (o.float() - ref).abs().max().item() < 2e-2
    one, _ = ops.attention(q, torch.cat(ks, 1), torch.cat(vs, 1))
    assert (o.float() - one.float()).abs().max().item() < 1e-2
    single = torch.ops.cosmos_b200.attn_fwd_sources(q, [ks[0].data_ptr()], [vs[0].data_ptr()], lens[:1], hkv, 128 ** -0.5, None)
    ref1, _ = ops.ref.attention(q.float(), ks[0].float(), vs[0].float())
    assert (single.float() - ref1).abs().max().item() < 2e-2


@pytest.mark.parametrize("normalize", [False, True])
def test_cfg_unipc_step_matches_the_sampler(normalize):
    """The fused CFG + UniPC kernel against the sampler's own fp32 step, over a whole schedule (first step without a
    corrector, later ones with it, the last one returning the prediction)."""
    from cosmos_b200.models import sampler as samplers
    torch.manual_seed(2)
    rows, d, steps = 300, 64, 6
    sig = samplers.shifted_sigmas(steps, 3.0, None, device="cpu")
    a, b = samplers.UniPCSampler(sig), samplers.UniPCSampler(sig)
    x = torch.randn(rows, d, device="cuda")
    xa, xb = x.clone(), x.clone()
    for i in range(steps):
        vc = torch.randn(rows, d, device="cuda").bfloat16()
        vu = torch.randn(rows, d, device="cuda").bfloat16()
        v = ops.ref.cfg_combine(vc, vu, 4.0, normalize)
        xa = a.step(xa, v)
        xb = ops.cfg_unipc_step(xb, vc, vu, 4.0, b, normalize)
        assert (xa - xb).abs().max().item() < 2e-4 * (1 + xa.abs().max().item()), i


@pytest.mark.parametrize("scheduler", ["euler", "unipc"])
def test_denoise_steps_through_a_cuda_graph_equal_the_eager_steps(scheduler):
    """Small sequences run the model evaluation of every denoise step from one CUDA graph captured at the first step
    of the generation; the latents must equal those of the eager steps, for both samplers and with a control stream."""
    from cosmos_b200.config import SamplingConfig, tiny128_config
    from cosmos_b200.models.generator import GeneratorEngine
    from cosmos_b200.models.mot import MoTModel

    cfg = tiny128_config(max_text_len=32, n_layers=2)
    model = MoTModel(cfg, dtype=torch.bfloat16, device=DEV)
    model.init_weights(seed=4)
    g = torch.Generator(device=DEV).manual_seed(9)
    ids_c = torch.randint(0, cfg.vocab_size, (1, 32), generator=g, device=DEV)
    ids_u = torch.randint(0, cfg.vocab_size, (1, 32), generator=g, device=DEV)
    outs = {}
    for limit in (0, 8192):
        eng = GeneratorEngine(model)
        eng.graph_max_tokens = limit
        st = eng.make_state(ids_c, ids_u, (3, 16, 16))
        st.control_tokens = torch.randn(1, st.n_video, cfg.patch_dim, generator=torch.Generator(device=DEV).manual_seed(3),
                                        device=DEV)
        sc = SamplingConfig(num_steps=4, guidance=4.0, shift=3.0, scheduler=scheduler, seed=5, control_guidance=1.5)
        outs[limit] = eng.sample(st, sc)
        assert (limit > 0) == bool(st.__dict__.get("_graphs"))
    assert torch.isfinite(outs[0]).all()
    assert (outs[0] - outs[8192]).abs().max().item() <= 1e-5 * (1 + outs[0].abs().max().item())


def test_attention_on_cta_pairs_matches_the_reference():
    """The CTA-pair variant of the forward kernel (cta_group::2 tiles; off by default) on shapes with an odd number of
    query blocks, causal and MoT masks, GQA and a batch."""
    k = torch.ops.cosmos_b200
    k.attn_set_cta_pair(True)
    try:
        torch.manual_seed(1)
        for (b, sq, skv, hq, hkv, mask, n_ar) in ((1, 777, 777, 4, 4, ops.MASK_CAUSAL, 0), (2, 600, 900, 2, 1, ops.MASK_FULL, 0),
                                                 (1, 1300, 1300, 4, 2, ops.MASK_MOT, 333)):
            q = torch.randn(b, sq, hq, 128, device=DEV).bfloat16()
            kk = torch.randn(b, skv, hkv, 128, device=DEV).bfloat16()
            v = torch.randn(b, skv, hkv, 128, device=DEV).bfloat16()
            o, lse = ops.attention(q, kk, v, mask=mask, n_ar=n_ar, return_lse=True)
            ro, rlse = ops.ref.attention(q.float(), kk.float(), v.float(), 128 ** -0.5, mask, n_ar, True)
            assert (o.float() - ro).abs().max().item() < 2e-2
            assert (lse - rlse).abs().max().item() < 1e-3
    finally:
        k.attn_set_cta_pair(False)


@pytest.mark.parametrize("b,v,flags", [(5, 151936, True), (3, 4097, True), (4, 1000, False), (2, 50, True)])
def test_sample_topk_selects_the_64_largest_penalised_logits(b, v, flags):
    """Radix-select kernel against torch.topk over the fp32 definition of the penalties. bf16 logits tie often, so the
    values are compared in order and every id is checked against the penalised row."""
    g = torch.Generator(device=DEV).manual_seed(v)
    logits = (torch.randn(b, v, device=DEV, generator=g) * 3).bfloat16()
    tokens = torch.randint(0, v, (b,), device=DEV, generator=g)
    any_ = (torch.rand(b, v, device=DEV, generator=g) < 0.3) if flags else None
    out_ = (any_ & (torch.rand(b, v, device=DEV, generator=g) < 0.5)) if flags else None
    pres = torch.rand(b, device=DEV, generator=g) * 2 if flags else None
    rep = 1 + torch.rand(b, device=DEV, generator=g) if flags else None
    off = 1000
    ref_any, ref_out = (any_.clone(), out_.clone()) if flags else (None, None)
    want = ops.sample_topk(logits.float(), ref_any, ref_out, tokens + off, pres, rep, off)      # PyTorch definition
    got = ops.sample_topk(logits, any_, out_, tokens + off, pres, rep, off)
    torch.cuda.synchronize()
    if flags:
        assert torch.equal(any_, ref_any) and torch.equal(out_, ref_out)
        assert out_[torch.arange(b), tokens].all()
    assert torch.equal(got[..., 0], want[..., 0])
    ids = got[..., 1].contiguous().view(torch.int32).long() - off
    k = min(64, v)
    pen = logits.float()
    if flags:
        pen = torch.where(ref_any, torch.where(pen > 0, pen / rep[:, None], pen * rep[:, None]), pen)
        pen = pen - pres[:, None] * ref_out.float()
    assert ((ids[:, :k] >= 0) & (ids[:, :k] < v)).all()
    assert torch.equal(pen.gather(1, ids[:, :k]), got[:, :k, 0])
    for r in range(b):
        assert ids[r, :k].unique().numel() == k


def test_sample_topk_with_all_logits_equal():
    logits = torch.full((2, 5000), 1.25, device=DEV, dtype=torch.bfloat16)
    got = ops.sample_topk(logits, None, None, None, None, None, 0)
    assert (got[..., 0] == 1.25).all()
    ids = got[..., 1].contiguous().view(torch.int32)
    assert all(ids[r].unique().numel() == 64 and ids[r].min() >= 0 and ids[r].max() < 5000 for r in range(2))


@pytest.mark.parametrize("n_src", [1, 2, 8])
def test_sample_pick_matches_the_definition(n_src):
    """Merge of the shards' candidates and the draw against the PyTorch definition on the same noise."""
    g = torch.Generator(device=DEV).manual_seed(n_src)
    b = 300
    vals = torch.randn(n_src, b, 64, device=DEV, generator=g).sort(dim=-1, descending=True).values * 2
    ids = torch.stack([torch.randperm(100000, device=DEV, generator=g)[:n_src * 64].view(n_src, 64) for _ in range(b)], 1)
    cand = torch.stack([vals, ids.to(torch.int32).view(torch.float32)], -1).view(n_src * b, 64, 2).contiguous()
    temp = torch.where(torch.rand(b, device=DEV, generator=g) < 0.2, torch.zeros(b, device=DEV),
                       0.3 + torch.rand(b, device=DEV, generator=g))
    top_k = torch.randint(1, 80, (b,), device=DEV, generator=g)
    top_p = 0.2 + 0.8 * torch.rand(b, device=DEV, generator=g)
    noise = torch.rand(b, 64, device=DEV, generator=g).clamp_min(1e-7)
    got = ops.sample_pick(cand, n_src, temp, top_k, top_p, noise, 90000, torch.empty(b, dtype=torch.long, device=DEV))
    want = ops.sample_pick(cand.cpu(), n_src, temp.cpu(), top_k.cpu(), top_p.cpu(), noise.cpu(), 90000,
                           torch.empty(b, dtype=torch.long))
    same = (got.cpu() == want).float().mean().item()
    assert same >= 0.99, f"only {same:.3f} of the draws agree"      # a nucleus boundary within rounding may differ
    greedy = temp.cpu() == 0
    assert torch.equal(got.cpu()[greedy], want[greedy]) and (got < 90000).all()


@pytest.mark.parametrize("b,hq,hkv,d", [(32, 32, 8, 4096), (1, 32, 8, 4096), (8, 8, 2, 1024), (300, 4, 4, 512)])
def test_gemm_decode_qkv_post_reduces_the_split_k_partials_in_the_glue_kernel(b, hq, hkv, d):
    """QKV projection + decode glue in two launches (partials reduced by the glue kernel) against the three-launch
    form (GEMM, split-K reduction, glue) and, through it, the fp32 definition."""
    torch.manual_seed(b)
    page, n_pages = 16, 2 * ((b + 15) // 16) + 1
    h = _rand(b, d)
    w = _rand((hq + 2 * hkv) * 128, d, scale=d ** -0.5)
    ang = torch.rand(b, 64, device=DEV) * 6.0
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    gq, gk = (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16(), (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16()
    slots = (torch.randperm(n_pages * page, device=DEV)[:b]).long()
    kc, vc = _rand(n_pages, hkv, page, 128), _rand(n_pages, hkv, page, 128)
    kc2, vc2 = kc.clone(), vc.clone()
    q = ops.gemm_decode_qkv_post(h, w, hq, cos, sin, gq, gk, 1e-6, slots, kc, vc)
    qkv = ops.gemm(h, w).view(b, hq + 2 * hkv, 128)
    q2 = ops.decode_qkv_post(qkv, hq, cos, sin, gq, gk, 1e-6, slots, kc2, vc2)
    torch.cuda.synchronize()
    _close(q, q2, 1e-2, 1e-2, "q")
    _close(kc, kc2, 1e-2, 1e-2, "k cache")
    _close(vc, vc2, 1e-2, 1e-2, "v cache")
    f = (h.float() @ w.float().t()).view(b, hq + 2 * hkv, 128)
    _close(q, ref.mrope(f[:, :hq], cos, sin, gq.float(), 1e-6), 4e-2, 4e-2, "q vs fp32")


def test_vae_channels_last_encoder_matches_pytorch():
    """Implicit-GEMM encoder (strided convolutions as stride-1 + even positions, 1x1 skips as GEMMs, chunked in time)
    against the fp32 PyTorch modules in one pass."""
    from cosmos_b200.models.vae import CausalVideoVAE
    from cosmos_b200.models.vae_cuda import CLEncoder
    torch.manual_seed(21)
    vae = CausalVideoVAE(16, (64, 128, 256, 256)).to(DEV).float().eval()
    video = torch.rand(1, 3, 17, 48, 64, device=DEV) * 2 - 1
    with torch.no_grad():
        want = vae.encode(video)
    enc = CLEncoder(vae)
    got = enc.encode(video, chunk_frames=8)
    assert got.shape == want.shape == (1, 16, 5, 6, 8)
    err = (got - want).abs()
    scale = want.abs().mean().item()
    assert err.mean().item() < 0.03 * scale and err.max().item() < 0.25 * want.abs().max().item(), \
        (err.mean().item(), err.max().item(), scale)
    other = enc.encode(video, chunk_frames=4)
    assert (other - got).abs().max().item() <= 0.02 * want.abs().max().item()   # chunking does not change the result


@pytest.mark.parametrize("n,off", [(4096, 0), (1003, 0), (2048, 3), (777, 8)])
def test_adamw_kernels_match_the_fp32_definition(n, off):
    """`rs_adamw` (gradients read from bf16 buffers, here one local source) and `adamw_shard` (fp32 reduced
    gradient): vector path, scalar tail and a source offset that rules the vector loads out."""
    k = torch.ops.cosmos_b200
    g = torch.Generator(device=DEV).manual_seed(n + off)
    full = torch.randn(off + n + 5, device=DEV, generator=g).bfloat16()
    lr, b1, b2, eps, wd, scale, step = 1e-2, 0.9, 0.95, 1e-8, 0.1, 0.5, 3

    def fresh():
        w = torch.randn(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))
        m = torch.randn(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(2)) * 0.1
        v = torch.rand(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(3)) * 0.1
        return w, m, v, torch.empty(n, device=DEV, dtype=torch.bfloat16)

    gr = full[off:off + n].float()
    w0, m0, v0, _ = fresh()
    gs = gr * scale
    m_ref = b1 * m0 + (1 - b1) * gs
    v_ref = b2 * v0 + (1 - b2) * gs * gs
    w_ref = w0 - lr * ((m_ref / (1 - b1 ** step)) / ((v_ref / (1 - b2 ** step)).sqrt() + eps) + wd * w0)
    ptrs = torch.tensor([full.data_ptr()], dtype=torch.int64, device=DEV)
    # pass 1: sum of squares (and the reduced gradient), pass 2: the update from the sources
    sq = torch.zeros(1, device=DEV)
    red = torch.empty(n, device=DEV)
    w, m, v, p = fresh()
    k.rs_adamw(ptrs, 1, off, w, m, v, p, 1.0, 0.0, b1, b2, eps, 0.0, step, 1, sq, red)
    assert torch.allclose(sq, (gr * gr).sum()[None], rtol=1e-4) and torch.equal(red, gr)
    k.rs_adamw(ptrs, 1, off, w, m, v, p, scale, lr, b1, b2, eps, wd, step, 0, None, None)
    for got, want in ((m, m_ref), (v, v_ref), (w, w_ref)):
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)
    assert torch.equal(p, w.bfloat16())
    w, m, v, p = fresh()
    k.adamw_shard(gr.contiguous(), w, m, v, p, scale, lr, b1, b2, eps, wd, step)
    for got, want in ((m, m_ref), (v, v_ref), (w, w_ref)):
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)
    assert torch.equal(p, w.bfloat16())
