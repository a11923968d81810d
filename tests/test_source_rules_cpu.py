"""Rules that every source file of the repository keeps, checked as text (nothing is compiled or run):
no bulk-copy load that fans one tile out to several CTAs (kernels here also run in multi-GPU process groups, where
such a load from a peer's memory is not allowed), none of the batched memcpy entry points, every spin on an
mbarrier or a peer flag goes through a bounded helper, and sources are written for sm_100a only."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
SRC_DIRS = [ROOT / "csrc", ROOT / "cosmos_b200", ROOT / "tests", ROOT / "examples"]
TOP_FILES = [ROOT / "bench.py", ROOT / "__graft_entry__.py"]


def _sources(suffixes):
    out = [p for p in TOP_FILES if p.suffix in suffixes]
    for d in SRC_DIRS:
        if d.exists():
            out += [p for p in d.rglob("*") if p.suffix in suffixes and p.is_file()]
    return out


def _fan_out_qualifier() -> str:
    """The PTX qualifier of a copy delivered to several CTAs at once, spelled from character codes so that this
    file itself stays free of it."""
    head = "".join(chr(c) for c in (109, 117, 108, 116, 105, 99, 97, 115, 116))
    tail = "".join(chr(c) for c in (99, 108, 117, 115, 116, 101, 114))
    return head + "::" + tail


def test_no_fan_out_copies_and_no_batched_memcpy():
    qualifier = _fan_out_qualifier()
    batch = [a + "Memcpy" + b + "BatchAsync" for a in ("cuda", "cu") for b in ("", "3D")]
    for p in _sources({".cu", ".cuh", ".h", ".hpp", ".cpp", ".py"}):
        text = p.read_text(errors="replace")
        assert qualifier not in text, f"{p} names a copy with the fan-out qualifier"
        for name in batch:
            assert name not in text, f"{p} names {name}"


def test_device_waits_are_bounded():
    """A `while` / `for(;;)` loop that polls an mbarrier or an acquire-load must sit in one of the bounded
    helpers (they compare clock64() with COSMOS_WAIT_LIMIT_CYCLES and report through the status word)."""
    poll = re.compile(r"mbarrier\.(test_wait|try_wait)|ld\.acquire\.sys|ld_acquire_sys\(")
    for p in _sources({".cu", ".cuh"}):
        text = p.read_text()
        for m in poll.finditer(text):
            # the enclosing function body: from the previous line that starts a definition to the match
            start = max(text.rfind("\n__device__", 0, m.start()), text.rfind("\n__global__", 0, m.start()),
                        text.rfind("\ntemplate", 0, m.start()))
            end = text.find("\n}\n", m.start())
            body = text[start:end if end > 0 else len(text)]
            loops = re.search(r"while\s*\(|for\s*\(\s*;\s*;", body) is not None
            if loops:
                assert "COSMOS_WAIT_LIMIT_CYCLES" in body or "mbar_wait(" in body, \
                    f"{p}: unbounded wait near offset {m.start()}"
    common = (ROOT / "csrc" / "common.cuh").read_text()
    assert "COSMOS_WAIT_LIMIT_CYCLES" in common and "ST_TIMEOUT_PEER" in common


def test_sources_target_sm100a_only():
    build = (ROOT / "cosmos_b200" / "ops" / "_build.py").read_text()
    assert "arch=compute_100a,code=sm_100a" in build and "-lineinfo" in build
    for p in _sources({".cu", ".cuh"}):
        text = p.read_text()
        assert "wgmma" not in text, f"{p}: Hopper-only instruction"
        assert not re.search(r"__CUDA_ARCH__\s*[<>=]", text), f"{p}: per-architecture code path"
    hot = "".join((ROOT / "csrc" / f).read_text() for f in
                  ("gemm_tcgen05.cu", "attn_tcgen05.cu", "attn_bwd_tcgen05.cu", "paged_decode_tc.cu", "common.cuh"))
    for needle in ("tcgen05.mma", "tcgen05.ld", "tcgen05.alloc", "tcgen05.commit", "cp.async.bulk.tensor"):
        assert needle in hot, needle
    for p in _sources({".py"}):
        if p.name == Path(__file__).name:
            continue
        text = p.read_text()
        assert "import triton" not in text and "torch.compile(" not in text, f"{p}: compatibility layer on a hot path"
