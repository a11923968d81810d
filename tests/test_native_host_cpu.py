"""Host runtime in C++ (csrc/host): the test program is built with the compiler's address + undefined-behaviour
sanitizers and with its thread sanitizer and must pass under both; a negative control shows that the thread
sanitizer does see the race the trailing barrier of the one-shot all-reduce exists to prevent. The torch-bound
classes are compared against their pure-Python stand-ins."""
import random
import shutil
import subprocess
from pathlib import Path

import pytest
import torch

HOST = Path(__file__).resolve().parents[1] / "csrc" / "host"


def _build(tmp: Path, name: str, flags):
    exe = tmp / name
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-Wall", "-Wextra", "-Werror", *flags, str(HOST / "host_tests.cpp"), "-o", str(exe),
           "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if r.returncode != 0 and ("cannot find" in r.stderr or "unrecognized" in r.stderr):
        pytest.skip("sanitizer runtime not installed: " + r.stderr.strip().splitlines()[-1])
    assert r.returncode == 0, r.stderr
    return exe


def _probe(exe: Path, tmp: Path):
    """Some containers forbid the address-space layout a sanitizer runtime needs; that is not a finding."""
    r = subprocess.run([str(exe), str(tmp), "no_such_case"], capture_output=True, text=True, timeout=120)
    if r.returncode != 0 and ("FATAL" in r.stderr or "unexpected memory mapping" in r.stderr):
        pytest.skip("sanitizer runtime cannot start here: " + r.stderr.strip().splitlines()[0])


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host compiler")
def test_host_runtime_under_address_and_ub_sanitizers(tmp_path):
    exe = _build(tmp_path, "host_asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"])
    _probe(exe, tmp_path)
    r = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("PASS ") == 6 and "FAIL" not in r.stdout
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host compiler")
def test_host_runtime_under_thread_sanitizer_and_negative_control(tmp_path):
    exe = _build(tmp_path, "host_tsan", ["-fsanitize=thread"])
    _probe(exe, tmp_path)
    r = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "data race" not in r.stderr, r.stdout + r.stderr
    assert r.stdout.count("PASS ") == 6
    # Without the trailing barrier a fast rank overwrites its input under a slow reader: must be reported.
    bad = subprocess.run([str(exe), str(tmp_path), "signal_without_trailing_barrier"], capture_output=True, text=True,
                         timeout=600)
    assert bad.returncode != 0 and "data race" in bad.stderr


def test_native_allocator_matches_the_python_stand_in():
    from cosmos_b200 import ops
    from cosmos_b200.serve.paged import _PyAllocator
    if not ops.load_extension(build_if_missing=False):
        pytest.skip("extension not built")
    nat = torch.classes.cosmos_b200.PagedKVAllocator(53, 16, 9)
    py = _PyAllocator(53, 16, 9)
    rnd, live, nxt = random.Random(3), [], 0
    for _ in range(3000):
        op = rnd.random()
        if op < 0.25 or not live:
            t = rnd.randint(1, 170)
            a, b = nat.extend(nxt, t), py.extend(nxt, t)
            assert a == b
            if a:
                live.append(nxt)
            nxt += 1
        elif op < 0.85:
            s = rnd.choice(live)
            assert nat.extend(s, 1) == py.extend(s, 1)
        else:
            s = live.pop(rnd.randrange(len(live)))
            nat.release(s), py.release(s)
        assert nat.num_free() == py.num_free()
        assert nat.can_allocate(40) == py.can_allocate(40)
    q = live[:6] + [10 ** 9]
    ta, la = torch.zeros(len(q), 9, dtype=torch.int32), torch.zeros(len(q), dtype=torch.int32)
    tb, lb = torch.zeros(len(q), 9, dtype=torch.int32), torch.zeros(len(q), dtype=torch.int32)
    nat.fill_tables(q, ta, la), py.fill_tables(q, tb, lb)
    assert torch.equal(ta, tb) and torch.equal(la, lb)
    for s in q:
        assert list(nat.blocks(s)) == py.blocks(s) and nat.length(s) == py.length(s)
    with pytest.raises(RuntimeError):
        nat.fill_tables(q, torch.zeros(2, 9, dtype=torch.int32), la)   # too few rows
    with pytest.raises(RuntimeError):
        torch.classes.cosmos_b200.PagedKVAllocator(0, 16, 4)
