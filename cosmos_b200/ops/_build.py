"""In-tree build of the sm_100a kernel library (``cosmos_b200/_C.so``).

``.cu`` files contain no torch headers and are compiled one by one with
``nvcc -gencode arch=compute_100a,code=sm_100a``; the torch glue (``bindings.cpp``,
``runtime.cpp``, ``safetensors_reader.cpp``, over the torch-free host runtime in ``csrc/host``) is
compiled with the host compiler and everything is linked into one
shared object that ``torch.ops.load_library`` loads. Objects are cached under ``build/``
keyed by a hash of the source, its headers and the flags, so rebuilds are incremental.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"
SO_PATH = ROOT / "cosmos_b200" / "_C.so"
SO_PATH_CHECKED = ROOT / "cosmos_b200" / "_C_check.so"  # the same library with -DCOSMOS_BOUNDS_CHECK

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-D_GLIBCXX_USE_CXX11_ABI=1", "-w"]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _torch_paths():
    import torch
    from torch.utils import cpp_extension

    inc = cpp_extension.include_paths()
    lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return inc, lib, abi


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(Path(p).read_bytes())
    return h.hexdigest()[:16]


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(map(str, cmd)) + "\n" + r.stdout)
    return r.stdout


def build(verbose: bool = False, force: bool = False, bounds_check: bool = False) -> Path:
    """Compile (if stale) and return the path of the shared object. With `bounds_check` the debug
    variant is built: indices that kernels read from tensors (cache slots, page ids) are compared with
    their limits on the device and a bad one is reported through the status word and skipped."""
    BUILD.mkdir(exist_ok=True)
    so_path = SO_PATH_CHECKED if bounds_check else SO_PATH
    extra = ["-DCOSMOS_BOUNDS_CHECK"] if bounds_check else []
    suffix = ".chk" if bounds_check else ""
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted((CSRC / "host").glob("*.hpp"))
    cu_files = sorted(CSRC.glob("*.cu"))
    cpp_files = sorted(CSRC.glob("*.cpp"))
    inc, torch_lib, abi = _torch_paths()
    cxx_flags = [f if not f.startswith("-D_GLIBCXX") else f"-D_GLIBCXX_USE_CXX11_ABI={abi}" for f in CXX_FLAGS]
    nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
    cuda_inc = os.path.join(_cuda_home(), "include")
    py_inc = sysconfig.get_paths()["include"]

    jobs = []
    objs = []
    for src in cu_files:
        tag = _digest([src] + headers, " ".join(NVCC_FLAGS + extra))
        obj = BUILD / f"{src.stem}.{tag}{suffix}.o"
        objs.append(obj)
        if force or not obj.exists():
            jobs.append([nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
    for src in cpp_files:
        tag = _digest([src] + headers, " ".join(cxx_flags + extra) + sys.version)
        obj = BUILD / f"{src.stem}.{tag}{suffix}.o"
        objs.append(obj)
        if force or not obj.exists():
            cmd = ["g++", *cxx_flags, *extra, "-I", str(CSRC), "-I", cuda_inc, "-I", py_inc]
            for i in inc:
                cmd += ["-isystem", i]
            cmd += ["-DTORCH_API_INCLUDE_EXTENSION_H", "-c", str(src), "-o", str(obj)]
            jobs.append(cmd)

    if jobs:
        if verbose:
            print(f"[cosmos_b200] compiling {len(jobs)} translation unit(s) for sm_100a", flush=True)
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(_run, jobs):
                if verbose and out.strip():
                    print(out)

    stamp = BUILD / f"link{suffix}.stamp"
    want = " ".join(o.name for o in objs)
    if force or jobs or not so_path.exists() or not stamp.exists() or stamp.read_text() != want:
        cmd = ["g++", "-shared", "-o", str(so_path), *map(str, objs),
               f"-L{torch_lib}", f"-L{_cuda_home()}/lib64", f"-Wl,-rpath,{torch_lib}",
               "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart"]
        _run(cmd)
        stamp.write_text(want)
        # drop stale objects of earlier source versions
        keep = {o.name for o in objs}
        for old in BUILD.glob("*.chk.o" if bounds_check else "*.o"):
            if old.name not in keep and old.name.endswith(".chk.o") == bounds_check:
                old.unlink()
    return so_path


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="Build the sm_100a kernel library in-tree.")
    ap.add_argument("--force", action="store_true", help="recompile every translation unit")
    ap.add_argument("--bounds-check", action="store_true",
                    help="build the debug variant (cosmos_b200/_C_check.so, -DCOSMOS_BOUNDS_CHECK) instead")
    a = ap.parse_args()
    print(build(verbose=True, force=a.force, bounds_check=a.bounds_check))
