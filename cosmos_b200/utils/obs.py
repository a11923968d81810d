"""Observability: NVTX ranges, CUDA-event phase timers (max over ranks), rank-0 structured
logging and the `benchmark.json` writer (the reference's `--benchmark` flag writes a file with an
`"average"` object, reference cookbooks/cosmos3/reasoner/run_with_cosmos_framework.ipynb:634-639)."""
from __future__ import annotations

import contextlib
import json
import os
import sys
import time
from collections import defaultdict
from pathlib import Path
from typing import Dict, List, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when CUDA is available, else a no-op."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """Times named phases with CUDA events on the current stream (wall clock on CPU) and reports
    per-phase totals, reduced with max over ranks when a process group is up."""

    def __init__(self):
        self.cuda = torch.cuda.is_available()
        self._open: Dict[str, object] = {}
        self._pairs: Dict[str, List] = defaultdict(list)
        self._wall: Dict[str, float] = defaultdict(float)

    @contextlib.contextmanager
    def phase(self, name: str):
        with nvtx_range(name):
            if self.cuda:
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                try:
                    yield
                finally:
                    e.record()
                    self._pairs[name].append((s, e))
            else:
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self._wall[name] += (time.perf_counter() - t0) * 1e3

    def summary_ms(self, group=None) -> Dict[str, float]:
        out = dict(self._wall)
        if self.cuda:
            torch.cuda.synchronize()
            for k, pairs in self._pairs.items():
                out[k] = out.get(k, 0.0) + sum(s.elapsed_time(e) for s, e in pairs)
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and out:
            keys = sorted(out)
            t = torch.tensor([out[k] for k in keys], dtype=torch.float64,
                             device="cuda" if (self.cuda and dist.get_backend() == "nccl") else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            out = {k: float(v) for k, v in zip(keys, t.tolist())}
        return out


class JsonlLogger:
    """Rank-0 structured logger: one JSON object per line to a file and/or stdout."""

    def __init__(self, path: Optional[str] = None, stdout: bool = True):
        self.rank = int(os.environ.get("RANK", "0"))
        self.fh = open(path, "a") if (path and self.rank == 0) else None
        self.stdout = stdout

    def log(self, **fields) -> None:
        if self.rank != 0:
            return
        line = json.dumps({"ts": round(time.time(), 3), **fields})
        if self.fh:
            self.fh.write(line + "\n")
            self.fh.flush()
        if self.stdout:
            print(line, file=sys.stdout, flush=True)


def write_benchmark_json(out_root, records: List[dict], extra: Optional[dict] = None) -> Path:
    avg: Dict[str, float] = {}
    keys = {k for r in records for k, v in r.items() if isinstance(v, (int, float)) and not isinstance(v, bool)}
    for k in sorted(keys):
        vals = [r[k] for r in records if k in r]
        avg[k] = sum(vals) / len(vals)
    path = Path(out_root) / "benchmark.json"
    path.write_text(json.dumps({"average": avg, "samples": records, **(extra or {})}, indent=1))
    return path
