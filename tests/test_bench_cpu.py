"""The parts of bench.py that need no GPU: the reference arm's line and the clock-sample reduction."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_json_line_and_exits_zero():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "3"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]


def test_clock_sampler_reduces_rows_to_median_max_and_reasons():
    sys.path.insert(0, str(ROOT))
    try:
        import bench
    finally:
        sys.path.pop(0)
    s = bench.ClockSampler(0)
    assert s.stop()["reasons"] == ["nvidia-smi unavailable"]            # never started: says so instead of guessing

    class Done:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

    s.proc = Done()
    row = lambda sm, pw, cap: ["0", str(sm), "1965", str(pw), "0x4", "Not Active", "Not Active", "Not Active", cap]  # noqa: E731
    s.rows = [row(1600, 990.5, "Active"), row(1590, 998.0, "Active"), row(1650, 700.0, "Not Active"),
              ["0", "[N/A]", "1965", "1", "0", "x", "x", "x", "x"], ["short"]]
    out = s.stop()
    assert out["sm_mhz"] == 1600 and out["sm_max_mhz"] == 1965 and out["power_w_max"] == 998.0
    assert out["samples"] == 3 and out["reasons"] == ["sw_power_cap"]
    assert bench.PUBLISHED_S_PER_VIDEO[1] / bench.PUBLISHED_STEPS > 3.0
