"""The commands in README.md, cookbooks/, examples/README.md and the profile notes name modules that exist and flags their parsers
know (checked against each entry point's --help text)."""
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
DOCS = ([ROOT / "README.md", ROOT / "examples" / "README.md"] + sorted((ROOT / "cookbooks").glob("*.md"))
        + sorted((ROOT / "profiles").glob("*.md")))
LAUNCHER_FLAGS = {"--nproc-per-node", "--master-addr", "--master-port", "--nnodes", "--standalone", "--local-addr"}


def _commands():
    """(entry point, set of flags) per documented command; a trailing backslash continues the line."""
    found = {}
    for doc in DOCS:
        text = doc.read_text().replace("\\\n", " ")
        for line in text.splitlines():
            m = re.search(r"(?:-m\s+(cosmos_b200[\w.]*)|\b(bench\.py))", line)
            if not m or line.lstrip().startswith("|"):
                continue
            entry = m.group(1) or m.group(2)
            tail = line[m.end():].split("#")[0]
            flags = {f.split("=")[0] for f in re.findall(r"(?<![\w-])(--[A-Za-z][\w-]*)", tail)}
            found.setdefault(entry, set()).update(flags - LAUNCHER_FLAGS)
    return found


CMDS = _commands()


def test_documented_entry_points_exist():
    assert {"cosmos_b200.scripts.inference", "cosmos_b200.serve.server", "cosmos_b200.train", "bench.py"} <= set(CMDS)
    for entry in CMDS:
        if entry == "bench.py":
            assert (ROOT / "bench.py").exists()
        else:
            assert (ROOT / (entry.replace(".", "/") + ".py")).exists(), f"{entry} is documented but missing"


@pytest.mark.parametrize("entry", sorted(e for e, f in CMDS.items() if f))
def test_documented_flags_are_known_to_the_entry_point(entry):
    cmd = [sys.executable, str(ROOT / "bench.py"), "--help"] if entry == "bench.py" else [sys.executable, "-m", entry, "--help"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    known = set(re.findall(r"(--[A-Za-z][\w-]*)", r.stdout))
    missing = sorted(CMDS[entry] - known)
    assert not missing, f"{entry}: documented flags not in --help: {missing}"
