"""The extension's error paths, on the CPU: every refusal is a Python exception with a message
that names the numbers involved. (Messages used to stream integers into an ostream, which crashed
the interpreter in builds on some hosts; numbers are now turned into strings first.)"""

import subprocess
import sys
import textwrap
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

# Run in a child process: if an error path crashes, the test fails instead of the test run dying.
PROBE = textwrap.dedent(
    """
    import sys, torch
    sys.path.insert(0, {root!r})
    from llmserve_b200.ops import build
    ext = build.load_core()
    lib = build.attention_library(64)
    calls = {{
        "not loaded": lambda: ext.attention_scratch_floats(48, 1, 1, 2),
        "wrong head size": lambda: ext.load_attention_library(lib, 32),
        "missing file": lambda: ext.load_attention_library("/nonexistent/attention.so", 64),
        "cpu tensor": lambda: ext.silu_mul(torch.zeros(2, 4), torch.zeros(2, 2)),
    }}
    for name, call in calls.items():
        try:
            call()
            print(name, "-> no error")
        except RuntimeError as e:
            print(name, "->", str(e).splitlines()[0])
    """
)


def test_refusals_are_exceptions_with_their_numbers():
    r = subprocess.run([sys.executable, "-c", PROBE.format(root=str(ROOT))], capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, f"the probe died with {r.returncode}:\n{r.stdout}\n{r.stderr[-2000:]}"
    out = dict(line.split(" -> ", 1) for line in r.stdout.splitlines() if " -> " in line)
    assert "head size 48" in out["not loaded"]
    assert "built for head size 64, not 32" in out["wrong head size"]
    assert "cannot load attention library" in out["missing file"]
    assert "must be a CUDA tensor" in out["cpu tensor"]
