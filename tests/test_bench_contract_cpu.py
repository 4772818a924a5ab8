"""bench.py's output contract, as far as it can be checked without a GPU: exactly one JSON line on stdout, everything
else on stderr; the reference arm answers ``unavailable`` (exit 0) where the reference cannot run."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero_without_a_gpu():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-800:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, p.stdout
    obj = json.loads(lines[0])
    assert obj["impl"] == "reference" and "unavailable" in obj and len(obj["unavailable"]) <= 300


def test_stdout_is_reserved_for_the_json_line():
    """Anything a library prints to file descriptor 1 after start-up lands on stderr; ``_emit`` still reaches stdout."""
    code = ("import os, sys; sys.path.insert(0, %r); import bench; bench._claim_stdout(); "
            "os.write(1, b'banner from a C library\\n'); print('python print'); bench._emit({'ok': 1})") % ROOT
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-500:]
    assert p.stdout.strip() == '{"ok": 1}', p.stdout
    assert "banner from a C library" in p.stderr and "python print" in p.stderr
