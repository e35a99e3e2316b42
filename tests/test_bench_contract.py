"""What bench.py answers without a GPU: more than one GPU is declined in one line with exit code 2, and the
reference arm says in one JSON line why it cannot run here."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_declined_in_one_line():
    p = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]
