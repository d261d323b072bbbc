"""What bench.py promises without a GPU: more than one GPU is refused with one line and status 2; the reference arm
says in one JSON line why it is unavailable and exits with 0."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line():
    for n in ("2", "8"):
        p = run("--gpus", n, "--steps", "2", "--warmup", "1")
        assert p.returncode == 2
        lines = [line for line in p.stdout.splitlines() if line.strip()]
        assert len(lines) == 1 and f"--gpus {n}" in lines[0]


def test_the_reference_arm_says_why_it_is_unavailable():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    lines = [line for line in p.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference" and isinstance(record["unavailable"], str) and "\n" not in record["unavailable"]
