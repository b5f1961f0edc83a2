"""What bench.py answers without a GPU: more than one GPU is refused with exit code 2, the
reference arm reports that the reference cannot be installed here."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args],
                          capture_output=True, text=True, cwd=ROOT, timeout=120)


def test_more_than_one_gpu_is_refused():
    r = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_is_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]
