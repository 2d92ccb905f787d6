"""What bench.py promises without a device: more than one GPU is refused with a line and exit code 2, and
the reference arm says why it is unavailable where there is no checkout of the reference to compile."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300)


def test_more_than_one_gpu_is_refused():
    proc = run("--gpus", "2", "--steps", "1", "--warmup", "0")
    assert proc.returncode == 2
    lines = [l for l in (proc.stdout + proc.stderr).splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable(tmp_path):
    """Without a checkout of the reference to compile, the arm prints one line that says so and exits 0."""
    proc = run("--impl", "reference", "--reference-dir", str(tmp_path / "nothing_here"))
    assert proc.returncode == 0
    record = json.loads(proc.stdout.strip().splitlines()[-1])
    assert record["impl"] == "reference" and "\n" not in record["unavailable"] and len(record["unavailable"]) > 10
