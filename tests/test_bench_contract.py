"""bench.py's command line where it needs no GPU: more than one GPU is refused with one line and exit code 2, and the
reference arm answers with its one-line record and exit code 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300, cwd=ROOT)


def test_more_than_one_gpu_is_refused_in_one_line():
    done = _bench("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert done.returncode == 2
    lines = [ln for ln in done.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and "--gpus 2" in lines[0]


def test_reference_arm_prints_its_record():
    done = _bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert done.returncode == 0
    lines = [ln for ln in done.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference"
    assert ("unavailable" in record and "\n" not in record["unavailable"]) or "value" in record
