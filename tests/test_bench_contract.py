"""What bench.py promises without a GPU: more than one GPU is refused with one line and exit code 2, and the
reference arm answers with exit code 0 and ONE JSON line marked `"impl": "reference"` -- either a measurement
(`value`) or the reason why there is none (`unavailable`)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused():
    proc = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert proc.returncode == 2
    assert len(proc.stdout.strip().splitlines()) == 1 and "one GPU" in proc.stdout


def test_reference_arm_answers_with_a_measurement_or_a_reason():
    proc = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert proc.returncode == 0
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert isinstance(line["unavailable"], str) and len(line["unavailable"].splitlines()) == 1 and line["unavailable"]
    else:
        assert line["value"] > 0 and line["metric"] and line["config"]
