"""What bench.py answers without a GPU: the reference arm and a request for several GPUs."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True,
                          text=True, timeout=120)


def test_reference_arm_says_why_it_is_unavailable():
    out = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3")
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_more_than_one_gpu_is_one_line_and_exit_code_two():
    out = _run("--gpus", "2", "--steps", "2", "--warmup", "3")
    assert out.returncode == 2
    assert len(out.stdout.strip().splitlines()) == 1 and "one GPU" in out.stdout
