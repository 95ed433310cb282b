"""What bench.py hands to the reference arm (no GPU needed): the arm must get the headline
shape's sizes as integers whatever flags the driver leaves out."""

import importlib.util
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_gets_whole_numbers(monkeypatch, capsys):
    bench = load_bench()
    seen = {}

    class FakeArm:
        @staticmethod
        def run(steps, warmup, batch, context, layers, points):
            seen.update(steps=steps, warmup=warmup, batch=batch, context=context, layers=layers,
                        points=points)
            return {"impl": "reference", "unavailable": "a stand-in"}

        @staticmethod
        def unavailable(why):
            return {"impl": "reference", "unavailable": why}

    class FakeSpec:
        class loader:
            @staticmethod
            def exec_module(mod):
                mod.run, mod.unavailable = FakeArm.run, FakeArm.unavailable

    monkeypatch.setattr(importlib.util, "spec_from_file_location", lambda *a, **k: FakeSpec)
    monkeypatch.setattr(importlib.util, "module_from_spec", lambda spec: type(sys)("fake_arm"))
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--gpus", "1", "--steps", "5",
                                      "--warmup", "3"])
    assert bench.main() == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert seen["layers"] == 32 and seen["context"] == 8192 and seen["batch"] == 8
    assert all(isinstance(seen[k], int) for k in ("steps", "warmup", "batch", "context", "layers"))


def test_more_than_one_gpu_is_refused_with_one_line(monkeypatch, capsys):
    bench = load_bench()
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "2"])
    assert bench.main() == 2
    assert "one GPU" in capsys.readouterr().out
