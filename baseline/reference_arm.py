"""The reference arm of the benchmark: grenver/mini-llm-stack itself, unmodified.

Runs the reference's stock serving path (``serve.engine.Engine`` with
``use_kernels=True``: its Triton flash attention for prompts and its Triton
paged attention for decoding, ``nn.Linear`` for the products) through its own
public calls ``Engine(...)``, ``submit`` and ``step`` (serve/engine.py:163-185,
229-256) on a model built by its own ``Transformer(ModelConfig(...))``
(train/model.py:220-244), at the layer sizes of the Llama-3-8B shape, and prints
one JSON line with the keys of the engine's own line and ``"impl": "reference"``.

Nothing of this repository's package is imported here: no model, no kernel, no
engine.  The reference tree is pure Python without a setup.py or
pyproject.toml, so it cannot be pip-installed; it is used from a plain copy
under ``baseline/_ref`` (made by ``ensure_tree`` from the checkout beside this
repository when there is one).

One difference cannot be avoided: the reference's attention has as many key and
value heads as query heads (train/model.py:79-82), so the 8 kv heads of the
shape are held as 32 (each repeated for its group of four query heads: the same
function of the input, four times the cache bytes and a third more q/k/v
weights).  The line names it in ``config.kv_heads``.
"""

from __future__ import annotations

import json
import os
import shutil
import sys
import time
import traceback
from pathlib import Path

HERE = Path(__file__).resolve().parent
TREE = HERE / "_ref"
# where a checkout of the reference may lie: named by the environment, or beside this repository
SOURCES = tuple(Path(p) for p in (os.environ.get("MLS_REFERENCE_TREE"),
                                  HERE.parent.parent / "reference") if p)

SHAPE = dict(vocab_size=128256, d_model=4096, n_layers=32, n_heads=32, max_seq_len=8192,
             rope_theta=500000.0, norm_eps=1e-5, tie_embeddings=False, ffn_mult=5.25)
PAGE = 16
PREFILL_TOKENS = 2048


def ensure_tree() -> str | None:
    """Make sure ``baseline/_ref`` holds the reference; the reason if it cannot."""
    if (TREE / "serve" / "engine.py").is_file():
        return None
    for src in SOURCES:
        if (src / "serve" / "engine.py").is_file():
            try:
                shutil.copytree(src, TREE, dirs_exist_ok=True,
                                ignore=shutil.ignore_patterns(".git", "__pycache__", "results"))
                return None
            except OSError as exc:
                return f"copying the reference tree failed: {exc}"
    return ("no copy of grenver/mini-llm-stack under baseline/_ref and no checkout to copy it "
            "from (it has no setup.py or pyproject.toml, so pip cannot install it)")


def unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": " ".join(str(why).split())[:600]}


def run(steps: int, warmup: int, batch: int = 8, context: int = 8192, layers: int = 32,
        points: bool = True) -> dict:
    why = ensure_tree()
    if why:
        return unavailable(why)
    sys.path.insert(0, str(TREE))
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        from serve.engine import Engine
        from train.config import ModelConfig
        from train.model import Transformer
    except Exception as exc:                       # noqa: BLE001 (the text goes into the line)
        return unavailable(f"importing the reference failed: {type(exc).__name__}: {exc}")

    try:
        return _measure(torch, Engine, ModelConfig, Transformer, steps, warmup, batch, context,
                        layers, points)
    except Exception as exc:                       # noqa: BLE001
        tail = traceback.format_exc().strip().splitlines()[-3:]
        return unavailable(f"the reference's own serving path failed on this GPU: "
                           f"{type(exc).__name__}: {exc} | {' / '.join(tail)}")


def _measure(torch, Engine, ModelConfig, Transformer, steps, warmup, batch, context, layers,
             points) -> dict:
    dev = "cuda"
    mc = ModelConfig(**dict(SHAPE, n_layers=layers))
    assert mc.ffn_hidden == 14336 and mc.head_dim == 128
    torch.manual_seed(0)
    # built where it will run and in the type it will run in: the reference's own
    # constructor and initialisation, without 35 GB of float32 on the host first
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = Transformer(mc).eval()
    finally:
        torch.set_default_dtype(old)
    gen = torch.Generator().manual_seed(1)

    def rand_tokens(n):
        return torch.randint(0, mc.vocab_size, (n,), generator=gen).tolist()

    def sync_time(fn):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3

    def decode(b, ctx, n_warm, n_timed):
        """(device ms, wall ms, h2d bytes, d2h bytes) a step of ``b`` requests that end
        at ``ctx`` tokens, through ``Engine.step``."""
        max_new = n_warm + n_timed + 3
        blocks = b * (-(-ctx // PAGE)) + 8
        eng = Engine(model, num_blocks=blocks, block_size=PAGE, max_batch=b, use_kernels=True,
                     device=dev, dtype=torch.bfloat16)
        reqs = [eng.submit(rand_tokens(ctx - max_new), max_new_tokens=max_new) for _ in range(b)]
        eng.step()                                  # admits all: the prompts, one decoded token
        for _ in range(n_warm):
            eng.step()
        assert len(eng.running) == b
        n0 = sum(len(r.generated) for r in reqs)

        def timed():
            for _ in range(n_timed):
                eng.step()

        dev_ms, wall_ms = sync_time(timed)
        assert len(eng.running) == b
        assert sum(len(r.generated) for r in reqs) - n0 == n_timed * b
        # what Engine.step copies a step (serve/engine.py:121-127, serve/kv_cache.py:110-121):
        # token ids and positions as int64, every request's block table as int32, its length
        table = sum(4 * len(eng.cache.tables[r.req_id]) for r in reqs)
        h2d = 8 * b + 8 * b + table + 4 * b
        d2h = 8 * b                                 # int(argmax) per request
        del eng
        torch.cuda.empty_cache()
        return dev_ms / n_timed, wall_ms / n_timed, h2d, d2h

    def prefill_ms():
        eng = Engine(model, num_blocks=PREFILL_TOKENS // PAGE + 8, block_size=PAGE, max_batch=1,
                     use_kernels=True, device=dev, dtype=torch.bfloat16)
        times = []
        for i in range(7):
            eng.submit(rand_tokens(PREFILL_TOKENS), max_new_tokens=1)
            ms, _ = sync_time(eng.step)             # admit = prefill + arg max; then it is done
            assert not eng.running and not eng.waiting
            if i >= 2:
                times.append(ms)
        del eng
        torch.cuda.empty_cache()
        return sorted(times)[len(times) // 2]

    pf_ms = prefill_ms()
    ms, wall, h2d, d2h = decode(batch, context, warmup, steps)
    pts = {}
    if points:
        quick = max(4, steps // 4)
        pts["decode_b1"] = round(1e3 / decode(1, context, 3, quick)[0], 1)
        for b in (1, batch):
            pts[f"decode_b{b}_ctx1024"] = round(b * 1e3 / decode(b, 1024, 3, quick)[0], 1)
    return {
        "metric": "decode tok/s at batch 8, Llama-3-8B shape, context 8192 "
                  "(batch 1/64 in points; prefill tok/s at 2,048 tokens in prefill)",
        "value": round(batch * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference",
        "config": {"model": "llama-3-8b-shape", "layers": layers, "layers_of_config": 32,
                   "hidden": mc.d_model, "heads": mc.n_heads,
                   "kv_heads": "32 (8 expanded x4, same function: the reference has no grouped "
                               "queries)",
                   "head_dim": mc.head_dim, "intermediate": mc.ffn_hidden,
                   "vocab": mc.vocab_size, "global_batch": batch, "seq_len": context,
                   "page_size": PAGE, "weights": "random N(0,0.02)", "parallelism": "none",
                   "path": "serve.engine.Engine(use_kernels=True).step, Triton attention, "
                           "nn.Linear",
                   "device": torch.cuda.get_device_name(0)},
        "e2e": {"value": round(batch * 1e3 / wall, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "prefill": {"value": round(PREFILL_TOKENS / pf_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pf_ms, 3)},
        "points": pts,
    }


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--no-points", action="store_true")
    a = ap.parse_args()
    print(json.dumps(run(a.steps, a.warmup, a.batch, a.context, a.layers, not a.no_points)))
