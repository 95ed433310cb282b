"""Trace replay: feed given token ids through the model step by step, write logits.

Nothing is sampled.  The program drives the same model, step function, cache
and kernels that generation uses: ``load_model`` -> ``ModelRunner.step``.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input holds one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are wanted; all entries of a step run as one batch.  ``end``: requests
that are finished after this step; their pages go back to the pool.  For a step
that wants something, ``OUT/<step>.f32`` receives the logits as little-endian
float32 [wanted, vocab], in the order of the entries and of ``want``.  After
every step the line ``done <step>`` is printed and flushed.

``--max-tokens`` is the most tokens live requests hold at any time, each
request's count rounded up to a multiple of 64; the page pool is made for
exactly that many, so pages are used again.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE_SIZE = 16          # divides 64, so the rounding of --max-tokens is kept
MAX_LIVE = 8            # state slots; a trace holds up to four live requests


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch

    from .batch import Entry
    from .runner import ModelRunner, load_model

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    model = load_model(args.model, dtype=args.dtype, device=args.device)
    num_blocks = max(1, (args.max_tokens + PAGE_SIZE - 1) // PAGE_SIZE)
    runner = ModelRunner(model, num_blocks=num_blocks, block_size=PAGE_SIZE,
                         max_requests=MAX_LIVE)
    ops = model.runtime.ops

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step_no = rec["step"]
        entries = [Entry(owner=e["id"], tokens=list(e["tokens"]), want=list(e.get("want", [])))
                   for e in rec.get("entries", [])]
        if entries:
            runner.reserve(entries)
            logits = runner.step(entries)
            if logits is not None:
                host = logits.to("cpu", torch.float32).contiguous().numpy()
                host.astype("<f4", copy=False).tofile(out_dir / f"{step_no}.f32")
            ops.check_status()
        for owner in rec.get("end", []):
            runner.release(owner)
        print(f"done {step_no}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
