"""Replay on the GPU against the plain implementation, in every way of cutting.

Each request alone and whole; most of it in one step and the last 32 tokens one
by one; in portions of changing size down to two tokens; and mixed, up to four
live requests, portions of some beside decoded tokens of others, with so few
pages that they are used again.  In float32 and in bfloat16, for five tiny
configurations: three with small heads, and two (D, E) whose heads of 64 and 128
send the bfloat16 runs through the tcgen05 / TMA attention kernels, the fused
gate-up product and the weight-major product that large models use.
"""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from engine_helpers import (Replayer, assert_close, make_folder, plain_logits, tokens_for)

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DTYPES = ["float32", "bfloat16"]
KEYS = ["A", "B", "C", "D", "E"]
LENGTHS = {"A": [5, 17, 33, 150], "B": [1, 9, 40, 77, 300], "C": [3, 64, 131, 260],
           "D": [2, 63, 129, 300, 515], "E": [1, 31, 130, 257, 600]}
BLOCKS = {"A": 24, "B": 24, "C": 24, "D": 40, "E": 40}      # pages for one request


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {(k, d): make_folder(tmp, k, d) for k in KEYS for d in DTYPES}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_each_request_alone_and_whole(folders, key, dtype):
    folder, cfg, w = folders[(key, dtype)]
    rp = Replayer(folder, dtype, num_blocks=BLOCKS[key])
    for i, n in enumerate(LENGTHS[key]):
        toks = {i: tokens_for(cfg["vocab_size"], n, 100 + i)}
        rp.step([(i, n)], toks, end=[i])
        assert_close(rp.logits(i), plain_logits(w, cfg, toks[i], dtype), dtype,
                     f"tiny-{key} {dtype} whole prompt of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_last_32_tokens_one_by_one(folders, key, dtype):
    folder, cfg, w = folders[(key, dtype)]
    n = {"A": 180, "B": 333, "C": 250, "D": 370, "E": 421}[key]
    toks = {"r": tokens_for(cfg["vocab_size"], n, 5)}
    rp = Replayer(folder, dtype, num_blocks=BLOCKS[key])
    rp.step([("r", n - 32)], toks)
    for _ in range(32):
        rp.step([("r", 1)], toks)
    assert_close(rp.logits("r"), plain_logits(w, cfg, toks["r"], dtype), dtype,
                 f"tiny-{key} {dtype} prompt then 32 decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_portions_of_changing_size(folders, key, dtype):
    folder, cfg, w = folders[(key, dtype)]
    sizes = [16, 7, 3, 2, 2, 5, 31, 2, 17, 64, 1, 2, 33, 9]
    if key in "DE":                # portions of more than one 128-row tile, and a long tail
        sizes = sizes + [130, 2, 70, 3, 129]
    n = sum(sizes)
    toks = {"r": tokens_for(cfg["vocab_size"], n, 6)}
    rp = Replayer(folder, dtype, num_blocks=BLOCKS[key])
    for s in sizes:
        rp.step([("r", s)], toks)
    assert_close(rp.logits("r"), plain_logits(w, cfg, toks["r"], dtype), dtype,
                 f"tiny-{key} {dtype} portions {sizes}")


def mixed_schedule(lens, portion=(13, 2, 29, 5, 2, 40, 3, 16)):
    """Up to four live requests; portions of some beside single tokens of others;
    finished requests give their pages to later ones."""
    ids = list(range(len(lens)))
    fed = {i: 0 for i in ids}
    waiting, live, steps = list(ids), [], []
    k = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        step, end = [], []
        for j, r in enumerate(live):
            left = lens[r] - fed[r]
            # the last 6 tokens of a request come one by one, the rest in portions;
            # one request a step sits out
            if (len(steps) + j) % 5 == 4 and len(live) > 1:
                continue
            n = 1 if left <= 6 else min(left - 6, portion[k % len(portion)])
            k += 1
            step.append((r, n))
            fed[r] += n
            if fed[r] == lens[r]:
                end.append(r)
        for r in end:
            live.remove(r)
        if step:
            steps.append((step, end))
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_mixed_with_pages_used_again(folders, key, dtype):
    folder, cfg, w = folders[(key, dtype)]
    lens = [70, 45, 9, 120, 33, 64, 17, 90, 2, 51]
    num_blocks = 16
    portion = (13, 2, 29, 5, 2, 40, 3, 16)
    if key in "DE":                # longer requests, portions of several query tiles
        lens = [200, 45, 9, 310, 33, 140, 17, 190, 2, 151]
        num_blocks = 36
        portion = (13, 2, 150, 5, 2, 40, 67, 16)
    toks = {i: tokens_for(cfg["vocab_size"], n, 40 + i) for i, n in enumerate(lens)}
    steps = mixed_schedule(lens, portion)
    # the pool holds what four live requests need at worst, rounded up to pages of
    # 16: far fewer pages than all requests together, so pages are used again
    rp = Replayer(folder, dtype, num_blocks=num_blocks)
    seen = set()
    reused = False
    for step, end in steps:
        rp.step(step, toks, end=end)
        for r, _ in step:
            if rp.runner.cache.has(r):
                pages = set(rp.runner.cache.pages_of(r))
                reused |= bool(pages & seen)
        for r in end:
            pass
        seen |= {p for r in rp.runner.cache.live() for p in rp.runner.cache.pages_of(r)}
    assert max(len(s) for s, _ in steps) == 4
    assert sum(lens) > num_blocks * 16 and reused
    for i in toks:
        assert_close(rp.logits(i), plain_logits(w, cfg, toks[i], dtype), dtype,
                     f"tiny-{key} {dtype} mixed, request {i}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_does_not_change_float32_bits_or_bf16_much(folders, dtype):
    """In float32 every kernel sums in an order that depends on the token's own
    position only, so whole, decoded and chunked runs agree bit for bit."""
    folder, cfg, w = folders[("B", dtype)]
    n = 140
    toks = {"r": tokens_for(cfg["vocab_size"], n, 9)}
    whole = Replayer(folder, dtype, num_blocks=16)
    whole.step([("r", n)], toks)
    cut = Replayer(folder, dtype, num_blocks=16)
    for s in [50, 2, 37, 1, 1, 1, 48]:
        cut.step([("r", s)], toks)
    a, b = whole.logits("r"), cut.logits("r")
    if dtype == "float32":
        assert torch.equal(a, b)
    else:
        assert_close(a, b, dtype, "bfloat16 whole against cut")


def test_folder_stored_in_32_bits_run_in_bfloat16(tmp_path):
    """Tensors stored in 32 bits stay 32-bit in a bfloat16 run: the activations are
    bfloat16, the products with those weights true float32."""
    folder, cfg, w = make_folder(tmp_path, "B", "float32", seed=11)
    n = 90
    toks = {"r": tokens_for(cfg["vocab_size"], n, 8)}
    rp = Replayer(folder, "bfloat16", num_blocks=16)
    model = rp.model
    assert model.blocks[0].ffn.w_down.dtype == torch.float32
    assert model.blocks[0].mixer.wqkv.dtype == torch.float32
    assert model.runtime.act_dtype == torch.bfloat16
    rp.step([("r", 60)], toks)
    for _ in range(30):
        rp.step([("r", 1)], toks)
    assert_close(rp.logits("r"), plain_logits(w, cfg, toks["r"], "bfloat16"), "bfloat16",
                 "float32 weights, bfloat16 activations")


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(folders, tmp_path, dtype):
    """The program itself: JSON lines in, ``done`` lines and .f32 files out."""
    folder, cfg, w = folders[("A", dtype)]
    t = {"a": tokens_for(256, 70, 1), "b": tokens_for(256, 20, 2), "c": tokens_for(256, 64, 3)}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": t["a"][:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": t["a"][40:68], "want": []},
                                {"id": "b", "tokens": t["b"][:18], "want": [17]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": t["b"][18:19], "want": [0]},
                                {"id": "a", "tokens": t["a"][68:70], "want": [0, 1]}],
         "end": ["a"]},
        {"step": 3, "entries": [{"id": "c", "tokens": t["c"], "want": [63]},
                                {"id": "b", "tokens": t["b"][19:20], "want": [0]}],
         "end": ["b", "c"]},
    ]
    out = tmp_path / f"out_{dtype}"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype",
         dtype, "--out", str(out), "--max-tokens", "192"],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    plain = {k: plain_logits(w, cfg, v, dtype) for k, v in t.items()}
    want = {0: [plain["a"][0], plain["a"][39]], 1: [plain["b"][17]],
            2: [plain["b"][18], plain["a"][68], plain["a"][69]],
            3: [plain["c"][63], plain["b"][19]]}
    for s, rows in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(len(rows), 256))
        assert_close(got, torch.stack(rows), dtype, f"trace_run step {s}")
