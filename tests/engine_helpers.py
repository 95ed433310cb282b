"""Helpers of the GPU tests: model folders, replay in process, plain logits."""

from __future__ import annotations

import torch
from safetensors.torch import load_file

import plain_llama as P
from mini_llm_stack_b200.config import config_from_dict
from mini_llm_stack_b200.engine.batch import Entry
from mini_llm_stack_b200.engine.runner import ModelRunner, load_model
from mini_llm_stack_b200.weights import write_random_model
from tiny_configs import CONFIGS, NORM_STD, plain_cfg

RND = {"float32": P.ident, "bfloat16": P.to_bf16}

# Largest |engine - plain| allowed, as a fraction of the largest |logit| of the
# compared rows.  float32: sums in another order only.  bfloat16: the plain
# implementation rounds where the engine stores, so what is left is a value
# that falls on the other side of a rounding step here and there.
TOL = {"float32": 5e-6, "bfloat16": 1e-2}


def make_folder(tmp_path, key: str, dtype: str, seed: int = 7, patch=None):
    """A model folder for tiny config ``key`` stored in ``dtype``; returns
    (folder, plain config dict, float32 weights by name as the file holds them)."""
    raw = dict(CONFIGS[key], **(patch or {}))
    cfg = config_from_dict(dict(raw, dtype=dtype))
    folder = tmp_path / f"tiny_{key}_{dtype}"
    write_random_model(folder, cfg, seed, NORM_STD[key])
    w = {n: t.float().clone() for n, t in load_file(str(folder / "model.safetensors")).items()}
    return folder, plain_cfg(raw), w


def tokens_for(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class Replayer:
    """Feeds requests through a ``ModelRunner`` and keeps every row of logits."""

    def __init__(self, folder, dtype, num_blocks, block_size=16, max_requests=8):
        self.model = load_model(folder, dtype=dtype)
        self.runner = ModelRunner(self.model, num_blocks=num_blocks, block_size=block_size,
                                  max_requests=max_requests)
        self.fed = {}
        self.rows = {}

    def step(self, portions, tokens, end=()):
        """``portions``: [(id, n_tokens)]; every fed place is wanted."""
        entries = []
        for rid, n in portions:
            b = self.fed.get(rid, 0)
            entries.append(Entry(rid, tokens[rid][b:b + n], list(range(n))))
        self.runner.reserve(entries)
        logits = self.runner.step(entries).float().cpu()
        at = 0
        for (rid, n) in portions:
            self.rows.setdefault(rid, []).append(logits[at:at + n])
            self.fed[rid] = self.fed.get(rid, 0) + n
            at += n
        for rid in end:
            self.runner.release(rid)
        self.model.runtime.ops.check_status()
        self.runner.cache.check()

    def logits(self, rid):
        return torch.cat(self.rows[rid], dim=0)


def plain_logits(w, cfg, tokens, dtype):
    return P.plain_forward(w, cfg, tokens, RND[dtype])


def assert_close(got, want, dtype, what=""):
    scale = want.abs().max().item()
    err = (got - want).abs()
    worst = err.max().item()
    if worst > TOL[dtype] * scale:
        row = int(err.max(dim=1).values.argmax())
        raise AssertionError(
            f"{what}: max |difference| {worst:.3e} > {TOL[dtype]:.0e} * {scale:.3f}; "
            f"first wrong row {int((err.max(dim=1).values > TOL[dtype] * scale).nonzero()[0])}, "
            f"worst row {row}")
    return worst / max(scale, 1e-30)
