"""The plain implementation against the reference's own outputs (CPU).

``tests/golden/make_golden.py`` loaded the same seeded weights into the
reference's ``Transformer`` and stored three rows of its logits.
"""

import json
from pathlib import Path

import pytest
import torch

import plain_llama as P
from mini_llm_stack_b200.config import config_from_dict
from mini_llm_stack_b200.weights import random_tensors
from tiny_configs import CONFIGS, NORM_STD, plain_cfg

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("key", ["A", "B"])
def test_plain_forward_matches_reference_rows(key):
    g = json.loads((GOLDEN / f"tiny_{key}.json").read_text())
    cfg = config_from_dict(dict(CONFIGS[key], dtype="float32"))
    w = dict(random_tensors(cfg, g["seed"], g["norm_std"]))
    logits = P.plain_forward(w, plain_cfg(CONFIGS[key]), g["tokens"])
    want = torch.tensor(g["logits"])
    assert torch.allclose(logits[g["rows"]], want, rtol=0, atol=2e-6)


def test_causality_future_tokens_leave_past_logits():
    # the reference's own check (tests/test_model.py:37-47)
    cfg = config_from_dict(dict(CONFIGS["C"], dtype="float32"))
    w = dict(random_tensors(cfg, 5, NORM_STD["C"]))
    toks = [(3 * i + 1) % 301 for i in range(60)]
    a = P.plain_forward(w, plain_cfg(CONFIGS["C"]), toks)
    toks2 = list(toks)
    toks2[45] = (toks2[45] + 7) % 301
    b = P.plain_forward(w, plain_cfg(CONFIGS["C"]), toks2)
    assert torch.allclose(a[:45], b[:45], rtol=1e-5, atol=1e-5)
    assert not torch.allclose(a[45:], b[45:], rtol=1e-5, atol=1e-5)


def test_window_hides_far_keys():
    q = torch.randn(2, 6, 8)
    k = torch.randn(1, 6, 8)
    v = torch.randn(1, 6, 8)
    full = P.plain_attention(q, k, v, 0.3)
    win = P.plain_attention(q, k, v, 0.3, window=3)
    assert torch.allclose(full[:, :3], win[:, :3], atol=1e-6)   # first 3 queries see all
    again = P.plain_attention(q[:, 5:], k[:, 3:], v[:, 3:], 0.3)
    assert torch.allclose(win[:, 5:], again, atol=1e-6)         # last sees keys 3..5 only


def test_sampling_rule():
    logits = torch.tensor([0.0, 1.0, 3.0, 3.0, -2.0])
    assert P.plain_sample(logits, 0.0, 0.5) == 2               # first maximum
    p = torch.softmax(logits / 0.7, 0)
    cum = torch.cumsum(p, 0)
    for u in (0.0, 0.2, 0.5, 0.9, 0.999):
        want = int((cum > u).nonzero()[0])
        assert P.plain_sample(logits, 0.7, u) == want
    us = [P.uniform_for(3, r, i) for r in range(4) for i in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) == len(us)
    assert 0.35 < sum(us) / len(us) < 0.65
