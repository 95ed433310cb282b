"""One layer at the Llama-3-8B layer sizes against the plain implementation.

The tiny configurations never reach the paths that large sizes take: several
waves of GEMM tiles, split-K in the weight-major orientation, the tcgen05
attention kernel with head 128 and four query heads a kv head, context splits in
decode attention.  One layer with a small vocabulary keeps the plain
implementation on the CPU affordable.
"""

import pytest
import torch

from engine_helpers import Replayer, assert_close, plain_logits, tokens_for
from mini_llm_stack_b200.config import config_from_dict
from mini_llm_stack_b200.weights import write_random_model
from safetensors.torch import load_file
from tiny_configs import plain_cfg

pytestmark = pytest.mark.gpu

BIG = dict(architecture="llama_dense", vocab_size=1000, d_model=4096, n_layers=1, n_heads=32,
           n_kv_heads=8, head_dim=128, intermediate_size=14336, max_seq_len=1024,
           rope_theta=500000.0, norm_eps=1e-5, tie_embeddings=False)


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("big")
    cfg = config_from_dict(dict(BIG, dtype="bfloat16"))
    write_random_model(tmp / "m", cfg, seed=4, norm_std=0.1)
    w = {n: t.float().clone() for n, t in load_file(str(tmp / "m" / "model.safetensors")).items()}
    return tmp / "m", plain_cfg(BIG), w


def test_prompt_portions_and_decoded_tokens_at_full_layer_size(big):
    folder, cfg, w = big
    n = 330
    toks = {"a": tokens_for(1000, n, 1), "b": tokens_for(1000, 70, 2)}
    rp = Replayer(folder, "bfloat16", num_blocks=40)
    rp.step([("a", 200)], toks)                          # a prompt portion: tcgen05 attention
    rp.step([("a", 98), ("b", 64)], toks)                # two portions in one step
    for _ in range(6):
        rp.step([("a", 1), ("b", 1)], toks)              # decoded tokens: split attention, swap GEMM
    rp.step([("a", 26)], toks, end=["a", "b"])
    want_a = plain_logits(w, cfg, toks["a"], "bfloat16")
    want_b = plain_logits(w, cfg, toks["b"], "bfloat16")
    assert_close(rp.logits("a"), want_a, "bfloat16", "full-size layer, request a")
    assert_close(rp.logits("b"), want_b, "bfloat16", "full-size layer, request b")


def test_own_gemm_everywhere_gives_the_same_logits(big, monkeypatch):
    folder, cfg, w = big
    toks = {"a": tokens_for(1000, 150, 3)}
    monkeypatch.setenv("MLS_B200_GEMM", "tcgen05")
    rp = Replayer(folder, "bfloat16", num_blocks=16)
    assert rp.model.runtime.ops.gemm_impl == "tcgen05"
    rp.step([("a", 140)], toks)
    for _ in range(10):
        rp.step([("a", 1)], toks)
    assert rp.model.runtime.ops.library_launches == 0    # no product went to the library
    assert_close(rp.logits("a"), plain_logits(w, cfg, toks["a"], "bfloat16"), "bfloat16",
                 "tcgen05 GEMM for every product")


def test_chained_launches_do_not_change_a_bit(big):
    """Kernels that start under their predecessors (and fetch weights and old keys
    before they wait) must give what plainly ordered launches give, every time: a
    kernel that read its input too early would show as a difference or as a run
    that differs from the next."""
    folder, cfg, w = big
    toks = {r: tokens_for(1000, 600, 5 + i) for i, r in enumerate("abc")}

    def run(chained):
        rp = Replayer(folder, "bfloat16", num_blocks=130)
        ops = rp.model.runtime.ops
        ops.CHAINED_UP_TO = 256 if chained else -1
        rp.step([("a", 500), ("b", 300)], toks)           # plain launches either way (many tokens)
        rp.step([("a", 40), ("b", 7), ("c", 100)], toks)  # a small mixed step
        for _ in range(30):
            rp.step([("a", 1), ("b", 1), ("c", 1)], toks)  # decoded tokens, graphs after the second
        assert ops._chained == chained
        return {r: rp.logits(r) for r in "abc"}

    plain = run(False)
    for _ in range(3):
        chained = run(True)
        for r in "abc":
            assert torch.equal(chained[r], plain[r]), f"request {r} differs under chained launches"
