"""Compare the plain implementation with the reference's own model, once.

Run on a machine that has the reference checked out:

    python tests/golden/make_golden.py /path/to/mini-llm-stack

For tiny-A and tiny-B it draws the weights with the engine's seeded generator,
loads them into the reference's ``train.model.Transformer`` on the CPU and
checks that ``tests/plain_llama.py`` gives the same logits.  The reference is
all-MHA (train/model.py:79-82), so grouped keys and values are loaded with
every kv head's rows repeated for its group, which is the same function; its
feed-forward width comes from ``ffn_mult`` (train/config.py:32-35), so the
block's ``mlp`` is rebuilt with the wanted width (``SwiGLU(d, hidden)``,
train/model.py:128).  The logits of a fixed token sequence are then written to
``tests/golden/tiny_<X>.json``; ``tests/test_plain.py`` checks the plain
implementation against these files wherever the tests run.
"""

import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

from tiny_configs import CONFIGS, NORM_STD, plain_cfg          # noqa: E402
import plain_llama as P                                        # noqa: E402
from mini_llm_stack_b200.config import config_from_dict        # noqa: E402
from mini_llm_stack_b200.weights import random_tensors         # noqa: E402

SEED = 20240607
TOKENS = {"A": [(7 * i * i + 3 * i + 1) % 256 for i in range(29)],
          "B": [(5 * i * i + i + 2) % 97 for i in range(41)]}


def reference_logits(ref_root, cfg, w, tokens):
    sys.path.insert(0, str(ref_root))
    from train.config import ModelConfig
    from train.model import SwiGLU, Transformer

    H, Hkv, hd, d = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["d_model"]
    assert d == H * hd, "the reference has head_dim = d_model / n_heads"
    mc = ModelConfig(vocab_size=cfg["vocab_size"], d_model=d, n_layers=cfg["n_layers"],
                     n_heads=H, max_seq_len=cfg["max_seq_len"], rope_theta=cfg["rope_theta"],
                     norm_eps=cfg["norm_eps"], tie_embeddings=cfg["tie_embeddings"])
    model = Transformer(mc).eval()
    G = H // Hkv

    def expand(t):      # [Hkv*hd, d] -> [H*hd, d], kv head h//G for q head h
        return t.view(Hkv, hd, d).repeat_interleave(G, dim=0).reshape(H * hd, d)

    with torch.no_grad():
        model.embed.weight.copy_(w["embed.weight"])
        if not cfg["tie_embeddings"]:
            model.lm_head.weight.copy_(w["lm_head.weight"])
        model.final_norm.weight.copy_(w["final_norm.weight"])
        for i, blk in enumerate(model.blocks):
            p = f"blocks.{i}"
            blk.mlp = SwiGLU(d, cfg["intermediate_size"])
            blk.attn_norm.weight.copy_(w[f"{p}.attn_norm.weight"])
            blk.mlp_norm.weight.copy_(w[f"{p}.mlp_norm.weight"])
            blk.attn.wq.weight.copy_(w[f"{p}.attn.wq.weight"])
            blk.attn.wk.weight.copy_(expand(w[f"{p}.attn.wk.weight"]))
            blk.attn.wv.weight.copy_(expand(w[f"{p}.attn.wv.weight"]))
            blk.attn.wo.weight.copy_(w[f"{p}.attn.wo.weight"])
            blk.mlp.w_gate.weight.copy_(w[f"{p}.mlp.w_gate.weight"])
            blk.mlp.w_up.weight.copy_(w[f"{p}.mlp.w_up.weight"])
            blk.mlp.w_down.weight.copy_(w[f"{p}.mlp.w_down.weight"])
        return model(torch.tensor([tokens]))[0].float()


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/mini-llm-stack")
    ref_root = Path(sys.argv[1])
    for key in ("A", "B"):
        raw = CONFIGS[key]
        cfg = config_from_dict(dict(raw, dtype="float32"))
        w = dict(random_tensors(cfg, SEED, NORM_STD[key]))
        ours = P.plain_forward(w, plain_cfg(raw), TOKENS[key])
        ref = reference_logits(ref_root, plain_cfg(raw), w, TOKENS[key])
        err = (ours - ref).abs().max().item()
        print(f"tiny-{key}: plain vs reference max abs difference {err:.3e} "
              f"(logits up to {ref.abs().max().item():.3f})")
        assert err < 2e-5, "the plain implementation does not follow the reference"
        out = {"config": key, "seed": SEED, "norm_std": NORM_STD[key], "tokens": TOKENS[key],
               "max_abs_diff_vs_reference": err,
               "rows": [0, len(TOKENS[key]) // 2, len(TOKENS[key]) - 1],
               "logits": [[round(float(v), 7) for v in ref[r]]
                          for r in (0, len(TOKENS[key]) // 2, len(TOKENS[key]) - 1)]}
        with open(HERE / f"tiny_{key}.json", "w") as fh:
            json.dump(out, fh)
            fh.write("\n")


if __name__ == "__main__":
    main()
