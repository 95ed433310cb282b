"""Command line: ``python -m mini_llm_stack_b200.api chat -p "..."``.

The reference's ``chat`` (serve/api.py:72-104,135-148): ``-p/--prompt``
(required), ``--max-new 64``; it loads ``checkpoints/model.pt``, encodes the
prompt with the checkpoint's character table (unknown characters dropped, an
empty prompt becomes ``[0]``: serve/api.py:67-69), runs
``Engine(num_blocks=512, block_size=16)`` and prints ``'prompt' -> 'completion'``.
Its ``--quant``, ``--speculative``, ``train`` and ``serve`` belong to parts this
engine does not have.

Here the model comes from ``--model DIR`` (config.json + model.safetensors) or
from ``--random-weights CONFIG.json --seed N``; ``write-random`` stores such a
random model as a folder.  Text becomes tokens through ``itos.json`` in the
folder (a list of characters, the reference's table) or, for a vocabulary of
at least 256, through its UTF-8 bytes; ``--token-ids`` gives ids directly.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def _tables(folder, vocab_size: int):
    """(encode, decode) for a model folder."""
    itos_path = Path(folder) / "itos.json" if folder else None
    if itos_path is not None and itos_path.is_file():
        itos = json.loads(itos_path.read_text(encoding="utf-8"))
        stoi = {c: i for i, c in enumerate(itos)}

        def encode(text):
            toks = [stoi[c] for c in text if c in stoi]       # serve/api.py:68
            return toks or [0]                                # serve/api.py:69

        return encode, lambda ids: "".join(itos[i] for i in ids if 0 <= i < len(itos))
    if vocab_size >= 256:
        return (lambda text: list(text.encode("utf-8")) or [0],
                lambda ids: bytes(i for i in ids if i < 256).decode("utf-8", "replace"))
    return None, lambda ids: " ".join(str(i) for i in ids)


def cmd_chat(args) -> int:
    from .config.engine_options import EngineOptions
    from .config.model_config import ConfigError
    from .config.registry import config_from_dict
    from .engine.llm import LLM

    opts = EngineOptions(num_blocks=args.num_blocks, block_size=args.block_size,
                         max_batch=args.max_batch,
                         max_tokens_per_step=args.max_tokens_per_step,
                         chunk_size=args.chunk_size, dtype=args.dtype, device=args.device,
                         kv_dtype=args.kv_dtype, seed=args.sample_seed)
    if args.model:
        llm = LLM.from_folder(args.model, options=opts)
        folder = args.model
    elif args.random_weights:
        raw = json.loads(Path(args.random_weights).read_text())
        llm = LLM.from_random(config_from_dict(raw), seed=args.seed, options=opts)
        folder = None
    else:
        raise SystemExit("give --model DIR or --random-weights CONFIG.json")
    encode, decode = _tables(folder, llm.config.vocab_size)
    if args.token_ids:
        prompt = [int(x) for x in args.token_ids.split(",") if x.strip()]
        shown = args.token_ids
    else:
        if args.prompt is None:
            raise SystemExit("give -p/--prompt or --token-ids")
        if encode is None:
            raise ConfigError("this model has no character table (itos.json) and fewer "
                              "than 256 tokens: give --token-ids")
        prompt = encode(args.prompt)
        shown = args.prompt
    out = llm.generate([prompt], max_new_tokens=args.max_new, temperature=args.temperature,
                       eos=args.eos)[0]
    if args.token_ids:
        print(f"{shown!r} -> {','.join(str(t) for t in out)!r}")
    else:
        print(f"{shown!r} -> {decode(out)!r}")                # serve/api.py:104
    return 0


def cmd_write_random(args) -> int:
    from .config.registry import config_from_dict
    from .weights.random_init import write_random_model

    raw = json.loads(Path(args.config).read_text())
    cfg = config_from_dict(raw)
    write_random_model(args.out, cfg, args.seed, args.norm_std)
    print(f"wrote {args.out}/config.json and model.safetensors (seed {args.seed})")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mini_llm_stack_b200.api")
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("chat", help="generate a continuation")
    c.add_argument("-p", "--prompt")
    c.add_argument("--max-new", type=int, default=64)
    c.add_argument("--model", help="folder with config.json and model.safetensors")
    c.add_argument("--random-weights", metavar="CONFIG.json")
    c.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    c.add_argument("--token-ids", help="prompt as comma-separated token ids")
    c.add_argument("--temperature", type=float, default=0.0)
    c.add_argument("--sample-seed", type=int, default=0)
    c.add_argument("--eos", type=int, default=None)
    c.add_argument("--dtype", choices=["bfloat16", "float32"], default=None)
    c.add_argument("--kv-dtype", choices=["bfloat16", "float32"], default=None,
                   help="must equal the run's dtype (the cache is kept in it)")
    c.add_argument("--device", default="cuda:0")
    c.add_argument("--num-blocks", type=int, default=512)     # serve/api.py:92
    c.add_argument("--block-size", type=int, default=16)
    c.add_argument("--max-batch", type=int, default=16)
    c.add_argument("--max-tokens-per-step", type=int, default=2048)
    c.add_argument("--chunk-size", type=int, default=2048)
    w = sub.add_parser("write-random", help="write a model folder with random weights")
    w.add_argument("--config", required=True, metavar="CONFIG.json")
    w.add_argument("--out", required=True)
    w.add_argument("--seed", type=int, default=0)
    w.add_argument("--norm-std", type=float, default=0.0)
    args = ap.parse_args(argv)
    return {"chat": cmd_chat, "write-random": cmd_write_random}[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
