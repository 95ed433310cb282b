"""A model put together from parts: embedding, blocks in a given order, head.

Reference (train/model.py:220-244): ``embed -> blocks -> final_norm -> lm_head``
with ``lm_head.weight`` being ``embed.weight`` when tied (train/model.py:228-229).
Here the order in which blocks run is a list of calls: a call names a block
(the same block may be called twice) and the cache slot it uses; a call may
read the slot an earlier call filled instead of owning one.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import CacheHandle, Part, ResidualStream, StepContext, TensorSpec


@dataclass(frozen=True)
class LayerCall:
    layer: int                    # index into ComposedModel.blocks
    cache_slot: Optional[int]     # index into ComposedModel.cache_specs()
    writes: bool = True           # False: reads a slot an earlier call filled


class TokenEmbedding(Part):
    """``x[t] = E[token[t]]``; no scaling, no position term (train/model.py:239)."""

    decode_capturable = prompt_capturable = True

    def __init__(self, vocab_size: int, d_model: int):
        self.vocab_size, self.d_model = int(vocab_size), int(d_model)
        self.weight = None

    def tensor_specs(self) -> dict:
        return {"weight": TensorSpec((self.vocab_size, self.d_model))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors["weight"].contiguous()

    def forward(self, step: StepContext):
        rt = self.runtime
        x = rt.buffer("residual", (step.n_tokens, self.d_model), rt.residual_dtype)
        rt.ops.embed(step.token_ids, self.weight, x, self.vocab_size)
        return x


class OutputHead(Part):
    """``logits = h @ W^T`` in float32; W is the embedding table when tied."""

    decode_capturable = prompt_capturable = True

    def __init__(self, vocab_size: int, d_model: int, tied_to: Optional[TokenEmbedding]):
        self.vocab_size, self.d_model = int(vocab_size), int(d_model)
        self.tied_to = tied_to
        self.weight = None

    def tensor_specs(self) -> dict:
        if self.tied_to is not None:
            return {}
        return {"weight": TensorSpec((self.vocab_size, self.d_model))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        w = self.tied_to.weight if self.tied_to is not None else tensors["weight"]
        self.weight = runtime.ops.prepare_weight(w)

    def forward(self, h, n_rows: int):
        rt = self.runtime
        logits = rt.buffer("logits", (n_rows, self.vocab_size), rt.logits_dtype)
        rt.ops.linear(h, self.weight, logits)
        return logits


class ComposedModel:
    """Embedding, blocks, the list of calls, final norm and output head."""

    def __init__(self, config, embedding: TokenEmbedding, blocks: list,
                 calls: list, final_norm, head: OutputHead,
                 names=("embed", "blocks", "final_norm", "lm_head"), aliases=None):
        self.config = config
        self._aliases = aliases          # callable: tensor name -> other names a file may use
        self.embedding, self.blocks, self.calls = embedding, list(blocks), list(calls)
        self.final_norm, self.head = final_norm, head
        self.names = tuple(names)
        self.runtime = None
        # one cache spec per slot, taken from the block of the call that owns it
        self._slot_specs = []
        for call in self.calls:
            if call.cache_slot is None:
                continue
            if call.writes:
                if call.cache_slot != len(self._slot_specs):
                    raise ValueError("cache slots must be numbered in call order")
                self._slot_specs.append(self.blocks[call.layer].cache_spec())
            elif not (0 <= call.cache_slot < len(self._slot_specs)):
                raise ValueError("a call reads a cache slot no earlier call owns")

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> dict:
        e, b, f, h = self.names
        out = {f"{e}.{n}": s for n, s in self.embedding.tensor_specs().items()}
        for i, blk in enumerate(self.blocks):
            for n, s in blk.tensor_specs().items():
                out[f"{b}.{i}.{n}"] = s
        out.update({f"{f}.{n}": s for n, s in self.final_norm.tensor_specs().items()})
        out.update({f"{h}.{n}": s for n, s in self.head.tensor_specs().items()})
        return out

    def name_aliases(self) -> dict:
        """For the names of ``tensor_specs`` and ``tied_names``: other spellings a
        weight file may use for the same tensor (the architecture's builder says which)."""
        if self._aliases is None:
            return {}
        names = list(self.tensor_specs()) + list(self.tied_names())
        return {n: a for n in names if (a := list(self._aliases(n)))}

    def tied_names(self) -> dict:
        """Names a file may hold although the model takes them from another."""
        e, _, _, h = self.names
        if self.head.tied_to is not None:
            return {f"{h}.weight": f"{e}.weight"}
        return {}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        e, b, f, h = self.names

        def sub(prefix):
            return {n[len(prefix) + 1:]: t for n, t in tensors.items()
                    if n.startswith(prefix + ".")}

        self.embedding.bind(sub(e), runtime)
        for i, blk in enumerate(self.blocks):
            blk.bind(sub(f"{b}.{i}"), runtime)
        self.final_norm.bind(sub(f), runtime)
        self.head.bind(sub(h), runtime)

    # -------------------------------------------------------------------- cache
    def cache_specs(self) -> list:
        return list(self._slot_specs)

    # ------------------------------------------------------------------- graphs
    def _all_parts(self) -> list:
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    @property
    def decode_capturable(self) -> bool:
        """Whether a step of single decoded tokens may be replayed from a CUDA graph:
        only if every part says so (``Part.decode_capturable``)."""
        return all(getattr(p, "decode_capturable", False) for p in self._all_parts())

    @property
    def prompt_capturable(self) -> bool:
        """The same for a step of any shape (``Part.prompt_capturable``)."""
        return all(getattr(p, "prompt_capturable", False) for p in self._all_parts())

    def decode_graph_key(self, step: StepContext) -> tuple:
        """What the parts add to the key of a decode step's graph, without repeats."""
        seen = []
        for p in self._all_parts():
            k = p.decode_graph_key(step)
            if k and k not in seen:
                seen.append(k)
        return tuple(seen)

    # ------------------------------------------------------------------ forward
    def forward(self, step: StepContext, handles: list):
        """Run the step's tokens; float32 logits [n_out, vocab] at ``out_rows``."""
        self.runtime.ops.begin_step(step.n_tokens)
        stream = ResidualStream(self.embedding.forward(step))
        none = CacheHandle()
        for call in self.calls:
            handle = none
            if call.cache_slot is not None:
                handle = handles[call.cache_slot]
                if not call.writes:
                    handle = handle.reader()
            self.blocks[call.layer].forward(stream, step, handle)
        if step.n_out == 0:
            stream.drop_pending()
            return None
        h = self.final_norm.forward(stream, rows=step.out_rows, n_rows=step.n_out)
        return self.head.forward(h, step.n_out)
