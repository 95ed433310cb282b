"""The arrangement of a layer's parts: the pre-norm residual block.

Reference (train/model.py:200-217): ``x = x + mixer(norm_a(x))``;
``x = x + feed_forward(norm_b(x))``.  The block owns the order and the names
its parts' tensors carry in a weight file; the parts own the math.
"""

from __future__ import annotations

from .base import CacheHandle, Part, ResidualStream, StepContext


class PreNormBlock(Part):
    def __init__(self, mixer_norm, mixer, ffn_norm, ffn,
                 names=("attn_norm", "attn", "mlp_norm", "mlp")):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.ffn_norm, self.ffn = ffn_norm, ffn
        self.names = tuple(names)

    def _named_parts(self):
        return list(zip(self.names,
                        (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)))

    def tensor_specs(self) -> dict:
        out = {}
        for prefix, part in self._named_parts():
            for n, s in part.tensor_specs().items():
                out[f"{prefix}.{n}"] = s
        return out

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        for prefix, part in self._named_parts():
            own = {n[len(prefix) + 1:]: t for n, t in tensors.items()
                   if n.startswith(prefix + ".")}
            part.bind(own, runtime)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def decode_capturable(self) -> bool:
        return all(getattr(p, "decode_capturable", False) for _, p in self._named_parts())

    @property
    def prompt_capturable(self) -> bool:
        return all(getattr(p, "prompt_capturable", False) for _, p in self._named_parts())

    def decode_graph_key(self, step: StepContext) -> tuple:
        return tuple(k for _, p in self._named_parts() if (k := p.decode_graph_key(step)))

    def forward(self, stream: ResidualStream, step: StepContext,
                cache: CacheHandle) -> None:
        h = self.mixer_norm.forward(stream)
        stream.push(self.mixer.forward(h, step, cache))
        h = self.ffn_norm.forward(stream)
        stream.push(self.ffn.forward(h, step))
