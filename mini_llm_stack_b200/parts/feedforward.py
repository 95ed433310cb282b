"""Dense SwiGLU feed-forward.

Reference (train/model.py:127-135): ``w_down(silu(w_gate x) * (w_up x))`` with
``silu(z) = z * sigmoid(z)``, no biases.  Gate and up share one projection
here (rows [gate | up]); ``silu(gate) * up`` is computed in float32.
"""

from __future__ import annotations

import torch

from .base import FeedForward, StepContext, TensorSpec


class SwiGLUFeedForward(FeedForward):
    def __init__(self, d_model: int, intermediate_size: int):
        self.d_model, self.intermediate_size = int(d_model), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> dict:
        d, i = self.d_model, self.intermediate_size
        return {
            "w_gate.weight": TensorSpec((i, d)),
            "w_up.weight": TensorSpec((i, d)),
            "w_down.weight": TensorSpec((d, i)),
        }

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        parts = [tensors["w_gate.weight"], tensors["w_up.weight"]]
        if parts[0].dtype != parts[1].dtype:
            parts = [p.float() for p in parts]
        self.w_gate_up = runtime.ops.prepare_weight(torch.cat(parts, dim=0))
        self.w_down = runtime.ops.prepare_weight(tensors["w_down.weight"])

    def forward(self, h, step: StepContext):
        rt = self.runtime
        t = h.shape[0]
        i = self.intermediate_size
        gu = rt.buffer("gate_up", (t, 2 * i), rt.act_dtype)
        rt.ops.linear(h, self.w_gate_up, gu)
        act = rt.buffer("ffn_act", (t, i), rt.act_dtype)
        rt.ops.swiglu(gu, act)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        rt.ops.linear(act, self.w_down, delta)
        return delta
