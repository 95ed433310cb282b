"""Dense SwiGLU feed-forward.

Reference (train/model.py:127-135): ``w_down(silu(w_gate x) * (w_up x))`` with
``silu(z) = z * sigmoid(z)``, no biases.  Gate and up share one projection
here; ``silu(gate) * up`` is computed in float32, in the projection's own
epilogue where the tcgen05 kernel takes the sizes.
"""

from __future__ import annotations

import torch

from .base import FeedForward, StepContext, TensorSpec


class SwiGLUFeedForward(FeedForward):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

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
        ops = runtime.ops
        # one kernel for projection and activation where the tensor-core kernel takes
        # the sizes: its weight holds gate and up rows interleaved in blocks of 16
        self.fused = (parts[0].dtype == torch.bfloat16
                      and ops.can_fuse_swiglu(self.d_model, self.intermediate_size))
        if self.fused:
            self.w_gate_up = ops.prepare_weight(ops.interleave_gate_up(parts[0], parts[1]))
        else:
            self.w_gate_up = ops.prepare_weight(torch.cat(parts, dim=0))
        self.w_down = ops.prepare_weight(tensors["w_down.weight"])

    def forward(self, h, step: StepContext):
        rt = self.runtime
        t = h.shape[0]
        i = self.intermediate_size
        act = rt.buffer("ffn_act", (t, i), rt.act_dtype)
        if self.fused:
            rt.ops.linear_swiglu(h, self.w_gate_up, act)
        else:
            gu = rt.buffer("gate_up", (t, 2 * i), rt.act_dtype)
            rt.ops.linear(h, self.w_gate_up, gu)
            rt.ops.swiglu(gu, act)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(act, self.w_down, delta)
