"""RMS norm with a learned weight.

Reference formula (train/model.py:29-33): ``xf = x.float()``;
``y = xf * rsqrt(mean(xf**2, -1) + eps)``; ``out = (y * w.float()).to(x.dtype)``.
eps sits inside the square root, added to the mean; the weight multiplies after
the normalisation; no bias.  All of it runs in float32 with one rounding at the
end.  The residual stream's pending addend is added in the same pass.
"""

from __future__ import annotations

from .base import Norm, ResidualStream, TensorSpec


class RMSNorm(Norm):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    def __init__(self, dim: int, eps: float):
        self.dim = int(dim)
        self.eps = float(eps)
        self.weight = None

    def tensor_specs(self) -> dict:
        return {"weight": TensorSpec((self.dim,), kind="vector", init="ones")}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors["weight"].contiguous()

    def forward(self, stream: ResidualStream, rows=None, n_rows: int = 0):
        """Add the pending delta into the stream, return the normalised rows.

        With ``rows`` (int32 row indices) only those rows are read, summed and
        normalised: the output is [n_rows, dim] and the stream itself is left
        as it was.
        """
        rt = self.runtime
        delta = stream.take_pending()
        if rows is None:
            t = stream.x.shape[0]
            h = rt.buffer("normed", (t, self.dim), rt.act_dtype)
            rt.ops.add_rmsnorm(stream.x, delta, self.weight, self.eps, h)
        else:
            h = rt.buffer("normed_rows", (n_rows, self.dim), rt.act_dtype)
            rt.ops.gather_add_rmsnorm(stream.x, delta, rows, n_rows, self.weight,
                                      self.eps, h)
        return h
