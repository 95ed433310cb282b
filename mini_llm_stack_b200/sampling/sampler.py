"""Greedy and temperature sampling.

The reference's engine takes ``int(logits.argmax(-1))`` (serve/engine.py:187-188);
its ``generate_naive`` draws from ``softmax(logits / temperature)`` with
``torch.multinomial`` on the global generator when ``temperature > 0``
(train/model.py:262-266).  It has no top-k or top-p, so neither exists here.

A draw here needs no generator state: the uniform number of a draw is a pure
function of (seed, request key, index of the output token), so a request
samples the same tokens whatever else is in its batch and however often it was
preempted and recomputed.  The token is the first index whose cumulative
probability exceeds that number (``sampling.cu``).
"""

from __future__ import annotations

import torch

_MASK = (1 << 64) - 1


def uniform_for(seed: int, request: int, index: int) -> float:
    """Uniform number in [0, 1) with 24 bits, from splitmix64's finaliser over a
    linear mix of the three keys."""
    z = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9
         + index * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


class Sampler:
    """Picks one token per row of float32 logits on the device."""

    def __init__(self, runtime, max_rows: int = 64):
        self.runtime = runtime
        self._cap = 0
        self._copied = torch.cuda.Event()        # the tokens of the last launch are on the host
        # the kernels' status word travels with the tokens: a kernel that refused its
        # input or gave up a wait is known in the step that ran it
        self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._grow(max_rows)

    def _grow(self, n: int) -> None:
        if n <= self._cap:
            return
        dev = self.runtime.device
        self._cap = max(n, 2 * self._cap)
        self._host = torch.empty((2, self._cap), dtype=torch.float32, pin_memory=True)
        self._dev = torch.empty((2, self._cap), dtype=torch.float32, device=dev)
        self._out = torch.empty(self._cap, dtype=torch.int32, device=dev)
        self._out_host = torch.empty(self._cap, dtype=torch.int32, pin_memory=True)

    def sample(self, logits, temperatures: list, uniforms: list) -> list:
        """Tokens for ``logits [n, V]``; row i is greedy if ``temperatures[i] <= 0``."""
        return self.finish(self.launch(logits, temperatures, uniforms))

    def launch(self, logits, temperatures: list, uniforms: list) -> int:
        """Start sampling and the copy of the tokens to the host; no wait."""
        n = logits.shape[0]
        self._grow(n)
        ops = self.runtime.ops
        if any(t > 0 for t in temperatures):
            self._host[0, :n] = torch.tensor(temperatures, dtype=torch.float32)
            self._host[1, :n] = torch.tensor(uniforms, dtype=torch.float32)
            self._dev[:, :n].copy_(self._host[:, :n], non_blocking=True)
            ops.sample(logits, self._dev[0, :n], self._dev[1, :n], self._out)
        else:
            ops.sample(logits, None, None, self._out)
        self._out_host[:n].copy_(self._out[:n], non_blocking=True)
        self._status_host.copy_(ops.status, non_blocking=True)
        self._copied.record(torch.cuda.current_stream(self.runtime.device))
        return n

    def device_tokens(self, n: int):
        """The tokens of the last ``launch`` where the kernel wrote them (int32 [n] on
        the device): a next step may read them there before the host has them."""
        return self._out[:n]

    def finish(self, n: int) -> list:
        """Wait for the tokens of the last ``launch`` (not for work queued after it).
        Raises ``KernelError`` if a kernel up to that launch set the status word."""
        self._copied.synchronize()
        code = int(self._status_host[0])
        if code:
            self.runtime.ops.raise_for_status(code)
        return self._out_host[:n].tolist()
