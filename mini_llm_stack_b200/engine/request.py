"""A request's record (the reference's ``Request``, serve/engine.py:36-50)."""

from __future__ import annotations

import time
from dataclasses import dataclass, field

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    req_id: int
    prompt: list
    max_new_tokens: int = 32
    eos_token: int | None = None
    temperature: float = 0.0
    seed: int = 0
    state: str = WAITING
    generated: list = field(default_factory=list)
    num_computed: int = 0              # tokens whose keys and values are in the cache
    preemptions: int = 0
    arrive_time: float = field(default_factory=time.perf_counter)
    first_token_time: float | None = None
    finish_time: float | None = None

    @property
    def tokens(self) -> list:
        return self.prompt + self.generated

    @property
    def n_tokens(self) -> int:
        return len(self.prompt) + len(self.generated)

    def token_slice(self, start: int, n: int) -> list:
        """``tokens[start:start + n]`` without building the whole list."""
        p = len(self.prompt)
        if start + n <= p:
            return self.prompt[start:start + n]
        if start >= p:
            return self.generated[start - p:start - p + n]
        return self.prompt[start:] + self.generated[:start + n - p]

    @property
    def remaining(self) -> int:
        """Tokens not yet run: the rest of the prompt, or the token sampled last."""
        return len(self.prompt) + len(self.generated) - self.num_computed
