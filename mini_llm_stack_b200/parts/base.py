"""What every part of a layer is made of: tensor specs, cache specs, interfaces.

A layer is put together from a mixer (attention here), a feed-forward, norms
and a position encoding, arranged by a block.  The reference wires these as
fixed ``nn.Module`` attributes of ``Block`` (train/model.py:200-217); here each
is an object built from its own sizes and constants, so one model may use
different parts in different layers and no part knows which model it is in.

Interfaces
----------
Every part:
    tensor_specs() -> {local name: TensorSpec}    tensors it needs
    bind(tensors, runtime)                        receive them (local names)
Norm:
    forward(stream, rows=None) -> h               stream.settle + normalise
Mixer:
    cache_spec() -> PagedKV | FixedState | None   what it keeps per request
    forward(h, step, cache) -> delta [T, d_model]
FeedForward:
    forward(h, step) -> delta [T, d_model]
PositionEncoding (rotary kind):
    rotate_and_store(qkv, step, cache, n_heads, n_kv_heads, head_dim)
Block:
    forward(stream, step, cache)                  runs its parts in its order
"""

from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Optional

import torch


# ----------------------------------------------------------------------------
# tensors
# ----------------------------------------------------------------------------
@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part needs: its shape, what it is, and how it is drawn.

    kind: "matrix" | "vector" (floating) or "table" (integer, kept as int32).
    init: "normal" (N(0, 0.02^2), train/model.py:232-236), "ones" (norm
    weights, train/model.py:27) or "zeros".
    """
    shape: tuple
    kind: str = "matrix"
    init: str = "normal"


# ----------------------------------------------------------------------------
# what a mixer keeps per request
# ----------------------------------------------------------------------------
@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every token (or of the last ``window`` tokens)."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """Per-request state whose size does not grow with the sequence."""
    shape: tuple
    dtype: torch.dtype = torch.float32


# ----------------------------------------------------------------------------
# what a step hands to the parts
# ----------------------------------------------------------------------------
@dataclass
class GroupView:
    """One paged cache group as a step sees it (device tensors)."""
    block_table: torch.Tensor        # [R, max_blocks] int32, -1 where no page
    slot_map: torch.Tensor           # [T] int32: page * block_size + offset
    block_size: int
    max_blocks: int


@dataclass
class StepContext:
    """A batch of (request, its next tokens) as device arrays plus host facts.

    Token t belongs to request ``req_of_token[t]``; request r owns tokens
    ``cu_q[r] .. cu_q[r+1]`` and will hold ``ctx_len[r]`` tokens after this
    step, so its i-th token of this step sits at absolute position
    ``ctx_len[r] - q_len[r] + i`` (the reference's bottom-right alignment,
    train/model.py:64-68).
    """
    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor          # [T] int32
    positions: torch.Tensor          # [T] int32
    req_of_token: torch.Tensor       # [T] int32
    cu_q: torch.Tensor               # [R+1] int32
    ctx_len: torch.Tensor            # [R+1] int32: the requests', then the longest of them
    state_slot: torch.Tensor         # [R] int32
    out_rows: torch.Tensor           # [n_out] int32
    n_out: int
    groups: dict = field(default_factory=dict)     # group id -> GroupView
    # host-side copies, for launch decisions only
    q_lens: list = field(default_factory=list)
    ctx_lens: list = field(default_factory=list)
    max_q_len: int = 0
    max_ctx_len: int = 0
    attn_tiles: dict = field(default_factory=dict)  # scratch for mixers' metadata


@dataclass
class CacheHandle:
    """What one layer call may touch of the cache.

    paged: ``k_pool``/``v_pool`` [n_kv_heads, num_blocks, block_size, head_dim]
    of this call's member of its group, ``group`` the id into
    ``StepContext.groups``, ``writes`` False if the call only reads a cache an
    earlier call filled.  fixed: ``state`` [max_slots, *shape].
    """
    kind: str = "none"               # "paged" | "fixed" | "none"
    group: int = -1
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    writes: bool = True
    state: Optional[torch.Tensor] = None
    window: Optional[int] = None

    def reader(self) -> "CacheHandle":
        """The same cache for a call that only reads it."""
        return replace(self, writes=False)


class ResidualStream:
    """The residual sum, kept in float32, with one pending addend.

    ``push(delta)`` defers an addition; the next norm adds it while it reads the
    row anyway (the reference adds eagerly: train/model.py:212-216).  A delta is a
    tensor [T, d_model] or the kernels' ``SplitParts`` (a product left as the parts
    of a cut along K, which ``add_rmsnorm`` adds up; ``.float()`` gives the tensor).
    """

    def __init__(self, x: torch.Tensor):
        self.x = x                   # [T, d_model] float32
        self.pending = None

    def push(self, delta) -> None:
        if self.pending is not None:
            raise RuntimeError("a delta is already pending on the residual stream")
        self.pending = delta

    def take_pending(self):
        p, self.pending = self.pending, None
        return p

    def drop_pending(self) -> None:
        """Forget the pending delta (the rows it belongs to are not wanted)."""
        p = self.take_pending()
        if hasattr(p, "release"):
            p.release()


class Part:
    """Base of every part; sizes and constants are constructor arguments.

    Capture into a CUDA graph is a part's own business.  The step function replays a
    step of single decoded tokens from a graph only if every part of the model says
    ``decode_capturable`` (its ``forward`` then only launches work on the current
    stream: no wait for the device, no read of device memory by the host, no launch
    that depends on values computed on the device) and keys the graph by the requests'
    token counts plus what each part's ``decode_graph_key(step)`` adds (whatever else,
    known on the host, changes its launches).  A step with portions of prompts is replayed
    (once its shape has come three times) only if every part says ``prompt_capturable``:
    the same promise for any step.  A part that says nothing is never captured.
    """

    decode_capturable = False
    prompt_capturable = False

    def tensor_specs(self) -> dict:
        return {}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime

    def decode_graph_key(self, step: "StepContext") -> tuple:
        return ()


class Norm(Part):
    def forward(self, stream: ResidualStream, rows=None, n_rows: int = 0):
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, h, step: StepContext, cache: CacheHandle):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h, step: StepContext):
        raise NotImplementedError


class PositionEncoding(Part):
    pass
