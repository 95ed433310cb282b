"""Grouped-query causal attention over the paged cache.

Reference (train/model.py:73-124, MHA only): q/k/v/o projections without bias,
``nn.Linear`` layout [out, in], output feature j belongs to head ``j // head_dim``;
RoPE on q and k; scores ``(q . k) * scale`` with ``scale = head_dim ** -0.5``
(train/model.py:62); causal mask bottom-right aligned: key j is hidden from
query i iff ``j > i + (Sk - Sq)`` (train/model.py:64-68); softmax and P.V in
float32; output heads concatenated head-major (train/model.py:122) and
projected by ``wo``.  Grouped queries: q head h reads kv head ``h // G``.  A
window w additionally hides keys ``j <= p - w`` from the query at position p.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from .base import CacheHandle, Mixer, PagedKV, StepContext, TensorSpec


@dataclass(frozen=True)
class AttentionPlan:
    """How one step's attention is launched (for one shape of heads)."""
    n_tiles: int          # tiles of the mma.sync tile kernel over the requests that are not small
    n_tiles_tc: int       # tiles of the tcgen05 kernel over the same requests
    n_tiles_tc_wide: int  # tiles of twice as many rows: the kernel takes these when they fill the SMs
    any_small: bool       # some request has so few rows that the context-split kernel takes it
    n_split: int          # parts the context of the small requests is cut into


def context_splits(tiles: list, n_kv: int, slots: int = 296, cluster_splits: int = 0,
                   longest: int = 0, cluster_slots: int = 0) -> int:
    """Context splits for decoding requests of ``tiles[i]`` key tiles (64 keys) each.

    The kernel cuts every request at the same multiples of tiles, the tiles of the step's
    longest context (``longest``, if a request that is not among these has more) shared
    out over the splits: a shorter request fills only its first splits, and the CTAs of
    the others leave at once.  ``slots`` CTAs of the split kernel run at a
    time (two an SM: 296 on a B200); the cost of a choice is its number of such waves of
    CTAs that have tiles times the tiles a CTA walks (plus six tiles' worth of start-up),
    plus what placing the empty CTAs costs, plus the merge's time, which grows with the
    number of parts (measured at batch 1: 16 parts beat 32).  Up to ``cluster_splits``
    parts are merged inside the split kernel while ``cluster_slots`` CTAs hold them all;
    beyond that a merge kernel follows, which costs about what two tiles take.  The
    cheapest choice wins; a split is never shorter than 256 keys.
    """
    longest = max(longest, max(tiles))
    forced = os.environ.get("MLS_B200_SPLITS")
    if forced:
        return max(1, min(int(forced), longest))
    best, best_cost = 1, None
    for s in range(1, max(1, min(64, longest // 4)) + 1):
        per = -(-longest // s)
        busy = sum(-(-t // per) for t in tiles) * n_kv
        grid = len(tiles) * n_kv * s
        cost = -(-busy // slots) * (per + 6) + 2.0 * (grid - busy) / slots
        if s > 1:
            cost += 0.3 * s
            if not (cluster_splits and s <= cluster_splits and grid <= (cluster_slots or slots)):
                cost += 2.0
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


class GroupedQueryAttention(Mixer):
    def __init__(self, d_model: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, position, window=None):
        if n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.d_model, self.n_heads, self.n_kv_heads = d_model, n_heads, n_kv_heads
        self.head_dim, self.scale, self.window = head_dim, float(scale), window
        self.position = position
        self.wqkv = self.wo = None

    def tensor_specs(self) -> dict:
        d, hd = self.d_model, self.head_dim
        return {
            "wq.weight": TensorSpec((self.n_heads * hd, d)),
            "wk.weight": TensorSpec((self.n_kv_heads * hd, d)),
            "wv.weight": TensorSpec((self.n_kv_heads * hd, d)),
            "wo.weight": TensorSpec((d, self.n_heads * hd)),
        }

    def cache_spec(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        parts = [tensors["wq.weight"], tensors["wk.weight"], tensors["wv.weight"]]
        if len({p.dtype for p in parts}) > 1:
            parts = [p.float() for p in parts]
        # one projection for q, k and v: rows [q heads | k heads | v heads]
        self.wqkv = runtime.ops.prepare_weight(torch.cat(parts, dim=0))
        self.wo = runtime.ops.prepare_weight(tensors["wo.weight"])
        self.position.bind({}, runtime)
        runtime.ops.require_attention(self.head_dim, self.n_heads, self.n_kv_heads)
        self._facts = runtime.ops.attention_facts(self.head_dim)

    # ---------------------------------------------------------- launch planning
    @property
    def decode_capturable(self) -> bool:
        """Forward only launches kernels; the position part has to agree."""
        return bool(getattr(self.position, "decode_capturable", False))

    @property
    def prompt_capturable(self) -> bool:
        return bool(getattr(self.position, "prompt_capturable", False))

    def plan(self, step: StepContext):
        """This step's ``AttentionPlan`` (None where the kernel in use needs none).

        Requests whose (token, head) rows of one kv head fit ``small_rows`` go to the
        context-split kernel, their context cut so that all SMs have work; the others
        are cut into tiles of rows.  Mixers with the same shape of heads share the
        plan of a step."""
        f = self._facts
        if not f["tensor_cores"]:
            return None
        group = self.n_heads // self.n_kv_heads
        key = ("gqa", group, self.n_kv_heads, self.head_dim)
        plan = step.attn_tiles.get(key)
        if plan is None:
            small = [q * group <= f["small_rows"] for q in step.q_lens]
            big = [q * group for q, s in zip(step.q_lens, small) if not s]
            n_small = sum(small)
            n_split = 1
            if n_small:
                keys = f.get("split_keys", 64)
                tiles = [-(-c // keys) for c, s in zip(step.ctx_lens, small) if s]
                n_split = context_splits(tiles, self.n_kv_heads, f["split_slots"],
                                         f.get("cluster_splits", 0),
                                         longest=-(-step.max_ctx_len // keys),
                                         cluster_slots=f.get("cluster_slots", 0))
            plan = AttentionPlan(
                n_tiles=sum(-(-r // f["tile_rows"]) for r in big),
                n_tiles_tc=sum(-(-r // f["tc_rows"]) for r in big),
                n_tiles_tc_wide=sum(-(-r // (2 * f["tc_rows"])) for r in big),
                any_small=n_small > 0, n_split=n_split)
            step.attn_tiles[key] = plan
        return plan

    def decode_graph_key(self, step: StepContext) -> tuple:
        """What, besides the number of requests, fixes this mixer's launches in a step
        of single tokens: the number of context splits."""
        plan = self.plan(step)
        if plan is None:
            return ()
        return ("gqa", self.n_kv_heads, self.n_heads // self.n_kv_heads, self.head_dim,
                plan.n_split)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt = self.runtime
        t = step.n_tokens
        hd = self.head_dim
        width = (self.n_heads + 2 * self.n_kv_heads) * hd
        qkv = rt.buffer("qkv", (t, width), rt.act_dtype)
        o = rt.buffer("attn_out", (t, self.n_heads * hd), rt.act_dtype)
        if getattr(self.position, "takes_parts", False):
            # the projection may stay in the parts it was cut into along K: the
            # rotation adds them up as it reads them
            src = rt.ops.linear_parts(h, self.wqkv, qkv)
            tables = (self.position.fused_tables()
                      if src is not qkv and step.max_q_len == 1 and cache.kind == "paged"
                      and hasattr(self.position, "fused_tables") else None)
            if tables is not None and rt.ops.can_fuse_rope_attention(
                    hd, step.groups[cache.group].block_size):
                # single decoded tokens: the attention kernel rotates and stores as well
                cos, sin, max_pos = tables
                rt.ops.attention_decode_fused(src, o, cache, step, cos, sin, max_pos,
                                              self.n_heads, self.n_kv_heads, hd, self.scale,
                                              self.window or 0, self.plan(step))
                delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
                return rt.ops.linear_parts(o, self.wo, delta)
            self.position.rotate_and_store(qkv, step, cache, self.n_heads, self.n_kv_heads,
                                           parts=None if src is qkv else src)
        else:
            rt.ops.linear(h, self.wqkv, qkv)
            self.position.rotate_and_store(qkv, step, cache, self.n_heads,
                                           self.n_kv_heads)
        rt.ops.paged_attention(qkv, o, cache, step, self.n_heads, self.n_kv_heads,
                               hd, self.scale, self.window or 0, plan=self.plan(step))
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(o, self.wo, delta)
