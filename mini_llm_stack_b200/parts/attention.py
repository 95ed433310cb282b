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

import torch

from .base import CacheHandle, Mixer, PagedKV, StepContext, TensorSpec


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

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt = self.runtime
        t = step.n_tokens
        hd = self.head_dim
        width = (self.n_heads + 2 * self.n_kv_heads) * hd
        qkv = rt.buffer("qkv", (t, width), rt.act_dtype)
        if getattr(self.position, "takes_parts", False):
            # the projection may stay in the parts it was cut into along K: the
            # rotation adds them up as it reads them
            src = rt.ops.linear_parts(h, self.wqkv, qkv)
            self.position.rotate_and_store(qkv, step, cache, self.n_heads, self.n_kv_heads,
                                           parts=None if src is qkv else src)
        else:
            rt.ops.linear(h, self.wqkv, qkv)
            self.position.rotate_and_store(qkv, step, cache, self.n_heads,
                                           self.n_kv_heads)
        o = rt.buffer("attn_out", (t, self.n_heads * hd), rt.act_dtype)
        rt.ops.paged_attention(qkv, o, cache, step, self.n_heads, self.n_kv_heads,
                               hd, self.scale, self.window or 0)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(o, self.wo, delta)
