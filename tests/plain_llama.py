"""A plain, slow implementation of the dense Llama-style decoder, for tests.

Whole sequences, no cache, one function for each part, float32 on the CPU (or
any device of the tensors given).  It shares no code with the engine: it takes
a plain dict of hyper-parameters and a dict of tensors by their file names.
Every function is written from the reference's formulas and cites them by the
file's path within grenver/mini-llm-stack.  ``tests/golden/make_golden.py``
compares it once with the reference's own ``Transformer`` on the CPU.

``rnd`` is the rounding applied where the engine stores an activation:
identity for the float32 path, a round trip through bfloat16 for the bfloat16
path (sums, softmax, norms and rotations stay in float32 either way).
"""

from __future__ import annotations


import torch


def ident(t):
    return t


def to_bf16(t):
    return t.to(torch.bfloat16).to(torch.float32)


def plain_rmsnorm(x, weight, eps):
    """train/model.py:29-33: ``x * rsqrt(mean(x^2) + eps)`` then ``* weight``, in
    float32; eps inside the root, weight after the normalisation."""
    x = x.float()
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x * weight.float()


def plain_rotary_tables(head_dim, max_pos, theta):
    """train/model.py:41-45: ``inv_freq = 1 / theta^(arange(0, hd, 2) / hd)``;
    ``freqs = outer(arange(max_pos), inv_freq)``; cos and sin in float32."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    t = torch.arange(max_pos).float()
    freqs = torch.outer(t, inv_freq)
    return freqs.cos(), freqs.sin()


def plain_rope(x, pos, cos, sin):
    """train/model.py:47-52 (rotate-half): ``x1, x2 = x.chunk(2, -1)``;
    ``cat(x1*cos - x2*sin, x2*cos + x1*sin)``.  x: [H, S, hd]; pos: [S]."""
    c = cos[pos].to(x.device)
    s = sin[pos].to(x.device)
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def plain_attention(q, k, v, scale, window=None):
    """train/model.py:55-70: ``scores = q k^T * scale`` in float32; key j hidden
    from query i iff ``j > i + (Sk - Sq)``; softmax; ``probs @ v``.
    q: [H, Sq, hd]; k, v: [Hkv, Sk, hd]; q head h reads kv head h // (H / Hkv).
    With ``window`` w, keys ``j <= p - w`` (p the query's position) are hidden too.
    """
    H, Sq, _ = q.shape
    Hkv, Sk, _ = k.shape
    G = H // Hkv
    k = k.repeat_interleave(G, dim=0)
    v = v.repeat_interleave(G, dim=0)
    scores = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    qi = torch.arange(Sq, device=q.device)[:, None] + (Sk - Sq)
    kj = torch.arange(Sk, device=q.device)[None, :]
    hidden = kj > qi
    if window is not None:
        hidden = hidden | (kj <= qi - window)
    scores = scores.masked_fill(hidden, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, v.float())


def plain_swiglu(x, w_gate, w_up, w_down, rnd=ident):
    """train/model.py:135: ``w_down(silu(w_gate x) * w_up x)``, no biases."""
    g = rnd(x @ w_gate.float().t())
    u = rnd(x @ w_up.float().t())
    a = rnd(torch.nn.functional.silu(g) * u)
    return rnd(a @ w_down.float().t())


def plain_mixer(h, w, prefix, cfg, cos, sin, pos, window, rnd=ident, kv_from=None):
    """train/model.py:86-123: q/k/v projections without bias, heads split as
    ``view(S, H, hd)``, RoPE on q and k, causal attention, heads concatenated
    head-major, ``wo``.  Returns (output [S, d], (k, v)) so that a later call
    may read this call's keys and values."""
    S = h.shape[0]
    H, Hkv, hd = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    q = rnd(h @ w[f"{prefix}.wq.weight"].float().t()).view(S, H, hd).transpose(0, 1)
    q = rnd(plain_rope(q, pos, cos, sin))
    if kv_from is None:
        k = rnd(h @ w[f"{prefix}.wk.weight"].float().t()).view(S, Hkv, hd).transpose(0, 1)
        v = rnd(h @ w[f"{prefix}.wv.weight"].float().t()).view(S, Hkv, hd).transpose(0, 1)
        k = rnd(plain_rope(k, pos, cos, sin))
    else:
        k, v = kv_from
    o = rnd(plain_attention(q, k, v, cfg["head_dim"] ** -0.5, window))
    o = o.transpose(0, 1).reshape(S, H * hd)
    return rnd(o @ w[f"{prefix}.wo.weight"].float().t()), (k, v)


def plain_forward(w, cfg, tokens, rnd=ident):
    """train/model.py:238-242 and :207-216: ``embed`` -> for every call
    ``x = x + attn(attn_norm(x))``; ``x = x + mlp(mlp_norm(x))`` -> ``final_norm``
    -> ``lm_head`` (the embedding table when tied, train/model.py:228-229).
    tokens: list or 1-D tensor of ids.  Returns float32 logits [S, V]."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    S = tokens.shape[0]
    eps = cfg["norm_eps"]
    cos, sin = plain_rotary_tables(cfg["head_dim"], cfg["max_seq_len"], cfg["rope_theta"])
    pos = torch.arange(S)
    x = w["embed.weight"].float()[tokens]
    order = cfg.get("layer_order") or list(range(cfg["n_layers"]))
    source = cfg.get("cache_source") or [None] * len(order)
    windows = cfg.get("layer_windows") or [None] * cfg["n_layers"]
    kept = {}
    for c, i in enumerate(order):
        p = f"blocks.{i}"
        h = rnd(plain_rmsnorm(x, w[f"{p}.attn_norm.weight"], eps))
        kv_from = kept[source[c]] if source[c] is not None else None
        a, kv = plain_mixer(h, w, f"{p}.attn", cfg, cos, sin, pos, windows[i], rnd, kv_from)
        kept[c] = kv
        x = x + a
        h = rnd(plain_rmsnorm(x, w[f"{p}.mlp_norm.weight"], eps))
        x = x + plain_swiglu(h, w[f"{p}.mlp.w_gate.weight"], w[f"{p}.mlp.w_up.weight"],
                             w[f"{p}.mlp.w_down.weight"], rnd)
    h = rnd(plain_rmsnorm(x, w["final_norm.weight"], eps))
    head = w["embed.weight"] if cfg["tie_embeddings"] else w["lm_head.weight"]
    return h @ head.float().t()


def uniform_for(seed: int, request: int, index: int) -> float:
    """The uniform number in [0, 1) for one draw; restates the documented rule of
    the engine's sampler (splitmix64 over seed, request and output index)."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9
         + index * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def plain_sample(logits, temperature, u):
    """train/model.py:262-266: ``temperature > 0`` -> draw from
    ``softmax(logits / temperature)``, else arg max.  The draw is the first index
    whose cumulative probability exceeds u (the engine's rule)."""
    if temperature <= 0:
        return int(torch.argmax(logits))
    z = logits.float() / temperature
    e = torch.exp(z - z.max())
    cum = torch.cumsum(e, dim=0)
    hit = torch.nonzero(cum > u * cum[-1])
    return int(hit[0]) if hit.numel() else logits.numel() - 1


def plain_generate(w, cfg, prompt, max_new, temperature=0.0, seed=0, request=0,
                   eos=None, rnd=ident):
    """train/model.py:256-268 (``generate_naive``): re-run the whole sequence for
    every new token, take the last row's logits, pick, append."""
    toks = list(prompt)
    out = []
    for i in range(max_new):
        logits = plain_forward(w, cfg, toks[-cfg["max_seq_len"]:], rnd)[-1]
        u = uniform_for(seed, request, i) if temperature > 0 else 0.0
        nxt = plain_sample(logits, temperature, u)
        toks.append(nxt)
        out.append(nxt)
        if eos is not None and nxt == eos:
            break
        if len(toks) >= cfg["max_seq_len"]:
            break
    return out
