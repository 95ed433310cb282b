"""Each part of a layer alone, bound to random weights, against its plain function."""

import pytest
import torch

import plain_llama as P
from mini_llm_stack_b200.cache.manager import CacheManager
from mini_llm_stack_b200.engine.batch import BatchBuilder, Entry
from mini_llm_stack_b200.ops.kernels import Runtime
from mini_llm_stack_b200.parts import (GroupedQueryAttention, OutputHead, PreNormBlock,
                                       ResidualStream, RMSNorm, RotaryPosition,
                                       SwiGLUFeedForward, TokenEmbedding)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 1e-5, torch.bfloat16: 1.5e-2}


@pytest.fixture(scope="module")
def rts():
    return {dt: Runtime(DEV, dt) for dt in DTYPES}


def draw(part, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in part.tensor_specs().items():
        t = torch.randn(spec.shape, generator=g) * (0.1 if spec.init == "normal" else 0.1)
        if spec.init == "ones":
            t = t + 1
        out[name] = t.to(dtype).to(DEV)
    return out


def rnd_of(dtype):
    return P.ident if dtype == torch.float32 else P.to_bf16


def close(got, want, dtype):
    return (got.float().cpu() - want).abs().max().item() <= TOL[dtype] * max(1e-6, want.abs().max().item())


def step_for(cache, entries, vocab=1000):
    for owner, tokens in entries:
        if not cache.has(owner):
            cache.admit(owner)
        assert cache.reserve(owner, len(tokens))
    return BatchBuilder(cache, DEV, vocab, 1 << 16).build(
        [Entry(o, t, [len(t) - 1]) for o, t in entries])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim, eps", [(96, 1e-6), (4096, 1e-5), (200, 3e-5)])
def test_norm_part_adds_the_pending_delta(rts, dtype, dim, eps):
    rt = rts[dtype]
    norm = RMSNorm(dim, eps)
    w = draw(norm, dtype, 1)
    norm.bind(w, rt)
    x = torch.randn(9, dim, device=DEV)
    delta = torch.randn(9, dim, device=DEV).to(dtype)
    stream = ResidualStream(x.clone())
    stream.push(delta)
    h = norm.forward(stream)
    assert stream.pending is None and torch.equal(stream.x, x + delta.float())
    want = rnd_of(dtype)(P.plain_rmsnorm((x + delta.float()).cpu(), w["weight"].float().cpu(), eps))
    assert close(h, want, dtype)
    # gathered rows leave the stream alone
    stream2 = ResidualStream(x.clone())
    stream2.push(delta)
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    hg = norm.forward(stream2, rows=rows, n_rows=2)
    assert torch.equal(stream2.x, x) and close(hg, want[[7, 2]], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(rts, dtype):
    rt = rts[dtype]
    emb = TokenEmbedding(301, 80)
    w = draw(emb, dtype, 2)
    emb.bind(w, rt)
    cache = CacheManager([], 4, 16, 2, 64, device=DEV)
    toks = [5, 300, 0, 17]
    step = step_for(cache, [("a", toks)], vocab=301)
    x = emb.forward(step)
    assert torch.equal(x, w["weight"].float()[toks])
    for tied in (True, False):
        head = OutputHead(301, 80, tied_to=emb if tied else None)
        hw = draw(head, dtype, 3)
        head.bind(hw, rt)
        h = torch.randn(3, 80, device=DEV).to(dtype)
        logits = head.forward(h, 3)
        table = w["weight"] if tied else hw["weight"]
        want = h.float().cpu() @ table.float().cpu().t()
        assert logits.dtype == torch.float32 and close(logits, want, torch.float32 if dtype == torch.float32 else dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, inter", [(64, 172), (96, 256), (80, 208)])
def test_feed_forward_part(rts, dtype, d, inter):
    rt = rts[dtype]
    ffn = SwiGLUFeedForward(d, inter)
    w = draw(ffn, dtype, 4)
    ffn.bind(w, rt)
    h = torch.randn(11, d, device=DEV).to(dtype)
    out = ffn.forward(h, None)
    f = {k: v.float().cpu() for k, v in w.items()}
    want = P.plain_swiglu(h.float().cpu(), f["w_gate.weight"], f["w_up.weight"], f["w_down.weight"],
                          rnd_of(dtype))
    assert close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, hd, d, window", [(4, 2, 16, 64, None), (3, 1, 32, 96, None),
                                                      (5, 5, 48, 80, 24), (8, 2, 64, 128, None)])
def test_attention_part_portion_after_cached_context(rts, dtype, heads, kv, hd, d, window):
    """The mixer with its position encoding: a prompt in two portions and a decoded
    token, against whole-sequence plain attention."""
    rt = rts[dtype]
    pos = RotaryPosition(hd, 10000.0, 256)
    mixer = GroupedQueryAttention(d, heads, kv, hd, hd ** -0.5, pos, window=window)
    w = draw(mixer, dtype, 5)
    mixer.bind(w, rt)
    cache = CacheManager([mixer.cache_spec()], 16, 16, 2, 256, device=DEV, kv_dtype=dtype)
    handle = cache.handles()[0]
    n = 70
    h_all = (torch.randn(n, d, device=DEV) * 0.5).to(dtype)
    outs = []
    at = 0
    for portion in (41, 28, 1):
        step = step_for(cache, [("r", [0] * portion)])
        outs.append(mixer.forward(h_all[at:at + portion].contiguous(), step, handle).clone())
        cache.commit("r", portion)
        at += portion
    got = torch.cat(outs)
    cfg = dict(n_heads=heads, n_kv_heads=kv, head_dim=hd)
    cos, sin = P.plain_rotary_tables(hd, 256, 10000.0)
    f = {f"m.{k}": v.float().cpu() for k, v in w.items()}
    want, _ = P.plain_mixer(h_all.float().cpu(), f, "m", cfg, cos, sin, torch.arange(n), window,
                            rnd_of(dtype))
    assert close(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, hd, d, window", [(4, 2, 64, 128, None), (8, 2, 128, 256, None),
                                                      (8, 2, 128, 256, 150), (4, 2, 32, 64, None)])
def test_what_a_page_held_before_does_not_reach_its_next_owner(rts, dtype, heads, kv, hd, d, window):
    """The whole pool is NaN, as a request that overflowed might have left its pages.
    A new request's keys and values go in through the mixer's position part, which
    clears the rest of every page it enters; the tensor-core kernels mask scores, not
    values, so a leftover NaN in a slot past the context would come out as 0 * NaN.
    Prompts of several tiles, portions of two tokens, decoded tokens; with a window,
    pages it has given back are read as zeros."""
    rt = rts[dtype]
    pos = RotaryPosition(hd, 10000.0, 1024)
    mixer = GroupedQueryAttention(d, heads, kv, hd, hd ** -0.5, pos, window=window)
    w = draw(mixer, dtype, 15)
    mixer.bind(w, rt)
    cache = CacheManager([mixer.cache_spec()], 48, 16, 2, 1024, device=DEV, kv_dtype=dtype)
    cache.paged[0].kv.fill_(float("nan"))
    handle = cache.handles()[0]
    portions = (131, 2, 1, 300, 1, 1, 2, 67, 1)
    n = sum(portions)
    h_all = (torch.randn(n, d, device=DEV) * 0.5).to(dtype)
    outs, at = [], 0
    for portion in portions:
        step = step_for(cache, [("r", [0] * portion)])
        outs.append(mixer.forward(h_all[at:at + portion].contiguous(), step, handle).float().clone())
        cache.commit("r", portion)
        at += portion
    got = torch.cat(outs)
    assert bool(torch.isfinite(got).all())
    cfg = dict(n_heads=heads, n_kv_heads=kv, head_dim=hd)
    cos, sin = P.plain_rotary_tables(hd, 1024, 10000.0)
    f = {f"m.{k}": v.float().cpu() for k, v in w.items()}
    want, _ = P.plain_mixer(h_all.float().cpu(), f, "m", cfg, cos, sin, torch.arange(n), window,
                            rnd_of(dtype))
    assert close(got, want, dtype)


@pytest.mark.parametrize("heads, kv, hd, d, window, block", [(4, 2, 64, 1024, None, 16),
                                                             (8, 2, 128, 1024, None, 16),
                                                             (8, 2, 128, 1024, 150, 8),
                                                             (32, 8, 128, 4096, None, 16)])
def test_decode_attention_that_rotates_and_stores_itself_gives_the_same_bits(
        rts, monkeypatch, heads, kv, hd, d, window, block):
    """Single decoded tokens: the attention kernel reads q, k and v as the K-parts of their
    projection, rotates, writes the cache and attends.  Outputs and pools must be, bit for
    bit, what the rotation kernel followed by the attention kernel gives; requests of
    different lengths, tokens that enter a page, a pool that held NaN before."""
    rt = rts[torch.bfloat16]

    def run(fused):
        monkeypatch.setenv("MLS_B200_FUSED_ROPE", "1" if fused else "0")
        pos = RotaryPosition(hd, 10000.0, 2048)
        mixer = GroupedQueryAttention(d, heads, kv, hd, hd ** -0.5, pos, window=window)
        mixer.bind(draw(mixer, torch.bfloat16, 25), rt)
        cache = CacheManager([mixer.cache_spec()], 300, block, 4, 2048, device=DEV,
                             kv_dtype=torch.bfloat16)
        cache.paged[0].kv.fill_(float("nan"))
        handle = cache.handles()[0]
        g = torch.Generator(device=DEV).manual_seed(3)
        lens = {"a": 700, "b": 31, "c": 1290}
        outs = []
        for r, n in lens.items():                      # the prompts, one request a step
            h = (torch.randn(n, d, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
            step = step_for(cache, [(r, [0] * n)])
            mixer.forward(h, step, handle).float()     # (a product left as parts is given back)
            cache.commit(r, n)
        used = []
        for i in range(20):                            # decoded tokens, all three a step
            h = (torch.randn(3, d, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
            step = step_for(cache, [(r, [0]) for r in lens])
            before = rt.ops.launches
            out = mixer.forward(h, step, handle)
            outs.append(out.float().clone())
            used.append(rt.ops.launches - before)
            for r in lens:
                cache.commit(r, 1)
        rt.ops.check_status()
        live = cache.paged[0].kv.clone()
        return torch.stack(outs), live, used

    fused, pool_f, n_f = run(True)
    plain, pool_p, n_p = run(False)
    assert max(n_f) < max(n_p)                         # one kernel fewer a step
    assert bool(torch.isfinite(fused).all())
    assert torch.equal(fused, plain)
    # the pools agree wherever a request's key or value lies (the rest is NaN or cleared)
    both = torch.isfinite(pool_p) | torch.isfinite(pool_f)
    assert torch.equal(torch.isfinite(pool_p), torch.isfinite(pool_f))
    assert torch.equal(pool_p[both], pool_f[both])


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part_wires_norms_mixer_and_feed_forward(rts, dtype):
    rt = rts[dtype]
    d, heads, kv, hd, inter, eps = 96, 3, 1, 32, 256, 1e-6
    block = PreNormBlock(RMSNorm(d, eps),
                         GroupedQueryAttention(d, heads, kv, hd, hd ** -0.5,
                                               RotaryPosition(hd, 5e5, 128)),
                         RMSNorm(d, eps), SwiGLUFeedForward(d, inter))
    w = draw(block, dtype, 6)
    assert set(w) == {"attn_norm.weight", "attn.wq.weight", "attn.wk.weight", "attn.wv.weight",
                      "attn.wo.weight", "mlp_norm.weight", "mlp.w_gate.weight",
                      "mlp.w_up.weight", "mlp.w_down.weight"}
    block.bind(w, rt)
    cache = CacheManager([block.cache_spec()], 8, 16, 2, 128, device=DEV, kv_dtype=dtype)
    n = 37
    x0 = torch.randn(n, d, device=DEV)
    stream = ResidualStream(x0.clone())
    step = step_for(cache, [("r", [0] * n)])
    block.forward(stream, step, cache.handles()[0])
    got = stream.x + stream.take_pending().float()
    f = {f"b.{k}": v.float().cpu() for k, v in w.items()}
    rnd = rnd_of(dtype)
    cfg = dict(n_heads=heads, n_kv_heads=kv, head_dim=hd)
    cos, sin = P.plain_rotary_tables(hd, 128, 5e5)
    x = x0.cpu()
    a, _ = P.plain_mixer(rnd(P.plain_rmsnorm(x, f["b.attn_norm.weight"], eps)), f, "b.attn", cfg,
                         cos, sin, torch.arange(n), None, rnd)
    x = x + a
    x = x + P.plain_swiglu(rnd(P.plain_rmsnorm(x, f["b.mlp_norm.weight"], eps)),
                           f["b.mlp.w_gate.weight"], f["b.mlp.w_up.weight"],
                           f["b.mlp.w_down.weight"], rnd)
    assert close(got, x, dtype)
