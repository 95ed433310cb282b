"""Each kernel alone against its plain reference, at other sizes than the engine's."""

import math

import pytest
import torch

import plain_llama as P
from mini_llm_stack_b200.cache.manager import CacheManager
from mini_llm_stack_b200.engine.batch import BatchBuilder, Entry
from mini_llm_stack_b200.ops.kernels import KernelError, Runtime
from mini_llm_stack_b200.parts.attention import GroupedQueryAttention
from mini_llm_stack_b200.parts.base import PagedKV

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def rts():
    return {dt: Runtime(DEV, dt) for dt in DTYPES}


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


# --------------------------------------------------------------------------- embed
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab, d", [(97, 96), (1000, 4097), (5, 8)])
def test_embed(rts, dtype, vocab, d):
    ops = rts[dtype].ops
    table = rand((vocab, d), dtype, 1)
    ids = torch.randint(0, vocab, (37,), generator=torch.Generator().manual_seed(2)).int().to(DEV)
    x = torch.empty((37, d), dtype=torch.float32, device=DEV)
    ops.embed(ids, table, x, vocab)
    assert torch.equal(x, table.float()[ids.long()])
    ops.check_status()
    ops.embed(torch.tensor([vocab], dtype=torch.int32, device=DEV), table, x[:1], vocab)
    with pytest.raises(KernelError, match="vocabulary"):
        ops.check_status()


# ---------------------------------------------------------------------------- norm
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, d, eps", [(5, 96, 1e-6), (33, 4096, 1e-5), (2, 1000, 3e-5),
                                          (1, 16, 1e-5), (3, 11008, 1e-5)])
def test_add_rmsnorm(rts, dtype, rows, d, eps):
    ops = rts[dtype].ops
    x = rand((rows, d), torch.float32, 3, 2.0)
    delta = rand((rows, d), dtype, 4)
    w = 1 + rand((d,), dtype, 5, 0.1)
    h = torch.empty((rows, d), dtype=dtype, device=DEV)
    want_x = x + delta.float()
    want_h = P.plain_rmsnorm(want_x.cpu(), w.cpu(), eps)
    xx = x.clone()
    ops.add_rmsnorm(xx, delta, w, eps, h)
    assert torch.equal(xx, want_x)                       # the residual sum is exact float32
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    assert torch.allclose(h.float().cpu(), want_h, rtol=tol, atol=tol)
    # no delta: x is left alone
    xx = x.clone()
    ops.add_rmsnorm(xx, None, w, eps, h)
    assert torch.equal(xx, x)
    assert torch.allclose(h.float().cpu(), P.plain_rmsnorm(x.cpu(), w.cpu(), eps), rtol=tol, atol=tol)
    # gathered rows: only those rows, x untouched
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    hg = torch.empty((2, d), dtype=dtype, device=DEV)
    xx = x.clone()
    ops.gather_add_rmsnorm(xx, delta, pick, 2, w, eps, hg)
    assert torch.equal(xx, x)
    assert torch.allclose(hg.float().cpu(), want_h[[rows - 1, 0]], rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, d", [(2048, 4096), (301, 1000), (777, 512), (296, 2056)])
def test_add_rmsnorm_of_many_rows_gives_the_bits_of_few_rows(rts, dtype, rows, d):
    """Prompts take a kernel that streams rows through shared memory; a row's result
    is bit for bit what it is in a batch of a few rows."""
    ops = rts[dtype].ops
    x = rand((rows, d), torch.float32, 41, 2.0)
    delta = rand((rows, d), dtype, 42)
    w = 1 + rand((d,), dtype, 43, 0.1)
    h = torch.empty((rows, d), dtype=dtype, device=DEV)
    xx = x.clone()
    ops.add_rmsnorm(xx, delta, w, 1e-5, h)
    ops.check_status()
    assert torch.equal(xx, x + delta.float())
    pick = torch.tensor([0, 1, rows // 2, rows - 5, rows - 1], device=DEV)
    x_few = x[pick].clone()
    h_few = torch.empty((5, d), dtype=dtype, device=DEV)
    ops.add_rmsnorm(x_few, delta[pick].contiguous(), w, 1e-5, h_few)
    assert torch.equal(h[pick], h_few)
    want = P.plain_rmsnorm((x + delta.float()).cpu(), w.cpu(), 1e-5)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    assert torch.allclose(h.float().cpu(), want, rtol=tol, atol=tol)
    # without a pending delta
    h2 = torch.empty((rows, d), dtype=dtype, device=DEV)
    ops.add_rmsnorm(xx, None, w, 1e-5, h2)
    assert torch.equal(h2, h)


def test_norm_weight_may_stay_float32_in_a_bfloat16_run(rts):
    ops = rts[torch.bfloat16].ops
    x = rand((4, 80), torch.float32, 6)
    w = 1 + rand((80,), torch.float32, 7, 0.1)
    h = torch.empty((4, 80), dtype=torch.bfloat16, device=DEV)
    ops.add_rmsnorm(x, None, w, 1e-5, h)
    assert torch.allclose(h.float().cpu(), P.plain_rmsnorm(x.cpu(), w.cpu(), 1e-5), rtol=8e-3, atol=8e-3)


# ------------------------------------------------------------------------ gemm f32
@pytest.mark.parametrize("m, n, k", [(1, 97, 96), (7, 300, 172), (130, 65, 33), (64, 64, 16),
                                     (3, 1000, 1023), (257, 129, 4096)])
def test_gemm_f32_is_true_float32_and_batch_invariant(rts, m, n, k):
    ops = rts[torch.float32].ops
    a, w = rand((m, k), torch.float32, 8), rand((n, k), torch.float32, 9)
    out = torch.empty((m, n), dtype=torch.float32, device=DEV)
    ops.linear(a, w, out)
    want = (a.double() @ w.double().t())
    err = (out.double() - want).abs().max().item()
    # a float32 running sum over k terms is off by about sqrt(k) roundings of its own
    # size; products rounded to TF32 (10-bit mantissa) would be off by sqrt(k) * 2^-11
    # of a product, some fifty times more
    bound = 4 * math.sqrt(k) * 2.0 ** -24 * want.abs().max().item()
    assert err <= bound and bound < math.sqrt(k) * 2.0 ** -11 / 5, (err, bound)
    # a row's result does not depend on what else is in the batch
    one = torch.empty((1, n), dtype=torch.float32, device=DEV)
    ops.linear(a[m // 2:m // 2 + 1].contiguous(), w, one)
    assert torch.equal(one[0], out[m // 2])


def test_linear_with_float32_weights_in_a_bfloat16_run(rts):
    ops = rts[torch.bfloat16].ops
    a, w = rand((5, 64), torch.bfloat16, 10), rand((24, 64), torch.float32, 11)
    out = torch.empty((5, 24), dtype=torch.bfloat16, device=DEV)
    ops.linear(a, w, out)
    want = (a.float() @ w.t()).to(torch.bfloat16)
    assert torch.equal(out, want) or torch.allclose(out.float(), want.float(), rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("m, n, k", [(1, 128, 64), (8, 6144, 4096), (37, 257, 200), (300, 96, 1000),
                                     (64, 1000, 4096), (2048, 512, 1024), (17, 4096, 14336),
                                     (129, 300, 72), (65, 128, 8), (33, 97, 4096),
                                     # 33 to 48 rows: tiles of 48 columns of tensor memory
                                     (40, 6144, 4096), (48, 1000, 520),
                                     # row counts whose 128-row tiles do not fill whole rounds of
                                     # CTAs: tiles of 96 + 128 rows, and of 64 + 96
                                     (2, 128256, 128), (5, 22016, 256), (64, 28672, 64),
                                     # more than 128 rows (pairs of CTAs on tiles of 256 x 256, or with
                                     # "tcgen05-tiles" one CTA a tile), ragged edges, many tiles a CTA
                                     (257, 513, 136), (600, 1000, 4096), (512, 6144, 4096),
                                     (2048, 4096, 4096), (130, 40, 64)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("impl", ["tcgen05", "tcgen05-tiles", "cublas"])
def test_linear_bf16(rts, m, n, k, out_dtype, impl):
    ops = rts[torch.bfloat16].ops
    a, w = rand((m, k), torch.bfloat16, 12), rand((n, k), torch.bfloat16, 13, 0.05)
    out = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
    ops.gemm_impl = impl
    try:
        ops.linear(a, ops.prepare_weight(w), out)
    finally:
        ops.gemm_impl = "auto"
    ops.check_status()
    want = a.float() @ w.float().t()
    scale = want.abs().max().item()
    # float32 sums over k in another order differ by about sqrt(k) roundings
    tol = max(1e-5, 4 * math.sqrt(k) * 2.0 ** -24) if out_dtype == torch.float32 else 5e-3
    assert (out.float() - want).abs().max().item() <= tol * scale + 1e-6


@pytest.mark.parametrize("m, n, k", [(1, 4096, 14336), (8, 4096, 4096), (33, 1000, 4104), (64, 96, 2048),
                                     (48, 4096, 4096)])
def test_product_left_as_parts_is_summed_by_the_next_norm(rts, m, n, k):
    """A product that only feeds the residual stream keeps its K-parts; add_rmsnorm
    adds them up, for all rows and for chosen rows, and the buffer is lent once."""
    from mini_llm_stack_b200.ops.kernels import SplitParts
    ops = rts[torch.bfloat16].ops
    a, w = rand((m, k), torch.bfloat16, 21), rand((n, k), torch.bfloat16, 22, 0.05)
    wp = ops.prepare_weight(w)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_impl = "tcgen05"
    try:
        parts = ops.linear_parts(a, wp, out)
        assert isinstance(parts, SplitParts) and parts.shape == (m, n)
        again = ops.linear_parts(a, wp, out)              # the buffer is taken: the ordinary way
        assert again is out
    finally:
        ops.gemm_impl = "auto"
    ops.check_status()
    want = a.float() @ w.float().t()
    scale = want.abs().max().item()
    tol = max(1e-5, 4 * math.sqrt(k) * 2.0 ** -24)
    x = rand((m, n), torch.float32, 23, 2.0)
    g = 1 + rand((n,), torch.bfloat16, 24, 0.1)
    rows = torch.tensor([m - 1, 0], dtype=torch.int32, device=DEV)
    hg = torch.empty((2, n), dtype=torch.bfloat16, device=DEV)
    xx = x.clone()
    ops.gather_add_rmsnorm(xx, SplitParts(parts.parts, None), rows, 2, g, 1e-5, hg)
    assert torch.equal(xx, x)                             # chosen rows leave the stream alone
    h = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    ops.add_rmsnorm(xx, parts, g, 1e-5, h)
    assert (xx - (x + want)).abs().max().item() <= tol * scale + 1e-6
    want_h = P.plain_rmsnorm((x + want).cpu(), g.cpu(), 1e-5)
    assert torch.allclose(h.float().cpu(), want_h, rtol=8e-3, atol=8e-3)
    assert torch.equal(hg[0], h[m - 1]) and torch.equal(hg[1], h[0])
    assert not ops._parts_busy                      # given back by the norm
    assert torch.allclose(out.float(), want, rtol=1e-2, atol=5e-3 * scale)   # the ordinary way's result


@pytest.mark.parametrize("m, inter, k", [(1, 14336, 4096), (8, 176, 64), (64, 256, 96), (33, 4096, 4096),
                                         (41, 1008, 512), (48, 14336, 4096),
                                         (8, 11008, 128), (3, 10000, 64),
                                          (300, 272, 200), (2048, 1024, 512), (129, 14336, 1024),
                                          # two tiles after three whole rounds, cut along K
                                          (512, 14336, 4096)])
def test_gate_up_projection_with_swiglu_epilogue(rts, m, inter, k):
    ops = rts[torch.bfloat16].ops
    a = rand((m, k), torch.bfloat16, 30)
    wg, wu = rand((inter, k), torch.bfloat16, 31, 0.08), rand((inter, k), torch.bfloat16, 32, 0.08)
    assert ops.can_fuse_swiglu(k, inter)
    out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(a, ops.interleave_gate_up(wg, wu), out)
    ops.check_status()
    g = (a.float() @ wg.float().t()).cpu()
    u = (a.float() @ wu.float().t()).cpu()
    want = torch.nn.functional.silu(g) * u
    assert (out.float().cpu() - want).abs().max().item() <= 8e-3 * want.abs().max().item() + 1e-6


@pytest.mark.parametrize("mode", ["always", "auto"])
@pytest.mark.parametrize("m, n, k, swiglu", [
    (600, 1000, 4096, False),      # twelve ragged tiles, no whole round, in six parts each
    (2500, 2048, 3080, False),     # a whole round, then six tiles in twelve parts; K ends inside a k-block
    (2048, 512, 1024, False), (300, 96, 1000, False),
    (512, 4096, 14336, False),     # few tiles and a long K: cut in "auto" too
    (512, 28672, 4096, True),      # two tiles after three whole rounds: cut in "auto" too
    (300, 2400, 512, True),        # twenty ragged tiles in halves
    (2048, 28672, 256, True)])     # eight tiles after twelve rounds, K too short for more than one part
def test_last_rounds_tiles_cut_along_k(rts, mode, m, n, k, swiglu):
    """A prompt's product on pairs of CTAs whose last round of tiles is cut along K: the
    pieces' float32 sums go through scratch and a second kernel adds them up."""
    ops = rts[torch.bfloat16].ops
    a, w = rand((m, k), torch.bfloat16, 41), rand((n, k), torch.bfloat16, 42, 0.05)
    out = torch.full((m, n // 2 if swiglu else n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_impl = "tcgen05"
    ops.set_gemm_tail_cut(mode)
    try:
        if swiglu:
            ops.linear_swiglu(a, w, out)
        else:
            ops.linear(a, ops.prepare_weight(w), out)
    finally:
        ops.gemm_impl = "auto"
        ops.set_gemm_tail_cut("auto")
    ops.check_status()
    want = a.float() @ w.float().t()
    if swiglu:
        both = want.view(m, n // 32, 2, 16)
        want = (torch.nn.functional.silu(both[:, :, 0]) * both[:, :, 1]).reshape(m, n // 2)
    assert (out.float() - want).abs().max().item() <= 8e-3 * want.abs().max().item() + 1e-6


# ------------------------------------------------------------------------- swiglu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("t, inter", [(3, 172), (17, 14336), (1, 5)])
def test_swiglu(rts, dtype, t, inter):
    ops = rts[dtype].ops
    gu = rand((t, 2 * inter), dtype, 14, 3.0)
    out = torch.empty((t, inter), dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    g, u = gu.float().cpu()[:, :inter], gu.float().cpu()[:, inter:]
    want = torch.nn.functional.silu(g) * u
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    assert torch.allclose(out.float().cpu(), want, rtol=tol, atol=tol)


# ----------------------------------------------------------------------- sampling
@pytest.mark.parametrize("vocab", [97, 256, 1000, 128256])
def test_argmax_and_temperature_sampling(rts, vocab):
    ops = rts[torch.float32].ops
    n = 6
    logits = rand((n, vocab), torch.float32, 15, 2.0)
    logits[1, vocab // 2] = logits[1].max() + 1
    logits[2, 3] = logits[2, vocab - 1] = logits[2].max() + 1          # a tie: first wins
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, None, None, out)
    assert out.tolist() == [int(torch.argmax(r)) for r in logits.cpu()]
    assert out[2].item() == 3
    temps = torch.tensor([0.8, 0.0, 1.5, 0.3, 1.0, 0.8], device=DEV)
    us = torch.tensor([0.0, 0.5, 0.999999, 0.37, 0.81, 0.5], device=DEV)
    ops.sample(logits, temps, us, out)
    for i in range(n):
        want = P.plain_sample(logits[i].cpu(), temps[i].item(), us[i].item())
        got = out[i].item()
        if got != want:      # u may sit within rounding of a step of the cumulative sum
            z = logits[i].cpu() / temps[i].item()
            cum = torch.cumsum(torch.softmax(z, 0), 0)
            assert abs(cum[min(got, want)].item() - us[i].item()) < 1e-5, (i, got, want)


@pytest.mark.parametrize("vocab", [4097, 5000, 50000, 128256])
def test_temperature_sampling_over_chunks_of_the_vocabulary(rts, vocab):
    """Large vocabularies are sampled in chunks on many SMs; many rows, temperatures and
    uniform numbers (0 and just below 1 among them) against the plain inverse CDF."""
    ops = rts[torch.float32].ops
    n = 48
    g = torch.Generator().manual_seed(vocab)
    logits = rand((n, vocab), torch.float32, 77, 3.0)
    logits[5, vocab - 1] += 30.0                     # nearly all weight on the last token
    logits[6, 0] += 30.0                             # ... on the first
    logits[7, 4096] += 30.0                          # ... on a chunk's first token
    temps = (torch.rand(n, generator=g) * 1.5 + 0.05).to(DEV)
    temps[9] = 0.0                                   # a greedy row among them
    us = torch.rand(n, generator=g).to(DEV)
    us[0], us[1], us[2] = 0.0, 0.99999994, 0.5
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, temps, us, out)
    assert out[9].item() == int(torch.argmax(logits[9]))
    assert out[5].item() == vocab - 1 or us[5].item() < 1e-6
    for i in range(n):
        want = P.plain_sample(logits[i].cpu(), temps[i].item(), us[i].item())
        got = out[i].item()
        if got != want:      # u may sit within rounding of a step of the cumulative sum
            z = logits[i].cpu().double() / temps[i].item()
            cum = torch.cumsum(torch.softmax(z, 0), 0)
            assert abs(cum[min(got, want)].item() - us[i].item()) < 1e-5, (i, got, want)
            assert abs(got - want) <= 64 or cum[max(got, want) - 1] - cum[min(got, want)] < 1e-5


# ------------------------------------------------------------------ rope and store
def owned_slots(block, pages, lens, starts, seed):
    """Slots as the cache hands them out: request r brings ``lens[r]`` tokens, the first
    at offset ``starts[r]`` of a page of its own; its tokens take consecutive slots and
    go on into further pages of its own.  Returns (int32 slots, set of (page, offset)
    the kernel must clear: the rest of the page a request's last token lies in, if that
    page was entered in this step)."""
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    slots, cleared = [], set()
    for n, s in zip(lens, starts):
        assert 0 <= s < block
        mine = [order.pop() for _ in range((s + n + block - 1) // block)]
        slots += [mine[(s + i) // block] * block + (s + i) % block for i in range(n)]
        last = s + n - 1
        if last // block > 0 or s == 0:
            cleared |= {(mine[last // block], o) for o in range(last % block + 1, block)}
    return torch.tensor(slots, dtype=torch.int32), cleared


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, hd, theta, block", [(4, 2, 16, 10000.0, 4), (3, 1, 32, 5e5, 8),
                                                         (5, 5, 48, 25000.0, 16), (8, 2, 128, 5e5, 16)])
def test_rope_store(rts, dtype, heads, kv, hd, theta, block):
    ops = rts[dtype].ops
    max_pos, pages, t = 200, 40, 23
    cos, sin = P.plain_rotary_tables(hd, max_pos, theta)
    qkv = rand((t, (heads + 2 * kv) * hd), dtype, 16)
    pos = torch.randint(0, max_pos, (t,), generator=torch.Generator().manual_seed(17)).int()
    # three requests: a single token entering a page, a portion that starts and ends
    # inside pages it already had or enters, a portion that ends at a page's last slot
    slots, cleared = owned_slots(block, pages, [1, 9, 13], [0, block - 3, (-13) % block], 18)
    k_pool = torch.full((kv, pages, block, hd), 7.0, dtype=dtype, device=DEV)
    v_pool = torch.full((kv, pages, block, hd), 7.0, dtype=dtype, device=DEV)
    src = qkv.float().cpu()
    got = qkv.clone()
    ops.rope_store(got, pos.to(DEV), cos.to(DEV), sin.to(DEV), slots.to(DEV), k_pool, v_pool, t,
                   heads, kv, hd, max_pos, True)
    ops.check_status()
    rnd = P.ident if dtype == torch.float32 else P.to_bf16
    q = src[:, :heads * hd].view(t, heads, hd).transpose(0, 1)
    k = src[:, heads * hd:(heads + kv) * hd].view(t, kv, hd).transpose(0, 1)
    v = src[:, (heads + kv) * hd:].view(t, kv, hd)
    want_q = rnd(P.plain_rope(q, pos.long(), cos, sin)).transpose(0, 1).reshape(t, heads * hd)
    want_k = rnd(P.plain_rope(k, pos.long(), cos, sin)).transpose(0, 1)      # [t, kv, hd]
    assert torch.equal(got.float().cpu()[:, :heads * hd], want_q)
    kp, vp = k_pool.float().cpu(), v_pool.float().cpu()
    touched = torch.zeros(pages, block, dtype=torch.bool)
    for i in range(t):
        pg, off = int(slots[i]) // block, int(slots[i]) % block
        assert torch.equal(kp[:, pg, off], want_k[i]) and torch.equal(vp[:, pg, off], v[i])
        touched[pg, off] = True
    # the rest of a page entered in this step is cleared (what its previous owner left
    # must not reach a tensor-core kernel as 0 * NaN); everything else is untouched
    zeroed = torch.zeros(pages, block, dtype=torch.bool)
    for pg, off in cleared:
        zeroed[pg, off] = True
    assert cleared and not bool((zeroed & touched).any())
    z = zeroed[None, :, :].expand(kv, pages, block)
    assert bool((kp[z] == 0.0).all()) and bool((vp[z] == 0.0).all())
    untouched = ~(touched | zeroed)[None, :, :].expand(kv, pages, block)
    assert bool((kp[untouched] == 7.0).all()) and bool((vp[untouched] == 7.0).all())
    # a call that reads another call's cache rotates its queries and writes nothing
    k2 = k_pool.clone()
    got2 = qkv.clone()
    ops.rope_store(got2, pos.to(DEV), cos.to(DEV), sin.to(DEV), slots.to(DEV), k_pool, v_pool, t,
                   heads, kv, hd, max_pos, False)
    assert torch.equal(k2, k_pool) and torch.equal(got2[:, :heads * hd], got[:, :heads * hd])


@pytest.mark.parametrize("heads, kv, hd, block, t", [(32, 8, 128, 16, 2048), (3, 1, 32, 8, 301),
                                                     (5, 5, 48, 16, 700), (4, 2, 64, 4, 296)])
def test_rope_store_of_many_tokens_gives_the_bits_of_few_tokens(rts, heads, kv, hd, block, t):
    """Prompts take a kernel that streams rows through shared memory (bfloat16, head
    halves of whole chunks); other sizes take the ordinary one: the same bits."""
    ops = rts[torch.bfloat16].ops
    max_pos = t + 50
    pages = (t + block - 1) // block + 3
    width = (heads + 2 * kv) * hd
    cos, sin = (x.to(DEV) for x in P.plain_rotary_tables(hd, max_pos, 5e5))
    qkv = rand((t, width), torch.bfloat16, 51)
    pos = torch.randint(0, max_pos, (t,), generator=torch.Generator().manual_seed(52)).int().to(DEV)
    slots = owned_slots(block, pages, [t], [0], 53)[0].to(DEV)     # one request's next t tokens
    pools = [torch.full((kv, pages, block, hd), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    many = qkv.clone()
    ops.rope_store(many, pos, cos, sin, slots, pools[0], pools[1], t, heads, kv, hd, max_pos, True)
    ops.check_status()
    few = qkv.clone()
    for at in range(0, t, 100):
        n = min(100, t - at)
        ops.rope_store(few[at:at + n], pos[at:at + n], cos, sin, slots[at:at + n], pools[2], pools[3],
                       n, heads, kv, hd, max_pos, True)
    assert torch.equal(many[:, :heads * hd], few[:, :heads * hd])
    assert torch.equal(pools[0], pools[2]) and torch.equal(pools[1], pools[3])
    reader = qkv.clone()                                  # a call that only rotates its queries
    k_before = pools[0].clone()
    ops.rope_store(reader, pos, cos, sin, slots, pools[0], pools[1], t, heads, kv, hd, max_pos, False)
    assert torch.equal(reader[:, :heads * hd], many[:, :heads * hd]) and torch.equal(k_before, pools[0])


@pytest.mark.parametrize("heads, kv, hd, block, n_parts", [(8, 2, 128, 16, 6), (3, 1, 32, 8, 3),
                                                           (5, 5, 48, 16, 2), (4, 2, 64, 4, 1)])
def test_rope_store_reads_rows_from_the_parts_of_a_product(rts, heads, kv, hd, block, n_parts):
    """Rows left as float32 K-parts give, bit for bit, what the summed and rounded
    rows give; the keys and values in qkv itself are not needed."""
    from mini_llm_stack_b200.ops.kernels import SplitParts
    ops = rts[torch.bfloat16].ops
    assert ops.rope_takes_parts(hd)
    max_pos, pages, t = 200, 40, 9
    width = (heads + 2 * kv) * hd
    cos, sin = (x.to(DEV) for x in P.plain_rotary_tables(hd, max_pos, 5e5))
    parts = rand((n_parts, t, width), torch.float32, 31)
    summed = parts[0].clone()
    for k in range(1, n_parts):
        summed += parts[k]
    qkv = summed.to(torch.bfloat16)
    pos = torch.randint(0, max_pos, (t,), generator=torch.Generator().manual_seed(32)).int().to(DEV)
    slots = owned_slots(block, pages, [4, 5], [0, block - 2], 33)[0].to(DEV)
    pools = [torch.full((kv, pages, block, hd), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    ops.rope_store(qkv, pos, cos, sin, slots, pools[0], pools[1], t, heads, kv, hd, max_pos, True)
    got = torch.full((t, width), 3.0, dtype=torch.bfloat16, device=DEV)
    ops.rope_store(got, pos, cos, sin, slots, pools[2], pools[3], t, heads, kv, hd, max_pos, True,
                   parts=SplitParts(parts, None))
    ops.check_status()
    assert torch.equal(got[:, :heads * hd], qkv[:, :heads * hd])
    assert torch.equal(pools[0], pools[2]) and torch.equal(pools[1], pools[3])
    assert bool((got[:, heads * hd:] == 3.0).all())


# ----------------------------------------------------------------------- attention
class AttnCase:
    """Requests with given context and portion lengths over a small page pool;
    keys and values are written into the pages the cache manager hands out."""

    def __init__(self, rt, heads, kv, hd, block, ctxs, q_lens, window=None, pages=None, seed=0,
                 poison=None):
        self.rt, self.heads, self.kv, self.hd = rt, heads, kv, hd
        dtype = rt.act_dtype
        need = sum((c + block - 1) // block for c in ctxs)
        pages = pages or need + 3
        self.cache = CacheManager([PagedKV(kv, hd, window)], pages, block, len(ctxs) + 1,
                                  max(ctxs) + 8, device=DEV, kv_dtype=dtype)
        self.handle = self.cache.handles()[0]
        if poison is not None:
            self.cache.paged[0].kv.fill_(poison)
        self.k = [rand((kv, c, hd), dtype, seed + 10 * i + 1) for i, c in enumerate(ctxs)]
        self.v = [rand((kv, c, hd), dtype, seed + 10 * i + 2) for i, c in enumerate(ctxs)]
        self.q = [rand((heads, n, hd), dtype, seed + 10 * i + 3) for i, n in enumerate(q_lens)]
        self.ctxs, self.q_lens, self.window, self.block = ctxs, q_lens, window, block

    def run(self):
        rt, cache = self.rt, self.cache
        entries = []
        for i, (c, n) in enumerate(zip(self.ctxs, self.q_lens)):
            cache.admit(i)
            # everything but the portion is already stored; a window gives pages back
            assert cache.reserve(i, c - n)
            cache.commit(i, c - n)
            assert cache.reserve(i, n)
            entries.append(Entry(i, [0] * n, []))
        for i, c in enumerate(self.ctxs):
            pages = cache.pages_of(i)
            for j in range(c):
                pg = pages[j // self.block]
                if pg >= 0:
                    self.handle.k_pool[:, pg, j % self.block] = self.k[i][:, j]
                    self.handle.v_pool[:, pg, j % self.block] = self.v[i][:, j]
        step = BatchBuilder(cache, DEV, 10, 1 << 20).build(entries)
        t = step.n_tokens
        width = (self.heads + 2 * self.kv) * self.hd
        qkv = torch.zeros((t, width), dtype=rt.act_dtype, device=DEV)
        at = 0
        for q in self.q:
            n = q.shape[1]
            qkv[at:at + n, :self.heads * self.hd] = q.transpose(0, 1).reshape(n, -1)
            at += n
        out = torch.empty((t, self.heads * self.hd), dtype=rt.act_dtype, device=DEV)
        # the part plans the launches (tiles, small requests, context splits)
        mixer = GroupedQueryAttention(self.heads * self.hd, self.heads, self.kv, self.hd,
                                      self.hd ** -0.5, position=None, window=self.window)
        rt.ops.require_attention(self.hd)
        mixer._facts = rt.ops.attention_facts(self.hd)
        rt.ops.paged_attention(qkv, out, self.handle, step, self.heads, self.kv, self.hd,
                               self.hd ** -0.5, self.window or 0, plan=mixer.plan(step))
        torch.cuda.synchronize()
        return out.float().cpu()

    def want(self):
        rows = []
        for q, k, v in zip(self.q, self.k, self.v):
            o = P.plain_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(),
                                  self.hd ** -0.5, self.window)
            rows.append(o.transpose(0, 1).reshape(q.shape[1], -1))
        return torch.cat(rows)


def attn_tol(dtype, ctx=64):
    """Largest |difference| as a fraction of the largest output.  float32: a sum
    over ctx keys is off by about sqrt(ctx) roundings (in the kernel and in the
    plain reference alike); bfloat16: the probabilities and the output are
    rounded to 8 bits."""
    if dtype == torch.float32:
        return max(2e-6, 4 * math.sqrt(ctx) * 2.0 ** -24)
    return 1.2e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, hd, block", [(4, 2, 16, 4), (3, 1, 32, 8), (5, 5, 48, 16),
                                                  (8, 2, 64, 16), (8, 2, 128, 16), (32, 1, 64, 32),
                                                  (2, 1, 256, 16), (6, 3, 80, 5)])
def test_attention_mixed_batch(rts, dtype, heads, kv, hd, block):
    # whole prompts, portions after cached context, single tokens, together
    ctxs = [7, 200, 45, 128, 1, 333, 65, 64]
    q_lens = [7, 1, 45, 3, 1, 70, 1, 64]
    case = AttnCase(rts[dtype], heads, kv, hd, block, ctxs, q_lens, seed=100 + hd)
    got, want = case.run(), case.want()
    assert (got - want).abs().max().item() <= attn_tol(dtype, 333) * want.abs().max().item()


@pytest.mark.parametrize("rows", [128, 256])
@pytest.mark.parametrize("heads, kv, hd, block", [(6, 2, 64, 8), (6, 1, 128, 32), (5, 1, 64, 16)])
def test_prompt_attention_with_groups_that_do_not_divide_a_row_tile(rts, rows, heads, kv, hd, block):
    """Three, five or six query heads a kv head: a tile of 128 rows then ends inside a token's
    heads, and a chain's last token differs from row to row."""
    ops = rts[torch.bfloat16].ops
    case = AttnCase(rts[torch.bfloat16], heads, kv, hd, block, [333, 130, 700, 90], [70, 130, 211, 43],
                    seed=17 + heads)
    ops.set_attention_rows(hd, rows)
    try:
        got = case.run()
    finally:
        ops.set_attention_rows(hd, 0)
    ops.check_status()
    want = case.want()
    assert (got - want).abs().max().item() <= attn_tol(torch.bfloat16, 700) * want.abs().max().item()


@pytest.mark.parametrize("rows", [128, 256])
@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("window", [None, 200])
def test_prompt_attention_as_two_row_tiles_and_as_two_key_halves(rts, rows, hd, window):
    """The tcgen05 prompt kernel's two ways to run two chains a CTA, each forced: 256 rows
    whose two halves walk the key tiles together, or 128 rows whose keys are split in
    halves.  Requests that end inside a row tile, inside a key tile, with one chain idle,
    with chains of different length, and long enough for the rings of tiles to wrap."""
    ops = rts[torch.bfloat16].ops
    ctxs = [333, 45, 700, 64, 1300, 130]
    q_lens = [70, 45, 300, 64, 515, 33]
    case = AttnCase(rts[torch.bfloat16], 8, 2, hd, 16, ctxs, q_lens, window=window, seed=7 + hd)
    ops.set_attention_rows(hd, rows)
    try:
        got = case.run()
    finally:
        ops.set_attention_rows(hd, 0)
    ops.check_status()
    want = case.want()
    assert (got - want).abs().max().item() <= attn_tol(torch.bfloat16, 1300) * want.abs().max().item()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ctx", [1, 15, 16, 17, 64, 65, 255, 256, 257, 1000, 3000])
def test_attention_decode_at_page_and_tile_edges(rts, dtype, ctx):
    case = AttnCase(rts[dtype], 8, 2, 64, 16, [ctx, max(1, ctx - 1)], [1, 1], seed=ctx)
    got, want = case.run(), case.want()
    assert (got - want).abs().max().item() <= attn_tol(dtype, ctx) * want.abs().max().item()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unused_slots_must_not_leak(rts, dtype):
    # the reference's poisoned-slot test (tests/test_serving.py:89-108): whatever lies
    # in the pool beyond a request's keys must not reach the result
    for q_lens in ([1, 1, 1], [5, 23, 12]):
        case = AttnCase(rts[dtype], 4, 2, 32, 16, [5, 23, 12], q_lens, seed=9, poison=1e6)
        got, want = case.run(), case.want()
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= attn_tol(dtype) * want.abs().max().item()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far, ctx, q_len", [(0, 700, 1), (3, 700, 1), (257, 900, 2), (0, 600, 90),
                                             (511, 513, 1), (640, 1500, 1)])
def test_one_far_key_among_hundreds_is_found(rts, dtype, far, ctx, q_len):
    """Random data would hide a lost key: here one key far back carries all the
    weight, so the output must be that key's value."""
    case = AttnCase(rts[dtype], 4, 2, 64, 16, [ctx], [q_len], seed=3)
    q, k, v = case.q[0], case.k[0], case.v[0]
    k.mul_(0.05)
    direction = torch.ones(64, dtype=q.dtype, device=DEV)
    q[:] = direction * 4
    k[:, far] = direction * 4                      # score 16 * 64 / 8 = 128 above all others
    got, want = case.run(), case.want()
    tol = attn_tol(dtype, ctx)
    mark = v[:, far].float().cpu().repeat_interleave(2, dim=0).reshape(1, -1)   # [1, H * hd]
    assert (got - mark).abs().max().item() < 2e-2
    assert (got - want).abs().max().item() <= tol * want.abs().max().item()


@pytest.mark.parametrize("far, ctx, q_len", [(123, 8192, 1), (4097, 8192, 1), (77, 8192, 300),
                                             (8000, 8192, 130)])
def test_far_key_at_the_full_context_with_the_8b_heads(rts, far, ctx, q_len):
    """The same at 8,192 keys with 32 query heads over 8 kv heads of 128: context
    splits, many waves of tiles, the tcgen05 kernel's rings wrapping many times."""
    case = AttnCase(rts[torch.bfloat16], 32, 8, 128, 16, [ctx], [q_len], seed=7)
    q, k, v = case.q[0], case.k[0], case.v[0]
    k.mul_(0.05)
    direction = torch.ones(128, dtype=q.dtype, device=DEV)
    q[:] = direction * 3
    k[:, far] = direction * 3                      # 9 * 128 / 11.3 = 102 above all others
    got = case.run()
    rts[torch.bfloat16].ops.check_status()
    mark = v[:, far].float().cpu().repeat_interleave(4, dim=0).reshape(1, -1)
    visible = torch.arange(ctx - q_len, ctx) >= far
    assert visible.all() or far > ctx - q_len
    assert (got[visible] - mark).abs().max().item() < 3e-2


@pytest.mark.parametrize("far, q_len", [(5, 1), (33001, 1), (17, 200), (39000, 1100)])
def test_far_key_in_a_context_of_forty_thousand(rts, far, q_len):
    """A context past 2^15 keys and 2,048 pages (positions, page numbers and tile counts
    that no longer fit 15 or 16 bits): one decoded token, a short portion and a long one
    each have to find the one key that stands out."""
    ctx = 40000
    case = AttnCase(rts[torch.bfloat16], 8, 2, 128, 16, [ctx], [q_len], seed=9)
    q, k, v = case.q[0], case.k[0], case.v[0]
    k.mul_(0.05)
    direction = torch.ones(128, dtype=q.dtype, device=DEV)
    q[:] = direction * 3
    k[:, far] = direction * 3                      # 9 * 128 / 11.3 = 102 above all others
    got = case.run()
    rts[torch.bfloat16].ops.check_status()
    mark = v[:, far].float().cpu().repeat_interleave(4, dim=0).reshape(1, -1)
    visible = torch.arange(ctx - q_len, ctx) >= far
    assert bool(visible.any())
    assert (got[visible] - mark).abs().max().item() < 3e-2
    if not bool(visible.all()):                    # rows before the key: an ordinary average
        assert got[~visible].abs().max().item() < 1.0


@pytest.mark.parametrize("far, ctx, q_len", [(55, 4096, 1), (2049, 4096, 700), (4000, 4096, 97)])
def test_far_key_with_heads_of_64(rts, far, ctx, q_len):
    """The same with 32 query heads over 8 kv heads of 64 (the Llama-3.2-1B geometry): the
    tcgen05 kernel and the split kernel compiled for the other head size they take."""
    case = AttnCase(rts[torch.bfloat16], 32, 8, 64, 16, [ctx], [q_len], seed=8)
    q, k, v = case.q[0], case.k[0], case.v[0]
    k.mul_(0.05)
    direction = torch.ones(64, dtype=q.dtype, device=DEV)
    q[:] = direction * 4
    k[:, far] = direction * 4                      # 16 * 64 / 8 = 128 above all others
    got = case.run()
    rts[torch.bfloat16].ops.check_status()
    mark = v[:, far].float().cpu().repeat_interleave(4, dim=0).reshape(1, -1)
    visible = torch.arange(ctx - q_len, ctx) >= far
    assert (got[visible] - mark).abs().max().item() < 3e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window, ctx, q_len", [(10, 50, 1), (16, 64, 1), (40, 200, 30), (33, 100, 100),
                                                (64, 1000, 1), (5, 300, 17)])
def test_window_edge(rts, dtype, window, ctx, q_len):
    """The key just outside the window carries a huge score and a huge value: it
    must not count; the key just inside must."""
    case = AttnCase(rts[dtype], 4, 2, 32, 16, [ctx], [q_len], window=window, seed=5)
    q, k, v = case.q[0], case.k[0], case.v[0]
    p_last = ctx - 1
    outside = p_last - window                      # hidden from the last query
    if outside >= 0:
        k[:, outside] = q[0, -1] * 3
        v[:, outside] = 1000.0
    got, want = case.run(), case.want()
    assert got[-1].abs().max().item() < 100         # the outside key did not leak in
    # earlier queries of the portion do see that key: compare row by row
    row_scale = want.abs().max(dim=1).values.clamp(min=1.0)
    assert bool(((got - want).abs().max(dim=1).values <= attn_tol(dtype, ctx) * row_scale).all())


@pytest.mark.parametrize("heads, kv, hd", [(4, 2, 64), (8, 2, 128)])
@pytest.mark.parametrize("window, ctx, q_len", [(150, 1000, 1), (77, 700, 2), (150, 900, 130),
                                                (200, 1300, 300), (77, 520, 300), (33, 400, 1)])
def test_window_edge_with_heads_of_64_and_128(rts, heads, kv, hd, window, ctx, q_len):
    """The same on the kernels bfloat16 takes for these head sizes: tcgen05 tiles whose
    first key tile starts at a window's edge, the TMA split kernel, and their zero-fill
    of pages the window has given back (the contexts are long enough for that).  The
    windows are no multiples of a tile of keys."""
    rt = rts[torch.bfloat16]
    case = AttnCase(rt, heads, kv, hd, 16, [ctx], [q_len], window=window, seed=6)
    q, k, v = case.q[0], case.k[0], case.v[0]
    outside = ctx - 1 - window                     # hidden from the last query
    k[:, outside] = q[0, -1] * 3
    v[:, outside] = 1000.0
    got, want = case.run(), case.want()
    rt.ops.check_status()
    assert -1 in case.cache.pages_of(0)            # pages were given back before the portion
    assert got[-1].abs().max().item() < 100
    row_scale = want.abs().max(dim=1).values.clamp(min=1.0)
    assert bool(((got - want).abs().max(dim=1).values
                 <= attn_tol(torch.bfloat16, ctx) * row_scale).all())


@pytest.mark.parametrize("hd, heads, kv", [(64, 8, 2), (128, 32, 8)])
@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8, 12])
@pytest.mark.parametrize("window", [None, 700])
def test_context_splits_merge_in_clusters_and_by_kernel(rts, monkeypatch, hd, heads, kv, splits,
                                                        window):
    """Decoded tokens over contexts cut into a forced number of stretches: two to eight
    stretches are merged inside clusters of the split kernel (through the CTAs' shared
    memory), more by the merge kernel.  Every request is cut at the same multiples of
    tiles (the longest request's, shared out over the stretches): the requests are of very
    different lengths, so the shorter ones fill only their first stretches, with and
    without a window that moves each request's first tile."""
    monkeypatch.setenv("MLS_B200_SPLITS", str(splits))
    rt = rts[torch.bfloat16]
    case = AttnCase(rt, heads, kv, hd, 16, [3000, 70, 1025, 1, 640], [1, 1, 1, 1, 2], window=window,
                    seed=31)
    got, want = case.run(), case.want()
    rt.ops.check_status()
    assert bool(torch.isfinite(got).all())
    assert (got - want).abs().max().item() <= attn_tol(torch.bfloat16, 3000) * want.abs().max().item()


def test_attention_refuses_head_sizes_it_does_not_have(rts):
    with pytest.raises(KernelError, match="steps of 16"):
        rts[torch.bfloat16].ops.require_attention(40)
    with pytest.raises(KernelError, match="steps of 16"):
        rts[torch.float32].ops.require_attention(272)


@pytest.mark.parametrize("block, window", [(8, None), (16, None), (32, None), (64, None),
                                           (16, 150), (32, 333)])
def test_bf16_attention_kernels_agree_with_each_other(rts, block, window):
    """tcgen05 tiles + TMA split kernel ("auto"), mma.sync kernels with TMA loads
    ("mma"), the same with plain asynchronous copies ("no_tma") and the CUDA-core
    kernel ("simt"), on the same pages; also with a window that has given pages back."""
    rt = rts[torch.bfloat16]
    ctxs, q_lens = [500, 77, 1200, 300, 2100], [1, 77, 2, 150, 1]
    got = {}
    try:
        for impl in ("auto", "mma", "no_tma", "simt"):
            rt.ops.attention_impl = impl
            got[impl] = AttnCase(rt, 8, 2, 128, block, ctxs, q_lens, window=window,
                                 seed=21).run()
    finally:
        rt.ops.attention_impl = "auto"
    rt.ops.check_status()
    scale = got["simt"].abs().max().item()
    assert (got["auto"] - got["simt"]).abs().max().item() <= 1.2e-2 * scale
    assert (got["no_tma"] - got["simt"]).abs().max().item() <= 1.2e-2 * scale
    assert (got["mma"] - got["simt"]).abs().max().item() <= 1.2e-2 * scale
    # the two mma.sync kernels do the same arithmetic on the same tiles
    assert (got["mma"] - got["no_tma"]).abs().max().item() <= 1e-3 * scale
