"""Other parts, registered and run from a test: a mixer with state of its own, a
routed feed-forward and a learned additive position encoding.

The mixer, its architecture and its configuration are defined here; no file of
the framework knows them.  The mixer keeps a fixed-size state per request (a
decaying sum of its inputs), so it needs a state slot instead of pages; the toy
model alternates it with the framework's attention, so one model holds a paged
group and a fixed-state group.
"""

from dataclasses import asdict, dataclass

import pytest
import torch

import plain_llama as P
from engine_helpers import Replayer, assert_close, tokens_for
from mini_llm_stack_b200.config import (config_from_folder, register_architecture,
                                        unregister_architecture)
from mini_llm_stack_b200.parts import (ComposedModel, FixedState, GroupedQueryAttention,
                                       LayerCall, Mixer, OutputHead, Part, PreNormBlock,
                                       RMSNorm, RotaryPosition, SwiGLUFeedForward, TensorSpec,
                                       TokenEmbedding)
from mini_llm_stack_b200.weights import write_random_model
from safetensors.torch import load_file

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class ToyConfig:
    architecture: str = "toy_decay"
    vocab_size: int = 53
    d_model: int = 48
    n_layers: int = 3
    n_heads: int = 3
    head_dim: int = 16
    intermediate_size: int = 72
    max_seq_len: int = 128
    decay: float = 0.75
    norm_eps: float = 1e-5
    rope_theta: float = 1000.0
    dtype: str = "float32"

    @classmethod
    def from_dict(cls, raw):
        return cls(**raw)

    def to_dict(self):
        return asdict(self)


class DecayMixer(Mixer):
    """``s_t = decay * s_{t-1} + h_t``; ``out_t = W s_t``.  State: s, per request.

    A step of single tokens runs on the device alone (indexed reads and writes of the
    state, one product), so the mixer agrees to be captured into the decode graph and
    adds its own word to the graph's key; portions of prompts walk their tokens on the
    host, which is never captured."""

    decode_capturable = True

    def __init__(self, d_model, decay):
        self.d, self.decay = d_model, decay

    def decode_graph_key(self, step):
        return ("decay", self.d)

    def tensor_specs(self):
        return {"w.weight": TensorSpec((self.d, self.d))}

    def cache_spec(self):
        return FixedState((self.d,), torch.float32)

    def bind(self, tensors, runtime):
        self.runtime = runtime
        self.w = tensors["w.weight"].float()

    def forward(self, h, step, cache):
        if step.max_q_len == 1 and self.decode_capturable:
            slots = step.state_slot.long()
            s = self.decay * cache.state[slots] + h.float()
            cache.state.index_copy_(0, slots, s)
            return (s @ self.w.t()).to(h.dtype)
        out = torch.empty_like(h)
        slots = step.state_slot.tolist()
        at = 0
        for r, n in enumerate(step.q_lens):
            s = cache.state[slots[r]]
            for i in range(n):
                s = self.decay * s + h[at + i].float()
                out[at + i] = (s @ self.w.t()).to(h.dtype)
            cache.state[slots[r]] = s
            at += n
        return out


def build_toy(cfg):
    emb = TokenEmbedding(cfg.vocab_size, cfg.d_model)
    blocks = []
    for i in range(cfg.n_layers):
        if i % 2 == 0:
            mixer = DecayMixer(cfg.d_model, cfg.decay)
        else:
            mixer = GroupedQueryAttention(
                cfg.d_model, cfg.n_heads, cfg.n_heads, cfg.head_dim, cfg.head_dim ** -0.5,
                RotaryPosition(cfg.head_dim, cfg.rope_theta, cfg.max_seq_len))
        blocks.append(PreNormBlock(RMSNorm(cfg.d_model, cfg.norm_eps), mixer,
                                   RMSNorm(cfg.d_model, cfg.norm_eps),
                                   SwiGLUFeedForward(cfg.d_model, cfg.intermediate_size),
                                   names=("norm_a", "mix", "norm_b", "ffn")))
    calls = [LayerCall(i, i, True) for i in range(cfg.n_layers)]
    return ComposedModel(cfg, emb, blocks, calls, RMSNorm(cfg.d_model, cfg.norm_eps),
                         OutputHead(cfg.vocab_size, cfg.d_model, tied_to=emb))


def plain_toy(w, cfg, tokens):
    """The toy model on whole sequences with the plain parts."""
    toks = torch.as_tensor(tokens)
    S = len(tokens)
    x = w["embed.weight"][toks]
    cos, sin = P.plain_rotary_tables(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta)
    attn_cfg = dict(n_heads=cfg.n_heads, n_kv_heads=cfg.n_heads, head_dim=cfg.head_dim)
    for i in range(cfg.n_layers):
        p = f"blocks.{i}"
        h = P.plain_rmsnorm(x, w[f"{p}.norm_a.weight"], cfg.norm_eps)
        if i % 2 == 0:
            s = torch.zeros(cfg.d_model)
            rows = []
            for t in range(S):
                s = cfg.decay * s + h[t]
                rows.append(s @ w[f"{p}.mix.w.weight"].t())
            a = torch.stack(rows)
        else:
            a, _ = P.plain_mixer(h, w, f"{p}.mix", attn_cfg, cos, sin, torch.arange(S), None)
        x = x + a
        h = P.plain_rmsnorm(x, w[f"{p}.norm_b.weight"], cfg.norm_eps)
        x = x + P.plain_swiglu(h, w[f"{p}.ffn.w_gate.weight"], w[f"{p}.ffn.w_up.weight"],
                               w[f"{p}.ffn.w_down.weight"])
    return P.plain_rmsnorm(x, w["final_norm.weight"], cfg.norm_eps) @ w["embed.weight"].t()


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    register_architecture("toy_decay", ToyConfig, build_toy)
    try:
        cfg = ToyConfig()
        write_random_model(tmp_path / "toy", cfg, seed=2, norm_std=0.1)
        assert config_from_folder(tmp_path / "toy") == cfg
        w = {n: t.float().clone() for n, t in
             load_file(str(tmp_path / "toy" / "model.safetensors")).items()}
        rp = Replayer(tmp_path / "toy", "float32", num_blocks=12, max_requests=3)
        cache = rp.runner.cache
        assert len(cache.paged) == 1 and len(cache.fixed) == 1
        assert cache.fixed[0].members == [0, 2] and cache.paged[0].members == [1]
        toks = {i: tokens_for(cfg.vocab_size, n, 60 + i) for i, n in enumerate([37, 21, 50, 9])}
        # portions and single tokens of three live requests; the fourth request
        # takes over the state slot and the pages of a finished one
        rp.step([(0, 20), (1, 2)], toks)
        rp.step([(0, 1), (1, 19), (2, 30)], toks, end=[1])
        rp.step([(0, 16), (2, 1), (3, 9)], toks, end=[0, 3])
        rp.step([(2, 19)], toks, end=[2])
        for i in toks:
            assert_close(rp.logits(i), plain_toy(w, cfg, toks[i]), "float32", f"toy request {i}")
        assert cache.slots.num_free == 3
    finally:
        unregister_architecture("toy_decay")


def plain_toy_generate(w, cfg, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(plain_toy(w, cfg, toks)[-1].argmax()))
    return toks[len(prompt):]


class HostWalkingDecayMixer(DecayMixer):
    """The same mixer without the device-only path: every step reads the slots on the
    host, so it must never be captured, and says so."""

    decode_capturable = False


def build_toy_host_walking(cfg):
    model = build_toy(cfg)
    for blk in model.blocks:
        if isinstance(blk.mixer, DecayMixer):
            blk.mixer.__class__ = HostWalkingDecayMixer
    return model


@pytest.mark.parametrize("capturable", [True, False])
def test_toy_mixer_through_the_scheduler_with_graphs_and_preemption(tmp_path, capturable):
    """The toy architecture through ``LLM.generate``: so few pages that requests give
    way and are recomputed (their state slots are given back, claimed again and start
    from zero), many decode-only steps in a row, CUDA graphs on by default.  With the
    capturable mixer those steps are replayed from a graph keyed also by the mixer's
    own word; with a mixer that reads device memory on the host nothing is captured.
    Either way the tokens are the plain implementation's."""
    from mini_llm_stack_b200.engine.llm import LLM
    name = "toy_decay" if capturable else "toy_decay_host"
    register_architecture(name, ToyConfig, build_toy if capturable else build_toy_host_walking)
    try:
        cfg = ToyConfig(architecture=name)
        write_random_model(tmp_path / "toy", cfg, seed=2, norm_std=0.1)
        w = {n: t.float().clone() for n, t in
             load_file(str(tmp_path / "toy" / "model.safetensors")).items()}
        prompts = [tokens_for(cfg.vocab_size, n, 90 + n) for n in (20, 31, 7, 26)]
        llm = LLM.from_folder(tmp_path / "toy", dtype="float32", num_blocks=7, max_batch=3,
                              chunk_size=16, max_tokens_per_step=24)
        assert llm.engine.runner.cuda_graphs and llm.model.decode_capturable == capturable
        got = llm.generate(prompts, max_new_tokens=24)
        eng = llm.engine
        assert eng.scheduler.preemptions > 0
        # at least three steps in a row in which every running request decoded one token
        runs, best = 0, 0
        for n in eng.step_tokens:
            runs = runs + 1 if n <= 3 else 0
            best = max(best, runs)
        assert best >= 3
        captured = [k for k, v in eng.runner._graphs.items()
                    if k != "moved" and isinstance(v, tuple)]
        if capturable:
            assert captured and all(repr(("decay", cfg.d_model)) in repr(k) for k in captured)
        else:
            assert not captured
        for p, g in zip(prompts, got):
            assert g == plain_toy_generate(w, cfg, p, 24)
        eng.cache.check()
        assert eng.cache.slots.num_free == 3 and eng.cache.num_free_pages() == 7
    finally:
        unregister_architecture(name)


# ---------------------------------------------------------------------------------------
# another feed-forward (routed) and another position encoding (learned, additive)
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class ToyRoutedConfig:
    architecture: str = "toy_routed"
    vocab_size: int = 61
    d_model: int = 64
    n_layers: int = 2
    n_heads: int = 2
    head_dim: int = 32
    intermediate_size: int = 48
    n_experts: int = 3
    max_seq_len: int = 96
    norm_eps: float = 1e-5
    dtype: str = "float32"

    @classmethod
    def from_dict(cls, raw):
        return cls(**raw)

    def to_dict(self):
        return asdict(self)


class RoutedFeedForward(Part):
    """Top-1 routing: each token goes to the expert with the largest router logit and
    is scaled by that expert's softmax weight.  The experts are the framework's SwiGLU."""

    def __init__(self, d_model, inter, n_experts):
        self.d, self.n = d_model, n_experts
        self.experts = [SwiGLUFeedForward(d_model, inter) for _ in range(n_experts)]

    def tensor_specs(self):
        out = {"router.weight": TensorSpec((self.n, self.d))}
        for e, ex in enumerate(self.experts):
            out.update({f"experts.{e}.{n}": s for n, s in ex.tensor_specs().items()})
        return out

    def bind(self, tensors, runtime):
        self.runtime = runtime
        self.router = tensors["router.weight"].float()
        for e, ex in enumerate(self.experts):
            pre = f"experts.{e}."
            ex.bind({n[len(pre):]: t for n, t in tensors.items() if n.startswith(pre)}, runtime)

    def forward(self, h, step):
        probs = torch.softmax(h.float() @ self.router.t(), dim=-1)      # float32 router
        weight, choice = probs.max(dim=-1)
        out = torch.zeros_like(h)
        for e, ex in enumerate(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                y = ex.forward(h[rows].contiguous(), step)
                out[rows] = (y.float() * weight[rows, None]).to(h.dtype)
        return out


class LearnedPositions(TokenEmbedding):
    """``x[t] = E[token[t]] + Pos[position[t]]``: a position encoding added once."""

    def __init__(self, vocab, d_model, max_pos):
        super().__init__(vocab, d_model)
        self.max_pos = max_pos

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.d_model)),
                "positions": TensorSpec((self.max_pos, self.d_model))}

    def bind(self, tensors, runtime):
        super().bind({"weight": tensors["weight"]}, runtime)
        self.table = tensors["positions"].float()

    def forward(self, step):
        x = super().forward(step)
        x += self.table[step.positions.long()]
        return x


class NoRotation(RotaryPosition):
    """Keys and values go into the pages unrotated: cos = 1, sin = 0."""

    def bind(self, tensors, runtime):
        self.runtime = runtime
        self.cos = torch.ones(self.max_positions, self.head_dim // 2, device=runtime.device)
        self.sin = torch.zeros(self.max_positions, self.head_dim // 2, device=runtime.device)


def build_toy_routed(cfg):
    emb = LearnedPositions(cfg.vocab_size, cfg.d_model, cfg.max_seq_len)
    blocks = []
    for _ in range(cfg.n_layers):
        mixer = GroupedQueryAttention(cfg.d_model, cfg.n_heads, cfg.n_heads, cfg.head_dim,
                                      cfg.head_dim ** -0.5,
                                      NoRotation(cfg.head_dim, 1.0, cfg.max_seq_len))
        blocks.append(PreNormBlock(RMSNorm(cfg.d_model, cfg.norm_eps), mixer,
                                   RMSNorm(cfg.d_model, cfg.norm_eps),
                                   RoutedFeedForward(cfg.d_model, cfg.intermediate_size,
                                                     cfg.n_experts)))
    calls = [LayerCall(i, i, True) for i in range(cfg.n_layers)]
    return ComposedModel(cfg, emb, blocks, calls, RMSNorm(cfg.d_model, cfg.norm_eps),
                         OutputHead(cfg.vocab_size, cfg.d_model, tied_to=None))


def plain_toy_routed(w, cfg, tokens):
    toks = torch.as_tensor(tokens)
    S = len(tokens)
    x = w["embed.weight"][toks] + w["embed.positions"][:S]
    for i in range(cfg.n_layers):
        p = f"blocks.{i}"
        h = P.plain_rmsnorm(x, w[f"{p}.attn_norm.weight"], cfg.norm_eps)
        H, hd = cfg.n_heads, cfg.head_dim
        q = (h @ w[f"{p}.attn.wq.weight"].t()).view(S, H, hd).transpose(0, 1)
        k = (h @ w[f"{p}.attn.wk.weight"].t()).view(S, H, hd).transpose(0, 1)
        v = (h @ w[f"{p}.attn.wv.weight"].t()).view(S, H, hd).transpose(0, 1)
        o = P.plain_attention(q, k, v, hd ** -0.5).transpose(0, 1).reshape(S, H * hd)
        x = x + o @ w[f"{p}.attn.wo.weight"].t()
        h = P.plain_rmsnorm(x, w[f"{p}.mlp_norm.weight"], cfg.norm_eps)
        probs = torch.softmax(h @ w[f"{p}.mlp.router.weight"].t(), dim=-1)
        weight, choice = probs.max(dim=-1)
        y = torch.zeros_like(h)
        for t in range(S):
            e = int(choice[t])
            pre = f"{p}.mlp.experts.{e}"
            y[t] = weight[t] * P.plain_swiglu(h[t:t + 1], w[f"{pre}.w_gate.weight"],
                                              w[f"{pre}.w_up.weight"], w[f"{pre}.w_down.weight"])[0]
        x = x + y
    return P.plain_rmsnorm(x, w["final_norm.weight"], cfg.norm_eps) @ w["lm_head.weight"].t()


def test_routed_feed_forward_and_learned_positions_without_framework_changes(tmp_path):
    from mini_llm_stack_b200.parts import Part  # noqa: F401  (the base the toy parts use)
    register_architecture("toy_routed", ToyRoutedConfig, build_toy_routed)
    try:
        cfg = ToyRoutedConfig()
        write_random_model(tmp_path / "routed", cfg, seed=5, norm_std=0.1)
        w = {n: t.float().clone() for n, t in
             load_file(str(tmp_path / "routed" / "model.safetensors")).items()}
        w["embed.positions"] *= 10            # make the positions matter
        from safetensors.torch import save_file
        save_file({n: t.contiguous() for n, t in w.items()},
                  str(tmp_path / "routed" / "model.safetensors"))
        rp = Replayer(tmp_path / "routed", "float32", num_blocks=12, max_requests=3)
        toks = {i: tokens_for(cfg.vocab_size, n, 80 + i) for i, n in enumerate([45, 30])}
        rp.step([(0, 17), (1, 2)], toks)
        rp.step([(0, 1), (1, 28)], toks, end=[1])
        rp.step([(0, 27)], toks, end=[0])
        for i in toks:
            want = plain_toy_routed(w, cfg, toks[i])
            assert_close(rp.logits(i), want, "float32", f"routed toy, request {i}")
        # every expert is used by some token, or the test shows nothing about routing
        h = torch.randn(200, cfg.d_model)
        assert len(set((h @ w["blocks.0.mlp.router.weight"].t()).argmax(-1).tolist())) == cfg.n_experts
    finally:
        unregister_architecture("toy_routed")
