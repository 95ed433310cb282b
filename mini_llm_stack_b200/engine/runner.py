"""The step function: run a batch of (request, next tokens) from the cache.

The reference has two runner calls: ``prefill`` for one whole prompt alone
(serve/engine.py:76-105) and ``decode_step`` for n sequences of one token each
(serve/engine.py:107-157); both follow the order norm -> q,k,v -> RoPE -> write
K/V -> attend -> wo + residual -> norm -> mlp + residual and advance the
lengths once after the last layer (serve/engine.py:103,155-156).  Only
``CachedModel.logits_for`` (serve/speculative.py:53-68) feeds a portion of a
sequence against cached context.  Here there is one ``step``: any mix of
portions (from two tokens up to a whole prompt) and single decoded tokens runs
as one batch and returns float32 logits at the wanted places only.
"""

from __future__ import annotations

import os
import time

import torch

from ..cache.manager import CacheError, CacheManager
from ..config.registry import build_model, config_from_folder
from ..ops.kernels import Runtime
from ..weights.loader import device_dtype, load_tensors
from ..weights.random_init import random_tensors
from .batch import BatchBuilder

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def load_model(folder, dtype: str | None = None, device="cuda:0"):
    """Model of a folder (config.json + model.safetensors), bound to a runtime."""
    config = config_from_folder(folder)
    run_dtype = _TORCH_DTYPES[dtype or config.dtype]
    runtime = Runtime(device, run_dtype)
    model = build_model(config)
    tensors = load_tensors(folder, model.tensor_specs(), model.tied_names(), run_dtype,
                           runtime.device, aliases=model.name_aliases())
    model.bind(tensors, runtime)
    return model


def random_model(config, seed: int, norm_std: float = 0.0, dtype: str | None = None,
                 device="cuda:0", fast: bool = False):
    """Model with random weights, without a folder in between.

    The tensors are those ``write_random_model`` would store for the same
    (config, seed, norm_std).  ``fast`` draws them on the device instead (other
    values, same distribution): a billion-parameter model is then ready in
    seconds, for measurements.
    """
    from ..weights.random_init import INIT_STD
    run_dtype = _TORCH_DTYPES[dtype or config.dtype]
    runtime = Runtime(device, run_dtype)
    model = build_model(config)
    tensors = {}
    if fast:
        gen = torch.Generator(device=runtime.device).manual_seed(int(seed))
        for name, spec in model.tensor_specs().items():
            if spec.init == "normal":
                t = torch.empty(spec.shape, dtype=run_dtype, device=runtime.device)
                t.normal_(0.0, INIT_STD, generator=gen)
            else:
                t = torch.ones(spec.shape, dtype=run_dtype, device=runtime.device)
                if spec.init == "zeros":
                    t.zero_()
            tensors[name] = t
    else:
        specs = model.tensor_specs()
        for name, t in random_tensors(config, seed, norm_std):
            # what a folder would hold, then what a load would make of it
            tensors[name] = t.to(device=runtime.device,
                                 dtype=device_dtype(t.dtype, specs[name].kind, run_dtype))
    model.bind(tensors, runtime)
    return model


class _Seen:
    """A step shape that has not been captured: how often it came, and how long the host
    took to issue it against how long the GPU took to run it."""

    __slots__ = ("count", "host_ms", "events")

    def __init__(self):
        self.count, self.host_ms, self.events = 0, 0.0, None

    def timed(self, forward):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        t0 = time.perf_counter()
        out = forward()
        self.host_ms = (time.perf_counter() - t0) * 1e3
        end.record()
        self.events = (start, end)
        return out

    def host_bound(self, share: float) -> bool:
        """Whether the last timed run was bound by the host (False while it still runs)."""
        if self.events is None or not self.events[1].query():
            return False
        return self.host_ms >= share * self.events[0].elapsed_time(self.events[1])


class ModelRunner:
    """A bound model, its cache and the step function over both."""

    def __init__(self, model, num_blocks: int, block_size: int = 16, max_requests: int = 16,
                 cuda_graphs: bool = True):
        self.model = model
        self.cuda_graphs = cuda_graphs
        # MLS_B200_PROMPT_GRAPHS=0: only steps of single decoded tokens replay from graphs
        self.prompt_graphs = os.environ.get("MLS_B200_PROMPT_GRAPHS", "1") != "0"
        self._graphs: dict = {}
        self._capture_stream = None
        self.runtime = model.runtime
        cfg = model.config
        self.cache = CacheManager(
            model.cache_specs(), num_blocks=num_blocks, block_size=block_size,
            max_requests=max_requests, max_seq_len=cfg.max_seq_len,
            device=self.runtime.device, kv_dtype=self.runtime.act_dtype)
        self.handles = self.cache.handles()
        self.builder = BatchBuilder(self.cache, self.runtime.device, cfg.vocab_size,
                                    cfg.max_seq_len)
        self.steps = 0

    def reserve(self, entries: list) -> None:
        """Pages for every entry's tokens; ``CacheError`` when they run out
        (entries before the failing one keep what they were given)."""
        for e in entries:
            if not self.cache.has(e.owner):
                if not self.cache.admit(e.owner):
                    raise CacheError("no state slot is free for a new request")
            if not self.cache.reserve(e.owner, len(e.tokens)):
                raise CacheError(
                    f"out of cache pages: request {e.owner!r} needs room for "
                    f"{len(e.tokens)} more tokens, {self.cache.num_free_pages()} pages free")

    @torch.no_grad()
    def step(self, entries: list):
        """Run the entries' tokens as one batch; float32 logits [n_out, vocab].

        Pages for the tokens must be reserved.  Keys and values of the tokens
        are written into the cache layer by layer before that layer attends;
        the requests' lengths advance once, after the last layer.
        """
        ctx = self.builder.build(entries)
        if self._may_replay(ctx):
            logits = self._decode_from_graph(ctx)
        else:
            logits = self.model.forward(ctx, self.handles)
        for e in entries:
            self.cache.commit(e.owner, len(e.tokens))
        self.steps += 1
        return logits

    @torch.no_grad()
    def step_prepared(self, prepared, token_ids, device_tokens=None):
        """``step`` for a batch of single tokens whose arrays were prepared ahead
        (``BatchBuilder.prepare``) and whose token ids are known only now: as a list
        on the host, or (``device_tokens``, int32 on the device, in the order of the
        entries) still on their way from the sampler."""
        ctx = self.builder.submit(prepared, token_ids)
        if device_tokens is not None:
            ctx.token_ids.copy_(device_tokens[:ctx.n_tokens])
        if self._may_replay(ctx):
            logits = self._decode_from_graph(ctx)
        else:
            logits = self.model.forward(ctx, self.handles)
        for owner in prepared.owners:
            self.cache.commit(owner, 1)
        self.steps += 1
        return logits

    GRAPHS_KEPT = 48             # captured steps kept; the oldest goes first
    PROMPT_SHAPE_SEEN = 3        # a step with portions is captured when its shape comes this often
    HOST_BOUND = 0.25            # ... and issuing it took the host this share of its time on the GPU

    def _may_replay(self, ctx) -> bool:
        """A step of single decoded tokens, all wanted, of a model whose parts all agree
        to be captured; or any other step, if they all agree to that too."""
        if not self.cuda_graphs:
            return False
        if ctx.max_q_len == 1 and ctx.n_out == ctx.n_tokens:
            return self.model.decode_capturable
        return self.prompt_graphs and self.model.prompt_capturable

    def _decode_from_graph(self, ctx):
        """A step replayed from a CUDA graph.

        A step launches the same kernels with the same arguments whenever the requests'
        token counts, the number of wanted rows and what the parts add to the key (the
        attention's cut of the context) are the same; only the arrays the batch builder
        has just copied to the device differ, and they lie at the same addresses.  The
        first step of a kind runs eagerly (which sizes every buffer), the second is
        captured, later ones replay.  A step with portions of prompts, whose shape may
        never come again, is captured when it has come ``PROMPT_SHAPE_SEEN`` times and
        the host had a part in its time: issuing its kernels one by one took at least
        ``HOST_BOUND`` of the time the GPU spent on them (small models, portions of a few
        hundred tokens: the gaps between their kernels go away).  A large step gains nothing
        from a graph.
        """
        ops = self.runtime.ops
        moved = (ops.generation, self.builder.generation)
        if moved != self._graphs.get("moved"):
            self._graphs = {"moved": moved}      # a buffer moved: the old graphs are stale
        decoding = ctx.max_q_len == 1
        shape = ctx.n_requests if decoding else tuple(ctx.q_lens)
        key = (shape, ctx.n_out, self.model.decode_graph_key(ctx))
        entry = self._graphs.pop(key, None)      # taken out and put back: the dict's order is by use
        if not isinstance(entry, tuple):
            seen = entry or _Seen()
            seen.count += 1
            if decoding:
                capture = seen.count >= 2
            else:
                capture = seen.count >= self.PROMPT_SHAPE_SEEN and seen.host_bound(self.HOST_BOUND)
            if not capture:
                self._keep(key, seen)
                if decoding:
                    return self.model.forward(ctx, self.handles)
                return seen.timed(lambda: self.model.forward(ctx, self.handles))
            before = (ops.launches, ops.library_launches)
            graph, logits = self._capture(lambda: self.model.forward(ctx, self.handles))
            entry = (graph, logits, ops.launches - before[0], ops.library_launches - before[1])
        self._keep(key, entry)
        graph, logits, own, lib = entry
        graph.replay()
        ops.launches += own
        ops.library_launches += lib
        return logits

    def _capture(self, forward):
        """Record what ``forward`` launches into a CUDA graph, on a side stream that waits
        for the current one.  (Without
        the collector run, device-wide wait and cache flush of ``torch.cuda.graph``, which
        made a capture cost 25-55 ms: a serving run captures dozens of step shapes.)"""
        device = self.runtime.device
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device)
        current = torch.cuda.current_stream(device)
        side = self._capture_stream
        side.wait_stream(current)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            graph.capture_begin()
            try:
                out = forward()
            finally:
                graph.capture_end()
        current.wait_stream(side)
        return graph, out

    def _keep(self, key, entry) -> None:
        self._graphs[key] = entry
        while len(self._graphs) > self.GRAPHS_KEPT + 1:          # + 1: the "moved" word
            oldest = next(k for k in self._graphs if k != "moved")
            del self._graphs[oldest]

    def release(self, owner) -> None:
        if self.cache.has(owner):
            self.cache.free(owner)
