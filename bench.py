"""Decode and prefill throughput of the engine at the Llama-3-8B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W]

One JSON line: ``value`` = decoded tokens a second at batch 8 with every request
near the context length (a step = one decode step of the whole batch), timed on
the device around the step function; ``e2e`` = the same through the Python entry
point (``Engine.step``: host token lists in, sampled tokens out); ``prefill`` =
one 2,048-token prompt in one step; ``roofline`` = bytes the decode step has to
read (every weight once + the live requests' cache) over its time, against the
measured copy bandwidth; ``points`` = decode at batch 1 and 64.

Weights are random (N(0, 0.02), drawn on the device), token ids uniform; the
caches of the decode runs are filled with random keys and values instead of
being computed, which changes no byte count and no kernel.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

# the Llama-3-8B shape: 32 layers, hidden 4096, 32 / 8 heads of 128, feed-forward 14336
MODEL = dict(architecture="llama_dense", vocab_size=128256, d_model=4096, n_layers=32,
             n_heads=32, n_kv_heads=8, head_dim=128, intermediate_size=14336,
             max_seq_len=8192, rope_theta=500000.0, norm_eps=1e-5, tie_embeddings=False,
             dtype="bfloat16")
FULL_LAYERS = 32
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            raw = json.loads(p.read_text())
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if k in raw and raw[k]:
                    out[k] = float(raw[k])
            return out, "measured"
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu: str = "0"):
        """``gpu``: what ``nvidia-smi -i`` takes: the UUID of the device in use (its
        index inside this process says nothing on a machine with several GPUs)."""
        self.rows, self.proc, self.thread, self.gpu = [], None, None, gpu

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self) -> int:
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, lo: int = 0, hi: int | None = None) -> dict:
        rows = [r for r in self.rows[lo:hi] if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            rows = [r for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower() == "active" for r in rows)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows),
                "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def device_uuid(torch) -> str:
    """The UUID of cuda:0 of this process, in nvidia-smi's spelling ("0" if unknown)."""
    try:
        u = str(torch.cuda.get_device_properties(0).uuid)
        return u if u.startswith("GPU-") else "GPU-" + u
    except Exception:                              # noqa: BLE001 (older torch: no uuid)
        return "0"


def weight_bytes(cfg, layers: int) -> int:
    d, hd = cfg["d_model"], cfg["head_dim"]
    per_layer = ((cfg["n_heads"] + 2 * cfg["n_kv_heads"]) * hd * d + d * cfg["n_heads"] * hd
                 + 3 * cfg["intermediate_size"] * d + 2 * d)
    return 2 * (per_layer * layers + cfg["vocab_size"] * d + d)


def kv_bytes_per_token(cfg, layers: int) -> int:
    return 2 * 2 * cfg["n_kv_heads"] * cfg["head_dim"] * layers


def prefill_flops(cfg, layers: int, t: int) -> float:
    d, hd = cfg["d_model"], cfg["head_dim"]
    lin = ((cfg["n_heads"] + 2 * cfg["n_kv_heads"]) * hd * d + d * cfg["n_heads"] * hd
           + 3 * cfg["intermediate_size"] * d)
    attn = 2 * 2 * cfg["n_heads"] * hd * (t * (t + 1) / 2)       # QK^T and PV, causal
    return layers * (2.0 * lin * t + attn) + 2.0 * cfg["vocab_size"] * d


# Llama-3.2-1B shape and Llama-2-7B shape, for the serving workloads
MODEL_1B = dict(architecture="llama_dense", vocab_size=128256, d_model=2048, n_layers=16,
                n_heads=32, n_kv_heads=8, head_dim=64, intermediate_size=8192, max_seq_len=8192,
                rope_theta=500000.0, norm_eps=1e-5, tie_embeddings=True, dtype="bfloat16")
MODEL_7B = dict(architecture="llama_dense", vocab_size=32000, d_model=4096, n_layers=32,
                n_heads=32, n_kv_heads=32, head_dim=128, intermediate_size=11008,
                max_seq_len=4096, rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=False,
                dtype="bfloat16")


def serve_workload(name: str, short: bool = False) -> dict:
    """Requests through the scheduler: chunked prompts beside decoding requests.

    mixed_1b: 64 requests at once, prompts of 16..4096 tokens (log-uniform), 256 new
    tokens each, Llama-3.2-1B shape.  poisson_7b: 128 requests arriving as a Poisson
    process, prompts of 128..2048 tokens, 128..512 new tokens, Llama-2-7B shape, with
    so few pages that requests are preempted and recomputed.  ``short``: a quarter of
    the requests (and of the new tokens of mixed_1b), for the decode line's ``points``.
    Returns the workload's line.
    """
    import random

    import torch

    sys.path.insert(0, str(ROOT))
    from mini_llm_stack_b200.config import config_from_dict
    from mini_llm_stack_b200.engine.engine import Engine
    from mini_llm_stack_b200.engine.runner import random_model

    rng = random.Random(7)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    if name == "mixed_1b":
        raw, max_batch, budget, n_req = MODEL_1B, 64, 4096, 16 if short else 64
        lens = [int(round(16 * (4096 / 16) ** rng.random())) for _ in range(n_req)]
        outs = [64 if short else 256] * n_req
        arrivals = [0.0] * n_req
        num_blocks = sum((a + b) // PAGE + 2 for a, b in zip(lens, outs))
    else:
        raw, max_batch, budget, n_req = MODEL_7B, 64, 4096, 32 if short else 128
        lens = [rng.randint(128, 2048) for _ in range(n_req)]
        outs = [rng.randint(128, 512) for _ in range(n_req)]
        t, arrivals = 0.0, []
        for _ in range(n_req):
            t += rng.expovariate(16.0)              # 16 requests a second
            arrivals.append(t)
        # room for about a third of the tokens all requests would hold at their ends
        num_blocks = sum((a + b) // PAGE + 1 for a, b in zip(lens, outs)) // 3
    cfg = config_from_dict(raw)
    model = random_model(cfg, seed=0, device=dev, fast=True)
    engine = Engine(model, num_blocks=num_blocks, block_size=PAGE, max_batch=max_batch,
                    max_tokens_per_step=budget, chunk_size=2048)
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lens]
    # warm-up: compile, size buffers, capture graphs
    for p in prompts[:2]:
        engine.submit(p[:64], max_new_tokens=4)
    engine.run_until_done()
    engine.finished.clear()
    engine.scheduler.preemptions = 0
    engine.step_tokens.clear()

    torch.cuda.synchronize()
    t0 = time.perf_counter()
    reqs, nxt = [], 0
    while nxt < n_req or engine.scheduler.has_work():
        now = time.perf_counter() - t0
        while nxt < n_req and arrivals[nxt] <= now:
            reqs.append(engine.submit(prompts[nxt], max_new_tokens=outs[nxt]))
            nxt += 1
        if engine.scheduler.has_work():
            engine.step()
        else:
            time.sleep(max(0.0, arrivals[nxt] - now))
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    model.runtime.ops.check_status()
    engine.cache.check()
    assert all(len(r.generated) == o for r, o in zip(reqs, outs))
    ttft = sorted(r.first_token_time - r.arrive_time for r in reqs)
    tpot = sorted((r.finish_time - r.first_token_time) / max(1, len(r.generated) - 1) for r in reqs)
    new_tokens = sum(outs)
    line = {
        "metric": f"served tokens/s, {name}", "value": round(new_tokens / wall, 1),
        "unit": "tokens/s", "n_gpus": 1, "impl": "ours", "dtype": "bf16", "data": "synthetic",
        "wall_s": round(wall, 3), "requests": n_req, "prompt_tokens": sum(lens),
        "new_tokens": new_tokens, "steps": len(engine.step_tokens),
        "mean_tokens_per_step": round(sum(engine.step_tokens) / len(engine.step_tokens), 1),
        "preemptions": engine.scheduler.preemptions,
        "ttft_s": {"p50": round(ttft[len(ttft) // 2], 4), "p99": round(ttft[-2], 4)},
        "tpot_ms": {"p50": round(tpot[len(tpot) // 2] * 1e3, 3), "p99": round(tpot[-2] * 1e3, 3)},
        "config": {"model": name, "device": torch.cuda.get_device_name(0),
                   "layers": raw["n_layers"], "hidden": raw["d_model"],
                   "heads": raw["n_heads"], "kv_heads": raw["n_kv_heads"],
                   "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"],
                   "vocab": raw["vocab_size"], "max_batch": max_batch, "token_budget": budget,
                   "page_size": PAGE, "num_blocks": num_blocks},
    }
    del engine, model
    torch.cuda.empty_cache()
    return line


def correctness_gate() -> None:
    """Nothing is timed before the engine has generated the right tokens: a tiny
    random model in float32 and in bfloat16 against the plain implementation (the
    reference's benchmarks are gated the same way: kaggle/kaggle_bench.py:46-54)."""
    import contextlib
    import io

    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry

    with contextlib.redirect_stdout(io.StringIO()):
        entry.smoke()


def reference_arm(args) -> int:
    """The unmodified reference through its own engine; nothing of this package."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("reference_arm",
                                                  ROOT / "baseline" / "reference_arm.py")
    arm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(arm)
    if args.gpus != 1:
        print(json.dumps(arm.unavailable("the reference's serving engine runs on one GPU")))
        return 0
    clocks = None
    try:
        import torch
        if torch.cuda.is_available():
            clocks = ClockSampler(device_uuid(torch))
            clocks.start()
    except Exception:                              # noqa: BLE001
        clocks = None
    # the arm runs the headline shape (Llama-3-8B): its own defaults where none was given
    line = arm.run(max(1, args.steps), max(3, args.warmup), args.batch,
                   args.context or MODEL["max_seq_len"], args.layers or MODEL["n_layers"],
                   not args.no_points)
    if clocks is not None:
        clocks.stop()
        if "unavailable" not in line:
            line["clocks"] = clocks.summary()
    print(json.dumps(line))
    return 0


def write_timeline(args, torch, runner, cache, ops, ctx, rand_tokens, Entry) -> int:
    """Start and end of every kernel of a decode step and of a prefill step.

    Kernels overlap where one was launched under its predecessor, which a list of
    durations cannot show.  Times are relative to the step's first kernel; numbers
    taken under the profiler are for reading the schedule, not for reporting."""
    from torch.autograd import DeviceType
    from torch.profiler import ProfilerActivity, profile

    ids = [f"t{i}" for i in range(args.batch)]
    for r in ids:
        cache.admit(r)
        assert cache.reserve(r, ctx - 16)
        cache.commit(r, ctx - 16)
    out = torch.empty(args.batch, dtype=torch.int32, device="cuda:0")

    def decode():
        e = [Entry(r, [5], [0]) for r in ids]
        runner.reserve(e)
        ops.sample(runner.step(e), None, None, out)

    def prefill():
        e = [Entry("prefill", rand_tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])]
        runner.reserve(e)
        runner.step(e)
        runner.release("prefill")

    def prefill_tail():
        # the last portion of a prompt of four: three portions' keys are in the cache already
        cache.admit("tail")
        assert cache.reserve("tail", 3 * PREFILL_TOKENS)
        cache.commit("tail", 3 * PREFILL_TOKENS)
        e = [Entry("tail", rand_tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])]
        runner.reserve(e)
        runner.step(e)
        runner.release("tail")

    lines = []
    steps = [("decode step", decode, 6), ("prefill step", prefill, 3)]
    if cache.num_blocks >= cache.pages_for(4 * PREFILL_TOKENS):
        steps.append((f"last {PREFILL_TOKENS} tokens of a prompt of {4 * PREFILL_TOKENS}",
                      prefill_tail, 2))
    for name, fn, warm in steps:
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn()
            torch.cuda.synchronize()
        evs = sorted((ev.time_range.start, ev.time_range.end, ev.name)
                     for ev in prof.events() if ev.device_type == DeviceType.CUDA)
        if fn is decode:
            for r in ids:
                runner.release(r)
        t0 = evs[0][0]
        lines.append(f"# {name}: batch {args.batch}, context {ctx}, {args.layers} layers, "
                     f"{len(evs)} kernels, {evs[-1][1] - t0:.1f} us")
        lines.append("start_us end_us dur_us kernel")
        for a, b, n in evs:
            short = n.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
            lines.append(f"{a - t0:8.1f} {b - t0:8.1f} {b - a:7.1f} {short[:60]}")
    with open(args.timeline, "w") as f:
        f.write("\n".join(lines) + "\n")
    print(json.dumps({"timeline": args.timeline, "lines": len(lines)}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="8b", choices=["8b", "1b", "7b"],
                    help="layer sizes of the decode line: Llama-3-8B (the contract's), "
                         "Llama-3.2-1B or Llama-2-7B shape")
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--no-serving", action="store_true",
                    help="skip the short serving workloads of points.served_*")
    ap.add_argument("--timeline", default=None, metavar="FILE",
                    help="instead of timing, record when each kernel of one decode step and of "
                         "one prefill step starts and ends (torch.profiler) and write the table "
                         "to FILE; use few --layers")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed_1b", "poisson_7b"],
                    help="decode: the contract's line; the others serve a request mix through "
                         "the scheduler and print their own line")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    import torch

    try:
        correctness_gate()
    except Exception as exc:                       # noqa: BLE001
        print(f"bench.py: the correctness gate failed, nothing is timed: "
              f"{type(exc).__name__}: {exc}", file=sys.stderr)
        return 1
    if args.workload != "decode":
        print(json.dumps(serve_workload(args.workload)))
        return 0

    sys.path.insert(0, str(ROOT))
    from mini_llm_stack_b200.config import config_from_dict
    from mini_llm_stack_b200.engine.batch import Entry
    from mini_llm_stack_b200.engine.engine import Engine
    from mini_llm_stack_b200.engine.runner import random_model

    pk, pk_src = peaks()
    shape = {"8b": MODEL, "1b": MODEL_1B, "7b": MODEL_7B}[args.shape]
    full_layers = shape["n_layers"]
    if args.layers is None:
        args.layers = full_layers
    if args.context is None:
        args.context = shape["max_seq_len"]
    raw = dict(shape, n_layers=args.layers)
    cfg = config_from_dict(raw)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    model = random_model(cfg, seed=0, device=dev, fast=True)
    ops = model.runtime.ops
    ctx = min(args.context, cfg.max_seq_len)
    max_b = max(args.batch, 1 if args.no_points else 64)
    pages_per_req = (ctx + PAGE - 1) // PAGE
    # room for every decoding request at its full context, and for the prompt of the prefill line
    engine = Engine(model, num_blocks=max(max_b * pages_per_req, PREFILL_TOKENS // PAGE) + 8,
                    block_size=PAGE,
                    max_batch=max_b, max_tokens_per_step=max(PREFILL_TOKENS, max_b),
                    chunk_size=PREFILL_TOKENS)
    runner, cache = engine.runner, engine.cache
    for g in cache.paged:                       # keys and values as a prefill would leave them
        for m in range(g.kv.shape[0]):
            g.kv[m].normal_(0.0, 1.0)
    gen = torch.Generator().manual_seed(1)

    def rand_tokens(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    if args.timeline:
        return write_timeline(args, torch, runner, cache, ops, ctx, rand_tokens, Entry)

    clocks = ClockSampler(device_uuid(torch))
    clocks.start()

    def timed(fn, n_warm, n_timed):
        for _ in range(n_warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = ops.launches
        e0.record()
        for _ in range(n_timed):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ops.check_status()           # a kernel that refused its input or gave up a wait: no number
        return e0.elapsed_time(e1) / n_timed, (ops.launches - l0)

    # ------------------------------------------------------------------ prefill
    def prefill_once():
        toks = rand_tokens(PREFILL_TOKENS)
        e = [Entry("prefill", toks, [PREFILL_TOKENS - 1])]
        runner.reserve(e)
        runner.step(e)
        runner.release("prefill")

    # ------------------------------------------------------------------- decode
    def decode_run(batch, n_warm, n_timed, end=None, temperature=0.0):
        """Device time of one decode step with ``batch`` requests that end at ``end``
        (the context length by default); every row sampled at ``temperature`` if that
        is positive, else by arg max."""
        torch.cuda.synchronize()
        time.sleep(1.0)                         # every point starts from a GPU at rest (see below)
        start = (end or ctx) - (n_warm + n_timed)
        ids = [f"d{batch}_{i}" for i in range(batch)]
        for r in ids:
            cache.admit(r)
            assert cache.reserve(r, start)
            cache.commit(r, start)              # the cache holds random keys and values
        last = [rand_tokens(1)[0] for _ in ids]
        out = torch.empty(batch, dtype=torch.int32, device=dev)
        temps = us = None
        if temperature > 0:
            temps = torch.full((batch,), float(temperature), dtype=torch.float32, device=dev)
            us = torch.rand(batch, dtype=torch.float32, device=dev)

        def one():
            e = [Entry(r, [t], [0]) for r, t in zip(ids, last)]
            runner.reserve(e)
            logits = runner.step(e)
            ops.sample(logits, temps, us, out)

        ms, launches = timed(one, n_warm, n_timed)
        mean_ctx = start + n_warm + (n_timed + 1) / 2
        for r in ids:
            runner.release(r)
        return ms, launches, mean_ctx

    mark0 = clocks.mark()
    # the decode line and the decode points first: the prompt steps that follow run under the
    # power cap, and decode steps timed right after them came out 1.2 % slower (4.46 against
    # 4.41 ms at batch 8, 6 % at batch 1; a second's pause between the two brought the times back)
    ms, launches, mean_ctx = decode_run(args.batch, warmup, steps)
    value = args.batch / ms * 1e3
    step_bytes = weight_bytes(raw, args.layers) + args.batch * mean_ctx * kv_bytes_per_token(
        raw, args.layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    points = {}
    if not args.no_points:
        for b in (1, 64):
            pms, _, _ = decode_run(b, 3, max(8, steps // 4))
            points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
        for b in (8, 64):                        # every row drawn at temperature 0.8
            pms, _, _ = decode_run(b, 3, max(8, steps // 4), temperature=0.8)
            points[f"decode_b{b}_temperature"] = round(b / pms * 1e3, 1)
        if ctx > 1024:                           # the same three batches early in a sequence
            for b in (1, 8, 64):
                pms, _, _ = decode_run(b, 3, max(8, steps // 4), end=1024)
                points[f"decode_b{b}_ctx1024"] = round(b / pms * 1e3, 1)

    # The prompt steps start from a rested GPU, as the decode line did: what ran before leaves
    # its mark for about a second (clocks under the power cap).  The median of single steps:
    # the first run at boost clocks, later ones under the power cap.
    torch.cuda.synchronize()
    time.sleep(1.0)
    prefill_ms = sorted(timed(prefill_once, 1 if i else 3, 1)[0] for i in range(9))[4]
    pf = prefill_flops(raw, args.layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3),
               "frac": round(pf / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    if not args.no_points:
        def prefill_in_four():                   # the same prompt in four portions of 512
            toks = rand_tokens(PREFILL_TOKENS)
            for at in range(0, PREFILL_TOKENS, 512):
                e = [Entry("prefill", toks[at:at + 512], [511])]
                runner.reserve(e)
                runner.step(e)
            runner.release("prefill")

        four_ms = sorted(timed(prefill_in_four, 1, 1)[0] for i in range(5))[2]
        points["prefill_4x512"] = round(PREFILL_TOKENS / four_ms * 1e3, 1)

    # ---------------------------------------------------- end to end (Engine API)
    # every request must still be decoding when the last one has finished its
    # prompt: the first to finish decodes during the others' portions
    portions = args.batch * (-(-ctx // PREFILL_TOKENS))
    max_new = portions + warmup + steps + 4
    prompt_len = ctx - max_new
    reqs = [engine.submit(rand_tokens(prompt_len), max_new_tokens=max_new)
            for _ in range(args.batch)]
    while any(r.remaining > 1 or not r.generated for r in reqs):
        engine.step()                            # prompts in portions, untimed
    torch.cuda.synchronize()
    time.sleep(1.0)                              # the prompts' mark on the clocks fades, as above
    for _ in range(warmup):
        engine.step()
    assert len(engine.running) == args.batch
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n0 = sum(len(r.generated) for r in reqs)
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    ops.check_status()
    e2e_tokens = sum(len(r.generated) for r in reqs) - n0
    assert len(engine.running) == args.batch and e2e_tokens == steps * args.batch
    h2d = runner.builder.last_bytes
    mark2 = clocks.mark()
    clocks.stop()
    if not args.no_points and not args.no_serving:
        # the other two workloads of the baseline's list, in short form, through the
        # scheduler (their models need the memory this one holds)
        del engine, runner, cache, model, reqs
        torch.cuda.empty_cache()
        for key, name in (("served_1b", "mixed_1b"), ("served_7b", "poisson_7b")):
            w = serve_workload(name, short=True)
            points[key] = w["value"]
            points[key + "_preemptions"] = w["preemptions"]

    line = {
        "metric": f"decode tok/s at batch {args.batch}, "
                  f"{ {'8b': 'Llama-3-8B', '1b': 'Llama-3.2-1B', '7b': 'Llama-2-7B'}[args.shape]} "
                  f"shape, context {ctx} "
                  "(batch 1/64 in points; prefill tok/s at 2,048 tokens in prefill)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": {"8b": "llama-3-8b-shape", "1b": "llama-3.2-1b-shape",
                             "7b": "llama-2-7b-shape"}[args.shape], "layers": args.layers,
                   "layers_of_config": full_layers, "hidden": raw["d_model"],
                   "heads": raw["n_heads"], "kv_heads": raw["n_kv_heads"],
                   "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"],
                   "vocab": raw["vocab_size"], "global_batch": args.batch, "seq_len": ctx,
                   "page_size": PAGE, "weights": "random N(0,0.02)", "parallelism": "none",
                   "l2": "inputs larger than L2 (weights and cache are read once a step)",
                   "peaks": pk_src, "device": torch.cuda.get_device_name(0),
                   "gate": "tiny model against the plain implementation: passed"},
        "e2e": {"value": round(e2e_tokens / e2e_s, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(h2d),
                # the sampled tokens and the kernels' status word
                "d2h_bytes_per_step": 4 * args.batch + 4},
        "gpu_launches": int(launches),
        "library_gemm_launches": int(getattr(ops, "library_launches", 0)),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(mark0, mark2),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
