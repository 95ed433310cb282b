"""Generation through the entry points on the GPU, against the plain implementation."""

import subprocess
import sys
from pathlib import Path

import pytest

import plain_llama as P
from engine_helpers import RND, make_folder, tokens_for
from mini_llm_stack_b200.engine.llm import LLM

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gen_models")
    out = {(k, d): make_folder(tmp, k, d) for k in "ABC" for d in ("float32", "bfloat16")}
    # heads of 64 and 128: bfloat16 runs go through the tcgen05 / TMA attention kernels,
    # the fused gate-up product and the weight-major products of large models
    out.update({(k, "bfloat16"): make_folder(tmp, k, "bfloat16") for k in "DE"})
    return out


def assert_tokens_are_maxima(w, cfg, prompt, generated, what=""):
    """Every generated token is, within the bfloat16 comparisons' tolerance, a largest
    logit of the plain implementation run on the sequence the engine itself produced
    (two runs may part at a near tie, so the tokens are not compared with each other)."""
    logits = P.plain_forward(w, cfg, list(prompt) + list(generated), RND["bfloat16"])
    for i, tok in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - 1e-2 * row.abs().max(), (what, i, tok)


def test_greedy_generation_matches_plain_token_for_token(folders):
    # tiny-A: 3 prompts of 5/17/33 tokens, 16 new tokens each, float32
    folder, cfg, w = folders[("A", "float32")]
    prompts = [tokens_for(256, n, 20 + n) for n in (5, 17, 33)]
    llm = LLM.from_folder(folder, dtype="float32", num_blocks=32, max_batch=4)
    got = llm.generate(prompts, max_new_tokens=16)
    for p, g in zip(prompts, got):
        assert g == P.plain_generate(w, cfg, p, 16)


def test_temperature_sampling_with_chunks_and_small_pages(folders):
    # tiny-B: 4 prompts of 1/9/40/77, portions of 16, pages of 8, temperature 0.8
    folder, cfg, w = folders[("B", "float32")]
    prompts = [tokens_for(97, n, 30 + n) for n in (1, 9, 40, 77)]
    llm = LLM.from_folder(folder, dtype="float32", num_blocks=64, block_size=8, max_batch=4,
                          chunk_size=16, max_tokens_per_step=40)
    got = llm.generate(prompts, max_new_tokens=12, temperature=0.8, seed=5)
    for i, (p, g) in enumerate(zip(prompts, got)):
        assert g == P.plain_generate(w, cfg, p, 12, temperature=0.8, seed=5, request=i)
    assert max(llm.engine.step_tokens) <= 40
    # the same requests alone, one at a time, draw the same tokens
    for i, p in enumerate(prompts):
        solo = LLM.from_folder(folder, dtype="float32", num_blocks=64, block_size=8)
        solo.engine._next_id = i
        assert solo.generate([p], max_new_tokens=12, temperature=0.8, seed=5)[0] == got[i]


@pytest.mark.parametrize("temperature", [0.0, 0.7])
def test_running_out_of_pages_does_not_change_the_output(folders, temperature):
    folder, cfg, w = folders[("C", "float32")]
    prompts = [tokens_for(301, n, 50 + n) for n in (20, 31, 7, 44, 12, 26)]
    roomy = LLM.from_folder(folder, dtype="float32", num_blocks=64, max_batch=6)
    want = roomy.generate(prompts, max_new_tokens=24, temperature=temperature, seed=3)
    assert roomy.engine.scheduler.preemptions == 0
    tight = LLM.from_folder(folder, dtype="float32", num_blocks=12, max_batch=6, chunk_size=24)
    got = tight.generate(prompts, max_new_tokens=24, temperature=temperature, seed=3)
    assert tight.engine.scheduler.preemptions > 0
    assert got == want
    assert tight.engine.cache.num_free_pages() == 12
    tight.engine.cache.check()
    if temperature == 0.0:
        assert got[2] == P.plain_generate(w, cfg, prompts[2], 24)


def test_bfloat16_greedy_tokens_are_maxima_of_the_plain_logits(folders):
    folder, cfg, w = folders[("B", "bfloat16")]
    prompts = [tokens_for(97, n, 70 + n) for n in (3, 50)]
    llm = LLM.from_folder(folder, dtype="bfloat16", num_blocks=32)
    got = llm.generate(prompts, max_new_tokens=10)
    for p, g in zip(prompts, got):
        logits = P.plain_forward(w, cfg, p + g, RND["bfloat16"])
        for i, tok in enumerate(g):
            row = logits[len(p) - 1 + i]
            assert row[tok] >= row.max() - 1e-2 * row.abs().max()


def test_eos_and_long_decoding(folders):
    folder, cfg, w = folders[("A", "float32")]
    p = tokens_for(256, 11, 99)
    ref = P.plain_generate(w, cfg, p, 200)
    llm = LLM.from_folder(folder, dtype="float32", num_blocks=32)
    assert llm.generate([p], max_new_tokens=200)[0] == ref        # 200 decoded tokens
    eos = ref[7]
    cut = ref[:ref.index(eos) + 1]
    assert llm.generate([p], max_new_tokens=200, eos=eos)[0] == cut


def test_command_line_chat(folders, tmp_path):
    folder, cfg, w = folders[("A", "float32")]
    p = tokens_for(256, 9, 4)
    want = P.plain_generate(w, cfg, p, 8)
    proc = subprocess.run(
        [sys.executable, "-m", "mini_llm_stack_b200.api", "chat", "--model", str(folder),
         "--dtype", "float32", "--token-ids", ",".join(map(str, p)), "--max-new", "8"],
        capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.strip().endswith(f"-> {','.join(map(str, want))!r}")
    # text goes in and out as bytes when the vocabulary has 256 entries
    proc = subprocess.run(
        [sys.executable, "-m", "mini_llm_stack_b200.api", "chat", "--model", str(folder),
         "--dtype", "float32", "-p", "kernel ", "--max-new", "5"],
        capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.startswith("'kernel ' -> ")


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_steps_launched_ahead_give_the_same_tokens(folders, temperature):
    """The next decode step starts before the host has read this step's tokens.  Requests
    that end on an end token (known one step late), by count, and one that arrives while
    a step is already on its way must come out as without launching ahead."""
    folder, cfg, w = folders[("B", "float32")]
    prompts = [tokens_for(97, n, 70 + n) for n in (3, 14, 29, 8)]
    free_run = [P.plain_generate(w, cfg, p, 40, temperature=temperature, seed=9, request=i)
                for i, p in enumerate(prompts)]
    # end tokens that do occur: request 0 ends early, request 2 in the middle
    eos = {0: free_run[0][5], 2: free_run[2][17]}
    news = {0: 40, 1: 23, 2: 40, 3: 40}

    def run(launch_ahead):
        llm = LLM.from_folder(folder, dtype="float32", num_blocks=64, block_size=8, max_batch=4,
                              launch_ahead=launch_ahead)
        eng = llm.engine
        reqs = [eng.submit(prompts[i], news[i], eos.get(i), temperature, 9) for i in range(3)]
        late = None
        while eng.step():
            if late is None and eng.steps == 6:           # a step may be on the device already
                late = eng.submit(prompts[3], news[3], None, temperature, 9)
        assert late is not None and not eng.step()
        eng.model.runtime.ops.check_status()
        eng.cache.check()
        assert eng.cache.num_free_pages() == 64
        return [list(r.generated) for r in reqs + [late]], eng

    ahead, eng = run(True)
    plain, _ = run(False)
    assert ahead == plain
    for i, got in enumerate(ahead):
        want = free_run[i][:news[i]]
        if i in eos:
            want = want[:want.index(eos[i]) + 1]
        assert got == want
    assert eng.launch_ahead


def test_many_requests_arriving_ending_and_giving_way_with_steps_launched_ahead(folders):
    """Forty requests with random lengths, end tokens and arrival steps over so few pages
    that some give way: launching ahead must not change a token, lose a page or a slot."""
    import random
    folder, cfg, w = folders[("C", "float32")]
    rng = random.Random(11)
    jobs = []
    for i in range(40):
        prompt = tokens_for(301, rng.randint(1, 60), 200 + i)
        jobs.append(dict(prompt=prompt, new=rng.randint(1, 40), eos=rng.choice([None, None, rng.randrange(301)]),
                         at=rng.randint(0, 120), temperature=rng.choice([0.0, 0.8])))

    def run(launch_ahead):
        llm = LLM.from_folder(folder, dtype="float32", num_blocks=20, max_batch=6, chunk_size=24,
                              max_tokens_per_step=48, launch_ahead=launch_ahead)
        eng = llm.engine
        reqs = [None] * len(jobs)
        step = 0
        while True:
            for i, j in enumerate(jobs):
                if j["at"] == step:
                    eng._next_id = i
                    reqs[i] = eng.submit(j["prompt"], j["new"], j["eos"], j["temperature"], 4)
            more = eng.step()
            step += 1
            if not more and all(r is not None for r in reqs):
                break
            assert step < 5000
        eng.model.runtime.ops.check_status()
        eng.cache.check()
        assert eng.cache.num_free_pages() == 20 and eng.cache.slots.num_free == 6
        return [list(r.generated) for r in reqs], eng.scheduler.preemptions

    ahead, pre_a = run(True)
    plain, pre_p = run(False)
    assert ahead == plain
    assert pre_a > 0 and pre_p > 0                        # pages did run out
    for i in (0, 7, 19, 33):
        j = jobs[i]
        want = P.plain_generate(w, cfg, j["prompt"], j["new"], temperature=j["temperature"], seed=4,
                                request=i)
        if j["eos"] is not None and j["eos"] in want:
            want = want[:want.index(j["eos"]) + 1]
        assert ahead[i] == want


# --------------------------------------------------------------------------------------
# bfloat16 through the scheduler, on the kernels large models use (heads of 64 and 128)
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("key", ["D", "E"])
def test_bfloat16_running_out_of_pages(folders, key):
    """Requests give way and are recomputed: the recomputation goes through the prompt
    kernels where the first run decoded, so the bits differ within rounding and every
    token is still a maximum of the plain logits."""
    folder, cfg, w = folders[(key, "bfloat16")]
    vocab = cfg["vocab_size"]
    prompts = [tokens_for(vocab, n, 50 + n) for n in (70, 131, 7, 44, 150, 26)]
    tight = LLM.from_folder(folder, dtype="bfloat16", num_blocks=30, max_batch=6, chunk_size=96,
                            max_tokens_per_step=128)
    got = tight.generate(prompts, max_new_tokens=40)
    assert tight.engine.scheduler.preemptions > 0
    tight.engine.cache.check()
    assert tight.engine.cache.num_free_pages() == 30
    for i, (p, g) in enumerate(zip(prompts, got)):
        assert len(g) == 40
        assert_tokens_are_maxima(w, cfg, p, g, f"tiny-{key} request {i}")


@pytest.mark.parametrize("key", ["D", "E"])
def test_bfloat16_steps_launched_ahead(folders, key):
    """Launching the next decode step before this one's tokens are on the host: end
    tokens known a step late, an end by count, a late arrival; bfloat16, CUDA graphs."""
    folder, cfg, w = folders[(key, "bfloat16")]
    vocab = cfg["vocab_size"]
    prompts = [tokens_for(vocab, n, 70 + n) for n in (3, 140, 29, 65)]
    news = {0: 40, 1: 23, 2: 40, 3: 30}

    def run(launch_ahead, eos):
        llm = LLM.from_folder(folder, dtype="bfloat16", num_blocks=64, max_batch=4,
                              launch_ahead=launch_ahead)
        eng = llm.engine
        reqs = [eng.submit(prompts[i], news[i], eos.get(i)) for i in range(3)]
        late = None
        while eng.step():
            if late is None and eng.steps == 6:
                late = eng.submit(prompts[3], news[3], None)
        assert late is not None and not eng.step()
        eng.cache.check()
        return [list(r.generated) for r in reqs + [late]], eng

    free, _ = run(False, {})
    eos = {0: free[0][5], 2: free[2][17]}          # end tokens that do occur
    ahead, eng = run(True, eos)
    assert any(k != "moved" and isinstance(v, tuple) for k, v in eng.runner._graphs.items())
    for i, g in enumerate(ahead):
        assert_tokens_are_maxima(w, cfg, prompts[i], g, f"tiny-{key} request {i}")
        if i in eos:
            assert g[-1] == eos[i] or len(g) == news[i]
            assert eos[i] not in g[:-1]
        else:
            assert len(g) == news[i]


def test_bfloat16_chunked_prompts_with_pages_of_eight(folders):
    folder, cfg, w = folders[("D", "bfloat16")]
    prompts = [tokens_for(cfg["vocab_size"], n, 30 + n) for n in (1, 9, 140, 77)]
    llm = LLM.from_folder(folder, dtype="bfloat16", num_blocks=96, block_size=8, max_batch=4,
                          chunk_size=48, max_tokens_per_step=80)
    got = llm.generate(prompts, max_new_tokens=20, temperature=0.0)
    assert max(llm.engine.step_tokens) <= 80
    for i, (p, g) in enumerate(zip(prompts, got)):
        assert_tokens_are_maxima(w, cfg, p, g, f"request {i}")


def test_a_kernels_refusal_raises_in_the_step_that_ran_it(folders):
    """The status word comes back with the sampled tokens.  The failure is made on the
    host: a token id outside the vocabulary slips past the batch builder (its check is
    switched off here); the embedding kernel answers with zeros and a status bit, and
    the step that ran it raises.  Nothing faults on the device."""
    from mini_llm_stack_b200.ops.kernels import KernelError
    folder, cfg, w = folders[("A", "float32")]
    llm = LLM.from_folder(folder, dtype="float32", num_blocks=32)
    eng = llm.engine
    eng.submit([5, 17, 3], max_new_tokens=3)
    eng.run_until_done()
    eng.runner.builder.vocab_size = 1 << 30
    eng.submit([5, 400, 7], max_new_tokens=4)            # 400 is not among 256 tokens
    with pytest.raises(KernelError, match="token id outside the vocabulary"):
        eng.step()
    eng.model.runtime.ops.check_status()                 # the word was cleared


@pytest.mark.parametrize("key, dtype", [("A", "float32"), ("D", "bfloat16"), ("C", "float32"),
                                        ("C", "bfloat16"), ("E", "bfloat16")])
def test_a_repeated_prompt_step_replays_from_a_graph_with_the_same_logits(folders, key, dtype):
    """Steps with portions of prompts are captured when their shape has come three times and
    the host was their bound (a tiny model always is): equal portions of several prompts,
    each beside the same number of decoding requests, give the logits of the step run
    kernel by kernel, to the bit (the same kernels with the same arguments)."""
    import torch
    from mini_llm_stack_b200.engine.batch import Entry
    from mini_llm_stack_b200.engine.runner import ModelRunner, load_model
    folder, cfg, w = folders[(key, dtype)]
    model = load_model(folder, dtype=dtype)
    runs = {}
    for graphs in (False, True):
        runner = ModelRunner(model, num_blocks=64, block_size=16, max_requests=8, cuda_graphs=graphs)
        gen = torch.Generator().manual_seed(5)
        rows = []
        # one request decodes throughout; five others bring a prompt of three portions of 24 each
        first = [Entry("d", torch.randint(0, cfg["vocab_size"], (9,), generator=gen).tolist(), [8])]
        runner.reserve(first)
        rows.append(runner.step(first).clone())
        for r in range(5):
            for portion in range(3):
                toks = torch.randint(0, cfg["vocab_size"], (24,), generator=gen).tolist()
                e = [Entry("d", [int(rows[-1][0].argmax())], [0]), Entry(f"p{r}", toks, [23])]
                runner.reserve(e)
                rows.append(runner.step(e).clone())
            runner.release(f"p{r}")
        torch.cuda.synchronize()
        model.runtime.ops.check_status()
        runs[graphs] = rows
        if graphs:
            captured = [k for k, v in runner._graphs.items() if k != "moved" and isinstance(v, tuple)]
            assert any(k[0] == (1, 24) for k in captured), captured
        runner.cache.check()
    assert len(runs[True]) == len(runs[False]) == 16
    for a, b in zip(runs[False], runs[True]):
        assert torch.equal(a, b)
