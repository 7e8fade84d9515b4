"""Generation through the Python entry point on the GPU: scheduler, cache, kernels, graphs, sampler."""

import pytest
import torch

import plain_llama
from conftest import TINY

pytestmark = pytest.mark.gpu

PROMPTS = [[5, 9, 200, 31, 7], list(range(40, 57)), [3] * 33, [100, 2], list(range(70))]


def llm(folder, name, dtype, **kw):
    from llmserve_b200 import LLM

    d = dict(dtype=dtype, block_size=TINY[name]["page_tokens"], num_kv_blocks=64,
             max_model_len=TINY[name]["max_position_embeddings"], max_num_seqs=8)
    d.update(kw)
    return LLM(str(folder), **d)


def assert_same_or_near_tie(folder, prompt, a, b):
    """Two bfloat16 runs of one greedy request through different kernels (a captured step is a
    padded batch, whose matrix products go to the library where the unpadded step's run this
    package's kernel) round differently, so they may part where two candidates are nearly tied.
    Up to there they must agree, and at the parting both choices must be within bfloat16
    rounding of the plain model's best; after it the sequences are different requests."""
    if a == b:
        return
    assert len(a) == len(b)
    i = next(k for k in range(len(a)) if a[k] != b[k])
    logits = plain_llama.model_logits(folder, list(prompt) + a[:i])[-1]
    bound = 0.03 * float(logits.abs().max())
    assert float(logits.max() - logits[a[i]]) <= bound and float(logits.max() - logits[b[i]]) <= bound, \
        (i, a[i], b[i], float(logits.max()), float(logits[a[i]]), float(logits[b[i]]))


def greedy(n):
    from llmserve_b200 import SamplingParams

    return SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_float32_equals_plain_greedy(sharp_dirs, name, graphs):
    outs = llm(sharp_dirs[name], name, "float32", cuda_graphs=graphs).generate(PROMPTS, greedy(10))
    for o, p in zip(outs, PROMPTS):
        assert o.outputs[0].token_ids == plain_llama.greedy(sharp_dirs[name], p, 10)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_bfloat16_picks_tokens_the_plain_model_also_ranks_first(sharp_dirs, name):
    """The engine's own tokens are replayed through the plain model: at every step the token the
    engine chose must be the plain model's best, or within bfloat16 rounding of it."""
    outs = llm(sharp_dirs[name], name, "bfloat16").generate(PROMPTS, greedy(10))
    for o, p in zip(outs, PROMPTS):
        gen = o.outputs[0].token_ids
        logits = plain_llama.model_logits(sharp_dirs[name], p + gen)[len(p) - 1 : -1]
        chosen = logits.gather(1, torch.tensor(gen)[:, None])[:, 0]
        gap = logits.max(-1).values - chosen
        assert (gap <= 0.03 * logits.abs().max(-1).values).all(), gap  # each step by its own largest logit


def test_graphs_portions_and_preemption_give_the_same_tokens(sharp_dirs):
    want = [o.outputs[0].token_ids for o in
            llm(sharp_dirs["B"], "B", "float32", cuda_graphs=False).generate(PROMPTS, greedy(12))]
    small = llm(sharp_dirs["B"], "B", "float32", max_num_batched_tokens=8)
    assert [o.outputs[0].token_ids for o in small.generate(PROMPTS, greedy(12))] == want
    tight = llm(sharp_dirs["B"], "B", "float32", num_kv_blocks=14, max_num_batched_tokens=16)
    assert [o.outputs[0].token_ids for o in tight.generate(PROMPTS, greedy(12))] == want
    assert tight.engine.scheduler.num_preemptions > 0
    tight.engine.manager.check_invariants()
    assert tight.engine.manager.usage() == 0.0
    assert tight.engine.stats()["kernel_set"] == "cuda-sm100a"


@pytest.mark.parametrize("name", ["B", "C"])
def test_preemption_in_bfloat16_with_captured_steps(sharp_dirs, name):
    """So few pages that requests are evicted and computed again, with captured steps of single
    tokens and of portions, in the precision that is served: the tokens are those of a roomy
    engine, up to a near-tie where a recomputed prompt meets other kernels (portions where the
    first pass decoded), and no page is lost."""
    pt = TINY[name]["page_tokens"]
    prompts = PROMPTS[:4]
    new = 2 * pt + 3  # every request outgrows the pages of its prompt twice
    roomy = llm(sharp_dirs[name], name, "bfloat16", cuda_graphs=False)
    want = [o.outputs[0].token_ids for o in roomy.generate(prompts, greedy(new))]
    pages = sum(-(-len(p) // pt) for p in prompts) + 1  # all prompts fit, their growth does not
    assert pages >= -(-(max(map(len, prompts)) + new) // pt)  # but each request alone does
    tight = llm(sharp_dirs[name], name, "bfloat16", num_kv_blocks=pages, max_num_batched_tokens=16)
    got = [o.outputs[0].token_ids for o in tight.generate(prompts, greedy(new))]
    assert tight.engine.scheduler.num_preemptions > 0
    for p, a, b in zip(prompts, got, want, strict=True):
        assert_same_or_near_tie(sharp_dirs[name], p, a, b)
    tight.engine.manager.check_invariants()
    assert tight.engine.manager.usage() == 0.0
    tight.engine.runner.ops.check_kernel_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_captured_steps_with_portions_give_the_same_tokens(sharp_dirs, name, dtype):
    """Steps that mix portions of prompts with single tokens, replayed as captured graphs of a
    padded batch (one-token rows first, then portion slots; padding sequences on the spare page):
    same tokens as the same steps run kernel by kernel. Greedy rows, a seeded temperature row (the
    sampling kernel inside the capture) and, in a second run, a row with penalties (sampled outside
    it, on rows gathered from the padded logits)."""
    import numpy as np

    from llmserve_b200 import SamplingParams

    rng = np.random.default_rng(5)
    v = TINY[name]["vocab_size"]
    prompts = [rng.integers(0, v, n).tolist() for n in (70, 33, 5, 90, 17, 64, 2, 45, 120, 9)]
    seeded = SamplingParams(temperature=0.8, top_p=0.9, seed=11, max_tokens=14, ignore_eos=True)
    penal = SamplingParams(temperature=0.0, repetition_penalty=1.7, frequency_penalty=0.2, max_tokens=14,
                           ignore_eos=True)
    for special in (seeded, penal):
        params = [greedy(10 + i) for i in range(len(prompts))]
        params[3] = special
        runs = {}
        for graphs in (False, True):
            m = llm(sharp_dirs[name], name, dtype, cuda_graphs=graphs, max_num_batched_tokens=24,
                    num_kv_blocks=200)
            if graphs:
                m.engine.runner._graphs().capture_after = 1
            runs[graphs] = [o.outputs[0].token_ids for o in m.generate(prompts, params)]
            if graphs:
                held = m.engine.runner.decode_graphs.graphs.values()
                mixed = [g for g in held if g.slots > 0 and g.graph is not None]
                assert len(mixed) >= 2 and any(g.batch > 0 for g in mixed)
                assert any(not g.sampled for g in mixed) == (special is penal)
                m.engine.manager.check_invariants()
                assert m.engine.manager.usage() == 0.0
        if dtype == "float32":
            assert runs[True] == runs[False]
        else:
            for k, (a, b) in enumerate(zip(runs[True], runs[False])):
                if k == 3:  # the sampled / penalised row: same length, tokens not comparable at a parting
                    assert len(a) == len(b)
                else:
                    assert_same_or_near_tie(sharp_dirs[name], prompts[k], a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_arrivals_give_the_same_tokens_with_and_without_graphs(sharp_dirs, dtype):
    """Requests of every sampling kind arrive at random moments into a cache so small that some are
    preempted; every step that can be captured is (decode steps, steps with portions, rows sampled
    inside and outside the capture). Token for token the same as with every kernel launched alone."""
    import random

    from llmserve_b200 import EngineConfig, LLMEngine, SamplingParams

    def run(graphs):
        eng = LLMEngine(EngineConfig(model=str(sharp_dirs["C"]), dtype=dtype, block_size=32,
                                     num_kv_blocks=26, max_model_len=1024, max_num_seqs=8,
                                     max_num_batched_tokens=48, cuda_graphs=graphs))
        if graphs:
            eng.runner._graphs().capture_after = 1
        rng = random.Random(4)
        todo = []
        for i in range(36):
            kind, n_out = rng.random(), rng.randrange(2, 40)
            if kind < 0.5:
                sp = SamplingParams(temperature=0.0, max_tokens=n_out, ignore_eos=True)
            elif kind < 0.8:
                sp = SamplingParams(temperature=0.9, top_p=0.9, top_k=40, seed=i, max_tokens=n_out, ignore_eos=True)
            elif kind < 0.9:
                sp = SamplingParams(temperature=0.0, repetition_penalty=1.3, max_tokens=n_out, ignore_eos=True)
            else:
                sp = SamplingParams(temperature=0.7, seed=i, logprobs=2, max_tokens=n_out, ignore_eos=True)
            todo.append(([rng.randrange(515) for _ in range(rng.choice([3, 17, 40, 90, 200]))], sp))
        outs, steps = {}, 0
        asked.clear()
        while todo or eng.has_unfinished_requests():
            for _ in range(rng.randrange(0, 3)):
                if todo:
                    prompt, sp = todo.pop(0)
                    asked[eng.add_request(prompt, sp)] = (prompt, sp)
            for o in eng.step():
                if o.finished:
                    outs[o.request_id] = o.outputs[0].token_ids
            steps += 1
            if steps % 25 == 0:
                eng.manager.check_invariants()
        eng.manager.check_invariants()
        assert eng.manager.usage() == 0.0
        return outs, eng

    asked = {}
    plain, _ = run(False)
    captured, eng = run(True)
    assert len(plain) == 36 and set(captured) == set(plain)
    if dtype == "float32":
        assert captured == plain
    else:
        for rid, (prompt, sp) in asked.items():
            if sp.greedy and not sp.has_penalties:
                assert_same_or_near_tie(sharp_dirs["C"], prompt, captured[rid], plain[rid])
            else:
                assert len(captured[rid]) == len(plain[rid])
    held = eng.runner.decode_graphs.graphs.values()
    assert sum(1 for g in held if g.slots) >= 3 and sum(1 for g in held if not g.slots) >= 3
    assert eng.scheduler.num_preemptions > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_seeded_sampling_is_the_same_alone_and_in_a_busy_batch(sharp_dirs, dtype):
    from llmserve_b200 import SamplingParams

    sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=123, max_tokens=10, ignore_eos=True)
    want = llm(sharp_dirs["C"], "C", dtype).generate([PROMPTS[1]], sp)[0].outputs[0].token_ids
    busy = llm(sharp_dirs["C"], "C", dtype, max_num_batched_tokens=8)
    params = [SamplingParams(temperature=1.0, max_tokens=9, ignore_eos=True), sp,
              SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)]
    outs = busy.generate([PROMPTS[0], PROMPTS[1], PROMPTS[2]], params)
    assert outs[1].outputs[0].token_ids == want
    assert len(set(want)) > 1
    # and the busy batch itself gives the same tokens every time it is run (its first request has
    # no seed and draws one)
    again = llm(sharp_dirs["C"], "C", dtype, max_num_batched_tokens=8).generate(
        [PROMPTS[0], PROMPTS[1], PROMPTS[2]], params)
    assert [o.outputs[0].token_ids for o in again[1:]] == [o.outputs[0].token_ids for o in outs[1:]]


def test_penalties_bans_and_logprobs_with_and_without_graphs(sharp_dirs):
    """Rows that need more than the sampling kernel replay the step up to the logits and are
    sampled outside the capture: same tokens and log-probabilities as without graphs, and the
    penalties do change what is generated."""
    from llmserve_b200 import SamplingParams

    sps = [SamplingParams(temperature=0.0, repetition_penalty=1.8, presence_penalty=0.4,
                          frequency_penalty=0.3, max_tokens=30, ignore_eos=True),
           SamplingParams(temperature=0.0, logprobs=3, max_tokens=30, ignore_eos=True),
           SamplingParams(temperature=0.9, top_p=0.9, seed=5, min_tokens=8, max_tokens=30)]
    runs = {}
    for graphs in (True, False):
        out = llm(sharp_dirs["C"], "C", "float32", cuda_graphs=graphs).generate(PROMPTS[:3], sps)
        runs[graphs] = out
    for a, b in zip(runs[True], runs[False]):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    lp_a, lp_b = runs[True][1].outputs[0].logprobs, runs[False][1].outputs[0].logprobs
    assert lp_a is not None and len(lp_a) == 30
    assert lp_a == pytest.approx(lp_b, abs=1e-4)
    plain = llm(sharp_dirs["C"], "C", "float32").generate(PROMPTS[:1], greedy(30))[0].outputs[0].token_ids
    assert runs[True][0].outputs[0].token_ids != plain


def test_long_generation_with_graphs_matches_stepwise(sharp_dirs):
    """120 decode steps: contexts cross page edges and the number of context partitions changes."""
    a = llm(sharp_dirs["C"], "C", "float32", cuda_graphs=True).generate(PROMPTS[:2], greedy(120))
    b = llm(sharp_dirs["C"], "C", "float32", cuda_graphs=False).generate(PROMPTS[:2], greedy(120))
    assert [o.outputs[0].token_ids for o in a] == [o.outputs[0].token_ids for o in b]
    assert a[0].outputs[0].token_ids == plain_llama.greedy(sharp_dirs["C"], PROMPTS[0], 120)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_changes_nothing(sharp_dirs, dtype):
    """Steps launched before the last one's tokens are read: same tokens, also when sequences stop
    at different times (stop tokens), which drops a step that was launched ahead."""
    from llmserve_b200 import SamplingParams

    free = plain_llama.greedy(sharp_dirs["A"], PROMPTS[0], 30)
    stop = next(t for i, t in enumerate(free) if i >= 9 and t not in free[:i])  # first met late
    params = [SamplingParams(temperature=0.0, max_tokens=30, stop_token_ids=[stop]),
              SamplingParams(temperature=0.0, max_tokens=17, ignore_eos=True),
              SamplingParams(temperature=0.9, top_k=40, seed=5, max_tokens=25, ignore_eos=True),
              SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)]
    outs = {}
    for ahead in (False, True):
        m = llm(sharp_dirs["A"], "A", dtype, run_ahead=ahead)
        res = m.generate(PROMPTS[:4], params)
        outs[ahead] = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in res]
        m.engine.manager.check_invariants()
        assert m.engine.manager.usage() == 0.0
    assert outs[True] == outs[False]
    if dtype == "float32":
        assert outs[True][0][0] == free[: free.index(stop) + 1] and outs[True][0][1] == "stop"
    assert [len(t) for t, _ in outs[True]][1:] == [17, 25, 30]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_that_are_never_cut(sharp_dirs, dtype):
    """``enable_chunked_prefill=False`` on the GPU: a prompt longer than the budget runs in a step
    of its own while the others pause; float32 tokens are the plain model's, bfloat16 tokens the
    same on two runs."""
    import numpy as np

    rng = np.random.default_rng(9)
    v = TINY["C"]["vocab_size"]
    prompts = [rng.integers(0, v, n).tolist() for n in (5, 70, 12, 33)]
    runs = []
    for _ in range(2):
        m = llm(sharp_dirs["C"], "C", dtype, enable_chunked_prefill=False, max_num_batched_tokens=40)
        runs.append([o.outputs[0].token_ids for o in m.generate(prompts, greedy(9))])
        m.engine.manager.check_invariants()
        assert m.engine.manager.usage() == 0.0
    assert runs[0] == runs[1]
    if dtype == "float32":
        assert runs[0] == [plain_llama.greedy(sharp_dirs["C"], p, 9) for p in prompts]


def test_abort_while_a_step_is_in_flight(sharp_dirs):
    from llmserve_b200 import SamplingParams

    m = llm(sharp_dirs["B"], "B", "float32")
    eng = m.engine
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    a = eng.add_request(PROMPTS[0], sp)
    b = eng.add_request(PROMPTS[1], sp)
    for _ in range(6):
        eng.step()
    assert eng._pending is not None  # a step was launched ahead
    eng.abort_request(a)
    done = {}
    while eng.has_unfinished_requests():
        for o in eng.step():
            if o.finished:
                done[o.request_id] = o
    assert done[b].outputs[0].token_ids == plain_llama.greedy(sharp_dirs["B"], PROMPTS[1], 40)
    eng.manager.check_invariants()
    assert eng.manager.usage() == 0.0


def test_cli_generates(sharp_dirs, capsys):
    from llmserve_b200.cli import main

    main(["generate", "--model", str(sharp_dirs["A"]), "--prompt-ids", "5,9,200,31,7", "--max-tokens", "6",
          "--dtype", "float32", "--max-model-len", "256", "--num-kv-blocks", "32", "--ignore-eos"])
    out = capsys.readouterr().out
    want = " ".join(map(str, plain_llama.greedy(sharp_dirs["A"], PROMPTS[0], 6)))
    assert want in out and "tok/s" in out
