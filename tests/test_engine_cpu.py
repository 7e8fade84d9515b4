"""The engine's host logic end to end on the CPU, with plain PyTorch kernels behind it."""

import pytest

import plain_llama
from conftest import TINY
from plain_ops import PlainOps


def engine(folder, name, **kw):
    from llmserve_b200 import EngineConfig, LLMEngine

    d = dict(model=str(folder), dtype="float32", device="cpu", block_size=TINY[name]["page_tokens"],
             num_kv_blocks=64, max_model_len=TINY[name]["max_position_embeddings"], max_num_seqs=8)
    d.update(kw)
    return LLMEngine(EngineConfig(**d), ops=PlainOps())


def run_all(eng):
    done = {}
    while eng.has_unfinished_requests():
        for o in eng.step():
            if o.finished:
                done[o.request_id] = o
        eng.manager.check_invariants()
    return done


PROMPTS = [[5, 9, 200, 31, 7], list(range(40, 57)), [3] * 33, [100, 2]]


def test_greedy_generation_matches_the_plain_model(sharp_dirs):
    from llmserve_b200 import SamplingParams

    eng = engine(sharp_dirs["A"], "A")
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    ids = [eng.add_request(p, sp) for p in PROMPTS]
    done = run_all(eng)
    for rid, p in zip(ids, PROMPTS):
        assert done[rid].outputs[0].token_ids == plain_llama.greedy(sharp_dirs["A"], p, 8)
        assert done[rid].outputs[0].finish_reason == "length"
    assert eng.manager.usage() == 0.0 and eng.stats()["num_running"] == 0


def test_portions_and_preemption_do_not_change_the_tokens(sharp_dirs):
    from llmserve_b200 import SamplingParams

    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    base = engine(sharp_dirs["B"], "B")
    ids = [base.add_request(p, sp) for p in PROMPTS]
    done = run_all(base)
    want = [done[i].outputs[0].token_ids for i in ids]
    small = engine(sharp_dirs["B"], "B", max_num_batched_tokens=8)  # many portions
    ids = [small.add_request(p, sp) for p in PROMPTS]
    done = run_all(small)
    assert [done[i].outputs[0].token_ids for i in ids] == want
    tight = engine(sharp_dirs["B"], "B", num_kv_blocks=9, max_num_batched_tokens=16)  # 72 tokens of cache
    ids = [tight.add_request(p, sp) for p in PROMPTS]
    done = run_all(tight)
    assert tight.scheduler.num_preemptions > 0
    assert [done[i].outputs[0].token_ids for i in ids] == want


def test_seeded_sampling_does_not_depend_on_the_batch(sharp_dirs):
    from llmserve_b200 import SamplingParams

    sp = SamplingParams(temperature=0.8, top_k=50, seed=123, max_tokens=10, ignore_eos=True)
    alone = engine(sharp_dirs["A"], "A")
    rid = alone.add_request(PROMPTS[1], sp)
    want = run_all(alone)[rid].outputs[0].token_ids
    busy = engine(sharp_dirs["A"], "A", max_num_batched_tokens=8)
    busy.add_request(PROMPTS[0], SamplingParams(temperature=1.0, max_tokens=9, ignore_eos=True))
    rid = busy.add_request(PROMPTS[1], sp)
    busy.add_request(PROMPTS[2], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    assert run_all(busy)[rid].outputs[0].token_ids == want
    assert len(set(want)) > 1


def test_stop_tokens_min_tokens_eos_logprobs_abort(sharp_dirs):
    from llmserve_b200 import SamplingParams

    eng = engine(sharp_dirs["A"], "A")
    free = plain_llama.greedy(sharp_dirs["A"], PROMPTS[0], 6)
    k = next(i for i in range(1, 6) if free[i] not in free[:i])  # first new token after the first
    rid = eng.add_request(PROMPTS[0], SamplingParams(temperature=0, max_tokens=6, stop_token_ids=[free[k]]))
    o = run_all(eng)[rid].outputs[0]
    assert o.token_ids == free[: k + 1] and o.finish_reason == "stop" and o.stop_reason == free[k]
    # the same stop token is banned until min_tokens is reached, so the continuation changes there
    rid = eng.add_request(PROMPTS[0], SamplingParams(temperature=0, max_tokens=6, min_tokens=k + 2,
                                                     stop_token_ids=[free[k]]))
    o = run_all(eng)[rid].outputs[0]
    assert o.token_ids[:k] == free[:k] and o.token_ids[k] != free[k] and len(o.token_ids) >= k + 2
    rid = eng.add_request(PROMPTS[1], SamplingParams(temperature=0, max_tokens=3, logprobs=2, ignore_eos=True))
    o = run_all(eng)[rid].outputs[0]
    assert len(o.logprobs) == 3 and all(lp <= 0 for lp in o.logprobs)
    assert o.top_logprobs[0][0][0] == o.token_ids[0] and abs(o.top_logprobs[0][0][1] - o.logprobs[0]) < 1e-5
    rid = eng.add_request(PROMPTS[2], SamplingParams(max_tokens=30, ignore_eos=True))
    eng.step()
    assert eng.manager.usage() > 0
    eng.abort_request(rid)
    assert eng.manager.usage() == 0.0 and not eng.has_unfinished_requests()


def test_intake_errors(tiny_dirs):
    from llmserve_b200 import SamplingParams

    eng = engine(tiny_dirs["A"], "A", num_kv_blocks=4)
    with pytest.raises(ValueError, match="empty"):
        eng.add_request([])
    with pytest.raises(ValueError, match="max_model_len"):
        eng.add_request([1] * 256)
    with pytest.raises(ValueError, match="never fit"):
        eng.add_request([1] * 60, SamplingParams(max_tokens=10))
    with pytest.raises(ValueError, match="token ids"):
        eng.add_request([1, 256])
    with pytest.raises(ValueError, match="tokenizer"):
        eng.add_request("hello")
    eng.add_request([1, 2], request_id="x")
    with pytest.raises(ValueError, match="duplicate"):
        eng.add_request([1, 2], request_id="x")
    with pytest.raises(ValueError):
        SamplingParams(top_p=0)
    with pytest.raises(ValueError):
        SamplingParams(n=2)


def test_llm_generate_returns_outputs_in_input_order(sharp_dirs):
    from llmserve_b200 import LLM, SamplingParams

    llm = LLM(str(sharp_dirs["C"]), ops=PlainOps(), dtype="float32", device="cpu", block_size=32,
              num_kv_blocks=16, max_model_len=256, max_num_seqs=2)
    outs = llm.generate(PROMPTS[:3], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert [o.prompt_token_ids for o in outs] == PROMPTS[:3]
    for o, p in zip(outs, PROMPTS):
        assert o.outputs[0].token_ids == plain_llama.greedy(sharp_dirs["C"], p, 4)
    one = llm.generate(PROMPTS[3], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    assert len(one) == 1 and len(one[0].outputs[0].token_ids) == 2


def test_penalties_from_the_token_state_equal_penalties_from_host_lists():
    """The sampler with state slots (tokens entered step by step into a [slots, vocab] state) and
    the sampler without (penalised tokens listed on the host every step) change the logits in the
    same way, also after a slot has passed to another request."""
    import torch

    from llmserve_b200.sampling.params import SamplingParams
    from llmserve_b200.sampling.sampler import SampleRow, Sampler

    V = 97
    g = torch.Generator().manual_seed(3)
    with_state = Sampler(PlainOps(), "cpu", max_slots=3)
    without = Sampler(PlainOps(), "cpu")
    pa = SamplingParams(temperature=0.0, repetition_penalty=1.7, presence_penalty=0.5, frequency_penalty=0.25)
    pb = SamplingParams(temperature=0.0, frequency_penalty=1.5)
    plain = SamplingParams(temperature=0.0)
    reqs = {"a": (pa, [5, 9, 9, 40], [], 0, 1), "b": (pb, [1, 2, 3], [], 2, 1), "c": (plain, [7], [], -1, 0)}
    for step in range(12):
        if step == 6:  # "a" ends; its slot goes to a new request with another prompt
            reqs["a"] = (pa, [60, 61, 5], [], 0, 2)
        logits = torch.randn(len(reqs), V, generator=g)
        logits[:, [5, 9, 40, 60, 1, 2]] += 3.0  # tokens that penalties will have to push down
        rows_s = [SampleRow(p, out, prompt, 0, slot=slot, epoch=ep) for p, prompt, out, slot, ep in reqs.values()]
        rows_h = [SampleRow(p, out, prompt, 0) for p, prompt, out, _, _ in reqs.values()]
        la, lb = logits.clone(), logits.clone()
        ta = with_state.sample(la, rows_s).token_ids
        tb = without.sample(lb, rows_h).token_ids
        assert ta == tb and torch.equal(la, lb)
        assert not torch.equal(la[0], logits[0]) and torch.equal(la[2], logits[2])
        for (_, _, out, _, _), t in zip(reqs.values(), ta):
            out.append(t)


def test_captured_batch_sizes_and_sampling_kinds():
    from llmserve_b200.engine.decode_graph import batch_sizes
    from llmserve_b200.sampling.params import SamplingParams
    from llmserve_b200.sampling.sampler import sample_kinds

    for limit in (1, 2, 5, 8, 64, 100, 256):
        sizes = batch_sizes(limit)
        assert sizes[0] == 1 and sizes[-1] == limit and sizes == sorted(set(sizes))
        # padding never adds more than half of the rows again (a third from 4 rows on)
        for n in range(1, limit + 1):
            b = next(x for x in sizes if x >= n)
            assert b <= max(n + 1, n * 3 // 2 + 1)
    greedy = SamplingParams(temperature=0.0)
    plain = SamplingParams(temperature=0.7)
    cut = SamplingParams(temperature=0.7, top_p=0.9)
    assert not greedy.has_cut and not plain.has_cut and cut.has_cut
    assert not SamplingParams(temperature=0.0, top_k=5).has_cut  # greedy rows are never cut
    assert sample_kinds([greedy]) == 1 and sample_kinds([plain]) == 2 and sample_kinds([cut]) == 1
    assert sample_kinds([greedy, plain, cut]) == 3


def test_padded_batch_of_a_captured_step_with_portions(tiny_dirs):
    """The batch that a captured step with portions of prompts runs (one-token rows first, padded;
    then portion slots, the unused ones and the remaining tokens as padding sequences on the spare
    page) gives the same logits as the step itself. Run here without a graph, on the CPU."""
    import numpy as np
    import torch

    from llmserve_b200.engine.batch import DeviceStep, StepEntry
    from llmserve_b200.engine.decode_graph import DecodeGraphs, row_bucket, slot_bucket, token_bucket

    assert [token_bucket(n) for n in (1, 64, 65, 513, 1024, 1025, 2049)] == [64, 64, 128, 576, 1024, 1152, 2304]
    assert [slot_bucket(n) for n in (1, 2, 8, 9)] == [8, 8, 8, 16]
    assert [row_bucket(n, 8) for n in (0, 1, 4, 5, 8)] == [0, 4, 4, 8, 8] and row_bucket(17, 256) == 64
    eng = engine(tiny_dirs["B"], "B", num_kv_blocks=200)
    runner = eng.runner
    graphs = DecodeGraphs(runner)
    graphs.max_mixed_tokens = 4096
    m = runner.manager
    v = TINY["B"]["vocab_size"]
    rng = np.random.default_rng(3)
    # five requests with some history in the cache
    history = {r: rng.integers(0, v, n).tolist() for r, n in zip("abcde", (7, 30, 1, 18, 44))}
    runner.run([StepEntry(r, t, []) for r, t in history.items()])
    # a step in the scheduler's order: single tokens and portions mixed; "c" unsampled, "f" new
    entries = [StepEntry("a", [5], [0]), StepEntry("b", rng.integers(0, v, 37).tolist(), [36]),
               StepEntry("c", [9], []), StepEntry("d", rng.integers(0, v, 2).tolist(), []),
               StepEntry("e", [11], [0]), StepEntry("f", rng.integers(0, v, 70).tolist(), [69])]
    m.admit("f")
    for e in entries:
        m.allocate(e.rid, len(e.tokens))
    shape = graphs.mixed_shape(entries)
    assert shape == (4, 8, 128)  # 3 single tokens -> 4; 3 portions -> 8 slots; 109 + 10 tokens -> 128
    assert graphs.mixed_shape(entries[:1] + entries[2:3]) is None  # no portion: the decode graphs' case
    assert graphs.mixed_shape([StepEntry("b", [1, 2, 3], [1])]) is None  # logits wanted inside a portion
    want = runner.step(entries)
    arrays, padded, index = graphs._fill_mixed(shape, entries)
    plans = graphs._plans_mixed(shape, padded)
    B, P, TP = shape
    assert index == [0, 4, 2, 6] and padded.q_lens.tolist() == [1, 1, 1, 1, 37, 2, 70, 2, 2, 2, 2, 11]
    assert arrays["positions"][B + 109 :].tolist() == [0, 1] * 4 + list(range(11))
    spare = runner.pools.spare_page(0)
    assert (arrays[("table", 0)][[3, 7, 11]] == spare).all() and (arrays["state_slots"][7:] == m.max_requests).all()
    for key, (mixer, _) in runner.planners.items():
        rows = mixer.plan_rows(B, P, TP)
        assert {n: a.shape[0] for n, a in plans[key].items()} == rows
        assert plans[key]["decode_seqs"].tolist() == [0, 1, 2, 3]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    step = DeviceStep(
        token_ids=t(arrays["token_ids"]), positions=t(arrays["positions"]), token_seq=t(arrays["token_seq"]),
        cu_q=t(arrays["cu_q"]), ctx_lens=t(arrays["ctx_lens"]), state_slots=t(arrays["state_slots"]),
        first_portion=t(arrays["first_portion"]), block_tables=[t(arrays[("table", 0)])],
        logit_rows=t(arrays["logit_rows"]), num_tokens=B + TP, num_seqs=B + P, num_logit_rows=B + P,
        max_decode_ctx=0, decode_splits=1,
        plans={k: {n: t(a) for n, a in p.items()} for k, p in plans.items()},
    )
    got = runner.model.forward(step, runner.pools)
    assert got.shape[0] == B + P
    torch.testing.assert_close(got[index], want, atol=1e-6, rtol=0)
    # a shape is captured the second time it is asked for
    rows = [None] * 4
    assert not graphs.accepts(entries, rows) and graphs.accepts(entries, rows)


def test_running_ahead_asks_for_the_pages_of_all_sequences_together(sharp_dirs):
    """Equal prompts reach a page's edge in the same step. With fewer free pages than sequences
    each of them alone could grow, all together cannot: the step must not be launched ahead."""
    from llmserve_b200 import SamplingParams

    pt = TINY["A"]["page_tokens"]
    eng = engine(sharp_dirs["A"], "A", num_kv_blocks=4)  # three sequences of one page, one page free
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    for _ in range(3):
        eng.add_request(list(range(1, pt - 1)), sp)  # pt - 2 tokens: the second next token needs a page
    eng.step()
    seqs = list(eng.scheduler.running)
    assert len(seqs) == 3 and eng.manager.num_free_pages(0) == 1
    assert all(eng.manager.can_allocate(s.seq_id, 3) for s in seqs)  # each alone fits
    assert not eng._pages_for_all(seqs, 3)
    assert eng._pages_for_all(seqs[:1], 3) and eng._pages_for_all(seqs, 2)
    done = run_all(eng)  # the scheduler preempts where pages run out; nothing raises
    assert len(done) == 3 and eng.scheduler.num_preemptions > 0
    assert len({tuple(o.outputs[0].token_ids) for o in done.values()}) == 1


class _ByteTokenizer:
    """Token = one byte of UTF-8 text: a character can be spread over up to four tokens."""

    eos_token_id = None

    def decode(self, ids, skip_special_tokens=True):
        return bytes(ids).decode("utf-8", errors="replace")

    def __call__(self, text, add_special_tokens=False):
        from types import SimpleNamespace

        return SimpleNamespace(input_ids=list(text.encode("utf-8")))


class _LetterTokenizer(_ByteTokenizer):
    """Token id -> one lower-case letter: every token sequence is valid text."""

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(97 + i % 26) for i in ids)

    def __call__(self, text, add_special_tokens=False):
        from types import SimpleNamespace

        return SimpleNamespace(input_ids=[ord(c) - 97 for c in text])


def test_text_stream_shows_whole_characters_only():
    from llmserve_b200.engine.detokenizer import TextStream, find_stop

    tok = _ByteTokenizer()
    prompt = list("say: ".encode())
    text = "héllo wörld → ok 🙂!"
    ids = prompt + list(text.encode())
    stream = TextStream(tok, prompt)
    shown = []
    for n in range(len(prompt) + 1, len(ids) + 1):
        piece = stream.push(ids[:n])
        assert "\N{REPLACEMENT CHARACTER}" not in piece
        shown.append(piece)
    assert "".join(shown) == text
    assert shown.count("") == len(text.encode()) - len(text)  # one silent step per continuation byte
    assert find_stop("abc STOP def", 5, ["STOP"]) == (4, "STOP")  # ends inside the new text
    assert find_stop("abc STOP defgh", 5, ["STOP"]) is None  # lies wholly in older text
    assert find_stop("xxabyy", 4, ["by", "ab", ""]) == (2, "ab")  # the one that begins first


def test_stop_strings_cut_the_text(sharp_dirs):
    from llmserve_b200 import SamplingParams

    tok = _LetterTokenizer()

    def run(**kw):
        eng = engine(sharp_dirs["A"], "A")
        eng.tokenizer = tok
        rid = eng.add_request("hello", SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True, **kw))
        return run_all(eng)[rid].outputs[0]

    free = run()
    assert len(free.text) == 12 and free.finish_reason == "length"
    assert free.token_ids == plain_llama.greedy(sharp_dirs["A"], [ord(c) - 97 for c in "hello"], 12)
    stop = free.text[5:8]
    at = free.text.find(stop)
    cut = run(stop=[stop])
    assert (cut.text, cut.finish_reason, cut.stop_reason) == (free.text[:at], "stop", stop)
    assert len(cut.token_ids) == at + 3  # the tokens of the stop string were generated
    kept = run(stop=[stop], include_stop_str_in_output=True)
    assert kept.text == free.text[: at + 3]


def test_a_kernel_that_gave_up_waiting_stops_the_engine(sharp_dirs):
    """A kernel of the product path that gives up a bounded wait records a code in a flag that
    the host reads after the step. Here a kernel set whose flag is raised by hand stands in for
    it: the step that follows must raise, not hand out tokens."""
    from llmserve_b200 import EngineConfig, LLMEngine, SamplingParams

    class Flagged(PlainOps):
        code = 0

        def check_kernel_errors(self):
            if self.code:
                code, self.code = self.code, 0
                raise RuntimeError(f"a CUDA kernel of llmserve_b200 gave up waiting (code {code})")

    ops = Flagged()
    eng = LLMEngine(EngineConfig(model=str(sharp_dirs["A"]), dtype="float32", device="cpu", block_size=16,
                                 num_kv_blocks=16, max_model_len=256, max_num_seqs=4), ops=ops)
    eng.add_request([1, 2, 3], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert eng.step()  # fine
    ops.code = 104
    with pytest.raises(RuntimeError, match="gave up waiting"):
        eng.step()


def test_context_partitions_fill_whole_waves():
    """148 SMs holding 7 blocks each run 1036 blocks at a time. The number of partitions per
    (sequence, head) avoids a last wave that is nearly empty, keeps partitions of 128 keys or
    more, and does not change while the context stays between two powers of two."""
    from llmserve_b200.ops.cuda_ops import choose_decode_splits

    def pick(batch, ctx=2118, heads=32):
        return choose_decode_splits(batch * heads, ctx, 148, 7)

    assert pick(1) == 17        # 544 blocks, partitions of 125 keys: as many as the 128-key rule allows
    assert pick(8) == 4         # 1024 blocks: one wave
    assert pick(12) in (2, 5)   # 768 or 1920 blocks, not 1152 (a second wave for 116 blocks)
    assert pick(24) == 4        # 3072 blocks: three waves, not 1536 (one and a half)
    assert pick(48) == 2        # 3072 blocks again
    assert pick(64) == 1        # 2048 blocks: two waves
    assert pick(8, ctx=100) == 1 and pick(8, ctx=300) <= 3
    assert len({pick(24, ctx=c) for c in range(2049, 4097, 97)}) == 1
    for batch in range(1, 70):
        for ctx in (1, 127, 129, 1000, 5000, 70000):
            s = pick(batch, ctx)
            assert 1 <= s <= 64 and (s == 1 or (ctx + 127) // 128 >= s)
    # occupancy unknown: about six blocks per SM, as before
    assert choose_decode_splits(256, 2118, 148, 0) == 4
    assert choose_decode_splits(0, 2118, 148, 7) == 1
