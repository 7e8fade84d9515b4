"""The scheduler's decisions, with no model: who runs, how many tokens, who is preempted."""

from llmserve_b200.cache import CacheManager, KVGroupSpec
from llmserve_b200.engine.scheduler import Scheduler, SchedulerConfig
from llmserve_b200.engine.sequence import Request, Sequence
from llmserve_b200.sampling import SamplingParams


def make(num_pages, page=4, **kw):
    cm = CacheManager([KVGroupSpec((0,), 1, 16, 0, page)], [num_pages], kw.get("max_num_seqs", 8))
    return Scheduler(SchedulerConfig(**kw), cm), cm


def seq(i, n_prompt):
    r = Request(f"q{i}", None, list(range(n_prompt)), SamplingParams(max_tokens=50))
    s = Sequence(i, r, r.prompt_token_ids, seed=i)
    r.seqs.append(s)
    return s


def run_step(sch, cm, out, new_token=True):
    """What the engine does after a forward pass: commit, and append a token where one was sampled."""
    for s in out.scheduled:
        cm.commit(s.seq.seq_id, s.num_new_tokens)
        s.seq.num_computed_tokens += s.num_new_tokens
        if new_token and s.seq.num_computed_tokens == s.seq.num_tokens:
            s.seq.output_token_ids.append(1)
    cm.check_invariants()


def plan(out):
    return [(s.seq.seq_id, s.num_new_tokens) for s in out.scheduled]


def test_prompts_are_cut_into_portions_under_the_budget_and_decodes_go_first():
    sch, cm = make(100, max_num_batched_tokens=16)
    a, b, c = seq(0, 10), seq(1, 30), seq(2, 3)
    for s in (a, b, c):
        sch.add(s)
    out = sch.schedule()
    assert plan(out) == [(0, 10), (1, 6)]  # b gets what is left of the budget
    run_step(sch, cm, out)
    out = sch.schedule()
    assert plan(out) == [(0, 1), (1, 15)]  # a decodes first, b's next portion takes the rest
    run_step(sch, cm, out)
    out = sch.schedule()
    assert plan(out) == [(0, 1), (1, 9), (2, 3)]  # b finishes its prompt, c is admitted behind it
    run_step(sch, cm, out)
    assert plan(sch.schedule()) == [(0, 1), (1, 1), (2, 1)]


def test_max_num_seqs_and_first_come_first_served():
    sch, cm = make(100, max_num_batched_tokens=64, max_num_seqs=2)
    seqs = [seq(i, 4) for i in range(3)]
    for s in seqs:
        sch.add(s)
    out = sch.schedule()
    assert plan(out) == [(0, 4), (1, 4)] and len(sch.waiting) == 1
    run_step(sch, cm, out)
    sch.finish(seqs[0])
    assert cm.num_free_pages() == 100 - 1  # its page is back at once
    assert plan(sch.schedule()) == [(1, 1), (2, 4)]


def test_when_pages_run_out_the_newest_running_sequence_is_preempted_and_recomputed():
    sch, cm = make(6, page=4, max_num_batched_tokens=64)
    a, b = seq(0, 11), seq(1, 11)
    sch.add(a)
    sch.add(b)
    out = sch.schedule()
    assert plan(out) == [(0, 11), (1, 11)] and cm.num_free_pages() == 0
    run_step(sch, cm, out)  # both now hold 12 tokens: pages full
    out = sch.schedule()
    assert plan(out) == [(0, 1), (1, 1)]  # token 12 still fits page 3
    run_step(sch, cm, out)
    out = sch.schedule()
    # a needs a fourth page: b (admitted last) is preempted, gives back its pages, goes to the front
    assert plan(out) == [(0, 1)] and [s.seq_id for s in out.preempted] == [1]
    assert b.num_computed_tokens == 0 and sch.waiting[0] is b and not cm.is_live(1)
    assert sch.num_preemptions == 1 and len(b.output_token_ids) == 2  # it keeps its tokens
    run_step(sch, cm, out)
    # nothing was admitted in the step of the preemption; b comes back when its 13 tokens fit
    out = sch.schedule()
    assert plan(out)[0] == (0, 1)
    while not any(s.seq.seq_id == 1 for s in out.scheduled):
        run_step(sch, cm, out)
        if a.num_tokens >= 16:
            sch.finish(a)
        out = sch.schedule()
    again = [s for s in out.scheduled if s.seq.seq_id == 1][0]
    assert again.num_new_tokens == b.num_tokens == 13  # prompt and generated tokens are recomputed


def test_a_sequence_that_cannot_grow_is_itself_preempted_when_it_is_the_newest():
    sch, cm = make(3, page=4, max_num_batched_tokens=64)
    a = seq(0, 12)
    sch.add(a)
    out = sch.schedule()
    run_step(sch, cm, out)
    out = sch.schedule()
    assert out.is_empty and [s.seq_id for s in out.preempted] == [0]  # needs a 4th page, has none
    assert cm.usage() == 0.0


def test_without_chunked_prefill_a_long_prompt_runs_alone():
    sch, cm = make(100, max_num_batched_tokens=8, enable_chunked_prefill=False)
    a, b = seq(0, 3), seq(1, 20)
    sch.add(a)
    out = sch.schedule()
    run_step(sch, cm, out)
    sch.add(b)
    out = sch.schedule()
    assert plan(out) == [(1, 20)]  # its own step, decodes pause (src/llmserve/scheduler.py:99-120)
    run_step(sch, cm, out)
    assert plan(sch.schedule()) == [(0, 1), (1, 1)]
