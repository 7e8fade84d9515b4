"""The sampling kernels against their plain versions and against the distributions they draw from."""

import pytest
import torch

from plain_ops import PlainOps

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from llmserve_b200.ops import get_ops

    return get_ops("cuda")


def params(R, temperature=1.0, top_k=-1, top_p=1.0, min_p=0.0, seed=0, draw=0):
    f = lambda v, dt: torch.full((R,), v, dtype=dt) if not torch.is_tensor(v) else v.to(dt)
    return (f(temperature, torch.float32), f(top_k, torch.int32), f(top_p, torch.float32),
            f(min_p, torch.float32), f(seed, torch.int64), f(draw, torch.int32))


def test_greedy_is_argmax_lowest_index_on_ties(ops):
    logits = torch.randn(9, 1031, generator=torch.Generator().manual_seed(0))
    logits[3, 77] = logits[3, 500] = 50.0
    got = ops.sample(logits.cuda(), *[p.cuda() for p in params(9, temperature=0.0)]).cpu()
    assert got.tolist() == logits.argmax(-1).tolist()
    assert got[3] == 77


@pytest.mark.parametrize("kw", [dict(), dict(top_k=5), dict(top_p=0.7), dict(min_p=0.2),
                                dict(top_k=40, top_p=0.9, min_p=0.05, temperature=0.7)])
def test_matches_plain_sampler_draw_for_draw(ops, kw):
    R, V = 6, 777
    logits = torch.randn(R, V, generator=torch.Generator().manual_seed(1)) * 2
    p = params(R, seed=torch.arange(R) * 7919 + 3, draw=torch.arange(R) * 5, **kw)
    got = ops.sample(logits.cuda(), *[x.cuda() for x in p]).cpu()
    ref = PlainOps().sample(logits, *p)
    assert got.tolist() == ref.tolist()


@pytest.mark.parametrize("V", [49152, 70001])  # the row kept in shared memory, and too long for it
@pytest.mark.parametrize("kw", [dict(top_k=50), dict(top_p=0.9), dict(top_p=0.999),
                                dict(top_k=1000, top_p=0.95, min_p=0.001, temperature=0.6),
                                dict(top_k=1), dict(top_p=1e-6)])
def test_cut_on_a_large_vocabulary(ops, V, kw):
    R = 5
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(R, V, generator=g) * 3
    logits[1, ::7] = float("-inf")           # banned tokens
    logits[2] = (logits[2] * 4).round() / 4  # many equal values: groups of ties across the cut
    logits[3, :] = 0.25                      # all equal: everything is kept or only ties matter
    p = params(R, seed=torch.arange(R) * 104729 + 11, draw=torch.arange(R) + 1, **kw)
    for rep in range(2):  # the same launch twice: the cut does not depend on the order of additions
        got = ops.sample(logits.cuda(), *[x.cuda() for x in p]).cpu()
        ref = PlainOps().sample_sorted(logits, *p)
        assert got.tolist() == ref.tolist()


def test_draws_follow_the_distribution_and_the_cuts(ops):
    V, N = 5, 20000
    probs = torch.tensor([0.4, 0.3, 0.15, 0.1, 0.05])
    logits = probs.log().repeat(N, 1).cuda()
    draw = torch.arange(N)
    got = ops.sample(logits, *[x.cuda() for x in params(N, seed=123, draw=draw)]).cpu()
    freq = torch.bincount(got.long(), minlength=V).float() / N
    assert (freq - probs).abs().max() < 0.015
    got = ops.sample(logits, *[x.cuda() for x in params(N, seed=5, draw=draw, top_k=2)]).cpu()
    freq = torch.bincount(got.long(), minlength=V).float() / N
    assert freq[2:].sum() == 0 and abs(freq[0] - 4 / 7) < 0.015
    # top_p 0.75: mass before token 2 is 0.7 < 0.75 so it is kept; before token 3 it is 0.85
    got = ops.sample(logits, *[x.cuda() for x in params(N, seed=6, draw=draw, top_p=0.75)]).cpu()
    freq = torch.bincount(got.long(), minlength=V).float() / N
    assert freq[3:].sum() == 0 and freq[2] > 0.1
    got = ops.sample(logits, *[x.cuda() for x in params(N, seed=7, draw=draw, min_p=0.5)]).cpu()
    freq = torch.bincount(got.long(), minlength=V).float() / N
    assert freq[2:].sum() == 0


def test_seeded_row_does_not_depend_on_the_batch(ops):
    V = 3000
    g = torch.Generator().manual_seed(4)
    row = torch.randn(1, V, generator=g)
    alone = ops.sample(row.cuda(), *[x.cuda() for x in params(1, seed=99, draw=3, temperature=0.8)]).cpu()
    batch = torch.cat([torch.randn(4, V, generator=g), row, torch.randn(2, V, generator=g)])
    seeds = torch.tensor([1, 2, 3, 4, 99, 5, 6])
    draws = torch.tensor([0, 9, 2, 2, 3, 1, 0])
    got = ops.sample(batch.cuda(), *[x.cuda() for x in params(7, seed=seeds, draw=draws, temperature=0.8)]).cpu()
    assert got[4] == alone[0]


def test_penalties_ban_and_logsumexp(ops):
    logits = torch.randn(3, 50, generator=torch.Generator().manual_seed(2))
    row = torch.tensor([0, 0, 2], dtype=torch.int32)
    tok = torch.tensor([4, 9, 49], dtype=torch.int32)
    cnt = torch.tensor([2, 0, 1], dtype=torch.int32)
    pres = torch.tensor([0.5, 0.5, 0.0])
    freq = torch.tensor([0.25, 0.25, 1.0])
    rep = torch.tensor([1.0, 1.3, 2.0])
    a, b = logits.clone().cuda(), logits.clone()
    ops.apply_penalties(a, *[x.cuda() for x in (row, tok, cnt, pres, freq, rep)])
    PlainOps().apply_penalties(b, row, tok, cnt, pres, freq, rep)
    assert torch.allclose(a.cpu(), b, atol=1e-6)
    ops.ban_tokens(a, row.cuda(), tok.cuda())
    assert torch.isinf(a[0, 4]) and torch.isinf(a[2, 49]) and torch.isfinite(a[1]).all()
    assert torch.allclose(ops.logsumexp(logits.cuda()).cpu(), torch.logsumexp(logits, -1), atol=1e-5)


def test_token_state_penalties_match_the_listed_ones(ops):
    """The dense penalties kernel reading a token state against the sparse one fed by lists."""
    R, V, slots = 4, 1031, 6
    g = torch.Generator().manual_seed(12)
    logits = torch.randn(R, V, generator=g)
    state = torch.zeros(slots, V, dtype=torch.int32)
    slot_of = [4, 0, 5, 2]
    prompts = [torch.randint(0, V, (50,), generator=g).tolist() for _ in range(R)]
    outs = [torch.randint(0, 40, (30,), generator=g).tolist() for _ in range(R)]  # repeats
    s, t, f = [], [], []
    for r in range(R):
        for x in set(prompts[r]):
            s.append(slot_of[r]); t.append(x); f.append(1)
        for x in outs[r]:
            s.append(slot_of[r]); t.append(x); f.append(0)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    state_gpu = state.cuda()
    ops.token_state_add(state_gpu, i32(s).cuda(), i32(t).cuda(), i32(f).cuda())
    PlainOps().token_state_add(state, i32(s), i32(t), i32(f))
    assert torch.equal(state_gpu.cpu(), state)
    pres = torch.tensor([0.5, 0.0, 1.0, 0.2]); freq = torch.tensor([0.25, 1.0, 0.0, 0.1])
    rep = torch.tensor([1.0, 1.3, 2.0, 0.8])
    rows = i32([0, 1, 2, 3])
    a = logits.clone().cuda()
    ops.apply_penalties_dense(a, rows.cuda(), i32(slot_of).cuda(), pres.cuda(), freq.cuda(), rep.cuda(), state_gpu)
    b = logits.clone()
    PlainOps().apply_penalties_dense(b, rows, i32(slot_of), pres, freq, rep, state)
    assert torch.allclose(a.cpu(), b, atol=1e-6)
    assert not torch.equal(b, logits)
