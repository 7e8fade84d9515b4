"""Ways of cutting the same requests into steps, and a driver that replays them on a runner.

A trace is a list of steps ``{"step": i, "entries": [{"id", "tokens", "want"}], "end": [ids]}``,
the format that ``bin/trace_run`` reads. Every position's logits are wanted, so any way of cutting
can be compared with the plain implementation position by position.
"""

from __future__ import annotations

import random

import torch


def make_requests(lengths, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def _entry(rid, tokens):
    return {"id": rid, "tokens": list(tokens), "want": list(range(len(tokens)))}


def _number(steps):
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def whole(requests):
    """Each request alone, in one step."""
    return _number([{"entries": [_entry(r, t)], "end": [r]} for r, t in requests.items()])


def decode_tail(requests, tail=32):
    """Most of a request in one step, then its last ``tail`` tokens one by one."""
    steps = []
    for r, t in requests.items():
        cut = max(1, len(t) - tail)
        steps.append({"entries": [_entry(r, t[:cut])], "end": []})
        for i in range(cut, len(t)):
            steps.append({"entries": [_entry(r, t[i : i + 1])], "end": []})
        steps[-1]["end"] = [r]
    return _number(steps)


def portions(requests, sizes=(7, 2, 33, 3, 64, 2, 5, 17)):
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    k = 0
    for r, t in requests.items():
        i = 0
        while i < len(t):
            n = min(sizes[k % len(sizes)], len(t) - i)
            k += 1
            steps.append({"entries": [_entry(r, t[i : i + n])], "end": []})
            i += n
        steps[-1]["end"] = [r]
    return _number(steps)


def mixed(requests, seed=0, max_live=4, tail=8, max_portion=40):
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others.

    A request is fed in random portions of 2..max_portion tokens until ``tail`` tokens are left,
    which then come one per step; now and then a live request sits a step out. When one ends the
    next is admitted, so the pages it held are handed out again.
    """
    rng = random.Random(seed)
    queue = list(requests)
    done = {r: 0 for r in requests}
    live: list[str] = []
    steps = []
    while queue or live:
        while queue and len(live) < max_live:
            live.append(queue.pop(0))
        entries, end = [], []
        for r in list(live):
            t = requests[r]
            left = len(t) - done[r]
            if len(live) > 1 and rng.random() < 0.15:
                continue  # this request is left out of the step
            if left > tail and left - tail >= 2:
                n = min(rng.randint(2, max_portion), left - tail)
                if left - tail - n == 1:
                    n += 1  # never leave a one-token portion before the tail
            else:
                n = 1
            entries.append(_entry(r, t[done[r] : done[r] + n]))
            done[r] += n
            if done[r] == len(t):
                end.append(r)
                live.remove(r)
        if entries:
            steps.append({"entries": entries, "end": end})
    return _number(steps)


def tokens_needed(requests, max_live=4, unit=64):
    """Pool size (in tokens) that lets any ``max_live`` requests be live at once."""
    sizes = sorted((-(-len(t) // unit) * unit for t in requests.values()), reverse=True)
    return sum(sizes[:max_live])


def replay(runner, steps):
    """Run ``steps`` on a ModelRunner; returns {(request id, position): logits row (CPU float32)}."""
    from llmserve_b200.engine.batch import StepEntry

    got = {}
    pos = {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        logits = runner.run(entries).float().cpu()
        row = 0
        for e in s["entries"]:
            p0 = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], p0 + w)] = logits[row]
                row += 1
            pos[e["id"]] = p0 + len(e["tokens"])
        assert row == logits.shape[0]
        for r in s["end"]:
            runner.finish(r)
            pos.pop(r, None)
        runner.manager.check_invariants()
    return got


def compare(got, expected, atol, rtol=0.0):
    """expected: {request id: logits [len, vocab]}. Returns the worst (error, id, position)."""
    worst = (0.0, None, None)
    n = 0
    for (rid, p), row in got.items():
        ref = expected[rid][p]
        err = (row - ref).abs().max().item()
        if err > worst[0]:
            worst = (err, rid, p)
        n += 1
    assert n == sum(v.shape[0] for v in expected.values()), "not every position was replayed"
    bound = atol + rtol * max(v.abs().max().item() for v in expected.values())
    # report the first wrong position of the worst request, which says where to look
    if worst[0] > bound:
        rid = worst[1]
        first = min(p for (r, p), row in got.items()
                    if r == rid and (row - expected[rid][p]).abs().max().item() > bound)
        raise AssertionError(
            f"max |engine - plain| = {worst[0]:.3e} > {bound:.3e} at request {rid} position "
            f"{worst[2]}; first wrong position of that request: {first}"
        )
    return worst
