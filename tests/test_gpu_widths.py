"""The engine at real layer widths against the plain implementation.

Two models of two layers each with the layer sizes of SmolLM2-1.7B (hidden 2048, 32 heads of 64,
feed-forward 8192, vocabulary 49152) and SmolLM2-360M (hidden 960, 15 query heads on 5 key heads,
feed-forward 2560: widths that are no multiple of 128 and three query heads per key head). These
are the shapes that a benchmark times: matrix products with 6144 / 16384 / 49152 output features
over 2048 and 8192 inputs, the work of a tile shared between blocks, single-token attention over
contexts of more than 2000 keys in partitions, prompt attention over many query tiles. One request is
2400 tokens long; it is replayed whole, with its last 32 tokens one by one, in portions of
changing size and mixed with other requests on a pool so small that pages are used again; then 8
and 40 requests decode side by side (40 rows go to the library's matrix product). The plain model
runs in float64 on the same device; logits are compared at a few hundred chosen positions (a
49152-entry row for every position would not fit).

float32 bound: 1e-4 absolute, the target stated for these sizes. bfloat16 bound: as in the other
GPU tests, a fraction of the largest logit.
"""

import random

import pytest
import torch

import plain_llama
import traces
from gpu_util import BF16_RTOL

pytestmark = pytest.mark.gpu

WIDE = {
    "1.7b": dict(vocab_size=49152, hidden_size=2048, intermediate_size=8192, num_hidden_layers=2,
                 num_attention_heads=32, num_key_value_heads=32, head_dim=64, rope_theta=130000.0,
                 rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=8192, seed=4),
    "360m": dict(vocab_size=49152, hidden_size=960, intermediate_size=2560, num_hidden_layers=2,
                 num_attention_heads=15, num_key_value_heads=5, head_dim=64, rope_theta=100000.0,
                 rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=8192, seed=5),
}
LONG = 2400
PAGE = 16
F32_BOUND = 1e-4


@pytest.fixture(scope="module")
def wide_dirs(tmp_path_factory):
    from llmserve_b200.config import LlamaConfig
    from llmserve_b200.weights import write_random_model

    out = {}
    for name, spec in WIDE.items():
        d = tmp_path_factory.mktemp(f"wide-{name}")
        cfg = LlamaConfig.from_dict({"model_type": "llama", **{k: v for k, v in spec.items() if k != "seed"}})
        write_random_model(d, cfg, spec["seed"])
        out[name] = d
    return out


def wanted_positions(n: int) -> list[int]:
    """The first tokens, every 97th, both sides of the edges of pages, tiles and partitions, and
    the last 40."""
    keep = set(range(min(4, n))) | set(range(0, n, 97)) | set(range(max(0, n - 40), n))
    for edge in (16, 64, 128, 256, 512, 1024, 2048, 2176):
        keep |= {p for p in (edge - 1, edge, edge + 1) if 0 <= p < n}
    return sorted(keep)


class Oracle:
    """Plain float64 logits of requests at their wanted positions, computed once per model."""

    def __init__(self, folder):
        self.cfg = plain_llama.read_config(folder)
        self.w = {k: v.to("cuda") for k, v in plain_llama.read_weights(folder, torch.float64).items()}
        self.known: dict[tuple, dict[int, torch.Tensor]] = {}

    def rows(self, tokens) -> dict[int, torch.Tensor]:
        key = tuple(tokens)
        if key not in self.known:
            want = wanted_positions(len(tokens))
            logits = plain_llama.forward(self.cfg, self.w, tokens, dtype=torch.float64, device="cuda",
                                         rows=want)
            self.known[key] = dict(zip(want, logits))
        return self.known[key]


@pytest.fixture(scope="module")
def oracles(wide_dirs):
    return {name: Oracle(d) for name, d in wide_dirs.items()}


def runner_for(folder, dtype, pool_tokens, max_num_seqs=4):
    from llmserve_b200.engine.runner import ModelRunner, load_model
    from llmserve_b200.ops import get_ops

    _, _, model = load_model(folder, dtype, "cuda", get_ops("cuda"), 4096)
    return ModelRunner(model, page_tokens=PAGE, num_pages=pool_tokens // PAGE, max_model_len=4096,
                       max_num_seqs=max_num_seqs, max_num_batched_tokens=4096)


def only_wanted(steps, requests):
    """Keep, in every entry, only the wanted places that :func:`wanted_positions` names."""
    pos = {}
    for s in steps:
        for e in s["entries"]:
            p0 = pos.get(e["id"], 0)
            keep = set(wanted_positions(len(requests[e["id"]])))
            e["want"] = [w for w in e["want"] if p0 + w in keep]
            pos[e["id"]] = p0 + len(e["tokens"])
    return steps


def check(got, requests, oracle, dtype):
    worst, scale, n = (0.0, None, None), 0.0, 0
    for (rid, p), row in got.items():
        ref = oracle.rows(requests[rid])[p]
        scale = max(scale, ref.abs().max().item())
        err = (row.double() - ref).abs().max().item()
        n += 1
        if err > worst[0]:
            worst = (err, rid, p)
    assert n == sum(len(wanted_positions(len(t))) for t in requests.values()), "a wanted position is missing"
    bound = F32_BOUND if dtype == "float32" else BF16_RTOL * scale
    assert worst[0] <= bound, (
        f"max |engine - plain| = {worst[0]:.3e} > {bound:.3e} at request {worst[1]} position {worst[2]} "
        f"(largest logit {scale:.2f})")
    return worst[0]


def requests_of(name, lengths, seed):
    return traces.make_requests(lengths, WIDE[name]["vocab_size"], seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["1.7b", "360m"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_every_way_of_cutting_at_real_widths(wide_dirs, oracles, name, mode, dtype):
    lengths = [LONG] if mode != "mixed" else [LONG, 150, 37, 420, 90, 64]
    reqs = requests_of(name, lengths, seed=31)
    if mode == "whole":
        steps = traces.whole(reqs)
    elif mode == "decode_tail":
        steps = traces.decode_tail(reqs, tail=32)
    elif mode == "portions":
        steps = traces.portions(reqs, sizes=(700, 2, 513, 33, 900, 3, 64, 130, 17))
    else:
        steps = traces.mixed(reqs, seed=3, max_live=4, tail=8, max_portion=600)
    runner = runner_for(wide_dirs[name], dtype, traces.tokens_needed(reqs))
    got = traces.replay(runner, only_wanted(steps, reqs))
    check(got, reqs, oracles[name], dtype)
    assert runner.manager.usage() == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,batch,ctx", [("1.7b", 8, 2100), ("1.7b", 40, 70), ("360m", 8, 2100),
                                            ("360m", 40, 70), ("1.7b", 1, 2300)])
def test_requests_decoding_side_by_side(wide_dirs, oracles, name, batch, ctx, dtype):
    """``batch`` requests with prompts of about ``ctx`` tokens (all lengths different), then twelve
    tokens each, one per step and all in the same step: rows 1, 8 (few-rows product) and 40
    (library product) over contexts that are cut into partitions."""
    rng = random.Random(batch * 1000 + ctx)
    lengths = [ctx + rng.randint(0, 40) + 12 for _ in range(batch)]
    reqs = requests_of(name, lengths, seed=batch)
    runner = runner_for(wide_dirs[name], dtype, sum(-(-n // 64) * 64 for n in lengths), max_num_seqs=batch)
    steps = [{"entries": [{"id": r, "tokens": t[:-12], "want": list(range(len(t) - 12))}], "end": []}
             for r, t in reqs.items()]
    for k in range(12, 0, -1):
        steps.append({"entries": [{"id": r, "tokens": [t[len(t) - k]], "want": [0]} for r, t in reqs.items()],
                      "end": list(reqs) if k == 1 else []})
    for i, s in enumerate(steps):
        s["step"] = i
    got = traces.replay(runner, only_wanted(steps, reqs))
    check(got, reqs, oracles[name], dtype)


@pytest.mark.parametrize("dtype,factor", [("float32", 4.0), ("bfloat16", 2.0)])
def test_sharp_attention_at_real_widths(wide_dirs, tmp_path, dtype, factor):
    """With random weights of deviation 0.02 the attention weights are nearly flat, and a key that
    is left out moves the logits little. Here the query and key projections are ``factor`` times
    larger, so the scores are ``factor`` squared times larger and every query's softmax is
    dominated by a few keys anywhere among its 2300: a partition, a tile or a page that is dropped
    or read twice then changes the logits far beyond rounding. (bfloat16 keeps eight bits of a
    query and a key, so an error of a score grows with the score; its factor is the smaller one.)"""
    import shutil

    from safetensors.torch import load_file, save_file

    name = "360m"
    shutil.copy(wide_dirs[name] / "config.json", tmp_path / "config.json")
    t = load_file(str(wide_dirs[name] / "model.safetensors"))
    for k in t:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            t[k] = (t[k].float() * factor).to(t[k].dtype)
    save_file(t, str(tmp_path / "model.safetensors"))
    del t
    reqs = requests_of(name, [2300], seed=77)
    oracle = Oracle(tmp_path)
    cuts = {"whole": traces.whole(reqs), "decode_tail": traces.decode_tail(reqs, tail=32),
            "portions": traces.portions(reqs, sizes=(900, 2, 513, 33, 700))}
    for cut, steps in cuts.items():
        runner = runner_for(tmp_path, dtype, traces.tokens_needed(reqs))
        try:
            check(traces.replay(runner, only_wanted(steps, reqs)), reqs, oracle, dtype)
        except AssertionError as e:
            raise AssertionError(f"{cut}: {e}") from None
