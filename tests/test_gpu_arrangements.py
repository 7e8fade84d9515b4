"""Arrangements of layers that the Llama checkpoints do not use, on the GPU with the real kernels:
a layer that runs twice, a layer that reads another layer's cache, and layers with a window whose
pages form a group of their own and come back while the request lives. The weights are those of a
tiny Llama folder; only the plan (which is data) differs. Compared with the plain implementation."""

import dataclasses

import pytest
import torch

import plain_llama
import traces
from conftest import TINY
from gpu_util import tolerances

pytestmark = pytest.mark.gpu


def build_runner(folder, change_plan, dtype, page_tokens, num_pages, max_len, max_num_seqs=4):
    from llmserve_b200.config.registry import load_model_config
    from llmserve_b200.engine.runner import ModelRunner, resolve_dtype
    from llmserve_b200.models.decoder import DecoderModel
    from llmserve_b200.ops import get_ops
    from llmserve_b200.parts.base import BuildEnv
    from llmserve_b200.weights import load_parameters

    arch, cfg = load_model_config(folder)
    plan = change_plan(arch.plan(cfg))
    ops = get_ops("cuda")
    tdtype = resolve_dtype(dtype)
    env = BuildEnv(ops=ops, dtype=tdtype, device=torch.device("cuda"), max_positions=max_len,
                   branch_dtype=ops.branch_dtype(tdtype))
    model = DecoderModel(plan, env)
    model.bind(load_parameters(folder, arch.checkpoint_layout(cfg), tdtype, "cuda"))
    return ModelRunner(model, page_tokens=page_tokens, num_pages=num_pages, max_model_len=max_len,
                       max_num_seqs=max_num_seqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["portions", "mixed", "decode_tail"])
def test_layer_twice_and_shared_cache(tiny_dirs, dtype, mode):
    from llmserve_b200.models.plan import RunEntry

    folder = tiny_dirs["B"]
    order = [(0, 0), (1, 1), (0, 2), (2, 1)]  # layer 0 twice; layer 2 reads layer 1's cache
    change = lambda plan: dataclasses.replace(plan, run_order=tuple(RunEntry(l, c) for l, c in order))
    reqs = traces.make_requests([45, 23, 70, 9, 130], TINY["B"]["vocab_size"], seed=3)
    pool = traces.tokens_needed(reqs) // 8
    runner = build_runner(folder, change, dtype, 8, pool, 512)
    assert len(runner.model.cache_needs()) == 3
    expected = {r: plain_llama.model_logits(folder, t, run_order=order) for r, t in reqs.items()}
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    atol, rtol = tolerances(dtype)
    traces.compare(got, expected, atol=atol, rtol=rtol)
    assert runner.manager.usage() == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,window", [("A", 20), ("C", 40)])
def test_window_layers_have_pages_of_their_own(tiny_dirs, dtype, name, window):
    """The last layer gets a window. Its group is given far fewer pages than the requests are long,
    so a page that the window has passed is used again by the same or another request while both
    live. C has head size 64: its portions take the mma.sync kernel (the tcgen05 one has no window),
    single tokens the split kernel."""
    folder = tiny_dirs[name]
    spec = TINY[name]
    n_layers = spec["num_hidden_layers"]
    page = spec["page_tokens"]

    def change(plan):
        last = plan.layers[-1]
        windowed = dataclasses.replace(last, mixer=dataclasses.replace(last.mixer, window=window))
        return dataclasses.replace(plan, layers=plan.layers[:-1] + (windowed,))

    lengths = [150, 97, 64, 201]
    reqs = traces.make_requests(lengths, spec["vocab_size"], seed=9)
    full_pages = traces.tokens_needed(reqs) // page
    # a windowed request holds the pages that overlap [computed - window + 1, computed + portion)
    longest_portion = 41  # traces.mixed cuts portions of at most 40 (+1) tokens
    per_request = -(-(window + longest_portion) // page) + 1
    runner = build_runner(folder, change, dtype, page, [full_pages, 4 * per_request],
                          spec["max_position_embeddings"])
    assert len(runner.manager.groups) == 2 and runner.manager.groups[1].window == window
    windows = [0] * (n_layers - 1) + [window]
    expected = {r: plain_llama.model_logits(folder, t, windows=windows) for r, t in reqs.items()}
    got = traces.replay(runner, traces.mixed(reqs, seed=2))
    atol, rtol = tolerances(dtype)
    traces.compare(got, expected, atol=atol, rtol=rtol)
    assert runner.manager.num_pages(1) == 4 * per_request < full_pages
    assert runner.manager.usage() == 0.0
