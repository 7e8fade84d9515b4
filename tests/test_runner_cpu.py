"""The step function, the cache and the model assembly on the CPU, with plain PyTorch kernels.

These tests exercise the host-side logic (flattening a ragged batch, block tables, pages that are
used again, layer order as data); the CUDA kernels have their own tests under ``-m gpu``.
"""

import pytest
import torch

import plain_llama
import traces
from conftest import TINY
from plain_ops import PlainOps


def cpu_runner(folder, name, num_pages, dtype="float32", max_num_seqs=4):
    from llmserve_b200.engine.runner import ModelRunner, load_model

    cfg = TINY[name]
    _, _, model = load_model(folder, dtype, "cpu", PlainOps(), cfg["max_position_embeddings"])
    return ModelRunner(model, page_tokens=cfg["page_tokens"], num_pages=num_pages,
                       max_model_len=cfg["max_position_embeddings"], max_num_seqs=max_num_seqs)


LENGTHS = {"A": [5, 17, 33, 70, 41, 64], "B": [1, 9, 40, 64, 130, 77], "C": [3, 66, 129, 50, 35]}


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_plain(tiny_dirs, name, mode):
    folder = tiny_dirs[name]
    reqs = traces.make_requests(LENGTHS[name], TINY[name]["vocab_size"], seed=11)
    expected = {r: plain_llama.model_logits(folder, t) for r, t in reqs.items()}
    pool_tokens = traces.tokens_needed(reqs)
    runner = cpu_runner(folder, name, pool_tokens // TINY[name]["page_tokens"])
    steps = getattr(traces, mode)(reqs)
    got = traces.replay(runner, steps)
    traces.compare(got, expected, atol=2e-5)
    assert runner.manager.usage() == 0.0


def test_layer_order_is_data(tiny_dirs):
    """A layer run twice and a layer that reads another layer's cache, against the plain model."""
    from llmserve_b200.config.registry import load_model_config
    from llmserve_b200.engine.runner import ModelRunner
    from llmserve_b200.models.decoder import DecoderModel
    from llmserve_b200.models.plan import RunEntry
    from llmserve_b200.parts.base import BuildEnv
    from llmserve_b200.weights import load_parameters
    import dataclasses

    folder = tiny_dirs["B"]
    arch, cfg = load_model_config(folder)
    order = [(0, 0), (1, 1), (0, 2), (2, 1)]  # layer 0 twice; layer 2 reads layer 1's cache
    plan = dataclasses.replace(arch.plan(cfg), run_order=tuple(RunEntry(l, c) for l, c in order))
    env = BuildEnv(PlainOps(), torch.float32, torch.device("cpu"), 512, torch.float32)
    model = DecoderModel(plan, env)
    model.bind(load_parameters(folder, arch.checkpoint_layout(cfg), torch.float32, "cpu"))
    assert len(model.cache_needs()) == 3
    runner = ModelRunner(model, page_tokens=8, num_pages=40, max_model_len=512, max_num_seqs=4)
    reqs = traces.make_requests([45, 23], 384, seed=3)
    expected = {r: plain_llama.model_logits(folder, t, run_order=order) for r, t in reqs.items()}
    got = traces.replay(runner, traces.portions(reqs, sizes=(5, 2, 11)))
    traces.compare(got, expected, atol=2e-5)


def test_window_layers_get_their_own_pages(tiny_dirs):
    """Layers with a window form a second group whose pages come back while the request lives."""
    from llmserve_b200.config.registry import load_model_config
    from llmserve_b200.engine.runner import ModelRunner
    from llmserve_b200.models.decoder import DecoderModel
    from llmserve_b200.parts.base import BuildEnv
    from llmserve_b200.weights import load_parameters
    import dataclasses

    folder = tiny_dirs["A"]
    arch, cfg = load_model_config(folder)
    plan = arch.plan(cfg)
    l1 = plan.layers[1]
    windowed = dataclasses.replace(l1, mixer=dataclasses.replace(l1.mixer, window=20))
    plan = dataclasses.replace(plan, layers=(plan.layers[0], windowed))
    env = BuildEnv(PlainOps(), torch.float32, torch.device("cpu"), 256, torch.float32)
    model = DecoderModel(plan, env)
    model.bind(load_parameters(folder, arch.checkpoint_layout(cfg), torch.float32, "cpu"))
    runner = ModelRunner(model, page_tokens=16, num_pages=[16, 5], max_model_len=256, max_num_seqs=2)
    assert len(runner.manager.groups) == 2
    reqs = traces.make_requests([150], 256, seed=9)
    expected = {r: plain_llama.model_logits(folder, t, windows=[0, 20]) for r, t in reqs.items()}
    got = traces.replay(runner, traces.portions(reqs, sizes=(9, 2, 17, 1, 1, 30)))
    traces.compare(got, expected, atol=2e-5)
    # 150 tokens need 10 pages in the full group; the windowed group never had more than 5
    assert runner.manager.num_pages(1) == 5


def test_step_refuses_bad_input(tiny_dirs):
    from llmserve_b200.engine.batch import StepEntry

    runner = cpu_runner(tiny_dirs["A"], "A", 8)
    with pytest.raises(ValueError, match="token ids"):
        runner.run([StepEntry("x", [1, 999], [])])
    runner.finish("x")
    runner.manager.admit("y")
    with pytest.raises(ValueError, match="block table"):
        runner.step([StepEntry("y", [1, 2, 3], [])])  # nothing allocated
    with pytest.raises(ValueError, match="twice"):
        runner.run([StepEntry("z", [1], []), StepEntry("z", [2], [])])
