"""Each part alone on the GPU, and a toy mixer with state of its own that the framework has never
seen: registered, built into a model and stepped without a change to the framework's files."""

import dataclasses
from dataclasses import dataclass
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_llama
import traces
from conftest import TINY

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env32():
    from llmserve_b200.ops import get_ops
    from llmserve_b200.parts import BuildEnv

    return BuildEnv(get_ops("cuda"), torch.float32, torch.device("cuda"), 128, torch.float32)


def test_norm_part(env32):
    from llmserve_b200.parts import NORMS, RMSNormSpec

    norm = NORMS.build(RMSNormSpec(72, 1e-4), env32)
    w = 1 + 0.1 * torch.randn(72)
    norm.bind({"weight": w.cuda()})
    x, r = torch.randn(5, 72), torch.randn(5, 72)
    xg = x.clone().cuda()
    h = norm.forward(xg, r.cuda())
    assert torch.allclose(xg.cpu(), x + r, atol=1e-6)
    assert torch.allclose(h.cpu(), plain_llama.rms_norm(x + r, w, 1e-4), atol=1e-5)


def test_rotary_part_tables(env32):
    from llmserve_b200.parts import POSITION_ENCODINGS, NoPositionSpec, RotarySpec

    for kw, scaling in [
        ({}, None),
        (dict(scaling_type="linear", factor=4.0), {"rope_type": "linear", "factor": 4.0}),
        (dict(scaling_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_positions=64),
         {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}),
    ]:
        pe = POSITION_ENCODINGS.build(RotarySpec(head_dim=48, theta=5000.0, **kw), env32)
        cos, sin = pe.rotary_tables()
        c, s = plain_llama.rope_tables(torch.arange(128), 48, 5000.0, scaling)
        assert torch.equal(cos.cpu(), c[:, :24]) and torch.equal(sin.cpu(), s[:, :24])
    assert POSITION_ENCODINGS.build(NoPositionSpec(), env32).rotary_tables() is None


def test_feed_forward_part(env32):
    from llmserve_b200.parts import FEED_FORWARDS, SwiGLUSpec

    ff = FEED_FORWARDS.build(SwiGLUSpec(40, 104), env32)
    g, u, d = torch.randn(104, 40) * 0.2, torch.randn(104, 40) * 0.2, torch.randn(40, 104) * 0.2
    ff.bind({"gate_up.weight": torch.cat([g, u]).cuda(), "down.weight": d.cuda()})
    x = torch.randn(9, 40)
    assert torch.allclose(ff.forward(x.cuda(), None).cpu(), plain_llama.swiglu(x, g, u, d), atol=1e-5)


# ------------------------------------------------------------------ a toy mixer with its own state
@dataclass(frozen=True)
class DecaySpec:
    hidden_size: int
    decay: float
    kind: str = "toy_decay"


def register_toy():
    from llmserve_b200.parts import MIXERS, Mixer, ParamDecl, StateNeed

    if "toy_decay" in MIXERS.classes:
        return

    @MIXERS.register("toy_decay")
    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + x_t W ; y_t = s_t. The state s lives in the request's slot."""

        def param_decls(self):
            h = self.spec.hidden_size
            return {"w.weight": ParamDecl((h, h), "matrix")}

        def bind(self, params):
            self.w = params["w.weight"]

        def cache_need(self):
            return StateNeed((self.spec.hidden_size,), torch.float32)

        def forward(self, h, step, cache):
            u = self.ops.linear(h, self.w, None, out_dtype=torch.float32)
            out = torch.empty_like(u)
            cu = step.host.cu_q.tolist()
            for i in range(step.num_seqs):
                slot = int(step.host.state_slots[i])
                s = cache.state[slot]
                if step.host.first_portion[i]:
                    s.zero_()
                for t in range(cu[i], cu[i + 1]):
                    s.mul_(self.spec.decay).add_(u[t])
                    out[t] = s
            return out


def toy_plain(w, cfg, ids, decay, mix_w):
    """Plain version: layer 0 is the toy mixer (own weight), layer 1 is attention."""
    x = w["model.embed_tokens.weight"][torch.as_tensor(ids)]
    pos = torch.arange(len(ids))
    for layer in range(2):
        p = f"model.layers.{layer}."
        h = plain_llama.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        if layer == 0:
            u = h @ mix_w.T
            s = torch.zeros(cfg["hidden"])
            a = torch.empty_like(u)
            for t in range(len(ids)):
                s = decay * s + u[t]
                a[t] = s
        else:
            a, _ = plain_llama.attention_block(h, w, p + "self_attn.", cfg, pos)
        x = x + a
        h = plain_llama.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        x = x + plain_llama.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                   w[p + "mlp.down_proj.weight"])
    x = plain_llama.rms_norm(x, w["model.norm.weight"], cfg["eps"])
    return x @ w["model.embed_tokens.weight"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped(tiny_dirs):
    from llmserve_b200.config import load_model_config
    from llmserve_b200.engine.runner import ModelRunner
    from llmserve_b200.models import DecoderModel
    from llmserve_b200.ops import get_ops
    from llmserve_b200.parts import BuildEnv
    from llmserve_b200.weights import load_parameters

    register_toy()
    folder = tiny_dirs["A"]
    arch, cfg = load_model_config(folder)
    plan = arch.plan(cfg)
    toy_layer = dataclasses.replace(plan.layers[0], mixer=DecaySpec(cfg.hidden_size, 0.9))
    plan = dataclasses.replace(plan, layers=(toy_layer, plan.layers[1]))
    env = BuildEnv(get_ops("cuda"), torch.float32, torch.device("cuda"), 256, torch.float32)
    model = DecoderModel(plan, env)
    params = load_parameters(folder, arch.checkpoint_layout(cfg), torch.float32, "cuda")
    params = {k: v for k, v in params.items() if not k.startswith("layers.0.mixer.")}
    mix_w = (torch.randn(64, 64, generator=torch.Generator().manual_seed(1)) * 0.05)
    params["layers.0.mixer.w.weight"] = mix_w.cuda()
    model.bind(params)
    runner = ModelRunner(model, page_tokens=16, num_pages=24, max_model_len=256, max_num_seqs=4)
    assert len(runner.pools.state) == 1 and runner.pools.state[0].shape == (1, 4, 64)
    assert len(runner.manager.groups) == 1 and runner.manager.groups[0].cache_ids == (1,)
    reqs = traces.make_requests([40, 23, 70, 9, 55, 31], 256, seed=13)
    pcfg, w = plain_llama.read_config(folder), plain_llama.read_weights(folder)
    expected = {r: toy_plain(w, pcfg, t, 0.9, mix_w) for r, t in reqs.items()}
    got = traces.replay(runner, traces.mixed(reqs, seed=4))  # slots are handed out again
    traces.compare(got, expected, atol=2e-5)
