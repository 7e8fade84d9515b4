"""Each part alone on the GPU, and a toy mixer with state of its own that the framework has never
seen: registered, built into a model and stepped without a change to the framework's files."""

import dataclasses
from dataclasses import dataclass

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

        needs_host_step = True  # the loop below reads the batch on the host: never captured

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
    # four request slots and the spare one for rows that pad a captured batch
    assert len(runner.pools.state) == 1 and runner.pools.state[0].shape == (1, 5, 64)
    assert len(runner.manager.groups) == 1 and runner.manager.groups[0].cache_ids == (1,)
    reqs = traces.make_requests([40, 23, 70, 9, 55, 31], 256, seed=13)
    pcfg, w = plain_llama.read_config(folder), plain_llama.read_weights(folder)
    expected = {r: toy_plain(w, pcfg, t, 0.9, mix_w) for r, t in reqs.items()}
    got = traces.replay(runner, traces.mixed(reqs, seed=4))  # slots are handed out again
    traces.compare(got, expected, atol=2e-5)


# ------------------------------------------------------------------ the attention part and the block alone
def test_attention_part_and_block_alone(tiny_dirs):
    """One PagedAttention part, then one PreNormBlock, built from specs and stepped on a ragged batch."""
    from llmserve_b200.cache import CacheManager, CachePools, KVGroupSpec
    from llmserve_b200.engine.batch import StepEntry, build_host_step
    from llmserve_b200.engine.runner import ModelRunner
    from llmserve_b200.ops import get_ops
    from llmserve_b200.parts import (BLOCKS, MIXERS, AttentionSpec, BuildEnv, PreNormBlockSpec,
                                     RMSNormSpec, RotarySpec, SwiGLUSpec)

    H, nq, nk, D, I, page = 96, 6, 3, 16, 200, 8
    env = BuildEnv(get_ops("cuda"), torch.float32, torch.device("cuda"), 64, torch.float32)
    aspec = AttentionSpec(H, nq, nk, D, D**-0.5, RotarySpec(D, 777.0), bias=True)
    bspec = PreNormBlockSpec(RMSNormSpec(H, 1e-5), aspec, RMSNormSpec(H, 2e-6), SwiGLUSpec(H, I))
    block = BLOCKS.build(bspec, env)
    g = torch.Generator().manual_seed(0)
    w = {n: (torch.randn(d.shape, generator=g) * (0.1 if d.role != "scale" else 0.05) + (d.role == "scale"))
         for n, d in block.param_decls().items()}
    block.bind({n: t.cuda() for n, t in w.items()})
    # the plain model's names for the same tensors
    q, kv = nq * D, nk * D
    pw = {"a.q_proj.weight": w["mixer.qkv.weight"][:q], "a.k_proj.weight": w["mixer.qkv.weight"][q : q + kv],
          "a.v_proj.weight": w["mixer.qkv.weight"][q + kv :], "a.q_proj.bias": w["mixer.qkv.bias"][:q],
          "a.k_proj.bias": w["mixer.qkv.bias"][q : q + kv], "a.v_proj.bias": w["mixer.qkv.bias"][q + kv :],
          "a.o_proj.weight": w["mixer.o.weight"], "a.o_proj.bias": w["mixer.o.bias"]}
    cfg = dict(heads=nq, kv_heads=nk, head_dim=D, theta=777.0, rope_scaling=None, bias=True)
    lens = [19, 1, 30]
    xs = [torch.randn(n, H, generator=g) for n in lens]
    manager = CacheManager([KVGroupSpec((0,), nk, D, 0, page)], [16], 4)
    pools = CachePools(manager.groups, [], [16], 4, torch.float32, "cuda")
    for i, n in enumerate(lens):
        manager.admit(i)
        manager.allocate(i, n)
    host = build_host_step([StepEntry(i, [0] * n, []) for i, n in enumerate(lens)], manager, 10, 64)
    # reuse the runner's upload by hand: a DeviceStep needs the attention plan of this mixer
    runner = ModelRunner.__new__(ModelRunner)
    runner.device, runner.pools, runner._staging, runner._staging_turn = env.device, pools, [], 0
    runner.planners = {block.mixer.plan_key(): (block.mixer, 0)}
    runner.last_h2d_bytes = 0
    step = runner.upload(host)
    x = torch.cat(xs).cuda()
    x_in = x.clone()
    x_out, pending = block.forward(x, None, step, pools.view(0, writes=True))
    got = (x_out if pending is None else x_out + pending.float()).cpu()
    # plain: per sequence, whole
    want = []
    for xi in xs:
        h = plain_llama.rms_norm(xi, w["norm_in.weight"], 1e-5)
        a, _ = plain_llama.attention_block(h, pw, "a.", cfg, torch.arange(xi.shape[0]))
        y = xi + a
        h = plain_llama.rms_norm(y, w["norm_post.weight"], 2e-6)
        want.append(y + plain_llama.swiglu(h, w["feed_forward.gate_up.weight"][:I],
                                           w["feed_forward.gate_up.weight"][I:], w["feed_forward.down.weight"]))
    assert (got - torch.cat(want)).abs().max() < 2e-5
    # the mixer alone, on the block's first norm output
    mixer = MIXERS.build(aspec, env)
    mixer.bind({k[len("mixer."):]: v.cuda() for k, v in w.items() if k.startswith("mixer.")})
    h = block.norm_in.forward(x_in.clone(), None)
    a = mixer.forward(h, step, pools.view(0, writes=True)).cpu()
    ref = torch.cat([plain_llama.attention_block(plain_llama.rms_norm(xi, w["norm_in.weight"], 1e-5), pw, "a.", cfg,
                                                 torch.arange(xi.shape[0]))[0] for xi in xs])
    assert (a - ref).abs().max() < 2e-5


# ------------------------------------------------------------------ toy feed-forward with routing, toy positions
@dataclass(frozen=True)
class TopOneSpec:
    hidden_size: int
    inner: int
    experts: int
    kind: str = "toy_top1"


@dataclass(frozen=True)
class SinusoidSpec:
    hidden_size: int
    base: float
    kind: str = "toy_sinusoid"


def register_toy_ffn_and_positions():
    from llmserve_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, ParamDecl, PositionEncoding

    if "toy_top1" not in FEED_FORWARDS.classes:
        @FEED_FORWARDS.register("toy_top1")
        class TopOne(FeedForward):
            """Router logits in float32, one expert per token: y = relu(h W1_e) W2_e * p_e."""

            def param_decls(self):
                s = self.spec
                d = {"router.weight": ParamDecl((s.experts, s.hidden_size), "matrix")}
                for e in range(s.experts):
                    d[f"w1.{e}.weight"] = ParamDecl((s.inner, s.hidden_size), "matrix")
                    d[f"w2.{e}.weight"] = ParamDecl((s.hidden_size, s.inner), "matrix")
                return d

            def bind(self, params):
                self.p = params

            def forward(self, h, step):
                logits = self.ops.linear(h, self.p["router.weight"], None, out_dtype=torch.float32)
                prob, pick = logits.softmax(-1).max(-1)
                out = torch.zeros(h.shape[0], self.spec.hidden_size, dtype=torch.float32, device=h.device)
                for e in range(self.spec.experts):
                    rows = (pick == e).nonzero()[:, 0]
                    if rows.numel():
                        a = torch.relu(self.ops.linear(h[rows].contiguous(), self.p[f"w1.{e}.weight"], None,
                                                       out_dtype=torch.float32))
                        out[rows] = self.ops.linear(a.contiguous(), self.p[f"w2.{e}.weight"], None,
                                                    out_dtype=torch.float32) * prob[rows, None]
                return out

    if "toy_sinusoid" not in POSITION_ENCODINGS.classes:
        @POSITION_ENCODINGS.register("toy_sinusoid")
        class Sinusoid(PositionEncoding):
            """Absolute positions added to the embedded tokens (the ``embed`` hook)."""

            def __init__(self, spec, env):
                super().__init__(spec, env)
                self.table = sinusoid_table(env.max_positions, spec.hidden_size, spec.base).to(env.device)

            def embed(self, x, positions):
                x += self.table[positions.long()]


def sinusoid_table(n, width, base):
    pos = torch.arange(n, dtype=torch.float64)[:, None]
    freq = base ** (-torch.arange(0, width, 2, dtype=torch.float64) / width)
    return torch.cat([(pos * freq).sin(), (pos * freq).cos()], dim=-1).float()


def test_toy_routed_feed_forward_and_absolute_positions(tiny_dirs):
    """Another feed-forward (routing) in layer 1 and another position encoding (absolute, added at
    the embedding; the attention layers then use none), registered here and stepped in every cut."""
    from llmserve_b200.config import load_model_config
    from llmserve_b200.engine.runner import ModelRunner
    from llmserve_b200.models import DecoderModel
    from llmserve_b200.ops import get_ops
    from llmserve_b200.parts import BuildEnv, NoPositionSpec
    from llmserve_b200.weights import load_parameters

    register_toy_ffn_and_positions()
    folder = tiny_dirs["A"]
    arch, cfg = load_model_config(folder)
    plan = arch.plan(cfg)
    H = cfg.hidden_size
    nopos = [dataclasses.replace(l, mixer=dataclasses.replace(l.mixer, position=NoPositionSpec())) for l in plan.layers]
    routed = dataclasses.replace(nopos[1], feed_forward=TopOneSpec(H, 48, 3))
    plan = dataclasses.replace(plan, layers=(nopos[0], routed), embed_position=SinusoidSpec(H, 50.0))
    env = BuildEnv(get_ops("cuda"), torch.float32, torch.device("cuda"), 256, torch.float32)
    model = DecoderModel(plan, env)
    params = load_parameters(folder, arch.checkpoint_layout(cfg), torch.float32, "cuda")
    params = {k: v for k, v in params.items() if not k.startswith("layers.1.feed_forward.")}
    g = torch.Generator().manual_seed(3)
    toy = {}
    for name, d in model.param_decls().items():
        if name.startswith("layers.1.feed_forward."):
            toy[name] = torch.randn(d.shape, generator=g) * (1.0 if "router" in name else 0.08)
    model.bind({**params, **{k: v.cuda() for k, v in toy.items()}})
    runner = ModelRunner(model, page_tokens=16, num_pages=24, max_model_len=256, max_num_seqs=4)
    reqs = traces.make_requests([40, 23, 70, 9, 55], 256, seed=17)
    pcfg, w = plain_llama.read_config(folder), plain_llama.read_weights(folder)
    table = sinusoid_table(256, H, 50.0)

    def plain(ids):
        T = len(ids)
        x = w["model.embed_tokens.weight"][torch.as_tensor(ids)] + table[:T]
        for layer in range(2):
            p = f"model.layers.{layer}."
            h = plain_llama.rms_norm(x, w[p + "input_layernorm.weight"], pcfg["eps"])
            qq = (h @ w[p + "self_attn.q_proj.weight"].T).view(T, pcfg["heads"], pcfg["head_dim"])
            kk = (h @ w[p + "self_attn.k_proj.weight"].T).view(T, pcfg["kv_heads"], pcfg["head_dim"])
            vv = (h @ w[p + "self_attn.v_proj.weight"].T).view(T, pcfg["kv_heads"], pcfg["head_dim"])
            a = plain_llama.attention(qq, kk, vv, pcfg["head_dim"] ** -0.5).reshape(T, -1)
            x = x + a @ w[p + "self_attn.o_proj.weight"].T
            h = plain_llama.rms_norm(x, w[p + "post_attention_layernorm.weight"], pcfg["eps"])
            if layer == 0:
                x = x + plain_llama.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                           w[p + "mlp.down_proj.weight"])
            else:
                prob, pick = (h @ toy["layers.1.feed_forward.router.weight"].T).softmax(-1).max(-1)
                y = torch.zeros_like(x)
                for e in range(3):
                    rows = pick == e
                    a1 = torch.relu(h[rows] @ toy[f"layers.1.feed_forward.w1.{e}.weight"].T)
                    y[rows] = (a1 @ toy[f"layers.1.feed_forward.w2.{e}.weight"].T) * prob[rows, None]
                x = x + y
        x = plain_llama.rms_norm(x, w["model.norm.weight"], pcfg["eps"])
        return x @ w["model.embed_tokens.weight"].T

    expected = {r: plain(t) for r, t in reqs.items()}
    got = traces.replay(runner, traces.mixed(reqs, seed=6))
    traces.compare(got, expected, atol=3e-5)


def test_toy_state_mixer_through_the_engine_with_graphs_on(tiny_dirs, tmp_path):
    """A whole architecture registered from this file alone (its own name in config.json, the toy
    mixer with state in layer 0) generates through ``LLM`` with CUDA graphs switched on: the toy
    mixer declares that it works from the host, so no step of this model is captured, and the
    tokens are the plain model's."""
    from llmserve_b200 import LLM, LlamaConfig, SamplingParams
    from llmserve_b200.config.registry import ARCHITECTURES, Architecture, register_architecture
    from llmserve_b200.models.llama import llama_checkpoint_layout, llama_plan
    from llmserve_b200.models.plan import ParamSource, Source
    from llmserve_b200.weights import write_random_model

    register_toy()

    class ToyConfig(LlamaConfig):
        architecture = "ToyDecayForCausalLM"

    def toy_plan(cfg):
        plan = llama_plan(cfg)
        first = dataclasses.replace(plan.layers[0], mixer=DecaySpec(cfg.hidden_size, 0.9))
        return dataclasses.replace(plan, layers=(first, *plan.layers[1:]))

    def toy_layout(cfg):
        layout = llama_checkpoint_layout(cfg)
        keep = tuple(e for e in layout.entries if not e.param.startswith("layers.0.mixer."))
        mine = ParamSource("layers.0.mixer.w.weight",
                           (Source("model.layers.0.toy.w.weight", (cfg.hidden_size, cfg.hidden_size)),))
        return dataclasses.replace(layout, entries=keep + (mine,))

    register_architecture(Architecture("ToyDecayForCausalLM", "toy_decay", ToyConfig, toy_plan, toy_layout))
    try:
        base = {k: v for k, v in TINY["A"].items() if k not in ("seed", "page_tokens")}
        cfg = ToyConfig.from_dict({"model_type": "llama", **base})
        write_random_model(tmp_path, cfg, seed=3)
        # sharper weights, so that greedy choices are no near-ties
        from safetensors.torch import load_file, save_file

        t = {k: (v.float() * 6).to(v.dtype) if v.dim() > 1 else v for k, v in
             load_file(str(tmp_path / "model.safetensors")).items()}
        save_file(t, str(tmp_path / "model.safetensors"))
        llm = LLM(str(tmp_path), dtype="float32", block_size=16, num_kv_blocks=32, max_model_len=256,
                  max_num_seqs=4, cuda_graphs=True)
        prompts = [[5, 9, 200, 31, 7], list(range(40, 70)), [3, 4]]
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
        graphs = llm.engine.runner.decode_graphs
        assert graphs is None or (not graphs.capturable and not graphs.graphs)
        pcfg, w = plain_llama.read_config(tmp_path), plain_llama.read_weights(tmp_path)
        mix_w = w["model.layers.0.toy.w.weight"]
        for p, o in zip(prompts, outs):
            ids = list(p)
            for _ in range(10):
                ids.append(int(toy_plain(w, pcfg, ids, 0.9, mix_w)[-1].argmax()))
            assert o.outputs[0].token_ids == ids[len(p):]
    finally:
        ARCHITECTURES.pop("ToyDecayForCausalLM", None)


def test_scales_around_the_stack_of_layers_are_data_of_the_plan(tiny_dirs):
    """A multiplier on the embedded tokens, a multiplier and a soft cap on the logits: set in the
    plan, not in the decoder. Compared with the plain model given the scaled embedding table (the
    head of configuration B is a tensor of its own) and the same two steps on its logits."""
    from llmserve_b200.config import load_model_config
    from llmserve_b200.engine.batch import StepEntry
    from llmserve_b200.engine.runner import ModelRunner
    from llmserve_b200.models import DecoderModel
    from llmserve_b200.ops import get_ops
    from llmserve_b200.parts import BuildEnv
    from llmserve_b200.weights import load_parameters

    folder = tiny_dirs["B"]
    arch, cfg = load_model_config(folder)
    plan = dataclasses.replace(arch.plan(cfg), embed_scale=3.0, logit_scale=0.25, logit_softcap=0.2)
    ids = traces.make_requests([37], cfg.vocab_size, seed=2)["r0"]
    w = plain_llama.read_weights(folder)
    w["model.embed_tokens.weight"] = w["model.embed_tokens.weight"] * 3.0
    want = plain_llama.forward(plain_llama.read_config(folder), w, ids)
    want = 0.2 * torch.tanh(want * 0.25 / 0.2)
    for dtype, bound in ((torch.float32, 1e-5), (torch.bfloat16, 0.03 * float(want.abs().max()))):
        env = BuildEnv(get_ops("cuda"), dtype, torch.device("cuda"), 512, torch.float32)
        model = DecoderModel(plan, env)
        model.bind(load_parameters(folder, arch.checkpoint_layout(cfg), dtype, "cuda"))
        runner = ModelRunner(model, page_tokens=8, num_pages=8, max_model_len=512, max_num_seqs=2)
        got = runner.run([StepEntry("r", ids, list(range(len(ids))))]).float().cpu()
        assert (got - want).abs().max() <= bound
