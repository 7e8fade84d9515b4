"""Configuration, registry and weight loading (no GPU)."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY, tiny_config


def test_config_reads_hf_keys_and_defaults():
    from llmserve_b200.config import ConfigError, LlamaConfig

    base = dict(vocab_size=100, hidden_size=48, intermediate_size=96, num_hidden_layers=2,
                num_attention_heads=6)
    c = LlamaConfig.from_dict(base)
    assert (c.num_key_value_heads, c.head_dim, c.rms_norm_eps, c.rope_theta) == (6, 8, 1e-6, 10000.0)
    assert (c.max_position_embeddings, c.tie_word_embeddings, c.attention_bias) == (4096, False, False)
    c = LlamaConfig.from_dict({**base, "head_dim": 16, "num_key_value_heads": 2, "eos_token_id": [2, 7],
                               "rope_parameters": {"rope_theta": 5e5, "rope_type": "default"}})
    assert (c.head_dim, c.q_size, c.kv_size, c.rope_theta, c.eos_token_ids) == (16, 96, 32, 5e5, (2, 7))
    assert c.kv_bytes_per_token(2) == 2 * 2 * 32 * 2
    for bad in ({"hidden_act": "gelu"}, {"mlp_bias": True}, {"num_key_value_heads": 4},
                {"rope_scaling": {"rope_type": "yarn", "factor": 2}}, {"model_type": "qwen3"},
                {"head_dim": 7}):
        with pytest.raises(ConfigError):
            LlamaConfig.from_dict({**base, **bad})
    with pytest.raises(ConfigError, match="required"):
        LlamaConfig.from_dict({"vocab_size": 3})
    assert LlamaConfig.from_dict(c.to_dict()) == c


def test_generation_config_adds_eos(tmp_path):
    from llmserve_b200.config import LlamaConfig

    (tmp_path / "config.json").write_text(json.dumps({**tiny_config("A").to_dict(), "eos_token_id": 2}))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [2, 9]}))
    assert LlamaConfig.from_pretrained(tmp_path).eos_token_ids == (2, 9)


def test_registry_picks_the_model_by_config(tiny_dirs, tmp_path):
    from llmserve_b200.config import ARCHITECTURES, load_model_config

    arch, cfg = load_model_config(tiny_dirs["B"])
    assert arch is ARCHITECTURES["LlamaForCausalLM"] and cfg.num_hidden_layers == 3
    plan = arch.plan(cfg)
    assert len(plan.layers) == 3 and [e.layer for e in plan.run_order] == [0, 1, 2]
    assert plan.layers[0].mixer.scale == 32**-0.5 and plan.layers[0].mixer.position.theta == 100000.0
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["MambaForCausalLM"]}))
    with pytest.raises(KeyError, match="no architecture registered"):
        load_model_config(tmp_path)
    d = tiny_config("A").to_dict()
    d.pop("architectures")
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert load_model_config(tmp_path)[0].name == "LlamaForCausalLM"


def test_random_model_is_reproducible_and_loads(tiny_dirs, tmp_path):
    from llmserve_b200.config import load_model_config
    from llmserve_b200.weights import load_parameters, write_random_model

    write_random_model(tmp_path, tiny_config("A"), TINY["A"]["seed"])
    a = load_file(str(tmp_path / "model.safetensors"))
    b = load_file(str(tiny_dirs["A"] / "model.safetensors"))
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert all(v.dtype == torch.bfloat16 for v in a.values())
    assert abs(a["model.norm.weight"].float().mean() - 1) < 0.05
    assert "lm_head.weight" not in a  # tied
    arch, cfg = load_model_config(tmp_path)
    for dt in (torch.bfloat16, torch.float32):
        p = load_parameters(tmp_path, arch.checkpoint_layout(cfg), dt, "cpu")
        assert p["layers.0.mixer.qkv.weight"].shape == (64 + 2 * 32, 64)
        assert p["layers.0.mixer.qkv.weight"].dtype == dt
        assert p["layers.1.norm_in.weight"].dtype == torch.float32  # scales are held in 32-bit
        q = a["model.layers.0.self_attn.q_proj.weight"].to(dt)
        assert torch.equal(p["layers.0.mixer.qkv.weight"][:64], q)
        gate_up = p["layers.1.feed_forward.gate_up.weight"]
        assert torch.equal(gate_up[160:], a["model.layers.1.mlp.up_proj.weight"].to(dt))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tiny_dirs, tmp_path):
    from llmserve_b200.config import load_model_config
    from llmserve_b200.weights import CheckpointError, load_parameters

    t = load_file(str(tiny_dirs["B"] / "model.safetensors"))
    (tmp_path / "config.json").write_text((tiny_dirs["B"] / "config.json").read_text())
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["lm_head.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)  # ignored, as the reference does
    t["model.layers.9.mlp.down_proj.weight"] = torch.zeros(2, 2)
    t["model.norm.weight"] = torch.zeros(7, dtype=torch.bfloat16)
    save_file(t, str(tmp_path / "model.safetensors"))
    arch, cfg = load_model_config(tmp_path)
    with pytest.raises(CheckpointError) as e:
        load_parameters(tmp_path, arch.checkpoint_layout(cfg), torch.float32, "cpu")
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.9.mlp.down_proj.weight"]
    assert err.wrong_shape == [("model.norm.weight", (7,), (128,))]
    msg = str(err)
    assert "missing tensors (2)" in msg and "unexpected tensors (1)" in msg and "wrong shapes (1)" in msg
    with pytest.raises(FileNotFoundError):
        load_parameters(tmp_path / "nothing", arch.checkpoint_layout(cfg), torch.float32, "cpu")


def test_a_32bit_scale_stays_32bit_and_integers_become_int32(tmp_path):
    from llmserve_b200.parts.base import role_dtype

    assert role_dtype("scale", torch.bfloat16, torch.float32) == torch.float32
    assert role_dtype("matrix", torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert role_dtype("matrix", torch.float32, torch.bfloat16) == torch.float32
    assert role_dtype("matrix", torch.bfloat16, torch.int64) == torch.int32


def test_no_cpu_fallback_on_the_product_path():
    from llmserve_b200.ops import CudaOps

    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="CUDA device only"):
            CudaOps("cuda")
    with pytest.raises(RuntimeError, match="CUDA device only"):
        CudaOps("cpu")
