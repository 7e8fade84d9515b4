"""Compare the plain implementation with the reference's own model code, once, on the CPU.

Run from the repository root with the reference checkout available:

    python tests/golden/make_golden.py /path/to/reference

For each case it writes a tiny random Llama folder (seeded, via the engine's random-weights mode),
loads the same tensors into the reference's ``llmserve.models.transformer.CausalLM``, runs the
reference's forward through its own paged cache with a reversed block table on a fixed token
sequence, checks that ``tests/plain_llama.py`` gives the same logits, and stores the reference's
logits in ``tests/golden/tiny_llama_reference_logits.safetensors`` together with the token ids, the
weights themselves and (in the file's metadata) each case's config.json. ``tests/test_plain.py``
replays the comparison from that file alone, without the reference and whatever random numbers
this machine's torch draws. The cases cover grouped and single key/value heads, tied and untied
heads, attention biases with head size 64, and the "linear" and "llama3" scalings of the rotary
frequencies (src/llmserve/models/layers.py:24-58, src/llmserve/config.py:47-49,64).
"""

from __future__ import annotations

import json
import sys
import tempfile
from pathlib import Path

import torch
from safetensors.torch import save_file

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

GOLDEN = Path(__file__).resolve().parent / "tiny_llama_reference_logits.safetensors"
CASES = {
    # name: (config overrides, seed, tokens)
    "gqa_tied": (dict(vocab_size=256, hidden_size=64, intermediate_size=160, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=16, rope_theta=10000.0,
                      rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=256), 0, 33),
    "mqa_untied": (dict(vocab_size=384, hidden_size=128, intermediate_size=352, num_hidden_layers=3,
                        num_attention_heads=4, num_key_value_heads=1, head_dim=32, rope_theta=100000.0,
                        rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=512), 2, 40),
    "bias_d64": (dict(vocab_size=131, hidden_size=96, intermediate_size=136, num_hidden_layers=1,
                      num_attention_heads=3, num_key_value_heads=1, head_dim=64, rope_theta=50000.0,
                      rms_norm_eps=3e-6, tie_word_embeddings=False, attention_bias=True,
                      max_position_embeddings=128), 7, 50),
    "rope_linear": (dict(vocab_size=97, hidden_size=48, intermediate_size=80, num_hidden_layers=1,
                         num_attention_heads=3, num_key_value_heads=3, head_dim=16, rope_theta=10000.0,
                         rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=256,
                         rope_scaling={"rope_type": "linear", "factor": 4.0}), 11, 120),
    "rope_llama3": (dict(vocab_size=97, hidden_size=48, intermediate_size=80, num_hidden_layers=1,
                         num_attention_heads=3, num_key_value_heads=1, head_dim=32, rope_theta=500000.0,
                         rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=256,
                         rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                       "high_freq_factor": 4.0, "original_max_position_embeddings": 64}),
                    13, 200),
}


def case_inputs(name):
    import plain_llama  # noqa: F401
    from llmserve_b200.config import LlamaConfig

    over, seed, n = CASES[name]
    cfg = LlamaConfig.from_dict({"model_type": "llama", **over})
    ids = torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed + 1))
    return cfg, seed, ids


def main(reference_root: str) -> None:
    import plain_llama
    from llmserve_b200.weights import write_random_model

    sys.path.insert(0, str(Path(reference_root) / "src"))
    from llmserve.attention import AttentionMetadata
    from llmserve.config import ModelConfig
    from llmserve.kv_cache import KVCache
    from llmserve.models.loader import load_state_dict_into
    from llmserve.models.transformer import CausalLM

    out, configs = {}, {}
    for name in CASES:
        cfg, seed, ids = case_inputs(name)
        with tempfile.TemporaryDirectory() as d:
            write_random_model(d, cfg, seed, store_dtype=torch.float32)
            w = plain_llama.read_weights(d)
            ours = plain_llama.model_logits(d, ids.tolist())
            rcfg = ModelConfig.from_dict(cfg.to_dict())
            ref = CausalLM(rcfg, max_positions=cfg.max_position_embeddings).eval()
            load_state_dict_into(ref, iter(w.items()), torch.float32)
        bs, n = 4, ids.shape[0]
        nblocks = -(-n // bs)
        cache = KVCache(rcfg, nblocks + 3, bs, torch.float32, "cpu")
        table = list(range(nblocks + 2, 2, -1))[:nblocks]  # reversed, not starting at 0
        meta = AttentionMetadata.build([n], [n], [table], bs, backend="torch")
        with torch.no_grad():
            hidden = ref(ids, torch.arange(n), cache.layers, meta)
            logits = ref.compute_logits(hidden)
        diff = (logits - ours).abs().max().item()
        print(f"{name}: max |reference - plain| = {diff:.3e}")
        assert diff < 1e-5, diff
        out[f"{name}.logits"] = logits.contiguous()
        out[f"{name}.ids"] = ids.to(torch.int32)
        for k, v in w.items():
            out[f"{name}.weights.{k}"] = v.contiguous()
        configs[name] = cfg.to_dict()
    save_file(out, str(GOLDEN), metadata={"configs": json.dumps(configs)})
    print("wrote", GOLDEN)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
