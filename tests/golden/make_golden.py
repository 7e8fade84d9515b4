"""Compare the plain implementation with the reference's own model code, once, on the CPU.

Run from the repository root with the reference checkout available:

    python tests/golden/make_golden.py /path/to/reference

It writes a tiny random Llama folder (seeded, via the engine's random-weights mode), loads the same
tensors into the reference's ``llmserve.models.transformer.CausalLM``, runs the reference's forward
through its own paged cache with a reversed block table on a fixed token sequence, checks that
``tests/plain_llama.py`` gives the same logits, and stores the reference's logits in
``tests/golden/tiny_llama_reference_logits.safetensors`` together with the token ids and a checksum
of the weights. ``tests/test_plain.py`` replays the comparison from that file without the
reference.
"""

from __future__ import annotations

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
}


def case_inputs(name):
    import plain_llama  # noqa: F401
    from llmserve_b200.config import LlamaConfig

    over, seed, n = CASES[name]
    cfg = LlamaConfig.from_dict({"model_type": "llama", **over})
    ids = torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed + 1))
    return cfg, seed, ids


def weights_checksum(w: dict[str, torch.Tensor]) -> torch.Tensor:
    return torch.stack([w[k].double().sum() for k in sorted(w)]).sum().reshape(1)


def main(reference_root: str) -> None:
    import plain_llama
    from llmserve_b200.weights import write_random_model

    sys.path.insert(0, str(Path(reference_root) / "src"))
    from llmserve.attention import AttentionMetadata
    from llmserve.config import ModelConfig
    from llmserve.kv_cache import KVCache
    from llmserve.models.loader import load_state_dict_into
    from llmserve.models.transformer import CausalLM

    out = {}
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
        out[f"{name}.checksum"] = weights_checksum(w)
    save_file(out, str(GOLDEN))
    print("wrote", GOLDEN)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
