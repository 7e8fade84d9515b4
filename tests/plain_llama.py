"""A plain, slow implementation of the Llama forward pass, written from the reference's formulas.

Whole sequences, no cache, no batching, float32 (or float64), one function per part. It runs on
the CPU unless a test names another device for the models with real layer widths (the same plain
torch operations, in float64, only faster). It shares no code with the engine: it reads
``config.json`` with ``json`` and the weights with ``safetensors`` by their checkpoint names.

It was compared once with the reference's own model code (``llmserve.models.transformer.CausalLM``
imported on the CPU); the script and its small outputs are in ``tests/golden/``.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


def read_config(folder) -> dict:
    """config.json with the reference's defaults filled in (src/llmserve/config.py:35-68)."""
    d = json.loads((Path(folder) / "config.json").read_text())
    nh = d["num_attention_heads"]
    rp = d.get("rope_parameters") or {}
    scaling = d.get("rope_scaling")
    if scaling is None and rp.get("rope_type", "default") != "default":
        scaling = rp
    return {
        "vocab": d["vocab_size"],
        "hidden": d["hidden_size"],
        "inter": d["intermediate_size"],
        "layers": d["num_hidden_layers"],
        "heads": nh,
        "kv_heads": d.get("num_key_value_heads", nh),
        "head_dim": d.get("head_dim") or d["hidden_size"] // nh,
        "eps": d.get("rms_norm_eps", 1e-6),
        "theta": rp.get("rope_theta", d.get("rope_theta", 10000.0)),
        "rope_scaling": scaling,
        "tied": d.get("tie_word_embeddings", False),
        "bias": d.get("attention_bias", False),
    }


def read_weights(folder, dtype=torch.float32) -> dict[str, torch.Tensor]:
    out = {}
    for f in sorted(Path(folder).glob("*.safetensors")):
        with safe_open(str(f), framework="pt") as fh:
            for name in fh.keys():  # noqa: SIM118
                out[name] = fh.get_tensor(name).to(dtype)
    return out


def rms_norm(x, weight, eps):
    """src/llmserve/models/layers.py:17-21: x * rsqrt(mean(x^2) + eps), then the weight."""
    return weight * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))


def rope_inverse_frequencies(head_dim, theta, scaling=None):
    """src/llmserve/models/layers.py:24-58, in float64."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type"))
    if kind == "linear":
        inv = inv / scaling["factor"]
    elif kind == "llama3":
        factor = scaling["factor"]
        low = scaling.get("low_freq_factor", 1.0)
        high = scaling.get("high_freq_factor", 4.0)
        old = scaling["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv
        scaled = torch.where(wavelen > old / low, inv / factor, inv)
        smooth = (old / wavelen - low) / (high - low)
        mid = (1 - smooth) * scaled / factor + smooth * scaled
        inv = torch.where((wavelen >= old / high) & (wavelen <= old / low), mid, scaled)
    elif kind not in (None, "default"):
        raise NotImplementedError(kind)
    return inv


def rope_tables(positions, head_dim, theta, scaling=None, dtype=torch.float32):
    """cos and sin ``[T, head_dim]`` (both halves alike), src/llmserve/models/layers.py:59-63."""
    inv = rope_inverse_frequencies(head_dim, theta, scaling).to(positions.device)
    ang = torch.outer(positions.to(torch.float64), inv)
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope(x, cos, sin):
    """src/llmserve/models/layers.py:86-90; x ``[T, heads, D]``, cos/sin ``[T, D]``."""
    half = x.shape[-1] // 2
    rotated = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos[:, None, :] + rotated * sin[:, None, :]


def attention(q, k, v, scale, window=0):
    """Causal softmax attention of one whole sequence; q ``[T, Hq, D]``, k, v ``[T, Hk, D]``.

    Query head h reads key/value head h // (Hq // Hk) (src/llmserve/attention.py:249-257 with
    ``enable_gqa``); key j is visible to query i iff j <= i, and i - j < window if window > 0.
    """
    T, hq, _ = q.shape
    group = hq // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    s = torch.einsum("thd,shd->hts", q, k) * scale
    i = torch.arange(T, device=q.device)[:, None]
    j = torch.arange(T, device=q.device)[None, :]
    visible = j <= i
    if window > 0:
        visible &= (i - j) < window
    s = s.masked_fill(~visible, float("-inf"))
    return torch.einsum("hts,shd->thd", s.softmax(-1), v)


def swiglu(x, w_gate, w_up, w_down):
    """src/llmserve/models/transformer.py:69-71: down(silu(gate(x)) * up(x))."""
    g = x @ w_gate.T
    return ((g * torch.sigmoid(g)) * (x @ w_up.T)) @ w_down.T


def attention_block(h, w, prefix, cfg, positions, window=0, kv_from=None):
    """Projections, rotary positions, attention and the output projection of one layer.

    Returns (output, (k, v)); ``kv_from`` replaces this layer's own keys and values (a layer that
    reads another layer's cache).
    """
    T = h.shape[0]
    D = cfg["head_dim"]
    q = h @ w[prefix + "q_proj.weight"].T
    k = h @ w[prefix + "k_proj.weight"].T
    v = h @ w[prefix + "v_proj.weight"].T
    if cfg["bias"]:
        q = q + w[prefix + "q_proj.bias"]
        k = k + w[prefix + "k_proj.bias"]
        v = v + w[prefix + "v_proj.bias"]
    q = q.view(T, cfg["heads"], D)
    k = k.view(T, cfg["kv_heads"], D)
    v = v.view(T, cfg["kv_heads"], D)
    cos, sin = rope_tables(positions, D, cfg["theta"], cfg["rope_scaling"], h.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    if kv_from is not None:
        k, v = kv_from
    o = attention(q, k, v, D**-0.5, window).reshape(T, cfg["heads"] * D)
    o = o @ w[prefix + "o_proj.weight"].T
    if cfg["bias"]:
        o = o + w[prefix + "o_proj.bias"]
    return o, (k, v)


def forward(cfg, w, token_ids, run_order=None, windows=None, dtype=torch.float32, device="cpu",
            rows=None):
    """Logits ``[T, vocab]`` for one whole sequence (src/llmserve/models/transformer.py:125-139).

    run_order: list of (layer, cache id); default every layer once with its own cache. An entry
    whose cache id was filled by an earlier entry reads that entry's keys and values.
    windows: per layer attention window (0 = all), default none.
    rows: positions whose logits are returned (default all; a large vocabulary times thousands of
    positions would not fit). The result comes back on the CPU.
    """
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=device)
    positions = torch.arange(ids.shape[0], device=device)
    w = {k: v.to(device=device, dtype=dtype) for k, v in w.items()}
    x = w["model.embed_tokens.weight"][ids]
    run_order = run_order or [(i, i) for i in range(cfg["layers"])]
    caches = {}
    for layer, cache in run_order:
        p = f"model.layers.{layer}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        win = windows[layer] if windows else 0
        a, kv = attention_block(h, w, p + "self_attn.", cfg, positions, win, caches.get(cache))
        caches.setdefault(cache, kv)
        x = x + a
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        x = x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"])
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long, device=device)]
    x = rms_norm(x, w["model.norm.weight"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return (x @ head.T).cpu()


def model_logits(folder, token_ids, dtype=torch.float32, **kw):
    return forward(read_config(folder), read_weights(folder, dtype), token_ids, dtype=dtype, **kw)


def greedy(folder, prompt, n_new):
    """Greedy continuation by recomputing the whole sequence each time."""
    cfg, w = read_config(folder), read_weights(folder)
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(forward(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt):]
