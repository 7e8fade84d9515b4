"""The Llama architecture as data: which parts each layer has and where its tensors come from.

Layer structure from src/llmserve/models/transformer.py:19-139; tensor names and the fusing of
q|k|v and gate|up from src/llmserve/models/loader.py:16-85.
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..parts.attention import AttentionSpec
from ..parts.blocks import PreNormBlockSpec
from ..parts.feed_forward import SwiGLUSpec
from ..parts.norms import RMSNormSpec
from ..parts.positions import RotarySpec
from .plan import CheckpointLayout, ModelPlan, ParamSource, RunEntry, Source


def llama_plan(cfg: LlamaConfig) -> ModelPlan:
    rs = cfg.rope_scaling
    position = RotarySpec(
        head_dim=cfg.head_dim,
        theta=cfg.rope_theta,
        scaling_type=rs.rope_type,
        factor=rs.factor,
        low_freq_factor=rs.low_freq_factor,
        high_freq_factor=rs.high_freq_factor,
        original_max_positions=rs.original_max_position_embeddings,
    )
    norm = RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps)
    layer = PreNormBlockSpec(
        norm_in=norm,
        mixer=AttentionSpec(
            hidden_size=cfg.hidden_size,
            num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim,
            scale=cfg.head_dim**-0.5,
            position=position,
            bias=cfg.attention_bias,
            window=0,
        ),
        norm_post=norm,
        feed_forward=SwiGLUSpec(cfg.hidden_size, cfg.intermediate_size),
    )
    n = cfg.num_hidden_layers
    return ModelPlan(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        layers=tuple(layer for _ in range(n)),
        run_order=tuple(RunEntry(i, i) for i in range(n)),
        final_norm=norm,
        tie_head=cfg.tie_word_embeddings,
    )


def llama_checkpoint_layout(cfg: LlamaConfig) -> CheckpointLayout:
    h, q, kv, i = cfg.hidden_size, cfg.q_size, cfg.kv_size, cfg.intermediate_size
    entries = [
        ParamSource(
            "embed.weight", (Source("model.embed_tokens.weight", (cfg.vocab_size, h)),), "embedding"
        ),
        ParamSource("final_norm.weight", (Source("model.norm.weight", (h,)),), "scale"),
    ]
    if not cfg.tie_word_embeddings:
        entries.append(ParamSource("head.weight", (Source("lm_head.weight", (cfg.vocab_size, h)),)))
    for n in range(cfg.num_hidden_layers):
        src, dst = f"model.layers.{n}.", f"layers.{n}."
        entries += [
            ParamSource(
                dst + "norm_in.weight", (Source(src + "input_layernorm.weight", (h,)),), "scale"
            ),
            ParamSource(
                dst + "norm_post.weight",
                (Source(src + "post_attention_layernorm.weight", (h,)),),
                "scale",
            ),
            ParamSource(
                dst + "mixer.qkv.weight",
                (
                    Source(src + "self_attn.q_proj.weight", (q, h)),
                    Source(src + "self_attn.k_proj.weight", (kv, h)),
                    Source(src + "self_attn.v_proj.weight", (kv, h)),
                ),
            ),
            ParamSource(dst + "mixer.o.weight", (Source(src + "self_attn.o_proj.weight", (h, q)),)),
            ParamSource(
                dst + "feed_forward.gate_up.weight",
                (
                    Source(src + "mlp.gate_proj.weight", (i, h)),
                    Source(src + "mlp.up_proj.weight", (i, h)),
                ),
            ),
            ParamSource(
                dst + "feed_forward.down.weight", (Source(src + "mlp.down_proj.weight", (h, i)),)
            ),
        ]
        if cfg.attention_bias:
            entries += [
                ParamSource(
                    dst + "mixer.qkv.bias",
                    (
                        Source(src + "self_attn.q_proj.bias", (q,)),
                        Source(src + "self_attn.k_proj.bias", (kv,)),
                        Source(src + "self_attn.v_proj.bias", (kv,)),
                    ),
                    "bias",
                ),
                ParamSource(
                    dst + "mixer.o.bias", (Source(src + "self_attn.o_proj.bias", (h,)),), "bias"
                ),
            ]
    return CheckpointLayout(
        entries=tuple(entries),
        ignored_substrings=("rotary_emb",),
        ignored_names=("lm_head.weight",) if cfg.tie_word_embeddings else (),
    )
