"""Causal self-attention over a paged key/value cache, with grouped query heads.

Per token (src/llmserve/models/transformer.py:37-59, src/llmserve/attention.py:231-307):

    qkv = h @ Wqkv^T (+ b)                      rows of Wqkv ordered q, then k, then v
    q, k = rotate(q, k; position)               if the position encoding has rotary tables
    cache[k, v at this token's slot] = k, v     before attention, so a portion attends to itself
    s_j = scale * q . k_j   for every key j of the same request with j <= position
                            (and j > position - window if the layer has a window)
    o = sum_j softmax(s)_j v_j                  query head h reads key/value head h // group
    out = o @ Wo^T (+ b)

``scale`` and ``window`` are parameters of the spec. Scores, softmax and the weighted sum run in
float32 inside the kernels.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import MIXERS, POSITION_ENCODINGS, Mixer, PagedKVNeed, ParamDecl, project_into


@dataclass(frozen=True)
class AttentionSpec:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: Any  # a position-encoding spec
    bias: bool = False
    window: int = 0  # 0: every earlier token; w: the last w tokens, the query's own included
    kind: str = "attention"


@MIXERS.register("attention")
class PagedAttention(Mixer):
    def __init__(self, spec: AttentionSpec, env) -> None:
        super().__init__(spec, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        self.position = POSITION_ENCODINGS.build(spec.position, env)
        self.rotary = self.position.rotary_tables()
        env.ops.check_attention_shape(spec.head_dim, env.dtype, spec.num_heads, spec.num_kv_heads)

    def param_decls(self):
        s = self.spec
        decls = {
            "qkv.weight": ParamDecl((self.q_size + 2 * self.kv_size, s.hidden_size), "matrix"),
            "o.weight": ParamDecl((s.hidden_size, self.q_size), "matrix"),
        }
        if s.bias:
            decls["qkv.bias"] = ParamDecl((self.q_size + 2 * self.kv_size,), "bias")
            decls["o.bias"] = ParamDecl((s.hidden_size,), "bias")
        return decls

    def bind(self, params):
        self.qkv_weight = params["qkv.weight"]
        self.o_weight = params["o.weight"]
        self.qkv_bias = params.get("qkv.bias")
        self.o_bias = params.get("o.bias")

    # what the cache manager has to keep for a layer of this kind
    def cache_need(self):
        s = self.spec
        return PagedKVNeed(s.num_kv_heads, s.head_dim, s.window)

    def reserve(self, max_seqs: int) -> None:
        """Allocate kernel scratch for up to ``max_seqs`` single-token sequences in a step."""
        if hasattr(self.ops, "reserve_attention_scratch"):
            self.ops.reserve_attention_scratch(self.spec.head_dim, max_seqs, self.spec.num_heads)

    # work lists depend only on the batch, the kernels' tile size and the group's page size
    def plan_key(self):
        return ("attention", self.env.dtype, self.spec.head_dim)

    def plan_step(self, host_step, group):
        return self.ops.attention_plan(host_step, self.env.dtype, self.spec.head_dim)

    def plan_rows(self, single: int, portions: int, tokens: int) -> dict[str, int]:
        """Most rows of each work list for a step of ``single`` one-token sequences and ``portions``
        longer ones that hold ``tokens`` tokens together. A captured step has lists of exactly this
        many rows; a shorter list is filled up by repeating its last row (a tile that is computed
        twice writes the same values twice)."""
        qt = self.ops.attention_q_tile(self.env.dtype, self.spec.head_dim)
        return {"tiles": tokens // qt + portions, "decode_seqs": single}

    accepts_residual = True

    def forward(self, h, step, cache, residual=None, may_defer=False):
        s = self.spec
        ops = self.ops
        tables = step.block_tables[cache.group]
        cos, sin = self.rotary if self.rotary is not None else (None, None)
        o = ops.project_attend(
            h, self.qkv_weight, self.qkv_bias,
            num_heads=s.num_heads,
            num_kv_heads=s.num_kv_heads,
            head_dim=s.head_dim,
            scale=s.scale,
            window=s.window,
            positions=step.positions,
            token_seq=step.token_seq,
            cos=cos,
            sin=sin,
            k_pages=cache.k,
            v_pages=cache.v,
            writes=cache.writes,
            block_tables=tables,
            page_tokens=cache.page_tokens,
            step=step,
            plan=step.plans[self.plan_key()],
            out_dtype=self.env.dtype,
        )
        return project_into(ops, o, self.o_weight, self.o_bias, self.env.residual_dtype, residual, may_defer)
