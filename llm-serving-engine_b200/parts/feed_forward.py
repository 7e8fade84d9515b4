"""Dense gated feed-forward (src/llmserve/models/transformer.py:62-71).

    gu = h @ Wgu^T          rows of Wgu: gate (first I rows), then up (last I rows)
    y  = (silu(gate) * up) @ Wdown^T,    silu(g) = g / (1 + exp(-g))

No biases. The activation is computed in float32 (src/llmserve/kernels/csrc/fused_ops.cpp:75-91).
"""

from __future__ import annotations

from dataclasses import dataclass

from .base import FEED_FORWARDS, FeedForward, ParamDecl, project_into


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def param_decls(self):
        s = self.spec
        return {
            "gate_up.weight": ParamDecl((2 * s.intermediate_size, s.hidden_size), "matrix"),
            "down.weight": ParamDecl((s.hidden_size, s.intermediate_size), "matrix"),
        }

    def bind(self, params):
        self.gate_up_weight = params["gate_up.weight"]
        self.down_weight = params["down.weight"]

    accepts_residual = True

    def forward(self, h, step, residual=None, may_defer=False):
        ops = self.ops
        a = ops.gated_silu(h, self.gate_up_weight, None, out_dtype=self.env.dtype)
        return project_into(ops, a, self.down_weight, None, self.env.residual_dtype, residual, may_defer)
