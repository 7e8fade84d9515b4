"""Root-mean-square norm (src/llmserve/models/layers.py:11-21).

``y = x * rsqrt(mean(x^2) + eps) * w`` with the statistics, the scaling and the weight multiply in
float32; the result is rounded once to the compute dtype. The residual add that precedes the norm
in a pre-norm block is part of the same kernel (src/llmserve/kernels/csrc/fused_ops.cpp:52-73).
"""

from __future__ import annotations

from dataclasses import dataclass

from .base import NORMS, Norm, ParamDecl


@dataclass(frozen=True)
class RMSNormSpec:
    size: int
    eps: float
    kind: str = "rmsnorm"


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    takes_pending_sums = True  # the kernel adds a product's pending sums as it reads the row

    def param_decls(self):
        return {"weight": ParamDecl((self.spec.size,), "scale")}

    def forward(self, x, residual=None, rows=None):
        return self.ops.add_rmsnorm(
            x, residual, self.weight, self.spec.eps, out_dtype=self.env.dtype, rows=rows
        )
