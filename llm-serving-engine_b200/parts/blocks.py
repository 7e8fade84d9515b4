"""Block arrangements.

``prenorm`` (src/llmserve/models/transformer.py:87-94, fused form :176-189):

    x <- x + mixer(norm_in(x));   x <- x + feed_forward(norm_post(x))

The residual stream ``x`` is float32 and is updated in place; each add is carried out by the norm
that reads ``x`` next, so a block returns its feed-forward output as ``pending``: a tensor, None
(already added), or pending sums of the kernel set (see ``parts.base.settle``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, settle


@dataclass(frozen=True)
class PreNormBlockSpec:
    norm_in: Any
    mixer: Any
    norm_post: Any
    feed_forward: Any
    kind: str = "prenorm"


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: PreNormBlockSpec, env) -> None:
        super().__init__(spec, env)
        self.children = {
            "norm_in": NORMS.build(spec.norm_in, env),
            "mixer": MIXERS.build(spec.mixer, env),
            "norm_post": NORMS.build(spec.norm_post, env),
            "feed_forward": FEED_FORWARDS.build(spec.feed_forward, env),
        }
        self.norm_in = self.children["norm_in"]
        self.mixer = self.children["mixer"]
        self.norm_post = self.children["norm_post"]
        self.feed_forward = self.children["feed_forward"]

    def forward(self, x, pending, step, cache):
        h = self.norm_in.forward(x, settle(pending, self.norm_in))
        if getattr(self.mixer, "accepts_residual", False):
            a = self.mixer.forward(h, step, cache, residual=x, may_defer=True)  # None: already added into x
        else:
            a = self.mixer.forward(h, step, cache)
        h = self.norm_post.forward(x, settle(a, self.norm_post))
        if getattr(self.feed_forward, "accepts_residual", False):
            return x, self.feed_forward.forward(h, step, residual=x, may_defer=True)
        return x, self.feed_forward.forward(h, step)
