"""A decoder-only language model assembled from a :class:`ModelPlan`.

Token embedding -> the blocks in run order -> final norm on the wanted rows -> output projection
(src/llmserve/models/transformer.py:125-139, 192-193). The model owns no sizes or constants of
its own: they all come with the plan (layer specs, run order, and the optional scale of the
embedded tokens and scale / soft cap of the logits).
"""

from __future__ import annotations

import torch

from ..parts.base import BLOCKS, NORMS, POSITION_ENCODINGS, BuildEnv, ParamDecl, role_dtype, settle
from .plan import ModelPlan


class DecoderModel:
    def __init__(self, plan: ModelPlan, env: BuildEnv) -> None:
        plan.validate()
        self.plan = plan
        self.env = env
        self.ops = env.ops
        self.blocks = [BLOCKS.build(spec, env) for spec in plan.layers]
        self.final_norm = NORMS.build(plan.final_norm, env)
        self.embed_position = (
            POSITION_ENCODINGS.build(plan.embed_position, env) if plan.embed_position is not None else None
        )
        self.embed_weight: torch.Tensor | None = None
        self.head_weight: torch.Tensor | None = None
        # which run of the order fills each cache layer
        self.writer_of: dict[int, int] = {}
        for k, e in enumerate(plan.run_order):
            self.writer_of.setdefault(e.cache, k)

    # ------------------------------------------------------------------ parameters
    def param_decls(self) -> dict[str, ParamDecl]:
        p = self.plan
        decls = {"embed.weight": ParamDecl((p.vocab_size, p.hidden_size), "embedding")}
        for i, block in enumerate(self.blocks):
            for name, decl in block.param_decls().items():
                decls[f"layers.{i}.{name}"] = decl
        for name, decl in self.final_norm.param_decls().items():
            decls[f"final_norm.{name}"] = decl
        if not p.tie_head:
            decls["head.weight"] = ParamDecl((p.vocab_size, p.hidden_size), "matrix")
        return decls

    def param_dtype(self, name: str) -> torch.dtype:
        return role_dtype(self.param_decls()[name].role, self.env.dtype)

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        decls = self.param_decls()
        absent = sorted(set(decls) - set(params))
        extra = sorted(set(params) - set(decls))
        if absent or extra:
            raise KeyError(f"model parameters: missing {absent}, unexpected {extra}")
        for name, decl in decls.items():
            t = params[name]
            want = role_dtype(decl.role, self.env.dtype)
            if tuple(t.shape) != tuple(decl.shape) or t.dtype != want or not t.is_contiguous():
                raise ValueError(
                    f"{name}: got {tuple(t.shape)} {t.dtype}, want {tuple(decl.shape)} {want} contiguous"
                )
        self.embed_weight = params["embed.weight"]
        self.head_weight = params["embed.weight"] if self.plan.tie_head else params["head.weight"]
        for i, block in enumerate(self.blocks):
            prefix = f"layers.{i}."
            block.bind({k[len(prefix):]: v for k, v in params.items() if k.startswith(prefix)})
        self.final_norm.bind(
            {k[len("final_norm."):]: v for k, v in params.items() if k.startswith("final_norm.")}
        )

    def parts(self):
        """Every part of the model, blocks and what they are made of."""
        for block in self.blocks:
            yield block
            yield from block.children.values()
        yield self.final_norm
        if self.embed_position is not None:
            yield self.embed_position

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> dict[int, object]:
        """cache id -> what the layer that fills it keeps per request (None: nothing)."""
        needs: dict[int, object] = {}
        for k, e in enumerate(self.plan.run_order):
            mixer = self.blocks[e.layer].mixer_part()
            need = mixer.cache_need() if mixer is not None else None
            if e.cache not in needs:
                needs[e.cache] = need
            elif needs[e.cache] != need:
                raise ValueError(
                    f"run {k} (layer {e.layer}) reads cache {e.cache}, which holds {needs[e.cache]}, "
                    f"but its mixer needs {need}"
                )
        return needs

    def step_planners(self):
        """Distinct (plan_key, mixer, cache id) whose work lists the runner builds once a step."""
        seen = {}
        for e in self.plan.run_order:
            mixer = self.blocks[e.layer].mixer_part()
            if mixer is None:
                continue
            key = mixer.plan_key()
            if key is not None and key not in seen:
                seen[key] = (mixer, e.cache)
        return seen

    # ------------------------------------------------------------------ forward
    def forward(self, step, pools) -> torch.Tensor:
        """Run this step's tokens; return float32 logits ``[len(step.logit_rows), vocab]``."""
        x = self.ops.embedding(step.token_ids, self.embed_weight)
        if self.plan.embed_scale != 1.0:
            x *= self.plan.embed_scale
        if self.embed_position is not None:
            self.embed_position.embed(x, step.positions)  # absolute encodings change x in place
        pending = None
        for k, e in enumerate(self.plan.run_order):
            view = pools.view(e.cache, writes=self.writer_of[e.cache] == k)
            x, pending = self.blocks[e.layer].forward(x, pending, step, view)
        if step.num_logit_rows == 0:
            if hasattr(pending, "resolve"):
                pending.resolve()  # nobody reads x any more, but the kernel set's sums must be taken
            return torch.empty(0, self.plan.vocab_size, dtype=torch.float32, device=x.device)
        rows = None if step.every_row_wanted else step.logit_rows
        h = self.final_norm.forward(x, settle(pending, self.final_norm), rows=rows)
        logits = self.ops.linear(h, self.head_weight, None, out_dtype=torch.float32)
        if self.plan.logit_scale != 1.0:
            logits *= self.plan.logit_scale
        if self.plan.logit_softcap > 0.0:
            cap = self.plan.logit_softcap
            logits = torch.tanh_(logits.div_(cap)).mul_(cap)
        return logits
