"""A decoder put together from a ``ModelPlan``: embedding, layers in run order, final norm, head.

``build_model(plan)`` builds every part through the part registry; the model
then lists its tensors (``tensor_specs``), receives them (``bind``), says what
cache each entry of the run order needs (``cache_needs``) and runs a step's
tokens (``forward``).  The loop over ``run_order`` is the only place where
layers are sequenced (crates/ferrisinfer-runtime/src/reference.rs:402-414 is the
reference's fixed ``for l in 0..L``).
"""

from __future__ import annotations

from typing import Optional

import torch

from .base import LayerCache, StepContext
from .plan import LayerPlan, ModelPlan, build_part


class DecoderModel:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.hidden_size, self.vocab_size = plan.hidden_size, plan.vocab_size
        self.embedding = build_part("embedding", plan.embedding)
        self.blocks = []
        for lp in plan.layers:
            self.blocks.append(self._build_layer(lp))
        self.final_norm = build_part("norm", plan.final_norm)
        self.output = build_part("output", plan.output)
        self.bound = False

    def _build_layer(self, lp: LayerPlan):
        return build_part(
            "block", lp.block,
            hidden_size=self.hidden_size,
            mixer=build_part("mixer", lp.mixer),
            feed_forward=build_part("feed_forward", lp.feed_forward),
            mixer_norm=build_part("norm", lp.mixer_norm),
            feed_forward_norm=build_part("norm", lp.feed_forward_norm),
        )

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model may be recorded into a CUDA graph."""
        return all(getattr(b, "graph_safe", False) for b in self.blocks)

    # ------------------------------------------------------------------ weights
    def tensor_specs(self) -> list:
        p = self.plan
        specs = list(self.embedding.tensor_specs(p.embedding_prefix))
        for lp, block in zip(p.layers, self.blocks):
            specs += block.tensor_specs(lp.prefix)
        specs += self.final_norm.tensor_specs(p.final_norm_prefix)
        specs += self.output.tensor_specs(p.output_prefix)
        names = [s.name for s in specs]
        if len(set(names)) != len(names):
            dup = sorted({n for n in names if names.count(n) > 1})
            raise ValueError(f"parts ask for the same tensor twice: {dup}")
        return specs

    def bind(self, tensors: dict) -> None:
        p = self.plan
        tensors = dict(tensors)
        self.embedding.bind(tensors, p.embedding_prefix)
        self.output.bind(tensors, p.output_prefix)
        for lp, block in zip(p.layers, self.blocks):
            block.bind(tensors, lp.prefix)
        self.final_norm.bind(tensors, p.final_norm_prefix)
        self.bound = True

    # -------------------------------------------------------------------- cache
    def cache_needs(self) -> list:
        """One entry per run-order step: the need of the step's own cache, or None when the
        step has none or reads another step's (``cache_of``)."""
        out = []
        for step in self.plan.run_order:
            need = self.blocks[step.layer].cache_need()
            out.append(need if step.cache_of is None else None)
        return out

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: StepContext, caches: list, logits_index: Optional[torch.Tensor],
                logits_out: Optional[torch.Tensor], greedy_out=None) -> Optional[torch.Tensor]:
        """Run the step's tokens through every run-order entry.  ``caches[i]`` is the
        LayerCache of entry i (None if it has no need).  Logits (fp32 [n, V]) are formed for the
        rows that ``logits_index`` names, into ``logits_out``; or, with ``greedy_out`` = (tokens int32 [n],
        probabilities fp32 [n]), each such row's best token and its probability instead of its logits."""
        T = ctx.num_tokens
        ctx.shared.clear()  # what parts share belongs to one pass; a context may be run again (to record a graph)
        h = ctx.workspace.get("residual", (T, self.hidden_size), torch.float32)
        self.embedding.forward(ctx.token_ids, h)
        for i, step in enumerate(self.plan.run_order):
            owner = i if step.cache_of is None else step.cache_of
            self.blocks[step.layer].forward(h, ctx, caches[owner], owns_cache=step.cache_of is None)
        if logits_index is None or logits_index.numel() == 0:
            return None
        n = logits_index.numel()
        y = ctx.workspace.get("final_normed", (n, self.hidden_size), ctx.act_dtype)
        self.final_norm.forward(h, y, row_index=logits_index)
        if greedy_out is not None:
            self.output.forward_greedy(y, greedy_out[0], greedy_out[1], ctx.workspace)
            return None
        self.output.forward(y, logits_out)
        return logits_out


def build_model(plan: ModelPlan) -> DecoderModel:
    return DecoderModel(plan)
