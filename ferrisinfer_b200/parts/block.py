"""How a layer's parts are arranged: the pre-norm residual block.

  h += mixer(norm_1(h));  h += feed_forward(norm_2(h))
(crates/ferrisinfer-runtime/src/reference.rs:244-249, 331-344, 362-368).  The sums are made in
the fp32 residual stream by the last matrix product of each branch.
"""

from __future__ import annotations

from .base import Block
from .plan import build_part, register_part


class PreNormResidualBlock(Block):
    def __init__(self, hidden_size: int, mixer, feed_forward, mixer_norm, feed_forward_norm,
                 mixer_prefix: str = "self_attn", feed_forward_prefix: str = "mlp",
                 mixer_norm_prefix: str = "input_layernorm",
                 feed_forward_norm_prefix: str = "post_attention_layernorm"):
        self.hidden_size = int(hidden_size)
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self._names = (mixer_prefix, feed_forward_prefix, mixer_norm_prefix, feed_forward_norm_prefix)

    def _children(self, prefix):
        m, f, n1, n2 = self._names
        return [
            (self.mixer_norm, f"{prefix}.{n1}"),
            (self.mixer, f"{prefix}.{m}"),
            (self.feed_forward_norm, f"{prefix}.{n2}"),
            (self.feed_forward, f"{prefix}.{f}"),
        ]

    def tensor_specs(self, prefix):
        out = []
        for part, p in self._children(prefix):
            out += part.tensor_specs(p)
        return out

    def bind(self, tensors, prefix):
        for part, p in self._children(prefix):
            part.bind(tensors, p)

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return bool(getattr(self.mixer, "graph_safe", False) and getattr(self.feed_forward, "graph_safe", False))

    def forward(self, h, ctx, cache, owns_cache):
        buf = ctx.workspace.get("block_normed", (h.shape[0], self.hidden_size), ctx.act_dtype)
        x = self.mixer_norm.lazy(h, buf)
        if not getattr(self.mixer, "accepts_lazy_norm", False) and hasattr(x, "materialize"):
            x = x.materialize()
        self.mixer.forward(x, h, ctx, cache, owns_cache)
        x = self.feed_forward_norm.lazy(h, buf)
        if not getattr(self.feed_forward, "accepts_lazy_norm", False) and hasattr(x, "materialize"):
            x = x.materialize()
        self.feed_forward.forward(x, h, ctx)


register_part("block", "pre_norm_residual", PreNormResidualBlock)
