"""Grouped-query attention over the paged cache, as a part.

  q = y Wq^T + bq, k = y Wk^T + bk, v = y Wv^T + bv       (reference.rs:251-268)
  q, k <- position encoding (rotary here)                  (reference.rs:291-297)
  k (after rotation) and v go to the cache                 (reference.rs:311-316)
  head hq reads kv head hq / (nh / nkv); s = (q . k) * scale; causal; softmax; sum w v
                                                           (kernel/cpu/attention.rs:729-781)
  h += o Wo^T                                              (reference.rs:331-337)
(paths under crates/ferrisinfer-runtime/src and crates/ferrisinfer-kernel/src).  The biases are
used iff the folder has them (crates/ferrisinfer-io/src/hf.rs:458-478); there is no output bias.

Unlike the reference, the step's keys and values are written to the cache BEFORE the
attention kernel runs, so one kernel serves whole prompts, portions and decoded tokens alike,
and q, k, v come from one fused [Q + 2 KV, H] matrix product.  ``window`` (keys the query sees,
itself included; None = all) is a parameter, as are the scale and every size.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, PagedKV, TensorSpec
from .plan import PartSpec, build_part, register_part


class GroupedQueryAttention(Mixer):
    accepts_lazy_norm = True  # x goes to ops.gemm and nowhere else

    @property
    def graph_safe(self):
        # its own work is kernels on device-resident metadata; the position encoding's ``apply`` may be anything
        return bool(getattr(self.position, "graph_safe", False))

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, window: Optional[int] = None, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} kv heads")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.num_kv_heads, self.head_dim = int(num_kv_heads), int(head_dim)
        self.window = None if window is None else int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = build_part("position", position) if isinstance(position, PartSpec) else position
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.qkv_weight = self.qkv_bias = self.o_weight = None

    # ------------------------------------------------------------------ weights
    def tensor_specs(self, prefix):
        H, Q, KV = self.hidden_size, self.q_size, self.kv_size
        return [
            TensorSpec(f"{prefix}.q_proj.weight", (Q, H), "matrix"),
            TensorSpec(f"{prefix}.k_proj.weight", (KV, H), "matrix"),
            TensorSpec(f"{prefix}.v_proj.weight", (KV, H), "matrix"),
            TensorSpec(f"{prefix}.q_proj.bias", (Q,), "bias", required=False),
            TensorSpec(f"{prefix}.k_proj.bias", (KV,), "bias", required=False),
            TensorSpec(f"{prefix}.v_proj.bias", (KV,), "bias", required=False),
            TensorSpec(f"{prefix}.o_proj.weight", (H, Q), "matrix"),
        ]

    def bind(self, tensors, prefix):
        w = [tensors.pop(f"{prefix}.{n}_proj.weight") for n in "qkv"]
        self.qkv_weight = torch.cat(w, dim=0).contiguous()
        biases = [tensors.pop(f"{prefix}.{n}_proj.bias", None) for n in "qkv"]
        if any(b is not None for b in biases):
            sizes = (self.q_size, self.kv_size, self.kv_size)
            parts = [
                b if b is not None else torch.zeros(n, dtype=torch.float32, device=self.qkv_weight.device)
                for b, n in zip(biases, sizes)
            ]
            self.qkv_bias = torch.cat(parts).contiguous()
        else:
            self.qkv_bias = None
        self.o_weight = tensors[f"{prefix}.o_proj.weight"]

    # -------------------------------------------------------------------- cache
    def cache_need(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window)

    # ------------------------------------------------------------------ forward
    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool):
        T = x.shape[0]
        nh, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        meta = ctx.paged[cache.group]
        qkv = ctx.workspace.get("attn_qkv", (T, self.q_size + 2 * self.kv_size), x.dtype)
        table = self.position.rotary_table(qkv.device)
        inv_freq, rotary = table if table is not None else (None, 0)
        slopes = self.position.score_slopes(nh, qkv.device)
        # a long step of prompt portions: rotation and cache write ride in the product's epilogue
        fused = False
        if (inv_freq is not None and ctx.max_q_len > 1 and T >= ops.QKV_ROPE_MIN_TOKENS
                and hasattr(self.position, "angles")):
            x = x.materialize() if hasattr(x, "materialize") else x
            fused = ops.qkv_rope_gemm_takes(x, self.qkv_weight, qkv, nh, nkv, d, rotary, cache.k)
        if fused:
            ops.qkv_rope_gemm(x, self.qkv_weight, self.qkv_bias, qkv, self.position.angles(ctx),
                              meta.slot_mapping if owns_cache else None, cache.k, cache.v, nh, nkv, d)
        else:
            ops.gemm(x, self.qkv_weight, self.qkv_bias, qkv)
            if table is None:
                self.position.apply(qkv, ctx.positions, nh, nkv, d)
        out = ctx.workspace.get("attn_out", (T, self.q_size), x.dtype)
        attended = ops.attention_step(qkv, out, cache.k, cache.v, meta, ctx, nh, nkv, d, inv_freq, rotary,
                                      self.window or 0, self.scale, write_kv=owns_cache, lazy_merge=True,
                                      rotated=fused, score_slopes=slopes)
        ops.gemm(attended, self.o_weight, None, h, accumulate=True)


register_part("mixer", "gqa_attention", GroupedQueryAttention)
