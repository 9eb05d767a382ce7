"""The Qwen2 dense decoder as a plan: which parts each layer has and in what order layers run.

Per layer (crates/ferrisinfer-runtime/src/reference.rs:163-370): RMSNorm -> grouped-query
attention with q/k/v bias and rotary positions -> residual -> RMSNorm -> SwiGLU -> residual;
then a final RMSNorm and the output head, tied to the embedding when the configuration says so
(crates/ferrisinfer-runtime/src/reference.rs:976-982).  Tensor names are those of the model
folder (crates/ferrisinfer-io/src/hf.rs:380-500).  Layers from ``max_window_layers`` on attend a
sliding window when ``use_sliding_window`` is set.
"""

from __future__ import annotations

from ..config.qwen2 import Qwen2Config
from ..config.registry import register_architecture
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, RunStep


def plan_qwen2(cfg: Qwen2Config) -> ModelPlan:
    cfg.validate()
    norm = PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    position = PartSpec("rotary", {"head_dim": cfg.head_dim, "rotary_dim": cfg.rotary_dim, "theta": cfg.rope_theta})
    feed_forward = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
    layers = []
    for l in range(cfg.num_hidden_layers):
        mixer = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "position": position,
            "window": cfg.layer_window(l),
        })
        layers.append(LayerPlan(prefix=f"model.layers.{l}", mixer=mixer, feed_forward=feed_forward,
                                mixer_norm=norm, feed_forward_norm=norm))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}),
        embedding_prefix="model.embed_tokens",
        layers=tuple(layers),
        run_order=tuple(RunStep(l) for l in range(cfg.num_hidden_layers)),
        final_norm=norm,
        final_norm_prefix="model.norm",
        output=PartSpec("linear_head", {
            "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
            "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None,
        }),
        output_prefix="lm_head",
        max_positions=cfg.max_position_embeddings,
        extra={"ignorable_tensors": ("lm_head.weight",) if cfg.tie_word_embeddings else ()},
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, plan_qwen2, replace=True)
