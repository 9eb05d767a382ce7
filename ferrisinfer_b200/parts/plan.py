"""The description of a model as data: parts by kind, layer by layer, and the run order.

An architecture's plan function turns its configuration into a ``ModelPlan``.
Nothing in a plan is code: each part is a ``PartSpec`` (a registered kind plus
its sizes and constants), each layer names its four parts, and ``run_order`` is
a list of ``RunStep`` that may name a layer twice (its weights are then shared
and every run has a cache of its own) or let a run read the cache that an
earlier run wrote (``cache_of``).

The reference hard-codes one block shape and loops ``for l in 0..L``
(crates/ferrisinfer-runtime/src/reference.rs:402-414); the plan is this
engine's way to keep that loop, the kinds of the parts and their sizes out of
the code that runs them.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartSpec:
    """A registered kind of part and the parameters it is built with."""

    kind: str
    params: dict = field(default_factory=dict)


@dataclass(frozen=True)
class TensorSpec:
    """One tensor that a part reads from the model folder.

    ``role`` decides the dtype on the device and the random initialisation:
    ``matrix`` / ``embedding``: the engine's compute dtype, N(0, 0.02);
    ``bias``: N(0, 0.02); ``norm``: 1 + N(0, 0.02); vectors (bias, norm) are
    held in 32-bit on the device (an exact widening of what the file stores);
    ``int_table``: int32, zeros.
    """

    name: str
    shape: tuple
    role: str = "matrix"
    required: bool = True


@dataclass(frozen=True)
class LayerPlan:
    """One layer: a block kind wiring two norms, a mixer and a feed-forward."""

    prefix: str  # tensor-name prefix, e.g. "model.layers.3"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block: PartSpec = PartSpec("pre_norm_residual")


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.

    ``layer``: index into ``ModelPlan.layers``.  ``cache_of``: None = this run
    has a cache of its own; an int = the index of an EARLIER run-order entry
    whose cache this run reads without writing.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    embedding_prefix: str
    layers: tuple
    run_order: tuple
    final_norm: PartSpec
    final_norm_prefix: str
    output: PartSpec
    output_prefix: str
    max_positions: int
    extra: dict = field(default_factory=dict)

    def validate(self) -> None:
        for i, step in enumerate(self.run_order):
            if not (0 <= step.layer < len(self.layers)):
                raise ValueError(f"run_order[{i}] names layer {step.layer}, which does not exist")
            if step.cache_of is not None:
                if not (0 <= step.cache_of < i):
                    raise ValueError(
                        f"run_order[{i}].cache_of={step.cache_of} must name an earlier entry"
                    )
                if self.run_order[step.cache_of].cache_of is not None:
                    raise ValueError(
                        f"run_order[{i}].cache_of={step.cache_of} names an entry that has no cache of its own"
                    )


# --------------------------------------------------------------------------- kinds
_PART_KINDS: dict[str, dict[str, Any]] = {
    "mixer": {},
    "feed_forward": {},
    "norm": {},
    "position": {},
    "block": {},
    "embedding": {},
    "output": {},
}


def register_part(family: str, kind: str, factory, *, replace: bool = False) -> None:
    """Register ``factory(**params) -> part`` under ``kind`` in ``family``
    (mixer, feed_forward, norm, position, block, embedding, output)."""
    table = _PART_KINDS[family]
    if kind in table and not replace:
        raise ValueError(f"{family} kind '{kind}' is already registered")
    table[kind] = factory


def build_part(family: str, spec: PartSpec, **extra):
    table = _PART_KINDS[family]
    if spec.kind not in table:
        raise KeyError(
            f"{family} kind '{spec.kind}' is not registered (registered: {', '.join(sorted(table))})"
        )
    return table[spec.kind](**spec.params, **extra)


def registered_parts(family: str) -> list[str]:
    return sorted(_PART_KINDS[family])
