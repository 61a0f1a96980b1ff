"""Transforms of the embedding's output or of the logits (``ModelSpec.embedding_transform``,
``ModelSpec.logits_transform``)."""
from __future__ import annotations

from ..config.spec import ScaleSpec, SoftCapSpec
from ..kernels import ops
from .base import Runtime, register_transform


@register_transform("soft_cap")
class SoftCap:
    """``cap * tanh(x / cap)`` on float32, in place."""

    @staticmethod
    def tensor_specs(spec: SoftCapSpec, prefix: str):
        return []

    def __init__(self, spec: SoftCapSpec, tensors, runtime: Runtime):
        if not spec.cap > 0:
            raise ValueError(f"a soft cap must be positive, got {spec.cap}")
        self.cap = float(spec.cap)

    def forward(self, x):
        return ops.soft_cap(x, self.cap)


@register_transform("scale")
class Scale:
    """``factor * x`` on float32, in place."""

    @staticmethod
    def tensor_specs(spec: ScaleSpec, prefix: str):
        return []

    def __init__(self, spec: ScaleSpec, tensors, runtime: Runtime):
        self.factor = float(spec.factor)

    def forward(self, x):
        return ops.scale(x, self.factor)
