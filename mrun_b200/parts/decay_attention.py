"""Linear attention with one decay a head (the formulas are with :class:`DecayAttentionSpec`).

One product makes [q | k | v | gate]; ``ops.decay_scan`` applies SiLU to q, k and v on the way
in and walks each request's tokens from the state it left (float32 [heads, dim, vdim] per
request); ``ops.gated_norm`` norms the heads' outputs together, applies the weight and the gate's
sigmoid; the output projection follows.  The state and everything inside the recurrence are
32-bit in both precisions.
"""
from __future__ import annotations

import torch

from ..cache.needs import FixedState
from ..config.spec import DecayAttentionSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_mixer


@register_mixer("decay_attention")
class DecayAttention:
    can_defer_output = True
    graph_safe = True

    @staticmethod
    def tensor_specs(spec: DecayAttentionSpec, prefix: str):
        inner = spec.heads * spec.vdim
        return [TensorSpec(f"{prefix}.q", (spec.heads * spec.dim, spec.hidden)),
                TensorSpec(f"{prefix}.k", (spec.heads * spec.dim, spec.hidden)),
                TensorSpec(f"{prefix}.v", (inner, spec.hidden)),
                TensorSpec(f"{prefix}.g", (inner, spec.hidden)),
                TensorSpec(f"{prefix}.o", (spec.hidden, inner)),
                TensorSpec(f"{prefix}.norm", (inner,), "norm")]

    def __init__(self, spec: DecayAttentionSpec, tensors, runtime: Runtime):
        if len(spec.decay) != spec.heads:
            raise ValueError(f"{len(spec.decay)} decays for {spec.heads} heads")
        self.spec = spec
        self.w_in = runtime.matrix(torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0))
        self.w_o = runtime.matrix(tensors["o"])
        self.norm_weight = runtime.vector_f32(tensors["norm"])
        self.decay = torch.tensor(spec.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.act = runtime.precision.act

    def activation_elements(self) -> int:
        s = self.spec
        return 2 * s.heads * s.dim + 5 * s.heads * s.vdim

    def cache_need(self):
        s = self.spec
        return FixedState((s.heads, s.dim, s.vdim), "float32", name="state")

    def forward(self, x, ctx, cache, defer_output: bool = False):
        s = self.spec
        if cache is None or not cache.writable:
            raise ValueError("a recurrent mixer needs a state of its own")
        qk, inner = s.heads * s.dim, s.heads * s.vdim
        y = ops.linear(x, self.w_in)
        o = ops.decay_scan(y[:, :qk], y[:, qk:2 * qk], y[:, 2 * qk:2 * qk + inner], self.decay, cache.states["state"], ctx,
                           s.heads, s.dim, s.vdim, silu_inputs=True)
        o = ops.gated_norm(o, self.norm_weight, y[:, 2 * qk + inner:], s.eps, 1, self.act)
        if defer_output:
            return ops.linear_or_pending(o, self.w_o)
        return ops.linear(o, self.w_o)
