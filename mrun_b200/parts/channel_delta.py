"""Gated delta rule with a decay per head and key channel (the formulas are with
:class:`ChannelDeltaSpec`).

One product makes [q | k | v | b | a1 x | g1 x]; two small products finish the low-rank decay and
gate projections (the decay's with 32-bit output, as it enters the recurrence).  One
``ops.causal_conv`` runs the three short convolutions with SiLU over the contiguous [q | k | v]
columns, from and into the request's last inputs; ``ops.delta_scan`` makes q and k unit vectors,
forms the decays and the write strengths and walks each request's tokens from the state it left
(float32 [heads, dim, vdim]); ``ops.gated_norm`` norms every head's output with the shared
weight and applies the gate; the output projection follows.
"""
from __future__ import annotations

import torch

from ..cache.needs import FixedState
from ..config.spec import ChannelDeltaSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_mixer


@register_mixer("channel_delta")
class ChannelDelta:
    can_defer_output = True
    graph_safe = True

    @staticmethod
    def tensor_specs(spec: ChannelDeltaSpec, prefix: str):
        qk, inner, keyed = spec.kv_heads * spec.dim, spec.heads * spec.vdim, spec.heads * spec.dim
        out = []
        for name, rows in (("q", qk), ("k", qk), ("v", inner)):
            out += [TensorSpec(f"{prefix}.{name}", (rows, spec.hidden)), TensorSpec(f"{prefix}.{name}.conv", (rows, spec.conv))]
        out += [TensorSpec(f"{prefix}.b", (spec.heads, spec.hidden)),
                TensorSpec(f"{prefix}.A_log", (spec.heads,), "log_rate"),
                TensorSpec(f"{prefix}.norm", (spec.vdim,), "norm"),
                TensorSpec(f"{prefix}.a1", (spec.decay_rank, spec.hidden)),
                TensorSpec(f"{prefix}.a2", (keyed, spec.decay_rank)),
                TensorSpec(f"{prefix}.dt_bias", (keyed,)),
                TensorSpec(f"{prefix}.g1", (spec.gate_rank, spec.hidden)),
                TensorSpec(f"{prefix}.g2", (inner, spec.gate_rank)),
                TensorSpec(f"{prefix}.o", (spec.hidden, inner))]
        return out

    def __init__(self, spec: ChannelDeltaSpec, tensors, runtime: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads={spec.heads} is not a multiple of kv_heads={spec.kv_heads}")
        self.spec = spec
        self.w_in = runtime.matrix(torch.cat([tensors[n] for n in ("q", "k", "v", "b", "a1", "g1")], dim=0))
        self.w_a2 = runtime.matrix(tensors["a2"])
        self.w_g2 = runtime.matrix(tensors["g2"])
        self.w_o = runtime.matrix(tensors["o"])
        self.conv_weight = runtime.vector_f32(torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0))
        self.a_log = runtime.vector_f32(tensors["A_log"])
        self.dt_bias = runtime.vector_f32(tensors["dt_bias"])
        self.norm_weight = runtime.vector_f32(tensors["norm"])
        self.act = runtime.precision.act
        self._state_dtype = runtime.precision.name
        self.channels = 2 * spec.kv_heads * spec.dim + spec.heads * spec.vdim

    def activation_elements(self) -> int:
        s = self.spec
        return 2 * self.channels + s.heads * (1 + 2 * s.dim + 3 * s.vdim) + s.decay_rank + s.gate_rank

    def cache_need(self):
        s = self.spec
        return (FixedState((s.heads, s.dim, s.vdim), "float32", name="state"),
                FixedState((s.conv - 1, self.channels), self._state_dtype, name="conv"))

    def forward(self, x, ctx, cache, defer_output: bool = False):
        s = self.spec
        if cache is None or not cache.writable:
            raise ValueError("a recurrent mixer needs a state of its own")
        qk, inner, C = s.kv_heads * s.dim, s.heads * s.vdim, self.channels
        y = ops.linear(x, self.w_in)
        at = C
        b = y[:, at:at + s.heads]; at += s.heads
        a1 = y[:, at:at + s.decay_rank]; at += s.decay_rank
        g1 = y[:, at:at + s.gate_rank]
        a = ops.linear(a1, self.w_a2, out_dtype=torch.float32)          # column slices: the products take row strides
        gate = ops.linear(g1, self.w_g2)
        qkv = ops.causal_conv(y[:, :C], self.conv_weight, cache.states["conv"], ctx, residual=False, silu=True)
        o = ops.delta_scan(qkv[:, :qk], qkv[:, qk:2 * qk], qkv[:, 2 * qk:], a, b, self.a_log, self.dt_bias,
                           cache.states["state"], ctx, s.heads, s.kv_heads, s.dim, s.vdim)
        o = ops.gated_norm(o, self.norm_weight, gate, s.eps, s.heads, self.act)
        if defer_output:
            return ops.linear_or_pending(o, self.w_o)
        return ops.linear(o, self.w_o)
