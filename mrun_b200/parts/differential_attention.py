"""Differential attention over the paged cache: two softmax maps a head over the same values,
combined as a1 - lambda * a2, normed per head and scaled (the formulas are with
:class:`DifferentialAttentionSpec`).

One product makes [q | k | v]; the rows of the q and k weights are reordered at load so that the
maps are outermost ([map][head][dim]), which makes each map a grouped-query attention of the
ordinary shape over key pages of its own.  ``ops.diff_rope_cache`` rotates q and k and stores k and v
in the pages; then either one kernel runs both maps, the combination and the head norm on CUDA
cores in 32-bit arithmetic (the 32-bit path, and every shape), or, in bfloat16 where the value
size is a multiple of the key size and the tensor-core attention kernels take that head size, each
(map, value chunk) pair goes through those kernels and ``ops.diff_combine`` finishes the heads.
lambda is one number a layer and is computed from its four vectors when the weights are bound.
"""
from __future__ import annotations

import math
import os

import torch

from ..cache.needs import PagedMaps
from ..config.spec import DifferentialAttentionSpec, TensorSpec
from ..kernels import ops
from ..kernels.attention import paged_attention, supports_tensor_cores
from .base import POSITIONS, Runtime, register_mixer

# False (``MRUN_DIFF_TENSOR_CORE=0`` in the environment): the one-kernel CUDA-core path for every
# step; the tests compare the two
TENSOR_CORE_MAPS = os.environ.get("MRUN_DIFF_TENSOR_CORE", "1") != "0"


class _MapCache:
    """One map's key pages and one chunk of the value pages, as the grouped-query kernels take them."""

    def __init__(self, k, v):
        self.k, self.v = k, v


@register_mixer("differential_attention")
class DifferentialAttention:
    can_defer_output = True

    @staticmethod
    def tensor_specs(spec: DifferentialAttentionSpec, prefix: str):
        out = [TensorSpec(f"{prefix}.q", (spec.heads * 2 * spec.dim, spec.hidden)),
               TensorSpec(f"{prefix}.k", (spec.kv_heads * 2 * spec.dim, spec.hidden)),
               TensorSpec(f"{prefix}.v", (spec.kv_heads * spec.vdim, spec.hidden)),
               TensorSpec(f"{prefix}.o", (spec.hidden, spec.heads * spec.vdim))]
        out += [TensorSpec(f"{prefix}.{name}", (spec.dim,)) for name in ("lq1", "lk1", "lq2", "lk2")]
        if spec.position is not None:
            out += POSITIONS.tensor_specs(spec.position, f"{prefix}.rotary_emb")
        return out

    def __init__(self, spec: DifferentialAttentionSpec, tensors, runtime: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads={spec.heads} is not a multiple of kv_heads={spec.kv_heads}")
        self.spec = spec
        H, G, D, V = spec.heads, spec.kv_heads, spec.dim, spec.vdim
        # head by head [map 1, map 2] -> maps outermost
        q = tensors["q"].view(H, 2, D, spec.hidden).transpose(0, 1).reshape(2 * H * D, spec.hidden)
        k = tensors["k"].view(G, 2, D, spec.hidden).transpose(0, 1).reshape(2 * G * D, spec.hidden)
        self.w_qkv = runtime.matrix(torch.cat([q, k, tensors["v"]], dim=0))
        self.w_o = runtime.matrix(tensors["o"])
        dot = lambda a, b: float((tensors[a].to(torch.float32) * tensors[b].to(torch.float32)).sum())
        self.lam = float(math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + spec.diff)
        self.position = POSITIONS.build(spec.position, {}, runtime) if spec.position is not None else None
        if self.position is not None:
            if getattr(self.position, "pairing", "half") != "half":
                raise ValueError("the differential attention rotates half-split pairs")
            if self.position.rotary_dim > D:
                raise ValueError(f"{self.position.rotary_dim} rotating features exceed the key size {D}")
        self.page_size = runtime.page_size
        self.act = runtime.precision.act
        # value chunks of the key size let a (map, chunk) pair go through the kernels for equal
        # key and value sizes
        # (groups of more than 16 query heads would leave the decode kernels and need a tile list made
        # on the host, which a captured decode step cannot have: they stay on the CUDA-core kernel)
        self.tensor_core = (TENSOR_CORE_MAPS and self.act == torch.bfloat16 and V % D == 0 and H // G <= 16
                            and supports_tensor_cores(self.act, D, H // G) and spec.window is None)
        self.chunks = V // D if self.tensor_core else 1

    graph_safe = True

    def activation_elements(self) -> int:
        s = self.spec
        return 2 * s.heads * s.dim + 2 * s.kv_heads * s.dim + s.kv_heads * s.vdim + 3 * s.heads * s.vdim

    def cache_need(self):
        s = self.spec
        return PagedMaps(2, s.kv_heads, s.dim, self.chunks, s.vdim // self.chunks, s.window)

    def forward(self, x, ctx, cache, defer_output: bool = False):
        s = self.spec
        H, G, D, V = s.heads, s.kv_heads, s.dim, s.vdim
        group = ctx.group(cache.group_key)
        qkv = ops.linear(x, self.w_qkv)
        rot = self.position.rotation(ctx) if self.position is not None else None
        slots = group.slot_mapping if cache.writable else None
        ops.diff_rope_cache(qkv, rot, self.position.rotary_dim if rot is not None else 0, slots, cache.k, cache.v,
                            H, G, D, V, self.page_size)
        out_scale = 1.0 - s.diff
        q = qkv[:, :2 * H * D]
        if not self.tensor_core:
            o = ops.diff_attention(q, cache.k, cache.v, group.block_tables, ctx.token_slot, ctx.positions, H, V,
                                   s.softmax_scale, self.lam, s.eps, out_scale, s.window or 0)
        else:
            tokens = qkv.shape[0]
            maps = torch.empty((2, self.chunks, tokens, H * D), dtype=qkv.dtype, device=qkv.device)
            for m in range(2):
                for c in range(self.chunks):
                    paged_attention(qkv[:, m * H * D:], qkv.stride(0), maps[m, c], _MapCache(cache.k[m], cache.v[c]),
                                    group, ctx, H, s.softmax_scale, 0)
            o = ops.diff_combine(maps, H, V, self.lam, s.eps, out_scale)
        if defer_output:
            return ops.linear_or_pending(o, self.w_o)
        return ops.linear(o, self.w_o)
