"""A mixture of gated experts whose choice is a table lookup by token id (the formulas are with
:class:`TableRoutedMLPSpec`).

The experts' gate and up matrices are stacked expert by expert ([gate | up] rows), and so are the
columns of the down matrices, as :mod:`routed` does for its experts.  A small step, and every
32-bit step, runs one product up over all experts, ``ops.clamped_glu`` with the token's weight of
each expert (zero for an expert the table does not name) and one product down whose accumulator
sums the weighted experts: every row's result depends on the row only, nothing is sorted, and the
step can be captured.  A bfloat16 step that would spend ``routed.SORT_MIN_SAVED_FLOPS`` or more
on experts the table did not name sorts its (token, expert) pairs by expert and runs grouped
products over the chosen experts only, as the routed feed-forward does.
"""
from __future__ import annotations

import torch

from ..config.spec import TableRoutedMLPSpec, TensorSpec
from ..kernels import ops
from . import routed
from .base import Runtime, register_feed_forward


@register_feed_forward("table_routed_mlp")
class TableRoutedMLP:
    @staticmethod
    def tensor_specs(spec: TableRoutedMLPSpec, prefix: str):
        out = []
        for e in range(spec.experts):
            out += [TensorSpec(f"{prefix}.e{e}.gate", (spec.expert_ff, spec.hidden)),
                    TensorSpec(f"{prefix}.e{e}.up", (spec.expert_ff, spec.hidden)),
                    TensorSpec(f"{prefix}.e{e}.down", (spec.hidden, spec.expert_ff))]
        out.append(TensorSpec(f"{prefix}.table", (spec.vocab, spec.top), f"table:{spec.experts}"))
        return out

    def __init__(self, spec: TableRoutedMLPSpec, tensors, runtime: Runtime):
        if not 1 <= spec.top <= spec.experts:
            raise ValueError(f"top={spec.top} of {spec.experts} experts")
        self.spec = spec
        names = [f"e{e}" for e in range(spec.experts)]
        self.w_up = runtime.matrix(torch.cat([t for n in names for t in (tensors[f"{n}.gate"], tensors[f"{n}.up"])], dim=0))
        self.w_down = runtime.matrix(torch.cat([tensors[f"{n}.down"] for n in names], dim=1))
        self.w_up_experts = self.w_up.view(spec.experts, 2 * spec.expert_ff, spec.hidden)
        self.w_down_experts = self.w_down.view(spec.hidden, spec.experts, spec.expert_ff).permute(1, 0, 2)
        table = tensors["table"]
        if table.is_floating_point():
            raise ValueError("the experts' table holds integers")
        self.table = table.to(device=runtime.device, dtype=torch.int32).contiguous()
        self.sortable = (runtime.precision.act == torch.bfloat16 and spec.top < spec.experts
                         and spec.hidden % 8 == 0 and spec.expert_ff % 8 == 0)

    def activation_elements(self) -> int:
        return 3 * self.spec.experts * self.spec.expert_ff + self.spec.experts

    def _sorted_forward(self, x, ctx):
        """Only the experts the table names: float32 [tokens, hidden]."""
        s = self.spec
        chosen = torch.empty((x.shape[0], s.top), dtype=torch.int32, device=x.device)
        weights = ops.table_route(ctx.token_ids, self.table, s.experts, chosen=chosen)
        ends, source, row_weight, dest = ops.moe_sort(chosen, weights)
        rows = ops.gather_rows(x, source)
        act = ops.clamped_glu(ops.grouped_linear(rows, self.w_up_experts, ends), row_weight, 1, s.expert_ff, s.limit, s.alpha)
        rows = ops.grouped_linear(act, self.w_down_experts, ends)
        return ops.combine_rows(None, rows, dest)

    def forward(self, x, ctx):
        s = self.spec
        saved = 6.0 * x.shape[0] * (s.experts - s.top) * s.expert_ff * s.hidden
        if self.sortable and saved >= routed.SORT_MIN_SAVED_FLOPS and x.shape[0] > 16 \
                and not torch.cuda.is_current_stream_capturing():
            return self._sorted_forward(x, ctx)
        weights = ops.table_route(ctx.token_ids, self.table, s.experts)
        act = ops.clamped_glu(ops.linear(x, self.w_up), weights, s.experts, s.expert_ff, s.limit, s.alpha)
        return ops.linear(act, self.w_down, out_dtype=torch.float32)
