"""Routed experts: ``experts`` small gated feed-forwards of which every row uses ``top``.

Router logits z = W_r x are formed in float32; the ``top`` largest choose (ties to the lower index) and the softmax over
the chosen logits alone weighs the experts' outputs. Each expert is down(act(gate x, up x)) with the spec's gated
activation. The experts' matrices are stacked when they are loaded ([experts, 2 ff, hidden] and [experts, hidden, ff]); a
step routes, groups its (row, choice) pairs by expert on the device, runs the two grouped products and sums a row's
choices in a fixed order (csrc/moe.cu). Nothing of a step's routing is read on the host.

``routing`` "sigmoid_groups": scores s = sigmoid(z); the choice goes by s + a stored correction, among the experts of the best
``keep_groups`` of ``groups`` equal groups of neighbours (a group's score: the sum of its two largest choice scores); the
weights are the chosen experts' s (without the correction) divided by their sum.

``routing`` "table": there is no router; an integer table [vocab, top] gives every token id its experts (the entries of a
row differ), each weighted 1 / top. ``shared``: one more expert of the same form that every row uses; its result (float32)
is added by the kernel that sums a row's choices.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import FeedForward
from .registry import build_feed_forward, register_feed_forward
from .spec import ParamInfo, RoutedExpertsSpec


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    takes_out_dtype = True

    def __init__(self, spec: RoutedExpertsSpec) -> None:
        super().__init__(spec)
        s = spec
        if not 0 < s.top <= s.experts or s.top > 32 or s.intermediate_size <= 0:
            raise ValueError(f"routed_experts: {s.top} of {s.experts} experts (at most 32 a row), ff {s.intermediate_size}")
        ops.glu_code(s.activation)          # refuses a name no kernel knows
        if s.routing not in ("softmax_top", "table", "sigmoid_groups"):
            raise ValueError(f"routed_experts: routing must be 'softmax_top', 'sigmoid_groups' or 'table', got {s.routing!r}")
        if s.routing == "sigmoid_groups" and (s.groups < 1 or not 1 <= s.keep_groups <= s.groups or s.experts % s.groups
                                              or (s.experts // s.groups) * s.keep_groups < s.top):
            raise ValueError(f"routed_experts: {s.experts} experts in {s.groups} groups of which {s.keep_groups} are kept "
                             f"cannot give {s.top} choices")
        if s.routing == "table" and s.vocab_size <= 0:
            raise ValueError("routed_experts: routing by a table needs the vocabulary's size")
        self.shared = build_feed_forward(s.shared) if s.shared is not None else None
        if self.shared is not None and not getattr(self.shared, "takes_out_dtype", False):
            raise ValueError("routed_experts: the shared expert must be able to return float32")
        self.table: Optional[torch.Tensor] = None
        self.w_router: Optional[torch.Tensor] = None
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def _names(self, e: int):
        s = self.spec
        p = f"{s.expert_prefix}{e}."
        return p + s.gate_name, p + s.up_name, p + s.down_name

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        W, F = s.hidden_size, s.intermediate_size
        if s.routing == "table":
            p = {s.table_name: ParamInfo((s.vocab_size, s.top), ("distinct_below", s.experts), integer=True)}
        else:
            p = {s.router_name: ParamInfo((s.experts, W), ("normal", W ** -0.5))}
            if s.routing == "sigmoid_groups":
                p[s.correction_name] = ParamInfo((s.experts,), ("normal", 0.1))
        for e in range(s.experts):
            g, u, d = self._names(e)
            p[g] = ParamInfo((F, W), ("normal", W ** -0.5))
            p[u] = ParamInfo((F, W), ("normal", W ** -0.5))
            p[d] = ParamInfo((W, F), ("normal", F ** -0.5))
        if self.shared is not None:
            for local, info in self.shared.parameters().items():
                p[s.shared_name + local] = info
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        if s.routing == "table":
            self.table = tensors[s.table_name].to(torch.int32).contiguous()
        else:
            self.w_router = tensors[s.router_name].contiguous()
            if s.routing == "sigmoid_groups":
                self.correction = tensors[s.correction_name].to(torch.float32).contiguous()
        if self.shared is not None:
            self.shared.load({local: tensors[s.shared_name + local] for local in self.shared.parameters()})
        names = [self._names(e) for e in range(s.experts)]
        self.w_gate_up = torch.stack([torch.cat([tensors[g], tensors[u]], dim=0) for g, u, _ in names]).contiguous()
        self.w_down = torch.stack([tensors[d] for _, _, d in names]).contiguous()

    def forward(self, x: torch.Tensor, ctx, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        s = self.spec
        if not x.is_contiguous():
            x = x.contiguous()
        if s.routing == "table":
            routing = ops.moe_route_table(ctx.token_ids, self.table, s.experts)
        elif s.routing == "sigmoid_groups":
            routing = ops.moe_route(x, self.w_router, s.top, scoring="sigmoid_groups", correction=self.correction, groups=s.groups,
                                    keep_groups=s.keep_groups)
        else:
            routing = ops.moe_route(x, self.w_router, s.top)
        add = self.shared.forward(x, ctx, out_dtype=torch.float32) if self.shared is not None else None
        out = ops.moe_experts(x, self.w_gate_up, self.w_down, routing, s.limit, act=s.activation, add=add)
        return out if out_dtype in (None, torch.float32) else out.to(out_dtype)
