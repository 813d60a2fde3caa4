"""Parts that act on the residual stream itself rather than on a branch of it.

"short_conv": a causal convolution over time on every channel, out = x + conv(x) (or conv(x) alone), whose last
``taps - 1`` inputs per request are state kept in the cache manager's slots, so a portion of a prompt or a single
decoded token continues where the request's earlier steps ended.

"token_input": a small input per layer that depends on the token id alone: a narrow gate read off the stream times the
token's slice of a table all layers share, projected back, RMS-normed and added.

"depth_average": after a layer, the stream becomes a weighted sum of the outputs of all layers so far and of the
embedding output. It owns only the weights; the sum itself is formed by the kernel that ends the layer's last branch
(``ops.branch_norm_add``) or by ``ops.history_average``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import StateNeed
from ..kernels import ops
from .base import Part
from .registry import register_stream_part
from ..kernels.linear import linear
from .spec import DepthAverageSpec, ParamInfo, ShortConvSpec, StreamCoefficientsSpec, TokenInputSpec


@register_stream_part("short_conv")
class ShortConv(Part):
    def __init__(self, spec: ShortConvSpec) -> None:
        super().__init__(spec)
        if spec.taps < 1 or spec.channels <= 0:
            raise ValueError(f"short_conv needs taps >= 1 and channels > 0, got {spec.taps} and {spec.channels}")
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        return {s.param_name: ParamInfo((s.channels, s.taps), ("normal", 0.3))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.param_name].contiguous()

    def state_needs(self) -> List[StateNeed]:
        s = self.spec
        # two copies: the kernel reads a request's old state in its portion's first rows while it writes the new one
        # from the last rows
        return [StateNeed((s.taps - 1, s.channels), "float32", phases=2)] if s.taps > 1 else []

    def forward(self, x: torch.Tensor, ctx, state_ids, out_dtype: torch.dtype) -> torch.Tensor:
        """x [tokens, channels] (float32 or ``out_dtype``) -> x + conv(x) in ``out_dtype``; the state moves on."""
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        state = ctx.cache.state_tensor(state_ids[0]) if self.spec.taps > 1 else None
        return ops.short_conv(out, x, self.weight, state, ctx.cu_seqlens, ctx.token_req, ctx.state_slots, ctx.state_phase,
                              add_input=self.spec.add_input)


@register_stream_part("depth_average")
class DepthAverage(Part):
    def __init__(self, spec: DepthAverageSpec) -> None:
        super().__init__(spec)
        if spec.terms < 1:
            raise ValueError("depth_average needs at least one term")
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        return {s.param_name: ParamInfo((s.terms,), ("normal_around", 0.2, 1.0 / s.terms))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.param_name].contiguous()


@register_stream_part("stream_coefficients")
class StreamCoefficients(Part):
    """The three small tensors of one sublayer over S residual streams: ``in`` [S] (how the sublayer's input is read off
    the streams), ``mix`` [S, S] (indexed [from, to]: how the streams are carried over) and ``out`` [S] (how the sublayer's
    result is added to each). It owns the tensors only; ``ops.hyper_step`` applies them."""

    def __init__(self, spec: StreamCoefficientsSpec) -> None:
        super().__init__(spec)
        if not 1 <= spec.streams <= 16:
            raise ValueError(f"stream_coefficients: {spec.streams} streams, 1 to 16 are supported")
        self.a_in: Optional[torch.Tensor] = None
        self.mix: Optional[torch.Tensor] = None
        self.b_out: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        s, n = self.spec, self.spec.streams
        return {s.in_name: ParamInfo((n,), ("normal_around", 0.2, 1.0 / n)), s.out_name: ParamInfo((n,), ("normal_around", 0.3, 1.0)),
                s.mix_name: ParamInfo((n, n), ("eye_plus_normal", 0.2))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.a_in = tensors[s.in_name].contiguous()
        self.b_out = tensors[s.out_name].to(self.a_in.dtype).contiguous()
        self.mix = tensors[s.mix_name].to(self.a_in.dtype).contiguous()


@register_stream_part("token_input")
class TokenInput(Part):
    """x <- x + rms(proj (gelu_tanh(gate x) * e)) * weight with e = table[token, offset : offset + dim]. The table is one
    tensor for all layers (its name is absolute); gate [dim, hidden], proj [hidden, dim], weight [hidden] (used as stored).
    The two products read the stream rounded to the model's type; the norm and the add are float32 on the stream."""

    def __init__(self, spec: TokenInputSpec) -> None:
        super().__init__(spec)
        s = spec
        if s.dim <= 0 or s.offset < 0 or s.offset + s.dim > s.table_width or s.vocab_size <= 0:
            raise ValueError(f"token_input: {s.dim} numbers at {s.offset} of a table row of {s.table_width}")
        self.table: Optional[torch.Tensor] = None
        self.w_gate: Optional[torch.Tensor] = None
        self.w_proj: Optional[torch.Tensor] = None
        self.weight: Optional[torch.Tensor] = None
        self.cols = -(-s.dim // 8) * 8          # the gate's rows, padded so that the narrow buffer's rows stay 16-byte aligned

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        return {s.table_name: ParamInfo((s.vocab_size, s.table_width), ("normal", 1.0)),
                s.gate_name: ParamInfo((s.dim, s.hidden_size), ("normal", s.hidden_size ** -0.5)),
                s.proj_name: ParamInfo((s.hidden_size, s.dim), ("normal", s.dim ** -0.5)),
                s.norm_name: ParamInfo((s.hidden_size,), ("normal_around", 0.1, 0.5))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.table = tensors[s.table_name].contiguous()
        g, p = tensors[s.gate_name], tensors[s.proj_name]
        if self.cols != s.dim:       # zero rows of the gate give gelu(0) = 0; zero columns of the projection add nothing
            g = torch.cat([g, torch.zeros((self.cols - s.dim, g.shape[1]), dtype=g.dtype, device=g.device)], dim=0)
            p = torch.cat([p, torch.zeros((p.shape[0], self.cols - s.dim), dtype=p.dtype, device=p.device)], dim=1)
        self.w_gate, self.w_proj = g.contiguous(), p.contiguous()
        self.weight = tensors[s.norm_name].contiguous()

    def forward(self, h: torch.Tensor, x_low: torch.Tensor, ctx, low: Optional[torch.Tensor] = None) -> torch.Tensor:
        """h float32 [tokens, hidden] is updated in place; ``x_low`` is h in the model's type (h itself in a float32 model);
        ``low``, when given, receives the new h rounded to the model's type."""
        s = self.spec
        g = linear(x_low, self.w_gate)
        ops.token_gate(g[:, : s.dim], ctx.token_ids, self.table, s.offset)
        y = linear(g, self.w_proj, out_dtype=torch.float32)
        ops.branch_norm_add(h, y, self.weight, s.eps, weight_offset=0.0, low=low)
        return h
