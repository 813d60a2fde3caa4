"""Block arrangements. "prenorm": norm -> mixer -> add, norm -> feed-forward -> add
(pegainfer-qwen3/src/unified_forward.rs:383-611). Each residual add is carried out by
the norm that follows it (the reference fuses the same way: flashinfer_norm.cu:39-132,
pegainfer-qwen3/src/batch_decode.rs:210-236)."""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import Block, CacheBinding, Part
from .norm import RmsNorm
from .registry import build_feed_forward, build_mixer, build_norm, build_stream_part, register_block
from .spec import BlockSpec


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: BlockSpec) -> None:
        super().__init__(spec)
        self._mixer = build_mixer(spec.mixer)
        self.feed_forward = build_feed_forward(spec.feed_forward)
        self.input_norm = build_norm(spec.input_norm)
        self.post_norm = build_norm(spec.post_norm)

    @property
    def mixer(self):
        return self._mixer

    def sub_parts(self) -> Dict[str, Part]:
        s = self.spec
        return {
            s.input_norm_name: self.input_norm,
            s.mixer_name: self._mixer,
            s.post_norm_name: self.post_norm,
            s.feed_forward_name: self.feed_forward,
        }

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx,
                binding: CacheBinding) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        x = self.input_norm(h, delta=pending)          # h += pending; x = norm(h)
        a = self._mixer.forward(x, ctx, binding)
        x = self.post_norm(h, delta=a)                 # h += a; x = norm(h)
        m = self.feed_forward.forward(x, ctx)
        return h, m


@register_block("branchnorm")
class BranchNormBlock(Block):
    """x <- x + norm(mixer(f(x))), then x <- x + norm(ff(x)): the norms sit on the branches' OUTPUTS and the branches
    read the stream itself. f is an optional filter over time (``input_conv``: f(x) = x + conv(x)); the feed-forward is
    optional; with ``depth_average`` the block's result X is kept and the stream that goes on is a weighted sum of the
    results of all blocks so far and of the embedding output.

    The stream is float32 whatever the model's type: the branches get it rounded to the model's type (by the filter, or
    by the kernel that ends the branch before), return float32, and one kernel norms a branch's output, adds it, and,
    after the block's last branch, forms the average. ``spec.input_norm`` is the norm of the mixer's output,
    ``spec.post_norm`` that of the feed-forward's.
    """

    def __init__(self, spec: BlockSpec) -> None:
        super().__init__(spec)
        self._mixer = build_mixer(spec.mixer)
        self.feed_forward = build_feed_forward(spec.feed_forward) if spec.feed_forward is not None else None
        self.mixer_norm = build_norm(spec.input_norm)
        self.ff_norm = build_norm(spec.post_norm) if spec.feed_forward is not None else None
        self.conv = build_stream_part(spec.input_conv) if spec.input_conv is not None else None
        self.depth = build_stream_part(spec.depth_average) if spec.depth_average is not None else None
        for n in (self.mixer_norm, self.ff_norm):
            if n is not None and not isinstance(n, RmsNorm):
                raise ValueError("a branchnorm block needs rms norms")

    wants_history = property(lambda self: self.depth is not None)
    stream_dtype = torch.float32

    @property
    def mixer(self):
        return self._mixer

    def sub_parts(self) -> Dict[str, Part]:
        s = self.spec
        parts: Dict[str, Part] = {s.input_norm_name: self.mixer_norm, s.mixer_name: self._mixer}
        if self.feed_forward is not None:
            parts[s.post_norm_name] = self.ff_norm
            parts[s.feed_forward_name] = self.feed_forward
        if self.conv is not None:
            parts[s.input_conv_name] = self.conv
        if self.depth is not None:
            parts[s.depth_average_name] = self.depth
        return parts

    def state_needs(self):
        return (self.conv.state_needs() if self.conv is not None else []) + self._mixer.state_needs()

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx,
                binding: CacheBinding) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if h.dtype != torch.float32 or pending is not None:
            raise RuntimeError("a branchnorm block takes a float32 stream with no branch pending")
        dtype = ctx.scratch["model_dtype"]
        n_conv = len(self.conv.state_needs()) if self.conv is not None else 0
        if self.conv is not None:
            u = self.conv.forward(h, ctx, binding.states[:n_conv], dtype)
        else:
            u = ctx.scratch.pop("stream_low", None)
            if u is None:
                u = h if dtype == torch.float32 else h.to(dtype)
        ctx.scratch.pop("stream_low", None)
        wide = {"out_dtype": torch.float32}      # parts that can, hand their branch back unrounded
        a = self._mixer.forward(u, ctx, dataclasses.replace(binding, states=binding.states[n_conv:]),
                                **(wide if getattr(self._mixer, "takes_out_dtype", False) else {}))
        hist = ctx.scratch.get("stream_history") if self.depth is not None else None
        low = torch.empty(h.shape, dtype=dtype, device=h.device) if dtype != torch.float32 else None

        def join(branch, norm, last, low_out):
            kw = {}
            if last and hist is not None:
                kw = dict(history=hist[0], n_prev=hist[1], coef=self.depth.weight)
                if self.depth.weight.numel() != hist[1] + 1:
                    raise RuntimeError(f"depth average: {self.depth.weight.numel()} weights for {hist[1] + 1} terms")
                hist[1] += 1
            ops.branch_norm_add(h, branch, norm.weight, norm.spec.eps, weight_offset=norm.spec.weight_offset, low=low_out, **kw)

        if self.feed_forward is None:
            join(a, self.mixer_norm, True, low)
        else:
            join(a, self.mixer_norm, False, low)
            m = self.feed_forward.forward(low if low is not None else h, ctx,
                                          **(wide if getattr(self.feed_forward, "takes_out_dtype", False) else {}))
            join(m, self.ff_norm, True, low)
        if low is not None:
            ctx.scratch["stream_low"] = low      # the stream as it goes on, rounded: what the next block's branch reads
        return h, None


@register_block("shared_norm")
class SharedNormBlock(Block):
    """x <- x + (mixer(h) + ff(h)) with h = norm(x): ONE norm whose output both sublayers read, and one add of their sum.
    The feed-forward is optional. With ``token_input`` the block ends with a per-token input (``stream.TokenInput``).

    The stream is float32 whatever the model's type. The norm reads it and writes h in the model's type; the sublayers
    return float32; one kernel adds both to the stream and leaves the new stream rounded to the model's type for the
    product that reads it next (the token input's gate)."""

    stream_dtype = torch.float32

    def __init__(self, spec: BlockSpec) -> None:
        super().__init__(spec)
        self._mixer = build_mixer(spec.mixer)
        self.feed_forward = build_feed_forward(spec.feed_forward) if spec.feed_forward is not None else None
        self.norm = build_norm(spec.input_norm)
        self.token_input = build_stream_part(spec.token_input) if spec.token_input is not None else None
        if not isinstance(self.norm, RmsNorm):
            raise ValueError("a shared_norm block needs an rms norm")
        for part in (self._mixer, self.feed_forward):
            if part is not None and not getattr(part, "takes_out_dtype", False):
                raise ValueError(f"a shared_norm block needs parts that can return float32, {type(part).__name__} cannot")

    @property
    def mixer(self):
        return self._mixer

    def sub_parts(self) -> Dict[str, Part]:
        s = self.spec
        parts: Dict[str, Part] = {s.input_norm_name: self.norm, s.mixer_name: self._mixer}
        if self.feed_forward is not None:
            parts[s.feed_forward_name] = self.feed_forward
        if self.token_input is not None:
            parts[s.token_input_name] = self.token_input
        return parts

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx,
                binding: CacheBinding) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if h.dtype != torch.float32 or h.dim() != 2 or pending is not None:
            raise RuntimeError("a shared_norm block takes one float32 stream with no branch pending")
        dtype = ctx.scratch["model_dtype"]
        ctx.scratch.pop("stream_low", None)
        x = self.norm(h, out_dtype=dtype)
        a = self._mixer.forward(x, ctx, binding, out_dtype=torch.float32)
        m = self.feed_forward.forward(x, ctx, out_dtype=torch.float32) if self.feed_forward is not None else None
        low = None
        if self.token_input is not None and dtype != torch.float32:
            low = torch.empty(h.shape, dtype=dtype, device=h.device)
        ops.add2_cast(h, a, m, low)
        if self.token_input is not None:
            self.token_input.forward(h, low if low is not None else h, ctx)
        return h, None


@dataclasses.dataclass
class PendingBranch:
    """A sublayer's result that has not reached the streams yet, with the coefficients it comes back by (None: added as
    it is). The kernel that opens the next sublayer, or the final norm, carries it out."""

    y: torch.Tensor
    coefficients: Optional[Part] = None
    # two results that were computed side by side and come back as c1 y + c2 y2 (formed by the kernel that carries them in)
    y2: Optional[torch.Tensor] = None
    c1: float = 1.0
    c2: float = 0.0


@register_block("hyper")
class HyperBlock(Block):
    """Pre-norm sublayers over ``streams`` residual streams X [tokens, S, hidden] in float32 (hyper-connections): a
    sublayer reads u = sum_s a[s] x_s through its norm, and its result y comes back as x'_r = sum_s M[s, r] x_s + b[r] y,
    every r from the old streams. With ``stream_coefficients`` off it is the plain pre-norm residual (a = b = 1, M = 1)
    on a float32 stream. The feed-forward is optional. ONE kernel ends a sublayer and opens the next (csrc/hyper.cu),
    across the border between two blocks too: the block hands its last result on as a ``PendingBranch``."""

    stream_dtype = torch.float32
    multi_stream = True

    def __init__(self, spec: BlockSpec) -> None:
        super().__init__(spec)
        self._mixer = build_mixer(spec.mixer)
        self.feed_forward = build_feed_forward(spec.feed_forward) if spec.feed_forward is not None else None
        self.input_norm = build_norm(spec.input_norm)
        self.post_norm = build_norm(spec.post_norm) if self.feed_forward is not None else None
        for n in (self.input_norm, self.post_norm):
            if n is not None and not isinstance(n, RmsNorm):
                raise ValueError("a hyper block needs rms norms")
        from .spec import StreamCoefficientsSpec
        self.mixer_streams = self.ff_streams = None
        if spec.stream_coefficients:
            self.mixer_streams = build_stream_part(StreamCoefficientsSpec(streams=spec.streams))
            if self.feed_forward is not None:
                self.ff_streams = build_stream_part(StreamCoefficientsSpec(streams=spec.streams))
        elif spec.streams != 1:
            raise ValueError("several streams need their coefficients")
        for part in (self._mixer, self.feed_forward):
            if part is not None and not getattr(part, "takes_out_dtype", False):
                raise ValueError(f"a hyper block needs parts that can return float32, {type(part).__name__} cannot")

    @property
    def mixer(self):
        return self._mixer

    def sub_parts(self) -> Dict[str, Part]:
        s = self.spec
        parts: Dict[str, Part] = {s.input_norm_name: self.input_norm, s.mixer_name: self._mixer}
        if self.feed_forward is not None:
            parts[s.post_norm_name] = self.post_norm
            parts[s.feed_forward_name] = self.feed_forward
        if self.mixer_streams is not None:
            parts[s.mixer_streams_name] = self.mixer_streams
        if self.ff_streams is not None:
            parts[s.feed_forward_streams_name] = self.ff_streams
        return parts

    @staticmethod
    def open_sublayer(X: torch.Tensor, pending: Optional[PendingBranch], reader: Optional[Part], norm: RmsNorm,
                      dtype: torch.dtype) -> torch.Tensor:
        """The pending result reaches the streams, and the next sublayer's input comes off them through its norm."""
        out = torch.empty((X.shape[0], X.shape[2]), dtype=dtype, device=X.device)
        c = pending.coefficients if pending is not None else None
        ops.hyper_step(X, y=pending.y if pending is not None else None, y2=pending.y2 if pending is not None else None,
                       c1=pending.c1 if pending is not None else 1.0, c2=pending.c2 if pending is not None else 0.0,
                       mix=c.mix if c is not None else None,
                       b_out=c.b_out if c is not None else None, a_in=reader.a_in if reader is not None else None,
                       norm_w=norm.weight, eps=norm.spec.eps, weight_offset=norm.spec.weight_offset, out=out)
        return out

    def forward(self, h: torch.Tensor, pending, ctx, binding: CacheBinding):
        if h.dim() != 3 or h.dtype != torch.float32 or h.shape[1] != self.spec.streams:
            raise RuntimeError(f"a hyper block takes float32 streams [tokens, {self.spec.streams}, hidden]")
        if pending is not None and not isinstance(pending, PendingBranch):
            raise RuntimeError("a hyper block follows hyper blocks only")
        dtype = ctx.scratch["model_dtype"]
        x = self.open_sublayer(h, pending, self.mixer_streams, self.input_norm, dtype)
        if getattr(self._mixer, "returns_pair", False):      # two sides whose weighted sum the next stream kernel forms
            a, a2, c1, c2 = self._mixer.forward(x, ctx, binding, out_dtype=torch.float32, as_pair=True)
            pending = PendingBranch(a, self.mixer_streams, y2=a2, c1=c1, c2=c2)
        else:
            pending = PendingBranch(self._mixer.forward(x, ctx, binding, out_dtype=torch.float32), self.mixer_streams)
        if self.feed_forward is not None:
            x = self.open_sublayer(h, pending, self.ff_streams, self.post_norm, dtype)
            m = self.feed_forward.forward(x, ctx, out_dtype=torch.float32)
            pending = PendingBranch(m, self.ff_streams)
        return h, pending


@dataclasses.dataclass
class PendingNormed:
    """A sublayer's result (float32) that has not reached the stream yet, and the norm it passes on its way there. The
    kernel that opens the next sublayer (also the next block's first), or the final norm, carries it out."""

    y: torch.Tensor
    norm: Part


@register_block("sandwich")
class SandwichBlock(Block):
    """x <- x + out_norm(mixer(in_norm(x))), then x <- x + out_norm'(ff(in_norm'(x))): a norm before AND behind each
    sublayer, four norms a layer (``input_norm`` / ``mixer_out_norm``, ``post_norm`` / ``feed_forward_out_norm``), all Dynamic
    Tanh. The feed-forward is optional.

    The stream is float32 whatever the model's type. ONE elementwise kernel stands between two sublayers: it norms the
    finished sublayer's result, adds it to the stream and forms the next sublayer's normed input in the model's type
    (csrc/sandwich_ops.cu), across the border between two blocks too: the block hands its last result on as a
    ``PendingNormed``. With ``ctx.scratch["stream_probe"]`` (a list) the block joins its last result at once and appends a
    copy of the stream, so that a test can look at the stream behind every layer."""

    stream_dtype = torch.float32

    def __init__(self, spec: BlockSpec) -> None:
        super().__init__(spec)
        from .norm import DynamicTanh
        self._mixer = build_mixer(spec.mixer)
        self.feed_forward = build_feed_forward(spec.feed_forward) if spec.feed_forward is not None else None
        self.input_norm = build_norm(spec.input_norm)
        self.mixer_out_norm = build_norm(spec.mixer_out_norm)
        self.post_norm = build_norm(spec.post_norm) if self.feed_forward is not None else None
        self.ff_out_norm = build_norm(spec.feed_forward_out_norm) if self.feed_forward is not None else None
        for n in (self.input_norm, self.mixer_out_norm, self.post_norm, self.ff_out_norm):
            if n is not None and not isinstance(n, DynamicTanh):
                raise ValueError("a sandwich block needs dyt norms")
        for part in (self._mixer, self.feed_forward):
            if part is not None and not getattr(part, "takes_out_dtype", False):
                raise ValueError(f"a sandwich block needs parts that can return float32, {type(part).__name__} cannot")

    @property
    def mixer(self):
        return self._mixer

    def sub_parts(self) -> Dict[str, Part]:
        s = self.spec
        parts: Dict[str, Part] = {s.input_norm_name: self.input_norm, s.mixer_name: self._mixer,
                                  s.mixer_out_norm_name: self.mixer_out_norm}
        if self.feed_forward is not None:
            parts[s.post_norm_name] = self.post_norm
            parts[s.feed_forward_name] = self.feed_forward
            parts[s.feed_forward_out_norm_name] = self.ff_out_norm
        return parts

    @staticmethod
    def open_sublayer(h: torch.Tensor, pending: Optional[PendingNormed], norm, dtype: torch.dtype) -> torch.Tensor:
        """The pending result reaches the stream through its norm, and the next sublayer's input comes off the stream
        through ``norm``: one kernel."""
        out = torch.empty(h.shape, dtype=dtype, device=h.device)
        ops.dyt_step(h, branch=pending.y if pending is not None else None, post=pending.norm.triple() if pending is not None else None,
                     pre=norm.triple(), out=out)
        return out

    def forward(self, h: torch.Tensor, pending, ctx, binding: CacheBinding):
        if h.dtype != torch.float32 or h.dim() != 2:
            raise RuntimeError("a sandwich block takes one float32 stream")
        if pending is not None and not isinstance(pending, PendingNormed):
            raise RuntimeError("a sandwich block follows sandwich blocks only")
        dtype = ctx.scratch["model_dtype"]
        x = self.open_sublayer(h, pending, self.input_norm, dtype)
        pending = PendingNormed(self._mixer.forward(x, ctx, binding, out_dtype=torch.float32), self.mixer_out_norm)
        if self.feed_forward is not None:
            x = self.open_sublayer(h, pending, self.post_norm, dtype)
            pending = PendingNormed(self.feed_forward.forward(x, ctx, out_dtype=torch.float32), self.ff_out_norm)
        probe = ctx.scratch.get("stream_probe")
        if probe is not None:
            ops.dyt_step(h, branch=pending.y, post=pending.norm.triple())
            probe.append(h.clone())
            pending = None
        return h, pending
