"""Attention mixer over the paged cache: grouped-query, causal, optional window,
optional per-head q/k norm, optional rotation.

One fused projection q|k|v (the reference also stores the three matrices as one,
pegainfer-qwen3/src/weights/load.rs:98-134), then the fused norm + rotation + cache
write, attention over the request's pages, and the output projection
(pegainfer-qwen3/src/unified_forward.rs:414-536). When the call reads another call's
cache only the query projection exists and nothing is written.

Queries / keys of ``qk_dim`` and values of ``v_dim`` numbers per head (``AttentionSpec.qk_dim``, ``v_dim``) run on the same
kernels: the cached row is ``head_dim`` (a multiple of 8 that holds both), the projections get zero rows up to it when
they are loaded (zeros change neither a score nor a value), and a per-head norm over qk_dim numbers is the norm over
head_dim with eps * qk_dim / head_dim whose result is long by sqrt(head_dim / qk_dim) in q and in k alike, which the
softmax scale takes back.

Optional, all from the spec: a short causal filter over time on every channel of q, k and v directly behind the
projections (its last taps - 1 input rows are per-request state); a query temperature that grows with the logarithm of the
position; a cap on the scores (cap * tanh(s / cap)); a distance bias slope_h * (i - j) with slope_h = 2^(-e (h + 1) / H);
a learned sink per head in the softmax's denominator; a sigmoid gate per head on the attention's output, read off the
mixer's input by rows appended to the fused projection. Temperature, cap, bias and sink are applied to the float32 scores
inside the attention kernels (csrc/oi_api.h, OiScoreMods).

Also from the spec: biases on q, k and v; a unit norm of q and k heads AFTER the rotation (root mean square over qk_dim
numbers, no weight) instead of the weighted norm before it; with a window, a number of first keys of the sequence that stay
visible behind it (their pages are kept). A layer with biases or the norm behind the rotation prepares its rows with one
kernel of its own (csrc/sandwich_ops.cu: bias, rotation, norm, cache write) and hands the attention kernels ready queries.
A bias in front of the filter is carried behind it: filter(u + b)_t = filter(u)_t + b * (sum of the taps that fall on
positions >= 0), a small table by position that the same kernel adds.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.manager import KvNeed, StateNeed
from ..kernels import attention as attn_kernels
from ..kernels import native, ops
from ..kernels.linear import linear
from .base import CacheBinding, Mixer
from .registry import build_position_encoding, register_mixer
from .spec import AttentionSpec, ParamInfo


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec: AttentionSpec) -> None:
        super().__init__(spec)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads ({s.num_heads}) must be a multiple of num_kv_heads ({s.num_kv_heads})")
        if s.head_dim % 8 or s.head_dim > 512:
            raise ValueError(f"head_dim {s.head_dim} unsupported: multiples of 8 up to 512")
        self.qk = s.qk_dim or s.head_dim
        self.vd = s.v_dim or s.head_dim
        if self.qk > s.head_dim or self.vd > s.head_dim:
            raise ValueError(f"head_dim {s.head_dim} must hold queries of {self.qk} and values of {self.vd} numbers")
        self.q_dim = s.num_heads * s.head_dim
        self.kv_dim = s.num_kv_heads * s.head_dim
        # a norm over qk of head_dim numbers (see the file's head)
        self.norm_eps_factor = self.qk / s.head_dim
        self.scale = s.softmax_scale * (self.qk / s.head_dim if (s.qk_norm is not None and self.qk != s.head_dim) else 1.0)
        self.position = build_position_encoding(s.position)
        if s.conv_taps < 0 or s.score_cap < 0.0 or s.distance_slope_exponent < 0.0:
            raise ValueError("attention: conv_taps, score_cap and distance_slope_exponent cannot be negative")
        if s.q_temperature is not None and int(s.q_temperature[1]) <= 0:
            raise ValueError(f"attention: the query temperature's period must be positive, got {s.q_temperature[1]}")
        self.qkv_cols = self.q_dim + 2 * self.kv_dim
        self.gate_off = self.qkv_cols                      # the gate's columns of the fused projection, behind q | k | v
        self.in_cols = -(-(self.qkv_cols + (s.num_heads if s.head_gate else 0)) // 8) * 8
        if s.keep_first < 0 or s.unit_norm_after_rotation_eps < 0.0:
            raise ValueError("attention: keep_first and the unit norm's eps cannot be negative")
        if s.unit_norm_after_rotation_eps > 0.0 and s.qk_norm is not None:
            raise ValueError("attention: q and k are normed before the rotation or behind it, not both")
        self.keep_first = int(s.keep_first) if s.window else 0
        # rows prepared by rope_norm_store (bias, rotation, unit norm, cache write) instead of the norm-then-rotate kernel
        self.own_prepare = bool(s.qkv_bias or s.unit_norm_after_rotation_eps > 0.0)
        if self.own_prepare and s.position.kind != "none" and getattr(s.position, "interleaved", False):
            raise ValueError("attention: the rotation in front of a unit norm turns the pairs (d, d + half)")
        self.bias_tab: Optional[torch.Tensor] = None
        self.has_mods = bool(s.sink or s.score_cap > 0.0 or s.distance_slope_exponent > 0.0 or s.q_temperature is not None
                             or self.keep_first > 0)
        self.w_conv: Optional[torch.Tensor] = None
        self.sinks: Optional[torch.Tensor] = None
        self.slopes: Optional[torch.Tensor] = None
        self.mods = None
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm_w: Optional[torch.Tensor] = None
        self.k_norm_w: Optional[torch.Tensor] = None
        self.tables = None

    def kv_need(self) -> Optional[KvNeed]:
        s = self.spec
        return KvNeed(s.num_kv_heads, s.head_dim, s.window, keep_first=self.keep_first)

    def state_needs(self):
        s = self.spec
        # two copies that take turns: the filter's kernel reads a request's old rows while it leaves the new ones
        return [StateNeed((s.conv_taps - 1, self.qkv_cols), "float32", phases=2)] if s.conv_taps > 1 else []

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        p = {
            s.q_name: ParamInfo((s.num_heads * self.qk, s.hidden_size)),
            s.k_name: ParamInfo((s.num_kv_heads * self.qk, s.hidden_size)),
            s.v_name: ParamInfo((s.num_kv_heads * self.vd, s.hidden_size)),
            s.o_name: ParamInfo((s.hidden_size, s.num_heads * self.vd)),
        }
        if s.qk_norm is not None:
            p[s.q_norm_name] = ParamInfo((self.qk,), ("one_plus_normal", 0.02))
            p[s.k_norm_name] = ParamInfo((self.qk,), ("one_plus_normal", 0.02))
        if s.conv_taps > 0:
            for name, rows in ((s.q_name, s.num_heads * self.qk), (s.k_name, s.num_kv_heads * self.qk), (s.v_name, s.num_kv_heads * self.vd)):
                p[name + s.conv_suffix] = ParamInfo((rows, s.conv_taps), ("normal_around", 0.2, 1.0 / s.conv_taps))
        if s.sink:
            p[s.sink_name] = ParamInfo((s.num_heads,), ("normal", 1.0))
        if s.head_gate:
            p[s.gate_name] = ParamInfo((s.num_heads, s.hidden_size), ("normal", s.hidden_size ** -0.5))
        if s.qkv_bias:
            for name, rows in ((s.q_name, s.num_heads * self.qk), (s.k_name, s.num_kv_heads * self.qk), (s.v_name, s.num_kv_heads * self.vd)):
                p[name + s.bias_suffix] = ParamInfo((rows,), ("normal", 0.1))
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        q, k, v = tensors[s.q_name], tensors[s.k_name], tensors[s.v_name]
        if not (q.dtype == k.dtype == v.dtype):
            raise ValueError("the q, k and v projections must be stored in one dtype to be fused")
        hd = s.head_dim

        def rows_padded(w, heads, size):       # [heads * size, in] -> [heads * head_dim, in], zero rows behind each head's
            if size == hd:
                return w
            out = torch.zeros((heads, hd, w.shape[1]), dtype=w.dtype, device=w.device)
            out[:, :size] = w.view(heads, size, -1)
            return out.view(heads * hd, -1)

        fused = [rows_padded(q, s.num_heads, self.qk), rows_padded(k, s.num_kv_heads, self.qk), rows_padded(v, s.num_kv_heads, self.vd)]
        if s.head_gate:
            g = tensors[s.gate_name]
            if g.dtype != q.dtype:
                raise ValueError("the gate's projection must be stored in the dtype of q, k and v to be fused")
            fused.append(g)
            if self.in_cols > self.qkv_cols + s.num_heads:
                fused.append(torch.zeros((self.in_cols - self.qkv_cols - s.num_heads, q.shape[1]), dtype=q.dtype, device=q.device))
        self.w_qkv = torch.cat(fused, dim=0).contiguous()
        if s.conv_taps > 0:
            names = ((s.q_name, s.num_heads, self.qk), (s.k_name, s.num_kv_heads, self.qk), (s.v_name, s.num_kv_heads, self.vd))
            self.w_conv = torch.cat([rows_padded(tensors[n + s.conv_suffix], heads, size) for n, heads, size in names], dim=0).contiguous()
        if s.sink:
            self.sinks = tensors[s.sink_name].to(torch.float32).contiguous()
        if s.qkv_bias:
            # the bias as the filter hands it on, by position: row m holds b * (sum of the taps j >= taps - 1 - m), the last
            # row b * (sum of all taps); without a filter the one row b
            names = ((s.q_name, s.num_heads, self.qk), (s.k_name, s.num_kv_heads, self.qk), (s.v_name, s.num_kv_heads, self.vd))
            b = torch.cat([rows_padded(tensors[n + s.bias_suffix].to(torch.float64)[:, None], heads, size)[:, 0] for n, heads, size in names])
            if s.conv_taps > 0:
                w = self.w_conv.to(torch.float64)
                tab = torch.stack([b * w[:, s.conv_taps - 1 - m:].sum(dim=1) for m in range(s.conv_taps)])
            else:
                tab = b[None, :]
            self.bias_tab = tab.to(torch.float32).contiguous()
        o = tensors[s.o_name]
        if self.vd != hd:
            wide = torch.zeros((o.shape[0], s.num_heads, hd), dtype=o.dtype, device=o.device)
            wide[:, :, : self.vd] = o.view(o.shape[0], s.num_heads, self.vd)
            o = wide.view(o.shape[0], s.num_heads * hd)
        self.w_o = o.contiguous()
        if self.spec.qk_norm is not None:
            def norm_padded(w):
                if self.qk == hd:
                    return w.contiguous()
                out = torch.zeros(hd, dtype=w.dtype, device=w.device)
                out[: self.qk] = w
                return out

            self.q_norm_w = norm_padded(tensors[s.q_norm_name])
            self.k_norm_w = norm_padded(tensors[s.k_norm_name])
            if self.q_norm_w.dtype != self.k_norm_w.dtype:
                self.k_norm_w = self.k_norm_w.to(self.q_norm_w.dtype)

    def prepare(self, device: torch.device, dtype: torch.dtype) -> None:
        self.tables = self.position.rotation_tables(device)
        s = self.spec
        if s.distance_slope_exponent > 0.0:
            h = torch.arange(1, s.num_heads + 1, dtype=torch.float64)
            self.slopes = torch.pow(2.0, -s.distance_slope_exponent * h / s.num_heads).to(torch.float32).to(device)
        if self.has_mods:
            coef, every = s.q_temperature if s.q_temperature is not None else (0.0, 0)
            self.mods = native.ScoreMods(sinks=None if self.sinks is None else self.sinks.data_ptr(),
                                         slopes=None if self.slopes is None else self.slopes.data_ptr(),
                                         softcap=float(s.score_cap), qt_coef=float(coef), qt_every=int(every),
                                         keep_first=self.keep_first)

    takes_out_dtype = True

    def forward(self, x: torch.Tensor, ctx, binding: CacheBinding, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        s = self.spec
        if binding.kv is None:
            raise RuntimeError("attention needs a cache binding")
        group = ctx.groups[binding.kv.group]
        k_cache, v_cache, page_stride = ctx.cache.kv_views(binding.kv)
        if binding.owns_kv:
            w = self.w_qkv
        elif s.head_gate or s.conv_taps > 0:
            raise RuntimeError("attention: a layer with a gate or a filter owns its cache")
        else:
            w = self.w_qkv[: self.q_dim]
        qkv = raw = linear(x, w)
        if s.conv_taps > 0:
            # the filter over time on the q | k | v columns; the request's last taps - 1 rows are carried in its state slot
            qkv = torch.empty((x.shape[0], self.qkv_cols), dtype=x.dtype, device=x.device)
            state = ctx.cache.state_tensor(binding.states[0]) if s.conv_taps > 1 else None
            ops.short_conv_act(qkv, raw[:, : self.qkv_cols], self.w_conv, state, ctx.cu_seqlens, ctx.token_req, ctx.state_slots,
                               ctx.state_phase, act="none", add_input=False)
        cos, sin = self.tables if self.tables is not None else (None, None)
        qn = s.qk_norm
        out = torch.empty((x.shape[0], self.q_dim), dtype=x.dtype, device=x.device)
        if self.own_prepare:
            # bias, rotation, unit norm and cache write in one kernel of the layer's own; the attention kernels get ready rows
            ops.rope_norm_store(qkv, s.num_heads, s.num_kv_heads, s.head_dim, self.qk, bias_tab=self.bias_tab, cos=cos, sin=sin,
                                unit_norm=s.unit_norm_after_rotation_eps > 0.0, eps=s.unit_norm_after_rotation_eps,
                                positions=ctx.positions, slots=group.slot_mapping if binding.owns_kv else None,
                                k_cache=k_cache if binding.owns_kv else None, v_cache=v_cache if binding.owns_kv else None,
                                page_stride=page_stride, page_size=ctx.cache.page_size, write_kv=binding.owns_kv)
            step = attn_kernels.attention_step(ctx, group, qkv, out, k_cache, page_stride, s.num_heads, s.num_kv_heads,
                                               s.head_dim, s.window, mods=self.has_mods, keep_first=self.keep_first)
            layer = attn_kernels.attention_layer(qkv, out, k_cache, v_cache, s.num_heads, s.num_kv_heads, s.head_dim, self.scale,
                                                 s.window, write_kv=False, rope_mode=0, mods=self.mods)
            attn_kernels.run_attention(step, layer)
            if s.head_gate:
                ops.head_gate(out, raw[:, self.gate_off: self.gate_off + s.num_heads], s.num_heads, s.head_dim)
            return linear(out, self.w_o, out_dtype=out_dtype)
        # One native call: the norm + rotation + cache write (in a kernel of its own, or inside the decode kernel when
        # the step is single tokens in one wave), then the attention kernel(s) that take the step's shape.
        step = attn_kernels.attention_step(ctx, group, qkv, out, k_cache, page_stride, s.num_heads, s.num_kv_heads,
                                           s.head_dim, s.window, cos=cos, q_norm_w=self.q_norm_w, mods=self.has_mods,
                                           keep_first=self.keep_first)
        layer = attn_kernels.attention_layer(
            qkv, out, k_cache, v_cache, s.num_heads, s.num_kv_heads, s.head_dim, self.scale, s.window,
            q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, eps=qn.eps * self.norm_eps_factor if qn else 0.0,
            weight_offset=qn.weight_offset if qn else 0.0, cos=cos, sin=sin, write_kv=binding.owns_kv, rope_mode=1,
            interleaved=bool(getattr(s.position, "interleaved", False)), mods=self.mods)
        attn_kernels.run_attention(step, layer)
        if s.head_gate:
            ops.head_gate(out, raw[:, self.gate_off: self.gate_off + s.num_heads], s.num_heads, s.head_dim)
        return linear(out, self.w_o, out_dtype=out_dtype)
