"""Attention over a cached low-rank latent, with a causal window and an optional sigmoid gate per head.

Per position the cache holds ONE vector c (``latent_rank`` numbers, normed): every head h forms its keys and values
from it, k = Wuk_h c and v = Wuv_h c. Because (q_h . Wuk_h c) = (Wuk_h^T q_h) . c and sum_s p_s Wuv_h c_s =
Wuv_h sum_s p_s c_s, the heads never need their keys and values spelled out: with q'_h = Wuk_h^T q_h the attention is
multi-query attention of ``num_heads`` queries over a single "kv head" whose keys AND values are the latent itself, and
it runs on the package's paged attention kernels with the cache's one plane given as both operands. The two
up-projections are applied either once at load time ("weights": Wq'_h = Wuk_h^T Wq_h and Wo'_h = Wo_h Wuv_h, formed in
float64 and rounded once to the weights' type: queries and outputs then come straight out of one product each) or in
every step ("runtime": one small product per head before and after the attention). Cached rows are padded with zeros to
a multiple of eight elements, which changes neither scores nor outputs.

With ``rope_dim`` > 0 every head's query has a rotated part behind its ``qk_dim`` unrotated numbers and the down-projection
one shared rotated key part behind the latent (not normed); their dot product is added to the score. The cached row is
then [latent, rotated key part] and the absorbed query [Wuk_h^T q_h, rotated query part]: still one multi-query attention
over one cached tensor, whose result's first ``latent_rank`` numbers are sum_s p_s c_s (the rest is not read). One kernel
norms the latent, turns the key part, stores both, and turns the heads' query parts in place. A sink (a learned number per
head in the softmax's denominator) is applied by the attention kernels; a gate per OUTPUT NUMBER (``gate_per`` "element")
sits between the value up-projection and the output projection, so the former then runs in every step.

A position encoding that turns neighbours (2 n, 2 n + 1) (``PositionSpec.interleaved``) costs nothing at run time: the rows
of the query projection's rotated part and of the down-projection's key part are reordered once, when the weights are
loaded, so that pair n sits at (n, n + rope_dim / 2); a dot product does not change when both sides are reordered alike.

A layer without a latent of its own (``has_latent`` False) reads the pages another layer wrote, with its own queries,
up-projections, window and gate.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.manager import KvNeed
from ..kernels import attention as attn_kernels
from ..kernels import native, ops
from ..kernels.linear import linear
from .base import CacheBinding, Mixer
from .registry import build_position_encoding, register_mixer
from .spec import LatentAttentionSpec, ParamInfo


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True
    takes_out_dtype = True

    def __init__(self, spec: LatentAttentionSpec) -> None:
        super().__init__(spec)
        s = spec
        for name in ("hidden_size", "num_heads", "qk_dim", "v_dim", "latent_rank"):
            if getattr(s, name) <= 0:
                raise ValueError(f"latent_attention: {name} must be positive, got {getattr(s, name)}")
        if s.absorb not in ("weights", "runtime"):
            raise ValueError(f"latent_attention: absorb must be 'weights' or 'runtime', got {s.absorb!r}")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"latent_attention: window must be positive, got {s.window}")
        if s.gate_per not in ("head", "element"):
            raise ValueError(f"latent_attention: gate_per must be 'head' or 'element', got {s.gate_per!r}")
        if s.rope_dim < 0 or s.rope_dim % 2:
            raise ValueError(f"latent_attention: rope_dim must be even and not negative, got {s.rope_dim}")
        if s.rope_dim:
            if s.position is None or s.position.kind == "none" or s.position.rotary_dim != s.rope_dim:
                raise ValueError("latent_attention: a rotated part needs a position encoding over exactly its numbers")
            if s.absorb != "weights":
                raise ValueError("latent_attention: a rotated part needs the key up-projection absorbed into the weights")
        self.position = build_position_encoding(s.position) if s.rope_dim else None
        self.tables = None
        # the values' up-projection is multiplied into the output projection unless a gate sits between the two
        self.absorb_values = s.absorb == "weights" and not (s.output_gate and s.gate_per == "element")
        self.gate_cols = (s.num_heads * s.v_dim if s.gate_per == "element" else s.num_heads) if s.output_gate else 0
        self.row = _round_up(s.latent_rank + s.rope_dim, 8)          # elements of a cached row
        if self.row > 512:
            raise ValueError(f"latent_attention: latent_rank {s.latent_rank} is beyond what the attention kernels take (512)")
        self.q_cols = s.num_heads * (self.row if s.absorb == "weights" else s.qk_dim)
        self.latent_off = self.q_cols
        self.gate_off = self.latent_off + (s.latent_rank + s.rope_dim if s.has_latent else 0)
        self.in_cols = _round_up(self.gate_off + self.gate_cols, 8)
        self.sinks: Optional[torch.Tensor] = None
        self.mods = None
        self.w_in: Optional[torch.Tensor] = None         # [in_cols, hidden]: queries | latent | gate | zero rows
        self.w_out: Optional[torch.Tensor] = None        # [hidden, heads * row] ("weights") or [hidden, heads * v_dim]
        self.w_latent_norm: Optional[torch.Tensor] = None
        self.w_up_k: Optional[torch.Tensor] = None       # "runtime": [heads, row, qk_dim]
        self.w_up_v: Optional[torch.Tensor] = None       # "runtime": [heads, v_dim, row]

    def kv_need(self) -> Optional[KvNeed]:
        return KvNeed(1, self.row, self.spec.window, planes=1)

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        H, W, R = s.num_heads, s.hidden_size, s.latent_rank
        p = {
            s.q_name: ParamInfo((H * (s.qk_dim + s.rope_dim), W), ("normal", W ** -0.5)),
            s.up_k_name: ParamInfo((H * s.qk_dim, R), ("normal", R ** -0.5)),
            s.up_v_name: ParamInfo((H * s.v_dim, R), ("normal", R ** -0.5)),
            s.out_name: ParamInfo((W, H * s.v_dim), ("normal", (H * s.v_dim) ** -0.5)),
        }
        if s.has_latent:
            p[s.down_name] = ParamInfo((R + s.rope_dim, W), ("normal", W ** -0.5))
            if s.latent_norm is not None:
                p[s.latent_norm_name] = ParamInfo((R,), ("one_plus_normal", 0.1))
        if s.output_gate:
            p[s.gate_name] = ParamInfo((self.gate_cols, W), ("normal", W ** -0.5))
        if s.sink:
            p[s.sink_name] = ParamInfo((H,), ("normal", 1.0))
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        H, W, R, D, V, row = s.num_heads, s.hidden_size, s.latent_rank, s.qk_dim, s.v_dim, self.row
        wq, wuk, wuv, wo = (tensors[n] for n in (s.q_name, s.up_k_name, s.up_v_name, s.out_name))
        dt, dev = wq.dtype, wq.device
        f64 = torch.float64
        uk = wuk.to(f64).view(H, D, R)
        uv = wuv.to(f64).view(H, V, R)
        P = s.rope_dim
        # where the rotated numbers go: as stored, or (interleaved pairs) evens first, then odds
        turn = torch.arange(P, device=dev)
        if P and s.position is not None and s.position.interleaved:
            turn = torch.cat([torch.arange(0, P, 2, device=dev), torch.arange(1, P, 2, device=dev)])
        if s.absorb == "weights":
            wq_heads = wq.to(f64).view(H, D + P, W)
            q_rows = torch.zeros((H, row, W), dtype=f64, device=dev)
            q_rows[:, :R] = torch.matmul(uk.transpose(1, 2), wq_heads[:, :D])                   # Wuk_h^T Wq_h
            q_rows[:, R: R + P] = wq_heads[:, D:][:, turn]                                      # the rotated part
            q_part = q_rows.view(H * row, W).to(dt)
            if self.absorb_values:
                out_cols = torch.zeros((W, H, row), dtype=f64, device=dev)
                out_cols[:, :, :R] = torch.einsum("whv,hvr->whr", wo.to(f64).view(W, H, V), uv)  # Wo_h Wuv_h
                self.w_out = out_cols.view(W, H * row).to(wo.dtype).contiguous()
            else:
                self.w_out = wo.contiguous()
                up_v = torch.zeros((H, V, row), dtype=wuv.dtype, device=dev)
                up_v[:, :, :R] = wuv.view(H, V, R)
                self.w_up_v = up_v.contiguous()
        else:
            q_part = wq
            self.w_out = wo.contiguous()
            up_k = torch.zeros((H, row, D), dtype=dt, device=dev)
            up_k[:, :R] = wuk.view(H, D, R).transpose(1, 2)
            up_v = torch.zeros((H, V, row), dtype=wuv.dtype, device=dev)
            up_v[:, :, :R] = wuv.view(H, V, R)
            self.w_up_k, self.w_up_v = up_k.contiguous(), up_v.contiguous()
        parts = [q_part]
        if s.has_latent:
            down = tensors[s.down_name]
            parts.append(torch.cat([down[:R], down[R:][turn]], dim=0) if P else down)
            if s.latent_norm is not None:
                self.w_latent_norm = tensors[s.latent_norm_name].contiguous()
            else:
                raise ValueError("latent_attention: a latent without a norm has no kernel")
        if s.output_gate:
            parts.append(tensors[s.gate_name])
        if s.sink:
            self.sinks = tensors[s.sink_name].to(torch.float32).contiguous()
            self.mods = native.ScoreMods(sinks=self.sinks.data_ptr())
        if any(p.dtype != dt for p in parts):
            raise ValueError("latent_attention: the input projections must be stored in one dtype to be fused")
        rows = sum(p.shape[0] for p in parts)
        if self.in_cols > rows:
            parts.append(torch.zeros((self.in_cols - rows, W), dtype=dt, device=dev))
        self.w_in = torch.cat(parts, dim=0).contiguous()

    def prepare(self, device: torch.device, dtype: torch.dtype) -> None:
        if self.position is not None:
            self.tables = self.position.rotation_tables(device)

    def forward(self, x: torch.Tensor, ctx, binding: CacheBinding, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        s = self.spec
        if binding.kv is None:
            raise RuntimeError("latent attention needs a cache binding")
        if binding.owns_kv != s.has_latent:
            raise RuntimeError("latent attention: a layer with a latent of its own owns its pages, one without reads another's")
        H, row, T = s.num_heads, self.row, x.shape[0]
        group = ctx.groups[binding.kv.group]
        pages, _, page_stride = ctx.cache.kv_views(binding.kv)
        proj = linear(x, self.w_in)                                        # [T, queries | latent | gate]
        if s.rope_dim:
            # one pass: the latent's norm, the key part's rotation, both stored; the heads' query parts turned in place
            ln = s.latent_norm
            cos, sin = self.tables
            ops.latent_rope_store(pages if s.has_latent else None, page_stride, proj, self.latent_off, s.latent_rank,
                                  self.w_latent_norm if s.has_latent else None, ln.eps if ln else 0.0, ln.weight_offset if ln else 0.0,
                                  cos, sin, ctx.positions, group.slot_mapping if s.has_latent else None, H, row, s.latent_rank,
                                  store=s.has_latent)
        elif s.has_latent:
            ln = s.latent_norm
            ops.latent_store(pages, page_stride, proj[:, self.latent_off: self.latent_off + s.latent_rank], self.w_latent_norm,
                             group.slot_mapping, s.latent_rank, ln.eps, ln.weight_offset)
        if s.absorb == "weights":
            q = proj[:, : H * row]
        else:
            q = torch.empty((T, H * row), dtype=x.dtype, device=x.device)
            for h in range(H):
                linear(proj[:, h * s.qk_dim: (h + 1) * s.qk_dim], self.w_up_k[h], out=q[:, h * row: (h + 1) * row])
        mixed = torch.empty((T, H * row), dtype=x.dtype, device=x.device)
        step = attn_kernels.attention_step(ctx, group, q, mixed, pages, page_stride, H, 1, row, s.window, mods=self.mods is not None)
        layer = attn_kernels.attention_layer(q, mixed, pages, pages, H, 1, row, s.softmax_scale, s.window,
                                             write_kv=False, rope_mode=0, mods=self.mods)
        attn_kernels.run_attention(step, layer)
        if s.output_gate and s.gate_per == "head":
            ops.head_gate(mixed, proj[:, self.gate_off: self.gate_off + H], H, row)
        if not self.absorb_values:
            heads_out = torch.empty((T, H * s.v_dim), dtype=x.dtype, device=x.device)
            for h in range(H):
                linear(mixed[:, h * row: (h + 1) * row], self.w_up_v[h], out=heads_out[:, h * s.v_dim: (h + 1) * s.v_dim])
            mixed = heads_out
            if s.output_gate and s.gate_per == "element":
                ops.head_gate(mixed, proj[:, self.gate_off: self.gate_off + H * s.v_dim], H * s.v_dim, 1)
        return linear(mixed, self.w_out, out_dtype=out_dtype)
