"""Recurrent mixers whose memory is a matrix per head, kept in the cache manager's state slots.

"matrix_memory" (the mLSTM cell of xLSTM): per head C [dim, vdim], a normaliser n [dim] and a running maximum m, all zero
at a request's start. With i = cap tanh(zi / cap) and f = logsigmoid(cap tanh(zf / cap)) (zi, zf: biased projections):
m' = max(f + m, i); C' = e^(f + m - m') C + e^(i - m') k v^T; n' likewise with k; the read-out is
C'^T q / (max(|n' . q|, e^(-m')) + 1e-6) with q scaled by dim^(-1/2). Each head's read-out is divided by its root mean
square, multiplied by a weight over all heads and by sigmoid(Wg x), then projected out.

"gated_delta" (gated delta rule): queries and keys per kv head and values per head pass a short causal filter over time
(its last taps - 1 inputs are state) and silu; q and k become unit vectors, q times dim^(-1/2); per head C <- diag(g) C,
d = beta (v - C^T k), C <- C + k d^T, read-out C^T q, with beta = sigmoid(Wb x) and one decay per head and key channel
g = exp(-exp(A) softplus(Wa2 Wa1 x + dt)). The read-out is normed per head over vdim with one weight shared by the heads,
gated by sigmoid(Wg2 Wg1 x), projected out.

"linear_attention" (linear attention with one fixed decay per head, "lightning attention"): q, k and v through silu; per
head S <- decay_h S + k v^T, read-out S^T q with no other scale; the concatenated heads are RMS-normed together with one
weight, multiplied by sigmoid(Wg x), projected out.

All run as ONE fused input product whose sums stay float32 (gates, decays and everything else that enters the
recurrence never pass through the model's type), the scan kernel over the step's rows (prompt portions and single tokens
alike, csrc/recurrent.cu), the norm-and-gate kernel, and the output product. The state lives in two copies that take
turns, like the short filter's.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import StateNeed
from ..kernels import ops
from ..kernels.linear import linear
from .base import CacheBinding, Mixer
from .registry import register_mixer
from .spec import GatedDeltaSpec, LinearAttentionSpec, MatrixMemorySpec, ParamInfo


def _pad8(n: int) -> int:
    return (n + 7) & ~7


@register_mixer("matrix_memory")
class MatrixMemory(Mixer):
    graph_safe = True
    takes_out_dtype = True

    def __init__(self, spec: MatrixMemorySpec) -> None:
        super().__init__(spec)
        s = spec
        if min(s.num_heads, s.qk_dim, s.v_dim) <= 0 or s.qk_dim > 512 or not s.gate_cap > 0:
            raise ValueError(f"matrix_memory: heads {s.num_heads}, dim {s.qk_dim} (at most 512), vdim {s.v_dim}, cap {s.gate_cap}")
        H, D, V = s.num_heads, s.qk_dim, s.v_dim
        # columns of the fused product: q | k | v | output gate | zi | zf
        self.off = {"q": 0, "k": H * D, "v": 2 * H * D, "g": 2 * H * D + H * V, "i": 2 * H * D + 2 * H * V,
                    "f": 2 * H * D + 2 * H * V + H}
        self.cols = 2 * H * D + 2 * H * V + 2 * H
        self.w_in: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        H, D, V, W = s.num_heads, s.qk_dim, s.v_dim, s.hidden_size
        std = W ** -0.5
        return {"q": ParamInfo((H * D, W), ("normal", std)), "k": ParamInfo((H * D, W), ("normal", std)),
                "v": ParamInfo((H * V, W), ("normal", std)), "g": ParamInfo((H * V, W), ("normal", std)),
                "o": ParamInfo((W, H * V), ("normal", (H * V) ** -0.5)), "norm": ParamInfo((H * V,), ("one_plus_normal", 0.1)),
                # random weights: a mild input gate around 0 and a forget gate near one keep the running maximum small, so
                # that both sides of the read-out's max(|n . q|, e^-m) occur and a rounding is not amplified by a tiny divisor
                "i": ParamInfo((H, W), ("normal", 0.3 * std)), "i.b": ParamInfo((H,), ("normal", 0.3)),
                "f": ParamInfo((H, W), ("normal", std)), "f.b": ParamInfo((H,), ("normal_around", 0.5, 4.0))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        rows = [tensors[n] for n in ("q", "k", "v", "g", "i", "f")]
        w = torch.cat(rows, dim=0)
        pad = _pad8(w.shape[0]) - w.shape[0]
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
        self.w_in = w.contiguous()
        self.w_o = tensors["o"].contiguous()
        self.norm_w = tensors["norm"].contiguous()
        self.bias_i = tensors["i.b"].contiguous()
        self.bias_f = tensors["f.b"].to(self.bias_i.dtype).contiguous()

    def state_needs(self) -> List[StateNeed]:
        s = self.spec
        return [StateNeed((s.num_heads, s.qk_dim * s.v_dim + s.qk_dim + 1), "float32", phases=2)]

    def forward(self, x: torch.Tensor, ctx, binding: CacheBinding, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        s = self.spec
        H, D, V = s.num_heads, s.qk_dim, s.v_dim
        z = linear(x, self.w_in, out_dtype=torch.float32)
        o = torch.empty((x.shape[0], H * V), dtype=torch.float32, device=x.device)
        ops.recurrent_scan(ops.SCAN_MATRIX_MEMORY, o, z, (self.off["q"], self.off["k"], self.off["v"]), z,
                           (self.off["i"], self.off["f"]), ctx.cache.state_tensor(binding.states[0]), ctx, H, H, D, V,
                           p0=self.bias_i, p1=self.bias_f, cap=s.gate_cap, q_scale=D ** -0.5)
        y = torch.empty((x.shape[0], H * V), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(y, o, z[:, self.off["g"]: self.off["g"] + H * V], self.norm_w, H, V, s.eps, weight_per_head=True)
        return linear(y, self.w_o, out_dtype=out_dtype)


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    graph_safe = True
    takes_out_dtype = True

    def __init__(self, spec: GatedDeltaSpec) -> None:
        super().__init__(spec)
        s = spec
        if min(s.num_heads, s.num_kv_heads, s.qk_dim, s.v_dim) <= 0 or s.num_heads % s.num_kv_heads or s.qk_dim > 512 or s.conv_taps < 1:
            raise ValueError(f"gated_delta: heads {s.num_heads}, kv heads {s.num_kv_heads}, dim {s.qk_dim} (at most 512), "
                             f"vdim {s.v_dim}, taps {s.conv_taps}")
        H, G, D, V = s.num_heads, s.num_kv_heads, s.qk_dim, s.v_dim
        self.filtered = 2 * G * D + H * V            # q | k | v: the columns that pass the filter
        self.ra = s.decay_rank or max(8, D // 4)
        self.rg = s.gate_rank or max(8, V // 4)

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        H, G, D, V, W, taps = s.num_heads, s.num_kv_heads, s.qk_dim, s.v_dim, s.hidden_size, s.conv_taps
        std = W ** -0.5
        return {
            "q": ParamInfo((G * D, W), ("normal", std)), "q.conv": ParamInfo((G * D, taps), ("normal", 0.5)),
            "k": ParamInfo((G * D, W), ("normal", std)), "k.conv": ParamInfo((G * D, taps), ("normal", 0.5)),
            "v": ParamInfo((H * V, W), ("normal", std)), "v.conv": ParamInfo((H * V, taps), ("normal", 0.5)),
            "b": ParamInfo((H, W), ("normal", std)), "A_log": ParamInfo((H,), ("normal", 0.5)),
            "norm": ParamInfo((V,), ("one_plus_normal", 0.1)),
            "a1": ParamInfo((self.ra, W), ("normal", std), free_dims=(0,)),
            "a2": ParamInfo((H * D, self.ra), ("normal", self.ra ** -0.5), free_dims=(1,)),
            "dt_bias": ParamInfo((H * D,), ("normal_around", 1.0, -2.0)),
            "g1": ParamInfo((self.rg, W), ("normal", std), free_dims=(0,)),
            "g2": ParamInfo((H * V, self.rg), ("normal", self.rg ** -0.5), free_dims=(1,)),
            "o": ParamInfo((W, H * V), ("normal", (H * V) ** -0.5)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        a1, a2, g1, g2 = tensors["a1"], tensors["a2"], tensors["g1"], tensors["g2"]
        if a1.shape[0] != a2.shape[1] or g1.shape[0] != g2.shape[1]:
            raise ValueError("gated_delta: the inner sizes of the low-rank decay and gate products do not match")
        self.ra, self.rg = a1.shape[0], g1.shape[0]
        # columns of the fused product: q | k | v | zb | a1 | g1, the low-rank parts on 8-column boundaries
        self.off_b = self.filtered
        self.off_a = _pad8(self.off_b + s.num_heads)
        self.off_g = self.off_a + _pad8(self.ra)
        cols = self.off_g + _pad8(self.rg)
        W = a1.shape[1]
        w = torch.zeros((cols, W), dtype=a1.dtype, device=a1.device)
        at = 0
        for n in ("q", "k", "v", "b"):
            t = tensors[n]
            w[at: at + t.shape[0]] = t
            at += t.shape[0]
        w[self.off_a: self.off_a + self.ra] = a1
        w[self.off_g: self.off_g + self.rg] = g1
        self.w_in = w.contiguous()
        # the second halves of the two low-rank products as ONE product over the neighbouring columns a1 | g1 of the fused
        # sums: a block-diagonal matrix [H D + H V, pad8(ra) + pad8(rg)] (its zeros add exact zeros to the sums)
        self.k_ag = _pad8(self.ra) + _pad8(self.rg)
        w_ag = torch.zeros((a2.shape[0] + g2.shape[0], self.k_ag), dtype=a2.dtype, device=a2.device)
        w_ag[: a2.shape[0], : self.ra] = a2
        w_ag[a2.shape[0]:, _pad8(self.ra): _pad8(self.ra) + self.rg] = g2
        self.w_ag = w_ag.contiguous()
        self.conv_w = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0).contiguous()
        self.dt_bias = tensors["dt_bias"].contiguous()
        self.a_log = tensors["A_log"].to(self.dt_bias.dtype).contiguous()
        self.norm_w = tensors["norm"].contiguous()
        self.w_o = tensors["o"].contiguous()

    def state_needs(self) -> List[StateNeed]:
        s = self.spec
        needs = [StateNeed((s.num_heads, s.qk_dim * s.v_dim), "float32", phases=2)]
        if s.conv_taps > 1:
            needs.append(StateNeed((s.conv_taps - 1, self.filtered), "float32", phases=2))
        return needs

    def forward(self, x: torch.Tensor, ctx, binding: CacheBinding, out_dtype: Optional[torch.dtype] = None,
                out_scale: float = 1.0) -> torch.Tensor:
        s = self.spec
        H, G, D, V = s.num_heads, s.num_kv_heads, s.qk_dim, s.v_dim
        T = x.shape[0]
        z = linear(x, self.w_in, out_dtype=torch.float32)
        qkv = torch.empty((T, self.filtered), dtype=torch.float32, device=x.device)
        conv_state = ctx.cache.state_tensor(binding.states[1]) if s.conv_taps > 1 else None
        ops.short_conv_act(qkv, z[:, : self.filtered], self.conv_w, conv_state, ctx.cu_seqlens, ctx.token_req, ctx.state_slots,
                           ctx.state_phase, act="silu")
        ag = linear(z[:, self.off_a: self.off_a + self.k_ag], self.w_ag, out_dtype=torch.float32)
        decay, gate = ag[:, : H * D], ag[:, H * D:]
        o = torch.empty((T, H * V), dtype=torch.float32, device=x.device)
        ops.recurrent_scan(ops.SCAN_GATED_DELTA, o, qkv, (0, G * D, 2 * G * D), z, (self.off_b, 0),
                           ctx.cache.state_tensor(binding.states[0]), ctx, H, G, D, V, p0=self.dt_bias, p1=self.a_log, decay=decay,
                           q_scale=D ** -0.5)
        y = torch.empty((T, H * V), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(y, o, gate, self.norm_w, H, V, s.eps, weight_per_head=False)
        return linear(y, self.w_o, out_dtype=out_dtype)


@register_mixer("linear_attention")
class LinearAttention(Mixer):
    graph_safe = True
    takes_out_dtype = True

    def __init__(self, spec: LinearAttentionSpec) -> None:
        super().__init__(spec)
        s = spec
        if min(s.num_heads, s.qk_dim, s.v_dim) <= 0 or s.qk_dim > 512 or len(s.decays) != s.num_heads:
            raise ValueError(f"linear_attention: heads {s.num_heads}, dim {s.qk_dim} (at most 512), vdim {s.v_dim}, "
                             f"{len(s.decays)} decays (one per head)")
        H, D, V = s.num_heads, s.qk_dim, s.v_dim
        # columns of the fused product: q | k | v | output gate
        self.off = {"q": 0, "k": H * D, "v": 2 * H * D, "g": 2 * H * D + H * V}
        self.cols = 2 * H * D + 2 * H * V
        self.w_in: Optional[torch.Tensor] = None
        self.decays: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        H, D, V, W = s.num_heads, s.qk_dim, s.v_dim, s.hidden_size
        std = W ** -0.5
        return {s.q_name: ParamInfo((H * D, W), ("normal", std)), s.k_name: ParamInfo((H * D, W), ("normal", std)),
                s.v_name: ParamInfo((H * V, W), ("normal", std)), s.gate_name: ParamInfo((H * V, W), ("normal", std)),
                s.out_name: ParamInfo((W, H * V), ("normal", (H * V) ** -0.5)),
                s.norm_name: ParamInfo((H * V,), ("one_plus_normal", 0.1))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        w = torch.cat([tensors[n] for n in (s.q_name, s.k_name, s.v_name, s.gate_name)], dim=0)
        pad = _pad8(w.shape[0]) - w.shape[0]
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
        self.w_in = w.contiguous()
        self.w_o = tensors[s.out_name].contiguous()
        self.norm_w = tensors[s.norm_name].contiguous()

    def prepare(self, device: torch.device, dtype: torch.dtype) -> None:
        self.decays = torch.tensor([float(d) for d in self.spec.decays], dtype=torch.float64).to(torch.float32).to(device)

    def state_needs(self) -> List[StateNeed]:
        s = self.spec
        return [StateNeed((s.num_heads, s.qk_dim * s.v_dim), "float32", phases=2)]

    def forward(self, x: torch.Tensor, ctx, binding: CacheBinding, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        s = self.spec
        H, D, V = s.num_heads, s.qk_dim, s.v_dim
        z = linear(x, self.w_in, out_dtype=torch.float32)
        o = torch.empty((x.shape[0], H * V), dtype=torch.float32, device=x.device)
        ops.recurrent_scan(ops.SCAN_LINEAR_DECAY, o, z, (self.off["q"], self.off["k"], self.off["v"]), z, (0, 0),
                           ctx.cache.state_tensor(binding.states[0]), ctx, H, H, D, V, p0=self.decays)
        y = torch.empty((x.shape[0], H * V), dtype=x.dtype, device=x.device)
        # the norm runs over all heads together: one "head" of H * V numbers
        ops.head_norm_gate(y, o, z[:, self.off["g"]: self.off["g"] + H * V], self.norm_w, 1, H * V, s.eps, weight_per_head=True)
        return linear(y, self.w_o, out_dtype=out_dtype)
