"""Plain, slow Bubalix: every mechanism as one function over a whole sequence [T, ...], written from the design's
equations with dense matrices and explicit loops. It shares no code with the engine and keeps no cache: a sequence is
always evaluated from its first token.

Notation: W x for a matrix stored [out, in]; rms(x) = x / sqrt(mean(x^2) + eps).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def time_filter(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start. u [T, C], w [C, taps]."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def softmax_with_sink(scores: torch.Tensor, visible: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """Row-wise weights exp(s_j) / (exp(sink) + sum_visible exp(s_j)); the sink has no key: the weights sum to less than 1."""
    s = scores.masked_fill(~visible, -math.inf)
    top = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))


def visibility(T: int, window: Optional[int]) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    return seen


def distance_slopes(heads: int, dtype) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=dtype)


def query_temperature(T: int, coef: float, every: int, dtype) -> torch.Tensor:
    p = torch.arange(T, dtype=dtype)
    return 1.0 + coef * torch.log(torch.floor((p + 1.0) / every) + 1.0)


def scored_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int], sink: torch.Tensor,
                     cap: Optional[float] = None, slopes: Optional[torch.Tensor] = None, temperature: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V] of one sequence -> [T, H, V]. Head h reads key/value head h // (H / G). The
    score of (i, j) is (t_i q_i . k_j) * scale, capped as cap * tanh(s / cap), minus slope_h * (i - j); keys j <= i within the
    window; the softmax's denominator holds exp(sink_h) as well."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    if temperature is not None:
        q = q * temperature[:, None, None]
    seen = visibility(T, window)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(q.dtype)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        if slopes is not None:
            s = s - slopes[head] * dist
        out[:, head] = softmax_with_sink(s, seen, sink[head]) @ v[:, g]
    return out


def attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    """Grouped-query attention without rotation: filtered q, k, v; a temperature on q; capped scores; a distance bias;
    a window; a sink; one gate per head."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    if m.get("conv"):
        q, k, v = time_filter(q, W[p + "q.conv"]), time_filter(k, W[p + "k.conv"]), time_filter(v, W[p + "v.conv"])
    temperature = query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype) if m.get("q_temp") else None
    out = scored_attention(q.view(T, H, D), k.view(T, G, D), v.view(T, G, V), m["scale"], m["mask"]["size"] if m.get("mask") else None,
                           W[p + "sink"], m.get("softcap"), distance_slopes(H, h.dtype), temperature)
    out = out * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return out.reshape(T, H * V) @ W[p + "o"].T


def rotary_frequencies(rot: dict, dtype=torch.float64):
    """(frequencies [dims / 2], amplitude): plain f_i = base^(-2 i / dims); with scaling, f_i mixed with f_i / factor by a
    ramp over i, and an amplitude 0.1 ln(factor) + 1 on cos and sin."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def turns(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns(sc["fast"])), 0)
    hi = min(math.ceil(turns(sc["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, ..., dims]: dimension i pairs with i + dims / 2; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p f_i."""
    T, half = x.shape[0], rot["dims"] // 2
    f, amp = rotary_frequencies(rot, x.dtype)
    a = torch.arange(T, dtype=x.dtype)[:, None] * f[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [half]
    c, s = (torch.cos(a) * amp).view(shape), (torch.sin(a) * amp).view(shape)
    u, v = x[..., :half], x[..., half:]
    return torch.cat([u * c - v * s, v * c + u * s], dim=-1)


def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Keys and values up-projected from a normed latent, plus one rotated key part all heads share; a sink; one gate per
    output number."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ W[p + "q"].T).view(T, H, D + R)
    down = h @ W[p + "dkv"].T
    c = rms(down[:, :C], eps) * W[p + "dkv.norm"]
    k_rot = rotate(down[:, C:], m["rot"])
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], m["rot"])
    k_plain = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, V)
    seen = visibility(T, m["mask"]["size"] if m.get("mask") else None)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        out[:, head] = softmax_with_sink(s, seen, W[p + "sink"][head]) @ v[:, head]
    out = out.reshape(T, H * V) * torch.sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


def expert(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def table_experts(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict, tokens: List[int]) -> torch.Tensor:
    """Each token's experts come from a table by its id, each weighted 1 / top; plus an expert every token uses."""
    top = mlp["router"]["top"]
    out = torch.zeros_like(h)
    for t, tok in enumerate(tokens):
        for e in W[p + "table"][tok].tolist():
            out[t] += expert(h[t:t + 1], W, f"{p}e{int(e)}.")[0] / top
    if mlp.get("shared"):
        out = out + expert(h, W, p + "shared.")
    return out


def token_input(x: torch.Tensor, W: Dict[str, torch.Tensor], p: str, layer: int, dim: int, tokens: List[int], eps: float) -> torch.Tensor:
    e = W["side.embed"][torch.tensor(tokens)][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ W[p + "gate"].T) * e) @ W[p + "proj"].T
    return x + rms(y, eps) * W[p + "norm"]


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, streams: Optional[list] = None,
            round_to=None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence. ``streams``: a list that receives the stream after every layer.
    ``round_to``: the sublayers' common input is rounded to this type (what the 16-bit engine does at least)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v.long()) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)] * (cfg["embedding"]["scale"] if cfg.get("embedding") else 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, eps) * (1.0 + W[p + "norm1"])
        if round_to is not None:
            h = h.to(round_to).to(dtype)
        if layer["type"] == "attention":
            mixed = attention(h, W, p + "mix.", layer["mixer"])
        else:
            mixed = latent_attention(h, W, p + "mix.", layer["mixer"], eps)
        ff = table_experts(h, W, p + "mlp.", layer["mlp"], tokens) if layer.get("mlp") else 0.0
        x = x + (mixed + ff)
        if cfg.get("token_side"):
            x = token_input(x, W, p + "side.", i, cfg["token_side"]["dim"], tokens, eps)
        if streams is not None:
            streams.append(x.clone())
    x = rms(x, eps) * (1.0 + W["final.norm"])
    return x @ W["head"].T
