"""Luzitar, written out plainly: one function per mechanism on whole sequences, slow, in float64 (or whatever type
the tensors come in). Shares no code with the package; the engine's tests compare against it.

Notation: W x is a matrix stored [out, in] applied to a column; t, i, j count positions from 0 in a sequence.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def dyt(x, p, name):
    """Dynamic tanh: tanh(alpha x) w + b, no mean and no variance."""
    return torch.tanh(p[name + ".alpha"] * x) * p[name] + p[name + ".b"]


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def causal_filter(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, C), dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j: j + T] * w[:, j]
    return y


def rotary_frequencies(rot: dict):
    """Frequencies of the pairs and the amplitude of cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, original, fast, slow = float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])

        def pair_of(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(pair_of(fast)), 0)
        hi = min(math.ceil(pair_of(slow)), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    return f, amp


def rotate(x, positions, rot: dict, interleaved: bool):
    """x [T, heads, d]: the first rot.dims numbers of every head are turned, the rest pass."""
    dims = int(rot["dims"])
    f, amp = rotary_frequencies(rot)
    ang = positions.to(torch.float64)[:, None] * f[None, :]
    cos, sin = (torch.cos(ang) * amp).to(x.dtype)[:, None, :], (torch.sin(ang) * amp).to(x.dtype)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2] = u * cos - v * sin
        out[..., dims // 2: dims] = v * cos + u * sin
    return out


def visible(T: int, window: Optional[int], keep_first: int):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def lightning(h, p, pre, m: dict, eps: float):
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ p[pre + "q"].T).view(T, H, D)
    k = silu(h @ p[pre + "k"].T).view(T, H, D)
    v = silu(h @ p[pre + "v"].T).view(T, H, V)
    out = torch.zeros((T, H, V), dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros((D, V), dtype=h.dtype)
        lam = float(m["decay"][hd])
        for t in range(T):
            S = lam * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    y = rms(out.reshape(T, H * V), eps, p[pre + "norm"]) * torch.sigmoid(h @ p[pre + "g"].T)
    return y @ p[pre + "o"].T


def attention(h, p, pre, m: dict, eps: float):
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)

    def proj(name):
        u = h @ p[pre + name].T + p[pre + name + ".b"]
        if m.get("conv"):
            u = causal_filter(u, p[pre + name + ".conv"])
        return u

    q, k, v = proj("q").view(T, H, D), proj("k").view(T, G, D), proj("v").view(T, G, V)
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"], False), rotate(k, pos, m["rot"], False)
    q, k = rms(q, eps), rms(k, eps)
    mask = m.get("mask") or {}
    ok = visible(T, int(mask["size"]) if mask.get("size") else None, int(mask.get("keep_first") or 0))
    out = torch.zeros((T, H, V), dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~ok, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * V) @ p[pre + "o"].T


def latent_and_key_part(h, p, pre, m: dict, eps: float):
    """What a latent layer caches per position: the normed latent and the rotated key part."""
    T = h.shape[0]
    R, P = int(m["kv_rank"]), int(m["rot_dim"])
    z = h @ p[pre + "dkv"].T
    c = rms(z[:, :R], eps, p[pre + "dkv.norm"])
    r = rotate(z[:, R: R + P].reshape(T, 1, P), torch.arange(T), m["rot"], True)[:, 0]
    return c, r


def latent_attention(h, p, pre, m: dict, eps: float, cached):
    T = h.shape[0]
    H, D, P, V, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    c, r = cached
    q = (h @ p[pre + "q"].T).view(T, H, D + P)
    qu = q[..., :D]
    qr = rotate(q[..., D:], torch.arange(T), m["rot"], True)
    ku = (c @ p[pre + "uk"].T).view(T, H, D)
    vv = (c @ p[pre + "uv"].T).view(T, H, V)
    ok = visible(T, None, 0)
    out = torch.zeros((T, H, V), dtype=h.dtype)
    for hd in range(H):
        s = (qu[:, hd] @ ku[:, hd].T + qr[:, hd] @ r.T) * float(m["scale"])
        s = s.masked_fill(~ok, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ vv[:, hd]
    return out.reshape(T, H * V) @ p[pre + "o"].T


def route(h, p, pre, router: dict, margins: Optional[list] = None):
    """Chosen experts [T, top] and their weights. ``margins`` collects, per row, how far the choice is from another one:
    the gap between the last chosen and the first unchosen choice score, and between the last kept and the first dropped
    group."""
    E, top = int(router["experts"]), int(router["top"])
    s = torch.sigmoid(h.to(torch.float64) @ p[pre + "router"].to(torch.float64).T)
    choice = s + p[pre + "correction"].to(torch.float64)
    margin = torch.full((h.shape[0],), float("inf"), dtype=torch.float64)
    groups = router.get("groups")
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        by_group = choice.view(-1, n, per)
        score = by_group.topk(min(2, per), dim=-1).values.sum(dim=-1)
        best = score.topk(keep, dim=-1).indices
        if keep < n:
            ranked = score.sort(dim=-1, descending=True).values
            margin = torch.minimum(margin, ranked[:, keep - 1] - ranked[:, keep])
        allowed = torch.zeros((h.shape[0], n), dtype=torch.bool)
        allowed.scatter_(1, best, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), float("-inf"))
    ids = choice.topk(top, dim=-1).indices
    ranked = choice.sort(dim=-1, descending=True).values
    if top < E:
        gap = ranked[:, top - 1] - ranked[:, top]
        margin = torch.minimum(margin, torch.where(torch.isfinite(ranked[:, top]), gap, torch.full_like(gap, float("inf"))))
    if margins is not None:
        margins.append(margin)
    w = s.gather(1, ids)
    w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    return ids, w.to(h.dtype)


def expert(h, p, pre, limit: float):
    g = torch.clamp(h @ p[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ p[pre + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ p[pre + "down"].T


def experts(h, p, pre, mlp: dict, margins: Optional[list] = None):
    ids, w = route(h, p, pre, mlp["router"], margins)
    out = torch.zeros_like(h)
    limit = float(mlp["expert"]["limit"])
    for t in range(h.shape[0]):
        for e, we in zip(ids[t].tolist(), w[t]):
            out[t] = out[t] + we * expert(h[t: t + 1], p, f"{pre}e{e}.", limit)[0]
    return out


def forward(cfg: dict, p: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None, dtype=torch.float64,
            round_to=None, margins: Optional[list] = None):
    """Logits [T, vocab] of one sequence in ``dtype``; ``layers_out`` collects the stream after every layer. ``round_to``:
    the sublayers' normed inputs are rounded to this type on the way (what a 16-bit engine does at least). ``margins``
    collects every routed layer's per-row distance from another choice."""
    p = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in p.items()}
    eps = float(cfg["norm"]["eps"])

    def dyt_in(x, name):
        h = dyt(x, p, name)
        return h.to(round_to).to(dtype) if round_to is not None else h
    x = dyt(p["embed"][torch.tensor(tokens)], p, "embed.norm")
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        m = layer["mixer"]
        h = dyt_in(x, pre + "norm1")
        if layer["type"] == "lightning":
            a = lightning(h, p, pre + "mix.", m, eps)
        elif layer["type"] == "attention":
            a = attention(h, p, pre + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                cached[i] = latent_and_key_part(h, p, pre + "mix.", m, eps)
                kv = cached[i]
            else:
                kv = cached[int(m["kv_from"])]
            a = latent_attention(h, p, pre + "mix.", m, eps, kv)
        else:
            raise ValueError(layer["type"])
        x = x + dyt(a, p, pre + "norm1b")
        if layer.get("mlp"):
            h = dyt_in(x, pre + "norm2")
            x = x + dyt(experts(h, p, pre + "mlp.", layer["mlp"], margins), p, pre + "norm2b")
        if layers_out is not None:
            layers_out.append(x.clone())
    x = dyt_in(x, "final.norm")
    logits = x @ p["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(logits / cap) if cap > 0 else logits
