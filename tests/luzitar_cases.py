"""Small Luzitar configurations for the tests, and what the tests share: model folders with random weights and the
float64 oracle of a whole sequence.

The configurations differ from one another in every size, and none of their sizes coincide by accident: key and value
sizes differ in both directions, head counts with and without grouping, rotated parts from two numbers to the whole head
with and without stretched waves, windows that straddle pages, of exactly a page and of one key, with none, one and many
kept first keys (also more than the window and more than a page), no window at all, one to five filter taps and none, latent
layers that read the cache of the layer before them or of one further back, one to four experts a row out of groups of
one to many experts with one or several groups kept or no groups at all, layers without a feed-forward, every order of the
three mixers. Softmax scales are about twice 1 / sqrt(dim): large enough that a key wrongly seen or missed moves the logits
far beyond rounding.
"""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List

import torch
from safetensors import safe_open


def lightning(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def attn(heads, kv_heads, dim, vdim, scale, window=None, keep_first=None, conv=None, rot=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if conv is not None:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = scaling
    return r


def latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, scaling=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot(rot_dim, base, scaling)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def moe(ff, experts, top, groups=None, limit=0.15):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}


STRETCH = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def model(vocab, width, layers, eps=1e-5, softcap=30.0):
    return {"architecture": "Luzitar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_softcap": softcap, "layers": layers}


# a latent layer first and a reader two layers behind it, values wider than keys, grouped heads, a window that straddles a
# page with kept keys that straddle another, three heads of linear attention, a layer without a feed-forward
CASE_A = model(211, 64, [
    latent(3, 16, 8, 24, 40, 0.4, base=10000.0, scaling=STRETCH, mlp=moe(24, 6, 2, groups=(3, 2))),
    attn(4, 2, 16, 24, 0.45, window=21, keep_first=19, conv=3, rot=rot(8, 1000.0, STRETCH), mlp=moe(16, 8, 3, groups=(2, 1), limit=0.05)),
    latent(2, 24, 8, 8, 40, 0.3, base=10000.0, scaling=STRETCH, kv_from=0, mlp=None),
    lightning(3, 8, 24, (0.5, 0.97, 1.0), mlp=moe(40, 3, 3)),
    attn(2, 2, 24, 8, 0.35, window=70, keep_first=3, conv=2, rot=rot(24, 50.0), mlp=moe(20, 5, 1)),
], eps=1e-5, softcap=12.0)
# linear attention first, attention without a window, without a filter, with one tap, without a rotation, without kept
# keys, with more kept keys than the window holds
CASE_B = model(97, 48, [
    lightning(2, 16, 8, (0.9, 0.99), mlp=moe(20, 4, 2, groups=(4, 3))),
    attn(3, 1, 16, 8, 0.5, window=16, keep_first=0, conv=1, rot=rot(16, 10000.0), mlp=moe(12, 2, 2, limit=0.4)),
    attn(6, 6, 8, 12, 0.6, rot=rot(4, 300.0), mlp=None),
    attn(2, 1, 40, 16, 0.3, window=1, keep_first=5, conv=5, mlp=moe(30, 12, 4, groups=(3, 2))),
    attn(2, 2, 8, 8, 0.7, window=6, keep_first=33, conv=2, rot=rot(2, 7.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5})),
], eps=1e-6, softcap=50.0)
# head sizes the tensor-core attention kernels take in bfloat16 (32, 64, 128), a window of exactly two pages, a wide latent
# with two readers, a wide linear attention
CASE_C = model(300, 128, [
    attn(6, 2, 32, 32, 0.3, window=32, keep_first=16, conv=4, rot=rot(16, 20000.0, {"factor": 2.0, "original": 128, "fast": 16.0, "slow": 2.0}),
         mlp=moe(48, 8, 3, groups=(2, 1))),
    latent(4, 32, 32, 32, 96, 0.25, base=1000000.0, mlp=moe(32, 6, 1, groups=(6, 2))),
    lightning(2, 64, 128, (0.8, 0.999), mlp=moe(64, 4, 2)),
    latent(2, 48, 32, 64, 96, 0.2, base=1000000.0, kv_from=1, mlp=None),
    attn(2, 1, 64, 64, 0.2, window=50, keep_first=1, conv=2, rot=rot(64, 10000.0), mlp=moe(64, 4, 2, groups=(1, 1))),
    latent(8, 16, 32, 16, 96, 0.3, base=1000000.0, kv_from=1, mlp=moe(16, 10, 4, groups=(5, 2))),
    attn(2, 2, 128, 128, 0.15, conv=3, rot=rot(32, 500.0), mlp=None),
], eps=1e-6, softcap=20.0)
# sizes that are multiples of nothing
CASE_D = model(101, 36, [
    attn(3, 1, 10, 6, 0.6, window=19, keep_first=7, conv=4, rot=rot(6, 100.0, {"factor": 8.0, "original": 32, "fast": 4.0, "slow": 0.5}),
         mlp=moe(14, 4, 4, groups=(2, 2))),
    lightning(5, 6, 10, (0.3, 0.6, 0.9, 0.95, 0.999), mlp=moe(50, 9, 2, groups=(3, 1))),
    latent(5, 6, 2, 10, 12, 0.7, base=100.0, scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 0.5}, mlp=moe(10, 7, 3)),
    latent(1, 20, 2, 12, 12, 0.4, base=100.0, scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 0.5}, kv_from=2, mlp=None),
    lightning(1, 20, 3, (0.75,), mlp=None),
], eps=1e-4, softcap=8.0)
# one layer of linear attention alone: a model without pages; a latent wider than 256 numbers with many experts
CASE_E = model(64, 80, [lightning(4, 12, 20, (0.2, 0.9, 0.99, 0.995), mlp=moe(16, 40, 2, groups=(8, 3)))], eps=1e-5, softcap=0.0)
CASE_F = model(64, 80, [latent(2, 24, 16, 16, 264, 0.35, base=10000.0, scaling=STRETCH, mlp=moe(16, 40, 2, groups=(8, 3)))], eps=1e-5)
CASES = {"A": (CASE_A, 31), "B": (CASE_B, 32), "C": (CASE_C, 33), "D": (CASE_D, 34), "E": (CASE_E, 35), "F": (CASE_F, 36)}


def make_folder(path: str, cfg: dict, seed: int) -> str:
    from openinfer_b200.config.base import resolve_architecture
    from openinfer_b200.weights import write_random_model

    config = resolve_architecture(cfg).config_cls.from_dict(cfg)
    write_random_model(config, path, seed)
    return path


def read_folder(path: str):
    with open(os.path.join(path, "config.json")) as fh:
        cfg = json.load(fh)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(path, "model.safetensors"), "pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return cfg, tensors


_ORACLE: Dict[tuple, tuple] = {}
CLOSE_CALL = 0.02       # a router's choice nearer than this to another one (in score units) may rightly fall either way in 16 bits


def _evaluate(path: str, tokens: List[int]):
    import plain_luzitar

    key = (path, tuple(tokens))
    if key not in _ORACLE:
        cfg, tensors = read_folder(path)
        margins: list = []
        logits = plain_luzitar.forward(cfg, tensors, list(tokens), dtype=torch.float64, margins=margins)
        size = logits.pow(2).mean().sqrt().item()
        # what rounding alone does in float32: the same formulas evaluated in float32
        single = plain_luzitar.forward(cfg, tensors, list(tokens), dtype=torch.float32).double()
        noise = (single - logits).abs().max().item() / size
        # and what 16-bit roundings of the sublayers' inputs alone do (float64 otherwise)
        half = plain_luzitar.forward(cfg, tensors, list(tokens), dtype=torch.float64, round_to=torch.bfloat16)
        noise16 = ((half - logits).abs().max().item() / size, (half - logits).abs().mean().item() / size)
        close = torch.stack(margins).min(dim=0).values < CLOSE_CALL if margins else torch.zeros(len(tokens), dtype=torch.bool)
        first_close = int(close.nonzero()[0]) if close.any() else len(tokens)
        _ORACLE[key] = (logits, noise, noise16, first_close)
    return _ORACLE[key]


def oracle(path: str, tokens: List[int]) -> torch.Tensor:
    """float64 logits [T, vocab] of the whole sequence by the plain implementation (cached per folder and sequence)."""
    return _evaluate(path, tokens)[0]


def float32_noise(path: str, tokens: List[int]) -> float:
    return _evaluate(path, tokens)[1]


def bfloat16_noise(path: str, tokens: List[int]):
    return _evaluate(path, tokens)[2]


def first_close_call(path: str, tokens: List[int]) -> int:
    """The first row at which some router's choice is a close call (the sequence's length if none is)."""
    return _evaluate(path, tokens)[3]


def tokens_for(cfg: dict, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(cfg["vocab"]) for _ in range(n)]


# Errors are measured against the root mean square of the reference logits of the sequence.
# float32 engine against the float64 oracle: 5e-5, or three times what rounding alone does to the plain implementation
# evaluated in float32 on that sequence where that is more.
F32_MAX_REL = 5e-5
F32_NOISE_FACTOR = 3.0
# bfloat16 engine: the bounds below, or four times what the roundings of the sublayers' inputs alone do to the float64
# plain implementation on that sequence where that is more (the engine rounds at more places: keys and values, the gate
# and up sums, the activations). Rows from a sequence's first close router call on are left out of the worst-row bound
# (the engine may rightly choose the other expert there, and state and cache carry the difference on), but of all rows at
# most one in ten may exceed it. One row in fifty (at least one) of the others may exceed it, by no more than half of it.
BF16_MAX_REL, BF16_MEAN_REL = 0.10, 0.02
BF16_NOISE_FACTOR = 4.0
BF16_ROWS_OVER, BF16_OVER_BY = 0.02, 1.5


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, noise: float = 0.0, noise16=(0.0, 0.0),
                  first_close: int = 1 << 30) -> None:
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    diff = (got - ref).abs()
    scale = ref.pow(2).mean().sqrt().item()
    worst, mean = diff.max().item() / scale, diff.mean().item() / scale
    row = int(diff.max(dim=1).values.argmax())
    if dtype == "float32":
        bound = max(F32_MAX_REL, F32_NOISE_FACTOR * noise)
        assert worst <= bound, f"{what}: float32 error {worst:.3e} of the logits' size (bound {bound:.3e}), worst row {row}"
    else:
        max_bound = max(BF16_MAX_REL, BF16_NOISE_FACTOR * noise16[0])
        mean_bound = max(BF16_MEAN_REL, BF16_NOISE_FACTOR * noise16[1])
        per_row = diff.max(dim=1).values / scale
        sure = per_row[:first_close]
        over = int((sure > max_bound).sum())
        assert (sure.numel() == 0 or sure.max().item() <= BF16_OVER_BY * max_bound) and over <= max(1, int(BF16_ROWS_OVER * sure.numel())), \
            f"{what}: bfloat16 error max {worst:.4f} (bound {max_bound:.4f}); worst row {row}, first close call {first_close}"
        assert int((per_row > max_bound).sum()) <= max(1, per_row.numel() // 10), f"{what}: bfloat16: more than one row in ten over {max_bound:.4f}"
        if first_close >= per_row.numel():
            assert mean <= mean_bound, f"{what}: bfloat16 mean error {mean:.5f} (bound {mean_bound:.5f})"
