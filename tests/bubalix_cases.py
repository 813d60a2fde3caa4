"""Small Bubalix configurations for the tests, and what the tests share: model folders with random weights and the
float64 oracle of a whole sequence.

The configurations differ from one another in every size, and none of their sizes coincide by accident: key and value
sizes differ in both directions, head counts with and without grouping, rotated parts of several sizes with and without
stretched waves, windows that straddle pages and windows of one page and of one key, one to five filter taps and none, a
query temperature whose period is passed several times within a test's sequences, with and without a cap, one to three
experts a token, layers without a feed-forward, without a shared expert, models without a side input and without an
embedding scale. Softmax scales are about twice 1 / sqrt(dim): large enough that a key wrongly seen or missed moves the
logits far beyond rounding.
"""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List

import torch
from safetensors import safe_open


def attn(heads, kv_heads, dim, vdim, scale, window=None, conv=None, q_temp=None, softcap=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if conv is not None:
        m["conv"] = conv
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, scaling=None, window=None, mlp=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling is not None:
        rot["scaling"] = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def moe(ff, experts, top, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


STRETCH = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def model(vocab, width, layers, eps=1e-5, scale=None, side=None):
    cfg = {"architecture": "Bubalix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if scale is not None:
        cfg["embedding"] = {"scale": scale}
    if side is not None:
        cfg["token_side"] = {"dim": side}
    return cfg


# a latent layer first, values wider than keys, grouped heads, a window that straddles a page, two experts a token, a layer
# without a feed-forward, a temperature whose period is 32
CASE_A = model(211, 64, [
    latent(3, 16, 8, 24, 40, 0.4, base=10000.0, scaling=STRETCH, mlp=moe(24, 5, 2, shared=40)),
    attn(4, 2, 16, 24, 0.45, window=21, conv=3, q_temp=(0.4, 32), softcap=12.0, mlp=moe(16, 7, 1, shared=32)),
    attn(2, 2, 24, 8, 0.35, window=70, conv=2, softcap=5.0, mlp=None),
    latent(2, 24, 4, 8, 20, 0.3, base=500.0, mlp=moe(40, 3, 3)),
], eps=1e-5, scale=0.7, side=6)
# attention only, no side input, no embedding scale, no cap, no temperature in one layer, no filter in another, one tap in
# a third, no window in one
CASE_B = model(97, 48, [
    attn(3, 1, 16, 8, 0.5, window=16, conv=1, q_temp=(0.8, 10), mlp=moe(20, 4, 2)),
    attn(6, 6, 8, 12, 0.6, softcap=30.0, mlp=moe(12, 2, 2, shared=24)),
    attn(2, 1, 40, 16, 0.3, window=1, conv=5, mlp=None),
], eps=1e-6)
# head sizes the tensor-core attention kernels take in bfloat16 (32, 64, 128), a window of exactly two pages, a wide latent
CASE_C = model(300, 128, [
    attn(6, 2, 32, 32, 0.3, window=32, conv=4, q_temp=(0.5, 64), softcap=20.0, mlp=moe(48, 8, 3, shared=64)),
    latent(4, 32, 32, 32, 96, 0.25, base=1000000.0, scaling={"factor": 2.0, "original": 128, "fast": 16.0, "slow": 2.0}, mlp=moe(32, 6, 1, shared=48)),
    attn(2, 1, 64, 64, 0.2, window=50, conv=2, q_temp=(0.3, 100), mlp=moe(64, 4, 2)),
    attn(2, 2, 128, 128, 0.15, conv=3, softcap=8.0, mlp=None),
], eps=1e-6, scale=2.0, side=16)
# sizes that are multiples of nothing
CASE_D = model(101, 36, [
    attn(3, 1, 10, 6, 0.6, window=19, conv=4, q_temp=(1.0, 7), softcap=3.0, mlp=moe(14, 4, 4, shared=10)),
    latent(5, 6, 2, 10, 12, 0.7, base=100.0, scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 0.5}, window=33, mlp=moe(50, 9, 2)),
    latent(1, 20, 6, 12, 50, 0.4, base=50000.0, mlp=None),
], eps=1e-4, scale=0.25, side=5)
# a latent wider than 256 numbers, many experts, one layer
CASE_E = model(64, 80, [
    latent(2, 24, 16, 16, 264, 0.35, base=10000.0, scaling=STRETCH, mlp=moe(16, 40, 2, shared=8)),
], eps=1e-5, side=3)
CASES = {"A": (CASE_A, 31), "B": (CASE_B, 32), "C": (CASE_C, 33), "D": (CASE_D, 34), "E": (CASE_E, 35)}


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


def _evaluate(path: str, tokens: List[int]):
    import plain_bubalix

    key = (path, tuple(tokens))
    if key not in _ORACLE:
        cfg, tensors = read_folder(path)
        logits = plain_bubalix.forward(cfg, tensors, list(tokens), dtype=torch.float64)
        size = logits.pow(2).mean().sqrt().item()
        # what rounding alone does in float32: the same formulas evaluated in float32
        single = plain_bubalix.forward(cfg, tensors, list(tokens), dtype=torch.float32).double()
        noise = (single - logits).abs().max().item() / size
        # and what 16-bit roundings of the sublayers' inputs alone do (float64 otherwise)
        half = plain_bubalix.forward(cfg, tensors, list(tokens), dtype=torch.float64, round_to=torch.bfloat16)
        noise16 = ((half - logits).abs().max().item() / size, (half - logits).abs().mean().item() / size)
        _ORACLE[key] = (logits, noise, noise16)
    return _ORACLE[key]


def oracle(path: str, tokens: List[int]) -> torch.Tensor:
    """float64 logits [T, vocab] of the whole sequence by the plain implementation (cached per folder and sequence)."""
    return _evaluate(path, tokens)[0]


def float32_noise(path: str, tokens: List[int]) -> float:
    return _evaluate(path, tokens)[1]


def bfloat16_noise(path: str, tokens: List[int]):
    return _evaluate(path, tokens)[2]


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
# and up sums, the activations).
# One row in fifty (at least one) may exceed the worst-row bound, by no more than half of it: tiny random models now and
# then turn one rounded latent or key into a row's largest error.
BF16_MAX_REL, BF16_MEAN_REL = 0.10, 0.015
BF16_NOISE_FACTOR = 4.0
BF16_ROWS_OVER, BF16_OVER_BY = 0.02, 1.5


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, noise: float = 0.0, noise16=(0.0, 0.0)) -> None:
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
        over = int((per_row > max_bound).sum())
        assert worst <= BF16_OVER_BY * max_bound and over <= max(1, int(BF16_ROWS_OVER * per_row.numel())) and mean <= mean_bound, \
            f"{what}: bfloat16 error max {worst:.4f} (bound {max_bound:.4f}) mean {mean:.5f} (bound {mean_bound:.5f}); worst row {row}"
