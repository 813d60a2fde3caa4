"""Luzitar configuration.

config.json of this design is nested: ``vocab``, ``width``, ``norm.eps``, ``logit_softcap`` and one entry per layer under
``layers``: ``type`` ("lightning", "attention" or "latent_attention"), the mixer's sizes and constants under ``mixer`` and
the feed-forward under ``mlp`` (``kind`` "moe", or null for none).

A "lightning" mixer has heads, dim, vdim and ``decay`` (one number per head). An "attention" mixer has heads, kv_heads,
dim, vdim and scale, and optionally ``conv`` (taps of a short filter over time on q, k and v), ``rot`` (dims, base, optional
scaling with factor, original, fast, slow) and ``mask`` (size, optionally keep_first). A "latent_attention" mixer has heads,
dim, rot_dim, vdim, kv_rank, scale and ``rot`` (dims = rot_dim, base, optional scaling), and either a down-projection of its
own or ``kv_from``: the index of an earlier latent layer whose cached latent and key part it reads. A "moe" feed-forward
has ``expert.ff``, ``expert.limit``, ``router.experts``, ``router.top`` and optionally ``router.groups`` (count, keep). Every
size comes from here or from a tensor's shape; nothing is assumed equal between layers.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Tuple

from .base import ConfigError, ModelConfig
from .delunex import _number, _positive_int
from .pilonex import _object

MIXER_TYPES = ("lightning", "attention", "latent_attention")
MLP_KINDS = ("moe",)


def _rotation(where: str, rot: Dict[str, Any]) -> int:
    dims = _positive_int(where, rot, "dims")
    if dims % 2:
        raise ConfigError(f"{where}: dims {dims} must be even")
    if not _number(where, rot, "base") > 1.0:
        raise ConfigError(f"{where}: base must be > 1")
    if rot.get("scaling") is not None:
        sc = _object(where, rot, "scaling")
        for key in ("factor", "original", "fast", "slow"):
            if not _number(where + ".scaling", sc, key) > 0.0:
                raise ConfigError(f"{where}.scaling: {key} must be > 0")
    return dims


@dataclasses.dataclass(frozen=True)
class LuzitarConfig(ModelConfig):
    architecture = "Luzitar"
    model_type = ""

    vocab: int
    width: int
    layers: Tuple[dict, ...]
    norm: dict
    logit_softcap: float = 0.0
    max_position_embeddings: int = 65536      # positions the rotation tables are made for
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"vocab and width must be positive, got {self.vocab} and {self.width}")
        if not isinstance(self.norm, dict) or not _number("norm", self.norm, "eps") > 0.0:
            raise ConfigError("norm.eps must be a number > 0")
        if isinstance(self.logit_softcap, bool) or not isinstance(self.logit_softcap, (int, float)) or self.logit_softcap < 0:
            raise ConfigError(f"logit_softcap must be a number >= 0, got {self.logit_softcap!r}")
        if not self.layers:
            raise ConfigError("'layers' must list at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                raise ConfigError(f"{where}: an object with a 'mixer' object is expected")
            if layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}: type {layer.get('type')!r} is not known (known: {', '.join(MIXER_TYPES)})")
            m, mw = layer["mixer"], where + ".mixer"
            heads = _positive_int(mw, m, "heads")
            for key in ("dim", "vdim"):
                _positive_int(mw, m, key)
            if layer["type"] == "lightning":
                decay = m.get("decay")
                if isinstance(decay, (int, float)) and not isinstance(decay, bool):
                    decay = [decay] * heads                  # one number for all heads
                if not isinstance(decay, (list, tuple)) or len(decay) != heads or any(
                        isinstance(d, bool) or not isinstance(d, (int, float)) or not 0.0 <= d <= 1.0 for d in decay):
                    raise ConfigError(f"{mw}: 'decay' must list one number in [0, 1] per head ({heads})")
            elif layer["type"] == "attention":
                _number(mw, m, "scale")
                kv = _positive_int(mw, m, "kv_heads")
                if heads % kv:
                    raise ConfigError(f"{mw}: {heads} heads do not divide into {kv} kv_heads")
                if m.get("conv") is not None:
                    _positive_int(mw, m, "conv")
                if m.get("rot") is not None:
                    if _rotation(mw + ".rot", _object(mw, m, "rot")) > int(m["dim"]):
                        raise ConfigError(f"{mw}: rot.dims is larger than dim")
                if m.get("mask") is not None:
                    mask = _object(mw, m, "mask")
                    _positive_int(mw + ".mask", mask, "size")
                    kf = mask.get("keep_first")
                    if kf is not None and (isinstance(kf, bool) or not isinstance(kf, int) or kf < 0):
                        raise ConfigError(f"{mw}.mask: keep_first must be an integer >= 0, got {kf!r}")
            else:
                _number(mw, m, "scale")
                for key in ("kv_rank", "rot_dim"):
                    _positive_int(mw, m, key)
                if _rotation(mw + ".rot", _object(mw, m, "rot")) != int(m["rot_dim"]):
                    raise ConfigError(f"{mw}: rot.dims must equal rot_dim {m['rot_dim']}")
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise ConfigError(f"{mw}: kv_from must name an earlier layer, got {src!r}")
                    other = self.layers[src]
                    if other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{mw}: kv_from {src} is not a latent layer with a down-projection of its own")
                    if any(other["mixer"].get(k) != m.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                        raise ConfigError(f"{mw}: kv_rank, rot_dim and rot must equal those of layer {src}")
            mlp = layer.get("mlp")
            if mlp is not None:
                fw = where + ".mlp"
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"{fw}: kind must be one of {', '.join(MLP_KINDS)}, or the mlp null")
                ex = _object(fw, mlp, "expert")
                _positive_int(fw + ".expert", ex, "ff")
                if not _number(fw + ".expert", ex, "limit") > 0.0:
                    raise ConfigError(f"{fw}.expert: limit must be > 0")
                router = _object(fw, mlp, "router")
                experts, top = _positive_int(fw + ".router", router, "experts"), _positive_int(fw + ".router", router, "top")
                count, keep = 1, 1
                if router.get("groups") is not None:
                    groups = _object(fw + ".router", router, "groups")
                    count, keep = _positive_int(fw + ".router.groups", groups, "count"), _positive_int(fw + ".router.groups", groups, "keep")
                if keep > count or experts % count or (experts // count) * keep < top:
                    raise ConfigError(f"{fw}.router: {experts} experts in {count} groups of which {keep} are kept cannot give {top} choices")

    def with_stop_token_ids(self, ids) -> "LuzitarConfig":
        return dataclasses.replace(self, stop_token_ids=tuple(int(i) for i in ids))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": dict(self.norm),
            "logit_softcap": self.logit_softcap, "layers": [dict(layer) for layer in self.layers],
        }
        if self.max_position_embeddings != 65536:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d
