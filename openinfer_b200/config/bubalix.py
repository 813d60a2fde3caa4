"""Bubalix configuration.

config.json of this design is nested: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, optionally
``token_side.dim`` (every layer then ends with a small input that depends on the token id), and one entry per layer
under ``layers``: ``type`` ("attention" or "latent_attention"), the mixer's sizes and constants under ``mixer`` and the
feed-forward under ``mlp`` (``kind`` "moe", or null for none).

An "attention" mixer has heads, kv_heads, dim, vdim and scale, and optionally ``conv`` (taps of a short filter over time
on q, k and v), ``q_temp`` (coef, every), ``softcap`` and ``mask.size`` (a sliding window). A "latent_attention" mixer has
heads, dim, rot_dim, vdim, kv_rank, scale and ``rot`` (dims, base, optional scaling with factor, original, fast, slow),
and optionally ``mask.size``. A "moe" feed-forward has ``expert.ff``, ``router.experts``, ``router.top`` and optionally
``shared.ff``. Every size comes from here or from a tensor's shape; nothing is assumed equal between layers.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig
from .delunex import _number, _positive_int
from .pilonex import _object

MIXER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("moe",)


@dataclasses.dataclass(frozen=True)
class BubalixConfig(ModelConfig):
    architecture = "Bubalix"
    model_type = ""

    vocab: int
    width: int
    layers: Tuple[dict, ...]
    norm: dict
    embedding: Optional[dict] = None
    token_side: Optional[dict] = None
    max_position_embeddings: int = 65536      # positions the rotation tables are made for
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"vocab and width must be positive, got {self.vocab} and {self.width}")
        if not isinstance(self.norm, dict) or not _number("norm", self.norm, "eps") > 0.0:
            raise ConfigError("norm.eps must be a number > 0")
        if self.embedding is not None:
            if not isinstance(self.embedding, dict):
                raise ConfigError("'embedding' must be an object")
            _number("embedding", self.embedding, "scale")
        if self.token_side is not None:
            if not isinstance(self.token_side, dict):
                raise ConfigError("'token_side' must be an object")
            _positive_int("token_side", self.token_side, "dim")
        if not self.layers:
            raise ConfigError("'layers' must list at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                raise ConfigError(f"{where}: an object with a 'mixer' object is expected")
            if layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}: type {layer.get('type')!r} is not known (known: {', '.join(MIXER_TYPES)})")
            m, mw = layer["mixer"], where + ".mixer"
            for key in ("heads", "dim", "vdim"):
                _positive_int(mw, m, key)
            _number(mw, m, "scale")
            if m.get("mask") is not None:
                _positive_int(mw + ".mask", _object(mw, m, "mask"), "size")
            if layer["type"] == "attention":
                heads, kv = _positive_int(mw, m, "heads"), _positive_int(mw, m, "kv_heads")
                if heads % kv:
                    raise ConfigError(f"{mw}: {heads} heads do not divide into {kv} kv_heads")
                if m.get("conv") is not None:
                    _positive_int(mw, m, "conv")
                if m.get("q_temp") is not None:
                    qt = _object(mw, m, "q_temp")
                    _number(mw + ".q_temp", qt, "coef")
                    _positive_int(mw + ".q_temp", qt, "every")
                if m.get("softcap") is not None and not _number(mw, m, "softcap") > 0.0:
                    raise ConfigError(f"{mw}: softcap must be > 0")
            else:
                for key in ("kv_rank", "rot_dim"):
                    _positive_int(mw, m, key)
                rot = _object(mw, m, "rot")
                dims = _positive_int(mw + ".rot", rot, "dims")
                if dims != int(m["rot_dim"]) or dims % 2:
                    raise ConfigError(f"{mw}: rot.dims {dims} must be even and equal rot_dim {m['rot_dim']}")
                if not _number(mw + ".rot", rot, "base") > 1.0:
                    raise ConfigError(f"{mw}.rot: base must be > 1")
                if rot.get("scaling") is not None:
                    sc = _object(mw + ".rot", rot, "scaling")
                    for key in ("factor", "original", "fast", "slow"):
                        if not _number(mw + ".rot.scaling", sc, key) > 0.0:
                            raise ConfigError(f"{mw}.rot.scaling: {key} must be > 0")
            mlp = layer.get("mlp")
            if mlp is not None:
                fw = where + ".mlp"
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"{fw}: kind must be one of {', '.join(MLP_KINDS)}, or the mlp null")
                _positive_int(fw + ".expert", _object(fw, mlp, "expert"), "ff")
                router = _object(fw, mlp, "router")
                experts, top = _positive_int(fw + ".router", router, "experts"), _positive_int(fw + ".router", router, "top")
                if top > experts:
                    raise ConfigError(f"{fw}.router: top {top} of {experts} experts")
                if mlp.get("shared") is not None:
                    _positive_int(fw + ".shared", _object(fw, mlp, "shared"), "ff")

    def with_stop_token_ids(self, ids) -> "BubalixConfig":
        return dataclasses.replace(self, stop_token_ids=tuple(int(i) for i in ids))

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding["scale"]) if self.embedding else 1.0

    @property
    def side_dim(self) -> int:
        return int(self.token_side["dim"]) if self.token_side else 0

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": dict(self.norm),
            "layers": [dict(layer) for layer in self.layers],
        }
        if self.embedding is not None:
            d["embedding"] = dict(self.embedding)
        if self.token_side is not None:
            d["token_side"] = dict(self.token_side)
        if self.max_position_embeddings != 65536:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d
