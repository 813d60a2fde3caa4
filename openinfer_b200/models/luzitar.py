"""Luzitar: how a ``LuzitarConfig`` becomes a ``ModelSpec``.

The embedded rows pass a Dynamic Tanh norm (tanh(alpha x) w + b); every layer is a "sandwich" block on a float32 stream,
x <- x + norm1b(mixer(norm1(x))), x <- x + norm2b(ff(norm2(x))), all four norms Dynamic Tanh; the final norm is one too,
and the logits are soft-capped. Layer types: "lightning" (linear attention with a fixed decay per head and a gated,
RMS-normed read-out), "attention" (grouped-query, biases on q, k and v, a short causal filter on them, a rotation of part of
each head in pairs (d, d + half) with ramp-stretched waves, a unit norm of q and k behind the rotation, a sliding window that
keeps the sequence's first keys) and "latent_attention" (keys and values from a cached low-rank latent plus one rotated key
part shared by all heads, pairs (2 d, 2 d + 1); a layer may read an earlier layer's cache). The feed-forward is a set of
routed experts (clamped gated activation) chosen by sigmoid scores with a correction, restricted to the best groups.
Tensor names: ``embed``, ``embed.norm``, ``head``, ``final.norm`` and per layer ``l<i>.`` + ``norm1``, ``norm1b``, ``norm2``,
``norm2b``, ``mix.*``, ``mlp.*``; a norm's bias and alpha lie beside its weight as ``<name>.b`` and ``<name>.alpha``.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.luzitar import LuzitarConfig
from ..parts.spec import (AttentionSpec, BlockSpec, LatentAttentionSpec, LayerCall, LinearAttentionSpec, ModelSpec, NormSpec,
                          PositionSpec, RoutedExpertsSpec)


def _pad8(n: int) -> int:
    return (n + 7) & ~7


def _position(cfg: LuzitarConfig, rot, interleaved: bool) -> PositionSpec:
    if not rot:
        return PositionSpec(kind="none")
    sc = rot.get("scaling")
    return PositionSpec(kind="rope", rotary_dim=int(rot["dims"]), theta=float(rot["base"]), max_positions=cfg.max_position_embeddings,
                        interleaved=interleaved, precise=True,
                        yarn=(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else None)


def _mixer(cfg: LuzitarConfig, layer: dict, eps: float):
    W, m = cfg.width, layer["mixer"]
    if layer["type"] == "lightning":
        decay = m["decay"] if isinstance(m["decay"], (list, tuple)) else [m["decay"]] * int(m["heads"])
        return LinearAttentionSpec(hidden_size=W, num_heads=int(m["heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]),
                                   decays=tuple(float(d) for d in decay), eps=eps)
    if layer["type"] == "attention":
        dim, vdim = int(m["dim"]), int(m["vdim"])
        mask = m.get("mask") or {}
        return AttentionSpec(
            hidden_size=W, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=_pad8(max(dim, vdim)),
            softmax_scale=float(m["scale"]), position=_position(cfg, m.get("rot"), False), qk_norm=None,
            window=int(mask["size"]) if mask.get("size") else None, qk_dim=dim, v_dim=vdim, q_name="q", k_name="k", v_name="v",
            o_name="o", conv_taps=int(m.get("conv") or 0), qkv_bias=True, unit_norm_after_rotation_eps=eps,
            keep_first=int(mask.get("keep_first") or 0))
    return LatentAttentionSpec(
        hidden_size=W, num_heads=int(m["heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]), latent_rank=int(m["kv_rank"]),
        softmax_scale=float(m["scale"]), latent_norm=NormSpec(kind="rms", size=int(m["kv_rank"]), eps=eps), window=None,
        output_gate=False, has_latent=m.get("kv_from") is None, rope_dim=int(m["rot_dim"]), position=_position(cfg, m["rot"], True),
        out_name="o")


def _feed_forward(cfg: LuzitarConfig, mlp):
    if not mlp:
        return None
    router = mlp["router"]
    groups = router.get("groups") or {}
    return RoutedExpertsSpec(
        hidden_size=cfg.width, intermediate_size=int(mlp["expert"]["ff"]), experts=int(router["experts"]), top=int(router["top"]),
        activation="swiglu_clamp", limit=float(mlp["expert"]["limit"]), routing="sigmoid_groups",
        groups=int(groups.get("count") or 1), keep_groups=int(groups.get("keep") or 1))


def build_spec(cfg: LuzitarConfig) -> ModelSpec:
    eps = float(cfg.norm["eps"])
    W = cfg.width
    norm = NormSpec(kind="dyt", size=W, eps=eps, param_name="")
    blocks, order = [], []
    for i, layer in enumerate(cfg.layers):
        ff = _feed_forward(cfg, layer.get("mlp"))
        blocks.append(BlockSpec(
            kind="sandwich", name=f"l{i}.", mixer=_mixer(cfg, layer, eps), feed_forward=ff, input_norm=norm, mixer_out_norm=norm,
            post_norm=norm if ff is not None else None, feed_forward_out_norm=norm if ff is not None else None,
            mixer_name="mix.", feed_forward_name="mlp.", input_norm_name="norm1", post_norm_name="norm2",
            mixer_out_norm_name="norm1b", feed_forward_out_norm_name="norm2b"))
        src = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
        order.append(LayerCall(i, read_cache_of=int(src)) if src is not None else i)
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W, blocks=tuple(blocks), order=tuple(order), final_norm=norm, embedding_name="embed",
        final_norm_name="final.norm", head_name="head", max_positions=cfg.max_position_embeddings,
        stop_token_ids=tuple(cfg.stop_token_ids), logit_soft_cap=float(cfg.logit_softcap), residual_dtype="float32",
        embedding_norm=norm, embedding_norm_name="embed.norm",
        embedding_init=("normal", 1.0))      # random weights: rows that the norm behind the table tells apart


register_architecture(LuzitarConfig.architecture, LuzitarConfig, build_spec)
