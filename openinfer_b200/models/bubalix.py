"""Bubalix: how a ``BubalixConfig`` becomes a ``ModelSpec``.

Every layer is a "shared_norm" block on a float32 stream: ONE norm (weight stored around zero, used as 1 + w) whose output
both the mixer and the feed-forward read, x <- x + (mixer(h) + ff(h)); then, when the model has a token side input, a small
gated product with a per-token embedding whose RMS-normed result is added. Layer types: "attention" (grouped-query, a short
causal filter on q, k and v, a query temperature, capped scores, a distance bias per head, a sliding window, a sink in the
softmax, one output gate per head; no rotation) and "latent_attention" (keys and values from a cached low-rank latent plus
one rotated key part shared by all heads, rotary waves stretched by a ramp, a sink, one output gate per output number).
The feed-forward is a set of experts chosen by the token id through a table, each weighted 1 / top, plus an expert every
token uses. Tensor names: ``embed``, ``head``, ``final.norm``, ``side.embed`` and per layer ``l<i>.`` + ``norm1``,
``mix.*``, ``mlp.*``, ``side.*``.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.bubalix import BubalixConfig
from ..parts.spec import (AttentionSpec, BlockSpec, GatedMlpSpec, LatentAttentionSpec, ModelSpec, NormSpec, PositionSpec,
                          RoutedExpertsSpec, TokenInputSpec)

DISTANCE_SLOPE_EXPONENT = 8.0     # head h of H takes 2^(-8 (h + 1) / H) * (i - j) off its scores


def _pad8(n: int) -> int:
    return (n + 7) & ~7


def _mixer(cfg: BubalixConfig, layer: dict, eps: float):
    W, m = cfg.width, layer["mixer"]
    window = int(m["mask"]["size"]) if m.get("mask") else None
    if layer["type"] == "attention":
        dim, vdim = int(m["dim"]), int(m["vdim"])
        qt = m.get("q_temp")
        return AttentionSpec(
            hidden_size=W, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=_pad8(max(dim, vdim)),
            softmax_scale=float(m["scale"]), position=PositionSpec(kind="none"), qk_norm=None, window=window, qk_dim=dim, v_dim=vdim,
            q_name="q", k_name="k", v_name="v", o_name="o", conv_taps=int(m.get("conv") or 0),
            q_temperature=(float(qt["coef"]), int(qt["every"])) if qt else None, score_cap=float(m.get("softcap") or 0.0),
            distance_slope_exponent=DISTANCE_SLOPE_EXPONENT, sink=True, head_gate=True)
    rot = m["rot"]
    sc = rot.get("scaling")
    position = PositionSpec(kind="rope", rotary_dim=int(rot["dims"]), theta=float(rot["base"]), max_positions=cfg.max_position_embeddings,
                            precise=True,
                            yarn=(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else None)
    return LatentAttentionSpec(
        hidden_size=W, num_heads=int(m["heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]), latent_rank=int(m["kv_rank"]),
        softmax_scale=float(m["scale"]), latent_norm=NormSpec(kind="rms", size=int(m["kv_rank"]), eps=eps), window=window,
        output_gate=True, gate_per="element", rope_dim=int(m["rot_dim"]), position=position, sink=True, out_name="o")


def _feed_forward(cfg: BubalixConfig, mlp):
    if not mlp:
        return None
    shared = mlp.get("shared")
    return RoutedExpertsSpec(
        hidden_size=cfg.width, intermediate_size=int(mlp["expert"]["ff"]), experts=int(mlp["router"]["experts"]),
        top=int(mlp["router"]["top"]), activation="silu", routing="table", vocab_size=cfg.vocab,
        shared=GatedMlpSpec(hidden_size=cfg.width, intermediate_size=int(shared["ff"]), activation="silu", gate_name="gate",
                            up_name="up", down_name="down") if shared else None)


def build_spec(cfg: BubalixConfig) -> ModelSpec:
    eps = float(cfg.norm["eps"])
    W = cfg.width
    norm = NormSpec(kind="rms", size=W, eps=eps, weight_offset=1.0, param_name="")
    side = cfg.side_dim
    blocks = []
    for i, layer in enumerate(cfg.layers):
        token_input = None
        if side:
            token_input = TokenInputSpec(hidden_size=W, dim=side, offset=i * side, vocab_size=cfg.vocab,
                                         table_width=side * len(cfg.layers), eps=eps)
        blocks.append(BlockSpec(
            kind="shared_norm", name=f"l{i}.", mixer=_mixer(cfg, layer, eps), feed_forward=_feed_forward(cfg, layer.get("mlp")),
            input_norm=norm, post_norm=None, mixer_name="mix.", feed_forward_name="mlp.", input_norm_name="norm1",
            token_input=token_input, token_input_name="side."))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W, blocks=tuple(blocks), order=tuple(range(len(blocks))), final_norm=norm,
        embedding_name="embed", final_norm_name="final.norm", head_name="head", max_positions=cfg.max_position_embeddings,
        stop_token_ids=tuple(cfg.stop_token_ids), embedding_scale=cfg.embedding_scale, residual_dtype="float32")


register_architecture(BubalixConfig.architecture, BubalixConfig, build_spec)
