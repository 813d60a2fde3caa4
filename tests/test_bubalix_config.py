"""Bubalix configuration and spec building (no GPU): keys, validation, tensor names and shapes, cache and state
registration, what the spec derives from the configuration, and the plain implementation's own mechanisms."""
import copy
import math

import pytest
import torch

import plain_bubalix as plain
from bubalix_cases import CASES, CASE_A, CASE_B, CASE_D, STRETCH, make_folder, read_folder, tokens_for

from openinfer_b200.cache.manager import CacheManager
from openinfer_b200.config.base import ConfigError, load_config, resolve_architecture
from openinfer_b200.parts.model import Model


def build(cfg):
    entry = resolve_architecture(cfg)
    config = entry.config_cls.from_dict(cfg)
    return config, entry.build_spec(config)


def test_registry_and_what_the_spec_takes_from_the_configuration():
    config, spec = build(CASE_A)
    assert type(config).__name__ == "BubalixConfig"
    assert spec.residual_dtype == "float32" and spec.embedding_scale == 0.7 and spec.vocab_size == 211 and spec.hidden_size == 64
    assert [b.kind for b in spec.blocks] == ["shared_norm"] * 4 and tuple(c.layer for c in spec.calls()) == (0, 1, 2, 3)
    lat, att, att2, lat2 = (b.mixer for b in spec.blocks)
    assert (lat.num_heads, lat.qk_dim, lat.rope_dim, lat.v_dim, lat.latent_rank) == (3, 16, 8, 24, 40)
    assert lat.softmax_scale == 0.4 and lat.sink and lat.output_gate and lat.gate_per == "element" and lat.window is None
    assert lat.position.yarn == (4.0, 64.0, 8.0, 1.0) and lat.position.theta == 10000.0 and lat.position.rotary_dim == 8
    assert lat2.position.yarn is None and lat2.position.theta == 500.0
    assert (att.num_heads, att.num_kv_heads, att.qk_dim, att.v_dim, att.window, att.conv_taps) == (4, 2, 16, 24, 21, 3)
    assert att.q_temperature == (0.4, 32) and att.score_cap == 12.0 and att.softmax_scale == 0.45 and att.sink and att.head_gate
    assert att.position.kind == "none" and att.qk_norm is None and att.head_dim % 8 == 0 and att.head_dim >= 24
    assert att2.q_temperature is None and att2.score_cap == 5.0 and att2.conv_taps == 2 and att2.window == 70
    ff = spec.blocks[0].feed_forward
    assert (ff.experts, ff.top, ff.intermediate_size, ff.routing, ff.shared.intermediate_size) == (5, 2, 24, "table", 40)
    assert spec.blocks[2].feed_forward is None and spec.blocks[3].feed_forward.shared is None
    assert [b.token_input.offset for b in spec.blocks] == [0, 6, 12, 18] and spec.blocks[0].token_input.table_width == 24
    plain_cfg, plain_spec = build(CASE_B)
    assert plain_spec.embedding_scale == 1.0 and all(b.token_input is None for b in plain_spec.blocks)
    assert plain_spec.blocks[1].mixer.conv_taps == 0 and plain_spec.blocks[1].mixer.window is None
    assert config.to_dict()["layers"][1]["mixer"]["q_temp"] == {"coef": 0.4, "every": 32}
    assert type(config).from_dict(config.to_dict()) == config


@pytest.mark.parametrize("name", list(CASES))
def test_tensor_names_and_shapes(name):
    cfg = CASES[name][0]
    _, spec = build(cfg)
    exp = Model(spec, torch.bfloat16).expected_tensors()
    W, n = cfg["width"], len(cfg["layers"])
    assert exp["embed"].shape == (cfg["vocab"], W) and exp["head"].shape == (cfg["vocab"], W) and exp["final.norm"].shape == (W,)
    side = cfg.get("token_side", {}).get("dim")
    assert ("side.embed" in exp) == bool(side)
    if side:
        assert exp["side.embed"].shape == (cfg["vocab"], side * n)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        assert exp[p + "norm1"].shape == (W,) and p + "norm2" not in exp
        H, D, V = m["heads"], m["dim"], m["vdim"]
        assert exp[p + "mix.sink"].shape == (H,) and exp[p + "mix.o"].shape == (W, H * V)
        if layer["type"] == "attention":
            G = m["kv_heads"]
            assert exp[p + "mix.q"].shape == (H * D, W) and exp[p + "mix.k"].shape == (G * D, W) and exp[p + "mix.v"].shape == (G * V, W)
            assert exp[p + "mix.g"].shape == (H, W)
            if m.get("conv"):
                taps = m["conv"]
                assert exp[p + "mix.q.conv"].shape == (H * D, taps) and exp[p + "mix.v.conv"].shape == (G * V, taps)
            else:
                assert p + "mix.q.conv" not in exp
        else:
            R, C = m["rot_dim"], m["kv_rank"]
            assert exp[p + "mix.q"].shape == (H * (D + R), W) and exp[p + "mix.dkv"].shape == (C + R, W)
            assert exp[p + "mix.dkv.norm"].shape == (C,) and exp[p + "mix.uk"].shape == (H * D, C) and exp[p + "mix.uv"].shape == (H * V, C)
            assert exp[p + "mix.g"].shape == (H * V, W)
        mlp = layer["mlp"]
        if mlp:
            E, F, top = mlp["router"]["experts"], mlp["expert"]["ff"], mlp["router"]["top"]
            assert exp[p + "mlp.table"].shape == (cfg["vocab"], top) and exp[p + "mlp.table"].integer
            assert exp[p + f"mlp.e{E - 1}.gate"].shape == (F, W) and exp[p + "mlp.e0.down"].shape == (W, F) and p + f"mlp.e{E}.up" not in exp
            assert (p + "mlp.shared.up" in exp) == bool(mlp.get("shared")) and p + "mlp.router" not in exp
            if mlp.get("shared"):
                assert exp[p + "mlp.shared.down"].shape == (W, mlp["shared"]["ff"])
        else:
            assert not any(k.startswith(p + "mlp.") for k in exp)
        if side:
            assert exp[p + "side.gate"].shape == (side, W) and exp[p + "side.proj"].shape == (W, side) and exp[p + "side.norm"].shape == (W,)


def test_random_folders_hold_what_the_design_stores(tmp_path):
    path = make_folder(str(tmp_path / "d"), CASE_D, 3)
    cfg, tensors = read_folder(path)
    assert cfg["architecture"] == "Bubalix" and cfg["layers"][0]["mixer"]["mask"] == {"size": 19}
    table = tensors["l0.mlp.table"]
    assert table.dtype == torch.int32 and table.shape == (101, 4) and int(table.min()) >= 0 and int(table.max()) < 4
    assert all(len(set(row)) == 4 for row in table.tolist())             # the entries of a row differ
    two = tensors["l1.mlp.table"]
    assert two.shape == (101, 2) and all(a != b for a, b in two.tolist()) and len({tuple(r) for r in two.tolist()}) > 10
    assert tensors["embed"].dtype == torch.bfloat16 and tensors["l1.mix.sink"].shape == (5,)
    config = load_config(path)
    model = Model(resolve_architecture(config.to_dict()).build_spec(config), torch.float32)
    from openinfer_b200.weights.loader import load_tensors
    loaded = load_tensors(path, model.expected_tensors(), torch.float32, "cpu")
    assert loaded["l0.mlp.table"].dtype == torch.int32 and loaded["l0.mix.q.conv"].dtype == torch.float32


def test_cache_and_state_registration():
    _, spec = build(CASE_A)
    model = Model(spec, torch.float32)
    cache = CacheManager(page_size=16)
    model.bind_cache(cache)
    kv = [b.kv for b in model.bindings]
    assert all(k is not None for k in kv) and len({(k.group, k.layer) for k in kv}) == 4
    windows = sorted((g.need.window is None, g.need.window) for g in cache.groups)
    assert windows == [(False, 21), (False, 70), (True, None), (True, None)] or windows == [(False, 21), (False, 70), (True, None)]
    # a latent layer caches one row of latent + rotated key part per token, padded to eight numbers
    rows = sorted(g.need.head_dim * g.need.num_kv_heads for g in cache.groups if g.need.window is None)
    assert rows[0] == 24 and rows[-1] == 48
    # attention layers with two or more taps keep taps - 1 projected rows of q | k | v; latent layers keep no state
    states = [len(b.states) for b in model.bindings]
    assert states == [0, 1, 1, 0]
    _, spec_b = build(CASE_B)
    model_b = Model(spec_b, torch.float32)
    model_b.bind_cache(CacheManager(page_size=16))
    assert [len(b.states) for b in model_b.bindings] == [0, 0, 1]        # one tap and no filter carry nothing


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "recurrent"), "type"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 6), "rot"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "dense"), "kind"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].__setitem__("every", 0), "every"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("softcap", -1.0), "softcap"),
    (lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c["norm"].__setitem__("eps", 0), "eps"),
    (lambda c: c.__setitem__("token_side", {"dim": 0}), "dim"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_bad_configs_are_refused(change, message):
    cfg = copy.deepcopy(CASE_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        build(cfg)


# ------------------------------------------------------------------------------- the plain implementation's own mechanisms
def test_plain_softmax_with_sink_and_visibility():
    s = torch.tensor([[0.3, -1.0, 2.0]], dtype=torch.float64)
    seen = torch.tensor([[True, False, True]])
    w = plain.softmax_with_sink(s, seen, torch.tensor(0.5, dtype=torch.float64))
    den = math.exp(0.3) + math.exp(2.0) + math.exp(0.5)
    assert torch.allclose(w, torch.tensor([[math.exp(0.3) / den, 0.0, math.exp(2.0) / den]], dtype=torch.float64))
    assert w.sum().item() < 1.0
    v = plain.visibility(6, 3)
    assert v[5].tolist() == [False, False, False, True, True, True] and v[1].tolist() == [True, True, False, False, False, False]
    assert plain.visibility(4, None)[3].all() and plain.visibility(4, 1).sum().item() == 4


def test_plain_filter_temperature_and_slopes():
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None].repeat(1, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    y = plain.time_filter(u, w)
    assert y[:, 0].tolist() == [100.0, 210.0, 321.0, 432.0, 543.0] and y[:, 1].tolist() == [1.0, 2.0, 3.0, 4.0, 5.0]
    t = plain.query_temperature(10, 0.5, 4, torch.float64)
    assert t[2] == 1.0 and abs(t[3].item() - (1 + 0.5 * math.log(2.0))) < 1e-12 and t[6] == t[3] and abs(t[7].item() - (1 + 0.5 * math.log(3.0))) < 1e-12
    sl = plain.distance_slopes(4, torch.float64)
    assert sl.tolist() == [2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8]


def test_plain_stretched_frequencies_and_rotation():
    """Short waves keep their frequency, long ones are divided by the factor, the ones between are mixed; cos and sin
    carry the amplitude; the rotation keeps lengths (times the amplitude) and its scores depend on distance alone."""
    rot = {"dims": 16, "base": 10000.0, "scaling": STRETCH}
    raw = 10000.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
    f, amp = plain.rotary_frequencies(rot)
    assert abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    ratio = (f / raw).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 0.25) < 1e-12 and any(0.25 < r < 1.0 for r in ratio)
    assert all(a >= b for a, b in zip(ratio, ratio[1:]))
    f0, amp0 = plain.rotary_frequencies({"dims": 16, "base": 10000.0})
    assert amp0 == 1.0 and torch.equal(f0, raw)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, 2, 16, generator=g, dtype=torch.float64)
    y = plain.rotate(x, rot)
    assert torch.allclose(y.norm(dim=-1), amp * x.norm(dim=-1))
    q = plain.rotate(x[:1].expand(9, 2, 16).contiguous(), rot)
    assert abs((q[3, 0] * q[1, 1]).sum().item() - (q[8, 0] * q[6, 1]).sum().item()) < 1e-9


def test_plain_forward_is_causal_and_every_mechanism_moves_the_logits(tmp_path):
    path = make_folder(str(tmp_path / "a"), CASE_A, 5)
    cfg, tensors = read_folder(path)
    toks = tokens_for(cfg, 50, 3)
    ref = plain.forward(cfg, tensors, toks)
    assert ref.shape == (50, cfg["vocab"]) and torch.isfinite(ref).all()
    assert torch.allclose(plain.forward(cfg, tensors, toks[:20]), ref[:20], atol=1e-10)
    size = ref.pow(2).mean().sqrt().item()

    def moved(change_cfg=None, change_tensors=None):
        c, t = copy.deepcopy(cfg), dict(tensors)
        if change_cfg:
            change_cfg(c)
        if change_tensors:
            change_tensors(t)
        return (plain.forward(c, t, toks) - ref).abs().max().item() / size

    # random weights keep the scores far below the cap: with the queries thirty times as long it bites
    sharp = dict(tensors)
    sharp["l1.mix.q"] = tensors["l1.mix.q"] * 30.0
    no_cap = copy.deepcopy(cfg)
    no_cap["layers"][1]["mixer"].pop("softcap")
    assert (plain.forward(no_cap, sharp, toks) - plain.forward(cfg, sharp, toks)).abs().max().item() / size > 1e-3
    assert moved(lambda c: c["layers"][1]["mixer"].pop("q_temp")) > 1e-4
    assert moved(lambda c: c["layers"][1]["mixer"].pop("conv")) > 1e-3
    assert moved(lambda c: c["layers"][0]["mixer"]["rot"].pop("scaling")) > 1e-4
    assert moved(lambda c: c.pop("token_side")) > 1e-3
    assert moved(lambda c: c["layers"][0]["mlp"].pop("shared")) > 1e-3
    assert moved(None, lambda t: t.__setitem__("l0.mix.sink", t["l0.mix.sink"] - 30.0)) > 1e-4
    assert moved(None, lambda t: t.__setitem__("l1.mix.sink", t["l1.mix.sink"] - 30.0)) > 1e-4
    assert moved(None, lambda t: t.__setitem__("l0.mlp.table", (t["l0.mlp.table"] + 1) % 5)) > 1e-3
