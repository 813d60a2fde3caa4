"""Luzitar configuration and spec building (no GPU): keys, validation, tensor names and shapes, cache and state
registration, pages kept for a sequence's first keys, and the plain implementation's own mechanisms."""
import copy
import math

import pytest
import torch

import plain_luzitar as plain
from luzitar_cases import CASES, CASE_A, CASE_B, CASE_D, CASE_E, STRETCH, make_folder, read_folder, tokens_for

from openinfer_b200.cache.manager import RELEASED, CacheManager, KvNeed
from openinfer_b200.config.base import ConfigError, load_config, resolve_architecture
from openinfer_b200.parts.model import Model


def build(cfg):
    entry = resolve_architecture(cfg)
    config = entry.config_cls.from_dict(cfg)
    return config, entry.build_spec(config)


def test_registry_and_what_the_spec_takes_from_the_configuration():
    config, spec = build(CASE_A)
    assert type(config).__name__ == "LuzitarConfig"
    assert spec.residual_dtype == "float32" and spec.logit_soft_cap == 12.0 and spec.vocab_size == 211 and spec.hidden_size == 64
    assert spec.embedding_norm.kind == "dyt" and spec.final_norm.kind == "dyt"
    assert [b.kind for b in spec.blocks] == ["sandwich"] * 5
    calls = spec.calls()
    assert [c.layer for c in calls] == [0, 1, 2, 3, 4] and [c.read_cache_of for c in calls] == [None, None, 0, None, None]
    lat, att, reader, lin, att2 = (b.mixer for b in spec.blocks)
    assert (lat.num_heads, lat.qk_dim, lat.rope_dim, lat.v_dim, lat.latent_rank, lat.has_latent) == (3, 16, 8, 24, 40, True)
    assert lat.position.interleaved and lat.position.yarn == (4.0, 64.0, 8.0, 1.0) and not lat.sink and not lat.output_gate and lat.window is None
    assert (reader.num_heads, reader.qk_dim, reader.v_dim, reader.has_latent) == (2, 24, 8, False)
    assert (att.num_heads, att.num_kv_heads, att.qk_dim, att.v_dim, att.window, att.keep_first, att.conv_taps) == (4, 2, 16, 24, 21, 19, 3)
    assert att.qkv_bias and att.unit_norm_after_rotation_eps == 1e-5 and att.qk_norm is None and not att.position.interleaved
    assert att.position.rotary_dim == 8 and att.position.yarn == (4.0, 64.0, 8.0, 1.0) and att.head_dim % 8 == 0 and att.head_dim >= 24
    assert att2.position.yarn is None and att2.position.theta == 50.0 and att2.keep_first == 3
    assert (lin.kind, lin.num_heads, lin.qk_dim, lin.v_dim, lin.decays) == ("linear_attention", 3, 8, 24, (0.5, 0.97, 1.0))
    ff = spec.blocks[0].feed_forward
    assert (ff.experts, ff.top, ff.intermediate_size, ff.routing, ff.groups, ff.keep_groups, ff.limit) == (6, 2, 24, "sigmoid_groups", 3, 2, 0.15)
    assert spec.blocks[1].feed_forward.limit == 0.05 and spec.blocks[2].feed_forward is None
    assert (spec.blocks[3].feed_forward.groups, spec.blocks[3].feed_forward.keep_groups) == (1, 1)
    _, spec_b = build(CASE_B)
    assert spec_b.blocks[2].mixer.window is None and spec_b.blocks[2].mixer.conv_taps == 0 and spec_b.blocks[3].mixer.position.kind == "none"
    assert type(config).from_dict(config.to_dict()) == config
    assert build(CASE_E)[1].logit_soft_cap == 0.0


@pytest.mark.parametrize("name", list(CASES))
def test_tensor_names_and_shapes(name):
    cfg = CASES[name][0]
    _, spec = build(cfg)
    exp = Model(spec, torch.bfloat16).expected_tensors()
    W = cfg["width"]
    want = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W)}

    def norm(n):
        want[n], want[n + ".b"], want[n + ".alpha"] = (W,), (W,), ()

    norm("embed.norm"), norm("final.norm")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        norm(p + "norm1"), norm(p + "norm1b")
        H, D, V = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "lightning":
            want.update({p + "mix.q": (H * D, W), p + "mix.k": (H * D, W), p + "mix.v": (H * V, W), p + "mix.g": (H * V, W),
                         p + "mix.o": (W, H * V), p + "mix.norm": (H * V,)})
        elif layer["type"] == "attention":
            G = m["kv_heads"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                want[p + "mix." + n], want[p + "mix." + n + ".b"] = (rows, W), (rows,)
                if m.get("conv"):
                    want[p + "mix." + n + ".conv"] = (rows, m["conv"])
            want[p + "mix.o"] = (W, H * V)
        else:
            R, P = m["kv_rank"], m["rot_dim"]
            want.update({p + "mix.q": (H * (D + P), W), p + "mix.uk": (H * D, R), p + "mix.uv": (H * V, R), p + "mix.o": (W, H * V)})
            if m.get("kv_from") is None:
                want.update({p + "mix.dkv": (R + P, W), p + "mix.dkv.norm": (R,)})
        mlp = layer.get("mlp")
        if mlp:
            norm(p + "norm2"), norm(p + "norm2b")
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            want[p + "mlp.router"], want[p + "mlp.correction"] = (E, W), (E,)
            for e in range(E):
                want.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
    assert {k: tuple(v.shape) for k, v in exp.items()} == want


def test_random_folders_load_back(tmp_path):
    path = make_folder(str(tmp_path / "m"), CASE_D, 3)
    cfg, tensors = read_folder(path)
    assert cfg["architecture"] == "Luzitar" and load_config(path).width == 36
    assert tensors["l0.norm1.alpha"].shape == () and tensors["l1.mix.norm"].shape == (50,)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())


def test_cache_and_state_registration():
    _, spec = build(CASE_A)
    model = Model(spec, torch.bfloat16)
    cache = CacheManager(page_size=16)
    model.bind_cache(cache)
    needs = [g.need for g in cache.groups]
    # the latent (read by layer 2 as well: one layer of pages), and the two attention layers with their windows and kept keys
    assert KvNeed(1, 48, None, planes=1) in needs
    assert KvNeed(2, 24, 21, keep_first=19) in needs and KvNeed(2, 24, 70, keep_first=3) in needs
    assert model.bindings[2].kv == model.bindings[0].kv and not model.bindings[2].owns_kv and model.bindings[0].owns_kv
    shapes = sorted(n.shape for n in cache.state_needs)
    # filter states of the two attention layers (taps - 1 rows of q | k | v columns), the linear attention's matrices
    assert shapes == sorted([(2, 4 * 24 + 2 * 2 * 24), (1, 2 * 24 + 2 * 2 * 24), (3, 8 * 24)])
    assert all(n.phases == 2 and n.dtype == "float32" for n in cache.state_needs)
    lone = Model(build(CASE_E)[1], torch.bfloat16)
    cache = CacheManager(page_size=16)
    lone.bind_cache(cache)
    assert cache.groups == [] and len(cache.state_needs) == 1


def test_pages_of_kept_first_keys_are_never_given_back():
    """A window of 20 keys that keeps the first 19 (two pages of 16): pages behind the window go back, the first two stay;
    without kept keys they go too."""
    for keep, stay in ((19, 2), (16, 1), (0, 0), (1, 1)):
        cache = CacheManager(page_size=16)
        cache.add_kv_layer(KvNeed(1, 8, 20, keep_first=keep))
        cache.add_state(__import__("openinfer_b200.cache.manager", fromlist=["StateNeed"]).StateNeed((1,), "float32"))
        cache.allocate(16, 2)
        cache.open("r")
        for n in (70, 1, 1, 30, 1):
            cache.reserve("r", n)
            cache.commit("r")
        table = list(cache.block_table("r", 0))
        total = 103
        first_needed = (total - 20 + 1) // 16
        assert all(p != RELEASED for p in table[:stay]) and all(p == RELEASED for p in table[stay:first_needed])
        assert all(p != RELEASED for p in table[first_needed:])
        cache.check()
        cache.close("r")
        assert cache.min_free_pages() == cache.num_pages


def _bad(change):
    cfg = copy.deepcopy(CASE_A)
    change(cfg)
    return cfg


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "not known"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("decay", [0.5, 0.9]), "one number"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("decay", [0.5, 0.9, 1.5]), "one number"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "do not divide"),
    (lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("keep_first", -1), "keep_first"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 18), "larger than dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 6), "must equal rot_dim"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 1), "not a latent layer"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2), "earlier layer"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_rank", 41), "must equal those"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 4), "cannot give"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 5), "cannot give"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "kind must be"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.__setitem__("logit_softcap", -1.0), "logit_softcap"),
    (lambda c: c.__setitem__("layers", []), "at least one layer"),
])
def test_bad_configs_are_refused(change, message):
    with pytest.raises(ConfigError) as e:
        build(_bad(change))
    assert message in str(e.value)


def test_plain_mechanisms():
    # dynamic tanh
    p = {"n": torch.tensor([2.0, -1.0]), "n.b": torch.tensor([0.5, 0.25]), "n.alpha": torch.tensor(0.5)}
    x = torch.tensor([[1.0, 4.0]])
    assert torch.allclose(plain.dyt(x, p, "n"), torch.tensor([[2.0 * math.tanh(0.5) + 0.5, -math.tanh(2.0) + 0.25]]))
    # visibility: a window of 3 that keeps the first 2 keys
    ok = plain.visible(7, 3, 2)
    assert ok[6].tolist() == [True, True, False, False, True, True, True] and ok[2].tolist() == [True, True, True] + [False] * 4
    assert plain.visible(4, None, 0).tolist() == torch.tril(torch.ones(4, 4, dtype=torch.bool)).tolist()
    # the filter: zeros before the start, the last tap on the row itself
    u = torch.arange(1.0, 5.0)[:, None]
    assert plain.causal_filter(u, torch.tensor([[100.0, 10.0, 1.0]]))[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0]
    # stretched waves: the ramp's ends, the amplitude
    f, amp = plain.rotary_frequencies({"dims": 8, "base": 1000.0, "scaling": STRETCH})
    plain_f = 1000.0 ** (-2.0 * torch.arange(4, dtype=torch.float64) / 8)
    assert abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-12 and abs(f[0] - plain_f[0]) < 1e-12 and abs(f[3] - plain_f[3] / 4.0) < 1e-12
    # rotation: neighbours against halves are the same turn in another order
    x = torch.randn(3, 2, 8, dtype=torch.float64)
    pos = torch.tensor([0, 5, 9])
    a = plain.rotate(x, pos, {"dims": 8, "base": 100.0}, True)
    order = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7])
    b = plain.rotate(x[..., order], pos, {"dims": 8, "base": 100.0}, False)
    assert torch.allclose(a[..., order], b) and torch.equal(a[0], x[0])
    # routing: groups shut experts out although their scores are larger; weights without the correction
    W = 4
    pr = {"r.router": torch.eye(4, W, dtype=torch.float64) * 4.0, "r.correction": torch.tensor([0.0, 0.0, 0.3, 0.0], dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.9, -1.0, 0.2]], dtype=torch.float64)
    ids, w = plain.route(h, pr, "r.", {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert sorted(ids[0].tolist()) == [0, 1] and abs(float(w.sum()) - 1.0) < 1e-12
    ids, w = plain.route(h, pr, "r.", {"experts": 4, "top": 2})
    assert sorted(ids[0].tolist()) == [0, 1]
    h2 = torch.tensor([[1.0, -1.0, 0.45, 0.4]], dtype=torch.float64)
    ids, w = plain.route(h2, pr, "r.", {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert sorted(ids[0].tolist()) == [2, 3]          # group 1's two scores (with the correction) beat group 0's one large score
    s = torch.sigmoid(h2[0] * 4.0)
    assert torch.allclose(w[0].sort().values, (s[2:] / s[2:].sum()).sort().values)


def test_plain_forward_is_causal_and_every_mechanism_moves_the_logits(tmp_path):
    path = make_folder(str(tmp_path / "m"), CASE_A, 5)
    cfg, tensors = read_folder(path)
    toks = tokens_for(cfg, 60, 1)
    ref = plain.forward(cfg, tensors, toks)
    assert ref.abs().max().item() <= cfg["logit_softcap"]
    other = plain.forward(cfg, tensors, toks[:40] + [(t + 1) % cfg["vocab"] for t in toks[40:]])
    assert torch.equal(ref[:40], other[:40]) and not torch.allclose(ref[40:], other[40:])
    size = ref.pow(2).mean().sqrt().item()

    def moved(change_cfg=None, change_tensors=None):
        c, t = copy.deepcopy(cfg), dict(tensors)
        if change_cfg:
            change_cfg(c)
        if change_tensors:
            change_tensors(t)
        return (plain.forward(c, t, toks) - ref).abs().max().item() / size

    L = lambda i: (lambda c: c["layers"][i]["mixer"])
    assert moved(lambda c: L(1)(c)["mask"].__setitem__("keep_first", 18)) > 1e-5
    assert moved(lambda c: L(1)(c)["mask"].__setitem__("size", 22)) > 1e-5
    assert moved(lambda c: L(1)(c).pop("conv")) > 1e-5
    assert moved(lambda c: L(1)(c)["rot"].pop("scaling")) > 1e-5
    assert moved(lambda c: L(3)(c).__setitem__("decay", [0.5, 0.9, 1.0])) > 1e-5
    assert moved(lambda c: c["layers"][0]["mlp"]["router"].pop("groups")) > 1e-5
    assert moved(lambda c: c["layers"][1]["mlp"]["expert"].__setitem__("limit", 0.02)) > 1e-5
    assert moved(lambda c: c.__setitem__("logit_softcap", 0.0)) > 1e-5
    assert moved(None, lambda t: t.__setitem__("l1.mix.k.b", t["l1.mix.k.b"] * 0)) > 1e-5
    assert moved(None, lambda t: t.__setitem__("l0.mlp.correction", t["l0.mlp.correction"] * -3)) > 1e-5
    assert moved(None, lambda t: t.__setitem__("embed.norm.alpha", t["embed.norm.alpha"] * 0.5)) > 1e-5
    assert moved(None, lambda t: t.__setitem__("l2.norm1b.b", t["l2.norm1b.b"] + 0.5)) > 1e-5
