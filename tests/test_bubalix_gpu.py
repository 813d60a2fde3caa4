"""Bubalix in the engine against the plain implementation: the design's kernels alone, every mechanism alone in a model
of one layer, whole prompts, decoding through cache and state, portions, mixed batches, pages and slots that are used
again, window edges, far keys, sinks, greedy generation through the scheduler, the command line and the trace program."""
import copy
import json
import math
import subprocess
import sys

import pytest
import torch

import plain_bubalix as plain
from bubalix_cases import (CASES, STRETCH, assert_logits, attn, bfloat16_noise, float32_noise, latent, make_folder, model, moe, oracle,
                           read_folder, tokens_for)
from helpers import (ROOT, count_page_handouts, replay_in_process, replay_trace_run, round64, trace_mixed, trace_portions,
                     trace_tail, trace_whole)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(str(tmp_path_factory.mktemp(f"bbx{n}")), cfg, seed) for n, (cfg, seed) in CASES.items()}


def runner_for(path, dtype, max_tokens=2048, max_requests=4, page_size=16, graphs=True):
    from openinfer_b200.engine.runner import ModelRunner
    r = ModelRunner.from_folder(path, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, page_size=page_size)
    r.cuda_graph = graphs
    return r


def compare(got, path, toks, dtype, what, rows=slice(None), noise=None):
    assert_logits(got, oracle(path, toks)[rows], dtype, what, noise=float32_noise(path, toks) if noise is None else noise,
                  noise16=bfloat16_noise(path, toks))


def check_trace(runner, path, requests, steps, dtype, what):
    got = replay_in_process(runner, steps)
    noise = max(float32_noise(path, toks) for toks in requests.values())
    for rid, toks in requests.items():
        compare(got[rid], path, toks, dtype, f"{what}/{rid}", noise=noise)
    runner.cache.check()
    assert runner.cache.min_free_pages() == runner.cache.num_pages and runner.cache.slot_pool.used_count == 0


def _dev(t, dtype=None):
    return t.to(device="cuda", dtype=dtype or t.dtype)


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


# ---------------------------------------------------------------------------------------------- kernels alone
def _paged_rows(rows, page, order, dtype, pages_total):
    """[S, heads, n] rows into pages [pages, page, heads, n] in the given page order."""
    S, heads, n = rows.shape
    pages = torch.zeros(pages_total, page, heads, n, dtype=dtype)
    for j in range(S):
        pages[order[j // page], j % page] = rows[j].to(dtype)
    return pages


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,P,window,cap,every,slopes,sink", [
    (4, 2, 16, 8, 21, 6.0, 16, True, True), (6, 6, 32, 16, None, 0.0, 0, False, True), (3, 1, 64, 4, 1, 3.0, 0, True, False),
    (8, 2, 128, 16, 100, 0.0, 50, False, False), (2, 1, 24, 16, 16, 30.0, 7, True, True), (5, 5, 40, 2, 33, 2.0, 1, True, True)])
def test_attention_kernel_with_modified_scores(dtype, nq, nkv, hd, P, window, cap, every, slopes, sink):
    """A portion of a prompt over a cached prefix beside a single decoded token, scores as the design's attention forms
    them: temperature by the row's position, cap, distance bias, window, sink. Every switch also off."""
    from openinfer_b200.kernels import native, ops
    g = torch.Generator().manual_seed(nq * 100 + hd)
    S0, new0, S1 = 70, 9, 131
    scale = 2.5 / math.sqrt(hd)                                       # sharp: scores reach the cap
    n0, n1 = -(-S0 // P), -(-S1 // P)
    pages_total = n0 + n1 + 5
    perm = torch.randperm(pages_total, generator=g).tolist()
    order = [perm[:n0], perm[n0: n0 + n1]]
    ks = [torch.randn(S, nkv, hd, generator=g) for S in (S0, S1)]
    vs = [torch.randn(S, nkv, hd, generator=g) for S in (S0, S1)]
    qs = [torch.randn(S, nq, hd, generator=g) for S in (S0, S1)]
    k_pages = _dev(_paged_rows(ks[0], P, order[0], dtype, pages_total) + _paged_rows(ks[1], P, order[1], dtype, pages_total))
    v_pages = _dev(_paged_rows(vs[0], P, order[0], dtype, pages_total) + _paged_rows(vs[1], P, order[1], dtype, pages_total))
    bt = torch.zeros(2, max(n0, n1), dtype=torch.int32)
    bt[0, :n0], bt[1, :n1] = torch.tensor(order[0]), torch.tensor(order[1])
    rows = [(0, p) for p in range(S0 - new0, S0)] + [(1, S1 - 1)]
    q = torch.stack([qs[r][p] for r, p in rows]).to(dtype)
    sinks = torch.randn(nq, generator=g) + 1.0
    slope_t = plain.distance_slopes(nq, torch.float32)
    sinks_d, slopes_d = _dev(sinks), _dev(slope_t)
    mods = native.ScoreMods(sinks=sinks_d.data_ptr() if sink else None, slopes=slopes_d.data_ptr() if slopes else None,
                            softcap=float(cap), qt_coef=0.6 if every else 0.0, qt_every=int(every))
    out = torch.empty(len(rows), nq * hd, device="cuda", dtype=dtype)
    ops.attention_generic(_dev(q).view(len(rows), -1), out, k_pages, v_pages, k_pages.stride(0), P, _dev(bt), _i32([r for r, _ in rows]),
                          _i32([p for _, p in rows]), nq, nkv, hd, scale, window, mods=mods)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for i, (r, p) in enumerate(rows):
        kk, vv = ks[r].to(dtype).double(), vs[r].to(dtype).double()
        qq = torch.zeros(p + 1, nq, hd, dtype=torch.float64)
        qq[p] = q[i].double()
        ref = plain.scored_attention(
            qq, kk[: p + 1], vv[: p + 1], scale, window, sinks.double() if sink else torch.full((nq,), -math.inf, dtype=torch.float64),
            cap or None, slope_t.double() if slopes else None, plain.query_temperature(p + 1, 0.6, every, torch.float64) if every else None)[p]
        assert (out[i].double().cpu().view(nq, hd) - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item()), f"row {i} ({r}, {p})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,rank,rot,page", [(3, 40, 8, 4), (1, 20, 4, 16), (5, 12, 2, 2), (2, 264, 16, 8), (4, 96, 32, 16)])
def test_latent_norm_rotation_and_store_kernel(dtype, heads, rank, rot, page):
    """One pass over the fused product: the latent normed and stored, the key part turned by its row's position and stored
    behind it, the heads' query parts turned in place; everything else of the product and of the pages is left alone."""
    from openinfer_b200.kernels import ops
    from openinfer_b200.parts.registry import build_position_encoding
    from openinfer_b200.parts.spec import PositionSpec
    g = torch.Generator().manual_seed(rank + rot)
    rot_cfg = {"dims": rot, "base": 1000.0, "scaling": STRETCH}
    spec = PositionSpec(kind="rope", rotary_dim=rot, theta=1000.0, max_positions=512, precise=True, yarn=(4.0, 64.0, 8.0, 1.0))
    cos, sin = build_position_encoding(spec).rotation_tables(torch.device("cuda"))
    row = -(-(rank + rot) // 8) * 8
    tokens, pages_total = 7, 9
    lat_off = heads * row
    width = lat_off + rank + rot + 11
    proj = (torch.randn(tokens, width, generator=g) * 2).to(dtype)
    w = (1 + 0.1 * torch.randn(rank, generator=g)).to(torch.bfloat16)
    positions = [0, 1, 77, 300, 5, 511, 64]
    slots = [3, 0, 6, page * pages_total - 1, -1, 8, 1]
    store = torch.full((pages_total, page, 1, row), 5.0, dtype=dtype, device="cuda")
    pd = _dev(proj.clone())
    ops.latent_rope_store(store, page * row, pd, lat_off, rank, _dev(w), 1e-5, 0.0, cos, sin, _i32(positions), _i32(slots), heads, row, rank)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    src = proj.double()
    f, amp = plain.rotary_frequencies(rot_cfg)

    def turn(x, p):                                        # one row's vector at position p
        a = p * f
        c, s = torch.cos(a) * amp, torch.sin(a) * amp
        u, v = x[..., : rot // 2], x[..., rot // 2:]
        return torch.cat([u * c - v * s, v * c + u * s], dim=-1)

    got = pd.double().cpu()
    flat = store.view(pages_total * page, row).double().cpu()
    for t in range(tokens):
        for h in range(heads):
            at = h * row + rank
            assert (got[t, at: at + rot] - turn(src[t, at: at + rot], positions[t])).abs().max().item() < tol * 8
            assert torch.equal(got[t, h * row: at], src[t, h * row: at])                       # the unrotated part
        assert torch.equal(got[t, lat_off + rank + rot:], src[t, lat_off + rank + rot:])       # what lies behind (gates)
        if slots[t] >= 0:
            c_ref = plain.rms(src[t, lat_off: lat_off + rank], 1e-5) * w.double()
            k_ref = turn(src[t, lat_off + rank: lat_off + rank + rot], positions[t])
            assert (flat[slots[t], :rank] - c_ref).abs().max().item() < tol * max(1.0, c_ref.abs().max().item())
            assert (flat[slots[t], rank: rank + rot] - k_ref).abs().max().item() < tol * 8
            assert (flat[slots[t], rank + rot:] == 0).all()
    untouched = [s for s in range(pages_total * page) if s not in slots]
    assert (flat[untouched] == 5.0).all()


def test_sum_of_sublayers_token_gate_and_table_routing_kernels():
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    # x <- x + a + b, with and without b, with and without the rounded copy; sizes that are and are not multiples of four
    for n, hidden in ((5, 36), (3, 101), (64, 256)):
        x, a, b = (torch.randn(n, hidden, generator=g) for _ in range(3))
        for with_b in (True, False):
            for low_dtype in (None, torch.bfloat16, torch.float32):
                xd = _dev(x.clone())
                low = torch.empty(n, hidden, dtype=low_dtype, device="cuda") if low_dtype else None
                ops.add2_cast(xd, _dev(a), _dev(b) if with_b else None, low)
                ref = x + a + (b if with_b else 0)
                assert (xd.cpu() - ref).abs().max().item() < 1e-6
                if low is not None:
                    assert torch.equal(low.cpu(), xd.cpu().to(low_dtype))
    # g <- gelu_tanh(g) * table[token, off : off + dim] on a slice of a wider buffer
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        for dim, off, width in ((6, 12, 24), (5, 0, 5), (16, 16, 64)):
            table = torch.randn(50, width, generator=g).to(torch.bfloat16)
            ids = [7, 0, 49, 7, 23]
            buf = (torch.randn(5, dim + 3, generator=g) * 3).to(dtype)
            bd = _dev(buf.clone())
            ops.token_gate(bd[:, :dim], _i32(ids), _dev(table), off)
            ref = plain.gelu_tanh(buf[:, :dim].double()) * table.double()[torch.tensor(ids)][:, off: off + dim]
            assert (bd[:, :dim].double().cpu() - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())
            assert torch.equal(bd[:, dim:].cpu(), buf[:, dim:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,W,F,E,top,shared", [(1, 40, 24, 5, 2, 16), (37, 64, 16, 3, 1, 0), (200, 96, 40, 16, 4, 24), (9, 36, 70, 40, 3, 10),
                                                   (64, 128, 96, 4, 4, 0), (300, 64, 32, 12, 1, 48),
                                                   (700, 72, 40, 3, 2, 16), (150, 64, 200, 2, 1, 0), (1100, 256, 136, 5, 3, 0)])
def test_experts_by_table_kernels(dtype, rows, W, F, E, top, shared):
    """Experts chosen by the token id through a table, each weighted 1 / top, plus an expert every row uses, against the
    plain statement row by row; a row's result does not depend on the rows beside it (steps whose experts have 64 rows and
    more on average take tiles of 128 rows, smaller ones tiles of 32, the smallest go pair by pair: the last three cases
    compare a row across them)."""
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(rows + E)
    vocab = 61
    x = torch.randn(rows, W, generator=g).to(dtype)
    table = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(vocab)]).to(torch.int32)
    tokens = torch.randint(0, vocab, (rows,), generator=g).tolist()
    Wt = {"table": table}
    names = [f"e{e}." for e in range(E)] + (["shared."] if shared else [])
    for p in names:
        ff = shared if p == "shared." else F
        Wt[p + "gate"] = (torch.randn(ff, W, generator=g) * W ** -0.5).to(torch.bfloat16)
        Wt[p + "up"] = (torch.randn(ff, W, generator=g) * W ** -0.5).to(torch.bfloat16)
        Wt[p + "down"] = (torch.randn(W, ff, generator=g) * ff ** -0.5).to(torch.bfloat16)
    mlp = {"router": {"experts": E, "top": top}, "shared": {"ff": shared} if shared else None}
    ref = plain.table_experts(x.double(), {k: (v.double() if v.is_floating_point() else v.long()) for k, v in Wt.items()}, "", mlp, tokens)
    gate_up = torch.stack([torch.cat([Wt[f"e{e}.gate"], Wt[f"e{e}.up"]]) for e in range(E)]).to(dtype)
    down = torch.stack([Wt[f"e{e}.down"] for e in range(E)]).to(dtype)
    add = None
    if shared:
        add = _dev(plain.expert(x.double(), {k: v.double() for k, v in Wt.items() if k.startswith("shared.")}, "shared.").float())

    def run(n):
        routing = ops.moe_route_table(_i32(tokens[:n]), _dev(table), E)
        return routing, ops.moe_experts(_dev(x[:n]), _dev(gate_up), _dev(down), routing, 0.0, act="silu",
                                        add=add[:n].contiguous() if add is not None else None)

    routing, out = run(rows)
    assert torch.equal(routing[0].cpu(), table[torch.tensor(tokens)]) and (routing[1].cpu() == 1.0 / top).all()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (out.double().cpu() - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())
    if rows > 100:
        assert torch.equal(run(90)[1], out[:90])
    if rows > 8:
        assert (run(3)[1].double().cpu() - ref[:3]).abs().max().item() < tol * max(1.0, ref.abs().max().item())


# ---------------------------------------------------------------------------------------------- mechanisms alone
def _one_layer(layer, width=48, vocab=83, **kw):
    return model(vocab, width, [layer], **kw)


MECHANISMS = {
    "plain grouped attention with a sink": _one_layer(attn(4, 2, 16, 16, 0.5)),
    "window": _one_layer(attn(2, 1, 16, 16, 0.5, window=18)),
    "filter of four taps": _one_layer(attn(2, 2, 8, 8, 0.7, conv=4)),
    "query temperature": _one_layer(attn(3, 1, 16, 8, 0.5, q_temp=(1.5, 9))),
    "cap that bites": _one_layer(attn(2, 1, 16, 24, 3.0, softcap=2.0)),
    "keys wider than values and heads of 264": _one_layer(attn(2, 1, 264, 40, 0.08, window=40, conv=2)),
    "latent without stretched waves": _one_layer(latent(3, 8, 4, 12, 20, 0.6, base=100.0)),
    "latent with stretched waves": _one_layer(latent(2, 16, 16, 8, 24, 0.5, base=10000.0, scaling=STRETCH)),
    "latent with one head": _one_layer(latent(1, 8, 2, 8, 8, 0.8)),
    "experts alone, all of them": _one_layer(attn(1, 1, 8, 8, 0.5, mlp=moe(20, 3, 3))),
    "one expert a token and a shared one": _one_layer(attn(1, 1, 8, 8, 0.5, mlp=moe(12, 9, 1, shared=30))),
    "side input": _one_layer(attn(1, 1, 8, 8, 0.5), side=7),
    "embedding scale": _one_layer(latent(1, 8, 2, 8, 8, 0.8), scale=3.0),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MECHANISMS))
def test_each_mechanism_alone(tmp_path, name, dtype):
    """A model of one layer with one mechanism switched on: a whole prompt, then portions of 2, 1, 5 and 3 tokens and
    decoding, two requests in the same trace."""
    cfg = MECHANISMS[name]
    path = make_folder(str(tmp_path / "m"), cfg, 7)
    requests = {"a": tokens_for(cfg, 75, 1), "b": tokens_for(cfg, 40, 2)}
    runner = runner_for(path, dtype, max_tokens=256)
    check_trace(runner, path, requests, trace_whole(requests), dtype, name)
    check_trace(runner, path, requests, trace_portions(requests, sizes=(2, 1, 5, 3, 30, 1, 1, 2)), dtype, name + "/portions")


def test_mechanisms_show_in_the_logits(tmp_path):
    """The comparison sees each mechanism: the plain implementation with the mechanism left out (or off by one) differs
    from the engine by far more than the bound. Weights are made so that it shows: sinks raised, queries lengthened."""
    cfg = model(83, 48, [attn(4, 2, 16, 8, 0.5, window=18, conv=3, q_temp=(1.5, 9), softcap=3.0, mlp=moe(20, 5, 2, shared=12)),
                         latent(3, 8, 4, 12, 20, 0.6, base=100.0, scaling=STRETCH)], side=5, scale=1.5)
    path = make_folder(str(tmp_path / "m"), cfg, 11)
    raw, tensors = read_folder(path)
    tensors = dict(tensors)
    tensors["l0.mix.sink"] = tensors["l0.mix.sink"] + 3.0
    tensors["l1.mix.sink"] = tensors["l1.mix.sink"] + 3.0
    tensors["l0.mix.q"] = tensors["l0.mix.q"] * 6.0
    from safetensors.torch import save_file
    save_file({k: v.contiguous() for k, v in tensors.items()}, path + "/model.safetensors")
    toks = tokens_for(cfg, 90, 4)
    runner = runner_for(path, "float32", max_tokens=256)
    got = replay_in_process(runner, trace_tail({"m": toks}, tail=40))["m"].double()
    ref = plain.forward(raw, tensors, toks)
    size = ref.pow(2).mean().sqrt().item()
    assert (got - ref).abs().max().item() < 1e-4 * size

    def without(change_cfg=None, change_tensors=None):
        c, t = copy.deepcopy(raw), dict(tensors)
        if change_cfg:
            change_cfg(c)
        if change_tensors:
            change_tensors(t)
        wrong = plain.forward(c, t, toks)
        return min((got[:50] - wrong[:50]).abs().max().item(), (got[50:] - wrong[50:]).abs().max().item()) / size

    # every change below moves the plain logits by 4e-4 of their size or more; the engine is within 1e-4 (in fact far closer)
    seen = max(2e-4, 20 * (got - ref).abs().max().item() / size)
    L0, L1 = (lambda c: c["layers"][0]["mixer"]), (lambda c: c["layers"][1]["mixer"])
    assert without(lambda c: L0(c).pop("softcap")) > seen
    assert without(lambda c: L0(c).pop("q_temp")) > seen
    assert without(lambda c: L0(c)["q_temp"].__setitem__("every", 10)) > seen            # floor((p + 1) / every): off by one
    assert without(lambda c: L0(c).pop("conv")) > seen
    assert without(lambda c: L0(c)["mask"].__setitem__("size", 17)) > seen
    assert without(lambda c: L0(c)["mask"].__setitem__("size", 19)) > seen
    assert without(lambda c: L1(c)["rot"].pop("scaling")) > seen
    assert without(lambda c: L1(c)["rot"].__setitem__("base", 200.0)) > seen
    assert without(None, lambda t: t.__setitem__("l0.mix.sink", t["l0.mix.sink"] - 40.0)) > seen
    assert without(None, lambda t: t.__setitem__("l1.mix.sink", t["l1.mix.sink"] - 40.0)) > seen
    assert without(None, lambda t: t.__setitem__("l0.mix.g", t["l0.mix.g"] * 0.0)) > seen
    assert without(None, lambda t: t.__setitem__("l1.mix.g", t["l1.mix.g"] * 0.0)) > seen
    assert without(None, lambda t: t.__setitem__("l0.mlp.table", (t["l0.mlp.table"] + 1) % 5)) > seen
    assert without(lambda c: c["layers"][0]["mlp"].pop("shared")) > seen
    assert without(lambda c: c.pop("token_side")) > seen
    assert without(lambda c: c.pop("embedding")) > seen
    assert without(lambda c: c["norm"].__setitem__("eps", 1e-1)) > seen


# ---------------------------------------------------------------------------------------------- the model
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_whole_prompts_and_decoding_match_plain(folders, name, dtype):
    """Whole prompts in one step (the first tokens of a sequence among them: one and two tokens); then most of a prompt
    in one step and its last 80 tokens one by one through recorded graphs, far enough for every window and several periods
    of the query temperature to pass over decoded tokens."""
    cfg = CASES[name][0]
    requests = {f"w{n}": tokens_for(cfg, n, 100 + n) for n in (1, 2, 37, 200)}
    runner = runner_for(folders[name], dtype)
    check_trace(runner, folders[name], requests, trace_whole(requests), dtype, f"{name}/whole")
    del requests["w1"], requests["w2"]
    check_trace(runner, folders[name], requests, trace_tail(requests, tail=80), dtype, f"{name}/decode")


@pytest.mark.parametrize("name", ["A", "D"])
def test_prefill_equals_token_by_token(folders, name):
    """A prompt fed one token a step from its first token on (cache and filter state carry everything) against the whole
    prompt in one step: the same logits up to rounding, and both the plain implementation's."""
    toks = tokens_for(CASES[name][0], 60, 5)
    runner = runner_for(folders[name], "float32")
    steps = [{"step": i, "entries": [{"id": "s", "tokens": [t], "want": [0]}], "end": ["s"] if i == len(toks) - 1 else []}
             for i, t in enumerate(toks)]
    one_by_one = replay_in_process(runner, steps)["s"]
    whole = replay_in_process(runner, trace_whole({"s": toks}))["s"]
    compare(one_by_one, folders[name], toks, "float32", "token by token")
    size = whole.pow(2).mean().sqrt().item()
    assert (one_by_one - whole).abs().max().item() < 2e-5 * size


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_portions_down_to_two_tokens(folders, name, dtype):
    cfg = CASES[name][0]
    requests = {"p0": tokens_for(cfg, 170, 1), "p1": tokens_for(cfg, 45, 2)}
    runner = runner_for(folders[name], dtype, graphs=False)
    check_trace(runner, folders[name], requests, trace_portions(requests), dtype, f"{name}/portions")
    check_trace(runner, folders[name], requests, trace_portions(requests, sizes=(2, 3, 1, 2, 4)), dtype, f"{name}/small portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("A", 16), ("B", 8), ("C", 16), ("D", 32), ("E", 16)])
def test_mixed_batches_with_pages_and_slots_used_again(folders, name, page, dtype):
    """Up to three live requests of unequal lengths, portions beside single tokens, in a pool that holds less than the
    sum of the requests and has three state slots: every request's logits are those of the request alone."""
    cfg = CASES[name][0]
    lens = [140, 3, 64, 97, 1, 33, 110, 18]
    requests = {f"m{i}": tokens_for(cfg, n, 50 + i) for i, n in enumerate(lens)}
    max_tokens = 384
    runner = runner_for(folders[name], dtype, max_tokens=max_tokens, max_requests=3, page_size=page)
    handed = count_page_handouts(runner.cache)
    steps = trace_mixed(requests, max_tokens, seed=3, max_live=3, tail=20)
    check_trace(runner, folders[name], requests, steps, dtype, f"{name}/mixed")
    assert max(handed.values()) >= 2, "no page was used a second time"


def test_a_slot_used_again_starts_from_zero(folders):
    """The same request twice through the one state slot, with another request's filter state left there in between."""
    name = "B"
    cfg = CASES[name][0]
    runner = runner_for(folders[name], "float32", max_requests=1)
    for seed in (1, 2, 1):
        toks = tokens_for(cfg, 50, seed)
        check_trace(runner, folders[name], {"r": toks}, trace_tail({"r": toks}, tail=10), "float32", f"slot/{seed}")


def test_window_edges_show_in_the_logits(tmp_path):
    """The comparison is sharp enough to see a window that is one key off: the plain implementation with a window one
    longer or one shorter differs from the engine by far more than the engine does from the right one, at prompt rows and
    at decoded ones. The model is made for it: sharp softmaxes, sinks far down, and in the layer with the long window few
    heads, so that the slope of the last one leaves the window's oldest key its weight."""
    from safetensors.torch import save_file
    cfg = model(120, 48, [
        attn(4, 2, 16, 24, 1.1, window=21, conv=3, q_temp=(0.4, 32), softcap=12.0, mlp=moe(16, 7, 1, shared=32)),
        attn(3, 1, 24, 40, 1.6, window=70, conv=2, softcap=8.0, mlp=None),
    ], eps=1e-5, scale=0.7, side=6)
    path = make_folder(str(tmp_path / "edges"), cfg, 77)
    raw, tensors = read_folder(path)
    tensors = dict(tensors)
    for layer in (0, 1):
        tensors[f"l{layer}.mix.sink"] = tensors[f"l{layer}.mix.sink"] - 20.0
    save_file({k: v.contiguous() for k, v in tensors.items()}, path + "/model.safetensors")
    toks = tokens_for(cfg, 150, 9)
    runner = runner_for(path, "float32", max_tokens=256)
    got = replay_in_process(runner, trace_tail({"e": toks}, tail=60))["e"].double()
    ref = plain.forward(raw, tensors, toks)
    scale = ref.pow(2).mean().sqrt().item()
    assert (got - ref).abs().max().item() < 2e-5 * scale
    for layer in (0, 1):
        for d in (-1, 1):
            off = json.loads(json.dumps(raw))
            off["layers"][layer]["mixer"]["mask"]["size"] += d
            wrong = plain.forward(off, tensors, toks)
            assert (got[75:90] - wrong[75:90]).abs().max().item() > 3e-4 * scale, "a window one key off would not be noticed in a prompt"
            assert (got[90:] - wrong[90:]).abs().max().item() > 3e-4 * scale, "a window one key off would not be noticed while decoding"
            assert (ref[:20] - wrong[:20]).abs().max().item() < 1e-9             # before any window is full the two agree


def test_windows_at_and_around_page_borders(tmp_path):
    """Windows of 15, 16, 17, 32 and 33 keys with pages of 16: the oldest key seen is the last of a page, the first of one,
    and one to either side; prompts and decoded tokens, portions that end inside a page."""
    for window in (15, 16, 17, 32, 33):
        cfg = _one_layer(attn(2, 1, 16, 16, 1.0, window=window, conv=2, softcap=10.0))
        path = make_folder(str(tmp_path / f"w{window}"), cfg, window)
        toks = tokens_for(cfg, 100, window)
        runner = runner_for(path, "float32", max_tokens=256)
        steps = trace_portions({"w": toks[:70]}, sizes=(13, 16, 3, 17, 21))
        steps[-1]["end"] = []
        steps += [{"step": 100 + i, "entries": [{"id": "w", "tokens": [t], "want": [0]}], "end": ["w"] if i == 29 else []}
                  for i, t in enumerate(toks[70:])]
        got = replay_in_process(runner, steps)["w"]
        compare(got, path, toks, "float32", f"window {window}")
        raw, tensors = read_folder(path)
        off = json.loads(json.dumps(raw))
        off["layers"][0]["mixer"]["mask"]["size"] = window + 1
        ref = oracle(path, toks)
        assert (ref - plain.forward(off, tensors, toks)).abs().max().item() > 1e-3 * ref.pow(2).mean().sqrt().item()


def test_a_far_key_among_hundreds_reaches_both_mixers(tmp_path):
    """No window, a sharp softmax, sinks far down: a row's weight sits on the few keys that match it best, wherever they
    are among 300. The engine follows the plain implementation while decoding, and a plain implementation that sees only the
    last 200 keys does not."""
    for layer in (attn(4, 2, 16, 24, 1.4, conv=2), latent(3, 16, 8, 12, 24, 1.2, base=10000.0)):
        cfg = _one_layer(layer)
        path = make_folder(str(tmp_path / layer["type"]), cfg, 11)
        raw, tensors = read_folder(path)
        tensors = dict(tensors)
        tensors["l0.mix.sink"] = tensors["l0.mix.sink"] - 20.0
        from safetensors.torch import save_file
        save_file({k: v.contiguous() for k, v in tensors.items()}, path + "/model.safetensors")
        toks = tokens_for(cfg, 300, 5)
        runner = runner_for(path, "float32", max_tokens=512)
        got = replay_in_process(runner, trace_tail({"f": toks}, tail=60))["f"].double()
        ref = plain.forward(raw, tensors, toks)
        scale = ref.pow(2).mean().sqrt().item()
        near = json.loads(json.dumps(raw))
        near["layers"][0]["mixer"]["mask"] = {"size": 200}
        wrong = plain.forward(near, tensors, toks)
        assert (ref[240:] - wrong[240:]).abs().max().item() > 1e-2 * scale, "lost far keys would not be noticed"
        assert (got - ref).abs().max().item() < 1e-4 * scale


def test_far_keys_reach_the_last_token_of_the_model(folders):
    """The latent layers see the first token from far away, also while decoding: with the first token changed the plain
    implementation's last logits move, and the engine follows the right one."""
    name = "A"
    cfg, tensors = read_folder(folders[name])
    toks = tokens_for(cfg, 300, 21)
    runner = runner_for(folders[name], "float32")
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:200], "want": []}], "end": []}]
    steps += [{"step": 1 + i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": ["x"] if i == 99 else []}
              for i, t in enumerate(toks[200:])]
    got = replay_in_process(runner, steps)["x"].double()
    ref = oracle(folders[name], toks)[200:]
    compare(got, folders[name], toks, "float32", "far keys", rows=slice(200, None))
    other = plain.forward(cfg, tensors, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])[200:]
    assert (ref - other).abs().max().item() > 100 * (got - ref).abs().max().item(), "the first token would not be missed"


def test_long_decoding(folders):
    """600 single-token steps behind a short prompt: filter state, windows, released pages and many periods of the query
    temperature over a long run."""
    name = "D"
    cfg = CASES[name][0]
    toks = tokens_for(cfg, 620, 77)
    runner = runner_for(folders[name], "float32", max_tokens=704)
    got = replay_in_process(runner, trace_tail({"l": toks}, tail=600))["l"]
    compare(got, folders[name], toks, "float32", "long decoding")


@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation_through_the_scheduler(folders, name):
    from openinfer_b200 import LLM, SamplingParams
    cfg, tensors = read_folder(folders[name])
    prompts = [tokens_for(cfg, n, 70 + n) for n in (1, 9, 33, 70)]
    n_new = 20

    def greedy(prompt):
        toks = list(prompt)
        for _ in range(n_new):
            toks.append(int(plain.forward(cfg, tensors, toks)[-1].argmax()))
        return toks[len(prompt):]

    want = [greedy(p) for p in prompts]
    llm = LLM(folders[name], dtype="float32", max_cache_tokens=512, max_prefill_tokens=13, max_decode_batch=3)
    assert llm.generate(prompts, max_tokens=n_new) == want
    assert llm.runner.cache.min_free_pages() == llm.runner.cache.num_pages
    assert [llm.generate([p], max_tokens=n_new)[0] for p in prompts] == want
    llm16 = LLM(folders[name], dtype="bfloat16", max_cache_tokens=512, max_decode_batch=4)
    sp = SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=5)
    a = llm16.generate(prompts, sp, max_tokens=12)
    assert a == llm16.generate(prompts, sp, max_tokens=12) and all(len(t) == 12 for t in a)
    assert llm16.runner.cache.slot_pool.used_count == 0


def test_command_line_and_trace_program(folders, tmp_path):
    name = "B"
    cfg, tensors = read_folder(folders[name])
    toks = [7, 8, 9]
    want = []
    for _ in range(5):
        want.append(int(plain.forward(cfg, tensors, toks + want)[-1].argmax()))
    out = subprocess.run([sys.executable, "-m", "openinfer_b200", "--model-path", folders[name], "--dtype", "float32",
                          "--prompt-ids", "7,8,9", "--max-tokens", "5", "--num-pages", "32"],
                         cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["token_ids"] == want and line["finish_reason"] == "length"
    name = "A"
    cfg = CASES[name][0]
    requests = {f"t{i}": tokens_for(cfg, n, 30 + i) for i, n in enumerate([80, 5, 130, 41, 1])}
    max_tokens = round64(130) + round64(80) + 64
    steps = trace_mixed(requests, max_tokens, seed=1, max_live=4, tail=16)
    for dtype in DTYPES:
        got = replay_trace_run(folders[name], dtype, steps, str(tmp_path / dtype), max_tokens, cfg["vocab"])
        for rid, t in requests.items():
            compare(got[rid], folders[name], t, dtype, f"trace_run/{dtype}/{rid}")
