"""Luzitar in the engine against the plain implementation: the design's kernels alone, every mechanism alone in a model
of one layer, whole prompts, decoding through cache and state, portions, mixed batches, pages and slots that are used
again, window edges and kept first keys, far keys, old state, greedy generation through the scheduler, the command line and
the trace program."""
import copy
import json
import math
import subprocess
import sys

import pytest
import torch

import plain_luzitar as plain
from luzitar_cases import (CASES, STRETCH, assert_logits, attn, bfloat16_noise, first_close_call, float32_noise, latent, lightning,
                           make_folder, model, moe, oracle, read_folder, rot, tokens_for)
from helpers import (ROOT, count_page_handouts, replay_in_process, replay_trace_run, round64, trace_mixed, trace_portions,
                     trace_tail, trace_whole)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(str(tmp_path_factory.mktemp(f"lzt{n}")), cfg, seed) for n, (cfg, seed) in CASES.items()}


def runner_for(path, dtype, max_tokens=2048, max_requests=4, page_size=16, graphs=True):
    from openinfer_b200.engine.runner import ModelRunner
    r = ModelRunner.from_folder(path, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, page_size=page_size)
    r.cuda_graph = graphs
    return r


def compare(got, path, toks, dtype, what, rows=slice(None), noise=None):
    start = rows.start or 0
    assert_logits(got, oracle(path, toks)[rows], dtype, what, noise=float32_noise(path, toks) if noise is None else noise,
                  noise16=bfloat16_noise(path, toks), first_close=max(0, first_close_call(path, toks) - start))


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


def save(path, tensors):
    from safetensors.torch import save_file
    save_file({k: v.contiguous() for k, v in tensors.items()}, path + "/model.safetensors")


# ---------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(1, 36), (7, 64), (33, 1030), (5, 4096)])
def test_dynamic_tanh_step_kernel(out_dtype, rows, width):
    """h += dyt(branch; post) and out = dyt(h; pre) in one pass, either half alone, gathered rows, and the norm in place."""
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(rows + width)
    h, br = torch.randn(rows, width, generator=g) * 2, torch.randn(rows, width, generator=g) * 3

    def trio(dtype):
        return (torch.rand(1, generator=g).to(dtype) + 0.3, (1 + 0.2 * torch.randn(width, generator=g)).to(dtype), (0.3 * torch.randn(width, generator=g)).to(dtype))

    def dyt(x, t):
        return torch.tanh(t[0].double() * x) * t[1].double() + t[2].double()

    post, pre = trio(torch.bfloat16), trio(torch.float32)
    tol = 1e-6 if out_dtype == torch.float32 else 1e-2
    hd, out = _dev(h.clone()), torch.empty(rows, width, device="cuda", dtype=out_dtype)
    ops.dyt_step(hd, branch=_dev(br), post=tuple(_dev(t) for t in post), pre=tuple(_dev(t) for t in pre), out=out)
    new_h = h.double() + dyt(br.double(), post)
    assert (hd.double().cpu() - new_h).abs().max().item() < 1e-5
    assert (out.double().cpu() - dyt(new_h, pre)).abs().max().item() < tol * 3
    hd2 = _dev(h.clone())
    ops.dyt_step(hd2, branch=_dev(br), post=tuple(_dev(t) for t in post))
    assert torch.equal(hd2, hd)
    idx = [rows - 1, 0, rows // 2]
    got = torch.empty(3, width, device="cuda", dtype=out_dtype)
    hd3 = _dev(h.clone())
    ops.dyt_step(hd3, branch=_dev(br), post=tuple(_dev(t) for t in post), pre=tuple(_dev(t) for t in pre), out=got, row_idx=_i32(idx))
    assert torch.equal(got, out[idx]) and torch.equal(hd3.cpu(), h)          # gathered rows leave the stream alone
    hd4 = _dev(h.clone())
    ops.dyt_step(hd4, pre=tuple(_dev(t) for t in pre), out=hd4)
    assert (hd4.double().cpu() - dyt(h.double(), pre)).abs().max().item() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,qk,rot_dims,taps,page", [(4, 2, 24, 16, 8, 3, 4), (6, 6, 16, 8, 4, 0, 16), (3, 1, 40, 40, 0, 5, 8),
                                                               (2, 1, 64, 64, 64, 1, 16), (5, 5, 16, 10, 6, 2, 2), (4, 2, 128, 128, 64, 4, 16),
                                                               (6, 2, 32, 24, 16, 3, 8), (2, 2, 256, 200, 128, 2, 16), (3, 1, 8, 8, 0, 2, 4),
                                                               (1, 1, 16, 16, 16, 0, 16)])
def test_bias_rotation_unit_norm_and_store_kernel(dtype, nq, nkv, hd, qk, rot_dims, taps, page):
    """One pass over the fused q | k | v rows: the bias by position, the rotation of the first numbers of q and k heads, the
    unit norm over qk numbers behind it, q in place, k and v to their slots; a padding row stores nothing."""
    from openinfer_b200.kernels import ops
    from openinfer_b200.parts.registry import build_position_encoding
    from openinfer_b200.parts.spec import PositionSpec
    g = torch.Generator().manual_seed(nq * 10 + hd)
    heads = nq + 2 * nkv
    tokens, pages_total = 6, 9
    x = torch.zeros(tokens, heads, hd)
    x[:, :, :qk] = torch.randn(tokens, heads, qk, generator=g) * 2
    x = x.to(dtype)
    n_tab = max(taps, 1)
    tab = torch.zeros(n_tab, heads, hd)
    tab[:, :, :qk] = torch.randn(n_tab, heads, qk, generator=g)
    positions = [0, 1, 2, 77, 300, 5]
    slots = [3, 0, 6, page * pages_total - 1, -1, 8]
    cos = sin = None
    rcfg = {"dims": rot_dims, "base": 1000.0, "scaling": STRETCH}
    if rot_dims:
        spec = PositionSpec(kind="rope", rotary_dim=rot_dims, theta=1000.0, max_positions=512, precise=True, yarn=(4.0, 64.0, 8.0, 1.0))
        cos, sin = build_position_encoding(spec).rotation_tables(torch.device("cuda"))
    k_pages = torch.full((pages_total, page, nkv, hd), 5.0, dtype=dtype, device="cuda")
    v_pages = torch.full((pages_total, page, nkv, hd), 5.0, dtype=dtype, device="cuda")
    xd = _dev(x.clone()).view(tokens, heads * hd)
    ops.rope_norm_store(xd, nq, nkv, hd, qk, bias_tab=_dev(tab.view(n_tab, -1)), cos=cos, sin=sin, unit_norm=True, eps=1e-5,
                        positions=_i32(positions), slots=_i32(slots), k_cache=k_pages, v_cache=v_pages, page_stride=k_pages.stride(0),
                        page_size=page, write_kv=True)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    got = xd.double().cpu().view(tokens, heads, hd)
    for t in range(tokens):
        y = x[t].double() + tab[min(positions[t], n_tab - 1)].double()
        qk_rows = y[: nq + nkv, :qk]
        if rot_dims:
            qk_rows = plain.rotate(qk_rows[None], torch.tensor([positions[t]]), rcfg, False)[0]
        qk_rows = plain.rms(qk_rows, 1e-5)
        assert (got[t, :nq, :qk] - qk_rows[:nq]).abs().max().item() < tol * 4, f"q of row {t}"
        assert got[t, :nq, qk:].abs().max().item() == 0 if qk < hd else True
        if slots[t] >= 0:
            pg, off = divmod(slots[t], page)
            assert (k_pages[pg, off].double().cpu()[:, :qk] - qk_rows[nq:]).abs().max().item() < tol * 4, f"k of row {t}"
            assert (v_pages[pg, off].double().cpu() - y[nq + nkv:]).abs().max().item() < tol * 4, f"v of row {t}"
    used = {divmod(s, page) for s in slots if s >= 0}
    for pg in range(pages_total):
        for off in range(page):
            if (pg, off) not in used:
                assert (k_pages[pg, off] == 5.0).all() and (v_pages[pg, off] == 5.0).all()


def _paged_rows(rows, page, order, dtype, pages_total):
    S, heads, n = rows.shape
    pages = torch.zeros(pages_total, page, heads, n, dtype=dtype)
    for j in range(S):
        pages[order[j // page], j % page] = rows[j].to(dtype)
    return pages


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,P,window,keep", [(4, 2, 16, 8, 21, 19), (6, 6, 32, 16, 16, 16), (3, 1, 64, 4, 1, 5), (8, 2, 128, 16, 100, 1),
                                                      (2, 1, 24, 16, 40, 70), (5, 5, 40, 2, 33, 0), (2, 1, 64, 16, 64, 17)])
def test_attention_kernels_with_kept_first_keys(dtype, nq, nkv, hd, P, window, keep):
    """A portion of a prompt over a cached prefix beside a single decoded token, through the general kernel and (bfloat16,
    heads of 32 / 64 / 128) the tensor-core kernels: a window, and the sequence's first keys visible behind it."""
    from openinfer_b200.kernels import native, ops
    g = torch.Generator().manual_seed(nq * 100 + hd)
    S0, new0, S1 = 150, 9, 131
    scale = 2.5 / math.sqrt(hd)
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
    mods = native.ScoreMods(keep_first=keep)
    out = torch.empty(len(rows), nq * hd, device="cuda", dtype=dtype)
    ops.attention_generic(_dev(q).view(len(rows), -1), out, k_pages, v_pages, k_pages.stride(0), P, _dev(bt), _i32([r for r, _ in rows]),
                          _i32([p for _, p in rows]), nq, nkv, hd, scale, window, mods=mods)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for i, (r, p) in enumerate(rows):
        kk, vv = ks[r].to(dtype).double()[: p + 1], vs[r].to(dtype).double()[: p + 1]
        ok = plain.visible(p + 1, window, keep)[p]
        for h in range(nq):
            s = (kk[:, h // (nq // nkv)] @ q[i, h].double()) * scale
            w = torch.softmax(s.masked_fill(~ok, -math.inf), dim=0)
            ref = w @ vv[:, h // (nq // nkv)]
            assert (out[i].double().cpu().view(nq, hd)[h] - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item()), f"row {i} head {h}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,W,E,top,groups,keep", [(1, 40, 6, 2, 3, 2), (37, 64, 8, 3, 2, 1), (200, 96, 12, 4, 2, 1), (9, 36, 40, 2, 8, 3),
                                                       (5, 48, 4, 4, 1, 1), (16, 32, 9, 1, 9, 2), (3, 64, 64, 8, 4, 4)])
def test_router_by_corrected_sigmoid_scores_within_groups(dtype, rows, W, E, top, groups, keep):
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(rows + E)
    x = torch.randn(rows, W, generator=g).to(dtype)
    w = (torch.randn(E, W, generator=g) * W ** -0.5 * 2).to(dtype)
    corr = torch.randn(E, generator=g) * 0.3
    ids, wts, _, _ = ops.moe_route(_dev(x), _dev(w), top, scoring="sigmoid_groups", correction=_dev(corr), groups=groups, keep_groups=keep)
    margins = []
    ref_ids, ref_w = plain.route(x.double(), {"r.router": w.double(), "r.correction": corr.double()}, "r.",
                                 {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}, margins)
    sure = margins[0] > 1e-4
    got_ids, got_w = ids.cpu().long(), wts.double().cpu()
    assert sure.sum() >= rows * 0.7
    for r in range(rows):
        if not sure[r]:
            continue
        assert sorted(got_ids[r].tolist()) == sorted(ref_ids[r].tolist()), f"row {r}"
        a = dict(zip(got_ids[r].tolist(), got_w[r].tolist()))
        for e, we in zip(ref_ids[r].tolist(), ref_w[r].tolist()):
            assert abs(a[e] - we) < 1e-5


@pytest.mark.parametrize("H,D,V", [(2, 16, 8), (3, 8, 24), (1, 20, 3), (2, 64, 128), (5, 6, 10), (1, 264, 16)])
def test_linear_attention_scan(H, D, V):
    """Two requests side by side, one a portion over old state and one a single token; the state is read from one copy and
    left in the other."""
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(H * D + V)
    lens, cols = [9, 1], 2 * H * D + H * V
    T = sum(lens)
    z = torch.randn(T, cols + 3, generator=g)
    decays = torch.tensor([0.3, 0.9, 1.0, 0.97, 0.999][:H])
    state = torch.randn(3, 2, H, D * V, generator=g)

    class Ctx:
        cu_seqlens, token_req = _i32([0, 9, 10]), _i32([0] * 9 + [1])
        state_slots, state_phase, num_requests = _i32([2, 0]), _i32([1, 0]), 2

    sd, zd = _dev(state.clone()), _dev(z.clone())
    o = torch.empty(T, H * V, device="cuda")
    ops.recurrent_scan(ops.SCAN_LINEAR_DECAY, o, zd, (0, H * D, 2 * H * D), zd, (0, 0), sd, Ctx, H, H, D, V, p0=_dev(decays))
    silu = lambda t: t * torch.sigmoid(t)
    row = 0
    for b, (n, slot, phase) in enumerate(zip(lens, [2, 0], [1, 0])):
        for h in range(H):
            S = state[slot, phase, h].double().view(V, D).T.clone()            # stored column by column
            for t in range(row, row + n):
                q, k = silu(z[t, h * D: (h + 1) * D].double()), silu(z[t, H * D + h * D: H * D + (h + 1) * D].double())
                v = silu(z[t, 2 * H * D + h * V: 2 * H * D + (h + 1) * V].double())
                S = float(decays[h]) * S + torch.outer(k, v)
                ref = S.T @ q
                assert (o[t, h * V: (h + 1) * V].double().cpu() - ref).abs().max().item() < 1e-4 * max(1.0, ref.abs().max().item())
            assert (sd[slot, 1 - phase, h].double().cpu().view(V, D).T - S).abs().max().item() < 1e-4 * max(1.0, S.abs().max().item())
            assert torch.equal(sd[slot, phase, h].cpu(), state[slot, phase, h])
        row += n
    assert torch.equal(sd[1].cpu(), state[1])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(1, 24), (9, 256), (3, 1030), (40, 2048)])
def test_norm_over_all_heads_and_gate(out_dtype, rows, width):
    """The read-outs of all heads normed together (one weight over the whole row) and gated: short rows by a warp, long rows
    by a block."""
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(rows + width)
    o, gate = torch.randn(rows, width + 8, generator=g) * 3, torch.randn(rows, width + 4, generator=g)
    w = (1 + 0.2 * torch.randn(width, generator=g)).to(torch.bfloat16)
    out = torch.empty(rows, width, device="cuda", dtype=out_dtype)
    ops.head_norm_gate(out, _dev(o)[:, :width], _dev(gate)[:, 2: 2 + width], _dev(w), 1, width, 1e-5, weight_per_head=True)
    ref = plain.rms(o[:, :width].double(), 1e-5, w.double()) * torch.sigmoid(gate[:, 2: 2 + width].double())
    assert (out.double().cpu() - ref).abs().max().item() < (1e-5 if out_dtype == torch.float32 else 3e-2) * max(1.0, ref.abs().max().item())


# ---------------------------------------------------------------------------------------------- mechanisms alone
def _one_layer(layer, width=48, vocab=83, **kw):
    return model(vocab, width, [layer], **kw)


W_ROT = rot(8, 1000.0, STRETCH)
MECHANISMS = {
    "norms alone around linear attention of one head": _one_layer(lightning(1, 8, 8, (0.9,))),
    "linear attention with decays from none to everything": _one_layer(lightning(4, 16, 24, (0.0, 0.5, 0.99, 1.0))),
    "plain grouped attention": _one_layer(attn(4, 2, 16, 16, 0.5)),
    "window": _one_layer(attn(2, 1, 16, 16, 0.5, window=18)),
    "window with kept first keys": _one_layer(attn(2, 1, 16, 16, 0.5, window=18, keep_first=5)),
    "filter of four taps": _one_layer(attn(2, 2, 8, 8, 0.7, conv=4)),
    "rotation of half a head, stretched": _one_layer(attn(3, 1, 16, 8, 0.5, rot=W_ROT)),
    "rotation of the whole head": _one_layer(attn(2, 1, 16, 24, 0.5, rot=rot(16, 100.0))),
    "keys wider than values and heads of 264": _one_layer(attn(2, 1, 264, 40, 0.08, window=40, keep_first=2, conv=2, rot=rot(64, 10000.0))),
    "latent without stretched waves": _one_layer(latent(3, 8, 4, 12, 20, 0.6, base=100.0)),
    "latent with stretched waves": _one_layer(latent(2, 16, 16, 8, 24, 0.5, base=10000.0, scaling=STRETCH)),
    "latent with one head": _one_layer(latent(1, 8, 2, 8, 8, 0.8)),
    "experts alone, all of them": _one_layer(lightning(1, 8, 8, (0.5,), mlp=moe(20, 3, 3))),
    "one expert a row out of the best of nine groups": _one_layer(lightning(1, 8, 8, (0.5,), mlp=moe(12, 9, 1, groups=(9, 1)))),
    "experts of the two best of four groups": _one_layer(lightning(1, 8, 8, (0.5,), mlp=moe(12, 16, 3, groups=(4, 2), limit=0.05))),
    "no cap on the logits": _one_layer(latent(1, 8, 2, 8, 8, 0.8), softcap=0.0),
    "a cap that bites": _one_layer(latent(1, 8, 2, 8, 8, 0.8), softcap=0.5),
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


def test_a_latent_read_by_a_later_layer(tmp_path):
    """Two readers of one latent, one directly behind it and one further back, with their own heads and sizes."""
    cfg = model(83, 48, [latent(3, 8, 4, 12, 20, 0.6, base=100.0, mlp=moe(12, 4, 2)), latent(2, 12, 4, 6, 20, 0.5, base=100.0, kv_from=0),
                         lightning(1, 8, 8, (0.9,)), latent(4, 6, 4, 10, 20, 0.7, base=100.0, kv_from=0)])
    path = make_folder(str(tmp_path / "m"), cfg, 3)
    requests = {"a": tokens_for(cfg, 90, 1), "b": tokens_for(cfg, 33, 2)}
    for dtype in DTYPES:
        runner = runner_for(path, dtype, max_tokens=256)
        check_trace(runner, path, requests, trace_tail(requests, tail=20), dtype, "readers")
        check_trace(runner, path, requests, trace_portions(requests, sizes=(2, 7, 1, 16, 3)), dtype, "readers/portions")


def test_the_stream_behind_every_layer(folders):
    """The residual stream after each layer, taken from the engine's blocks, against the plain implementation's."""
    name = "A"
    cfg, tensors = read_folder(folders[name])
    toks = tokens_for(cfg, 40, 9)
    ref = []
    plain.forward(cfg, tensors, toks, layers_out=ref)
    runner = runner_for(folders[name], "float32", graphs=False)
    runner.stream_probe = []
    replay_in_process(runner, trace_whole({"s": toks}))
    assert len(runner.stream_probe) == len(ref)
    for i, (got, want) in enumerate(zip(runner.stream_probe, ref)):
        assert (got.double().cpu() - want).abs().max().item() < 2e-5 * max(1.0, want.abs().max().item()), f"layer {i}"


def test_mechanisms_show_in_the_logits(tmp_path):
    """The comparison sees each mechanism: the plain implementation with the mechanism left out (or off by one) differs
    from the engine by far more than the engine does from the right one."""
    cfg = model(83, 48, [
        attn(4, 2, 16, 8, 1.0, window=18, keep_first=4, conv=3, rot=rot(8, 100.0, STRETCH), mlp=moe(20, 6, 2, groups=(3, 2), limit=0.1)),
        lightning(2, 8, 12, (0.8, 0.98)),
        latent(3, 8, 4, 12, 20, 0.9, base=100.0, scaling=STRETCH)], softcap=3.0)
    path = make_folder(str(tmp_path / "m"), cfg, 11)
    raw, tensors = read_folder(path)
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

    seen = max(5e-5, 20 * (got - ref).abs().max().item() / size)
    L0, L1, L2 = (lambda c: c["layers"][0]["mixer"]), (lambda c: c["layers"][1]["mixer"]), (lambda c: c["layers"][2]["mixer"])
    assert without(lambda c: L0(c).pop("conv")) > seen
    assert without(lambda c: L0(c)["mask"].__setitem__("size", 17)) > seen
    assert without(lambda c: L0(c)["mask"].__setitem__("size", 19)) > seen
    assert without(lambda c: L0(c)["mask"].__setitem__("keep_first", 0)) > seen
    assert without(lambda c: L0(c)["rot"].pop("scaling")) > seen
    assert without(lambda c: L0(c)["rot"].__setitem__("base", 200.0)) > seen
    assert without(lambda c: L0(c).pop("rot")) > seen
    assert without(lambda c: L1(c).__setitem__("decay", [0.8, 0.9])) > seen
    assert without(lambda c: L2(c)["rot"].pop("scaling")) > seen
    assert without(lambda c: c["layers"][0]["mlp"]["router"].pop("groups")) > seen
    assert without(lambda c: c["layers"][0]["mlp"]["expert"].__setitem__("limit", 5.0)) > seen
    assert without(lambda c: c.__setitem__("logit_softcap", 0.0)) > seen
    assert without(lambda c: c["norm"].__setitem__("eps", 1e-1)) > seen
    assert without(None, lambda t: t.__setitem__("l0.mix.q.b", t["l0.mix.q.b"] * 0)) > seen
    assert without(None, lambda t: t.__setitem__("l0.mix.v.b", t["l0.mix.v.b"] * 0)) > seen
    assert without(None, lambda t: t.__setitem__("l0.mlp.correction", t["l0.mlp.correction"] * -3)) > seen
    assert without(None, lambda t: t.__setitem__("l1.mix.g", t["l1.mix.g"] * 0)) > seen
    assert without(None, lambda t: t.__setitem__("l1.mix.norm", t["l1.mix.norm"] * 0 + 1)) > seen
    assert without(None, lambda t: t.__setitem__("embed.norm.alpha", t["embed.norm.alpha"] * 0.5)) > seen
    assert without(None, lambda t: t.__setitem__("l1.norm1b.b", t["l1.norm1b.b"] + 0.3)) > seen
    assert without(None, lambda t: t.__setitem__("final.norm.alpha", t["final.norm.alpha"] * 0.5)) > seen


# ---------------------------------------------------------------------------------------------- the model
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_whole_prompts_and_decoding_match_plain(folders, name, dtype):
    """Whole prompts in one step (the first tokens of a sequence among them: one and two tokens); then most of a prompt
    in one step and its last 80 tokens one by one through recorded graphs, far enough for every window to pass over decoded
    tokens."""
    cfg = CASES[name][0]
    requests = {f"w{n}": tokens_for(cfg, n, 100 + n) for n in (1, 2, 37, 200)}
    runner = runner_for(folders[name], dtype)
    check_trace(runner, folders[name], requests, trace_whole(requests), dtype, f"{name}/whole")
    del requests["w1"], requests["w2"]
    check_trace(runner, folders[name], requests, trace_tail(requests, tail=80), dtype, f"{name}/decode")


@pytest.mark.parametrize("name", ["A", "D"])
def test_prefill_equals_token_by_token(folders, name):
    """A prompt fed one token a step from its first token on (cache, filter state and matrix state carry everything)
    against the whole prompt in one step: the same logits up to rounding, and both the plain implementation's."""
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
@pytest.mark.parametrize("name,page", [("A", 16), ("B", 8), ("C", 16), ("D", 32), ("E", 16), ("F", 16)])
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
    if runner.cache.groups:
        assert max(handed.values()) >= 2, "no page was used a second time"


def test_a_slot_used_again_starts_from_zero(folders):
    """The same request twice through the one state slot, with another request's matrix and filter state left there in
    between."""
    name = "D"
    cfg = CASES[name][0]
    runner = runner_for(folders[name], "float32", max_requests=1)
    for seed in (1, 2, 1):
        toks = tokens_for(cfg, 50, seed)
        check_trace(runner, folders[name], {"r": toks}, trace_tail({"r": toks}, tail=10), "float32", f"slot/{seed}")


def sharpen(path, layer=0, kinds=("q", "k", "v"), by=6.0, out_by=8.0):
    """Random weights made so that single keys decide rows: longer projections (the scores spread, the values differ from
    key to key) and a longer output projection (the mixer's result weighs in the stream)."""
    _, tensors = read_folder(path)
    tensors = dict(tensors)
    for n in kinds:
        tensors[f"l{layer}.mix.{n}"] = tensors[f"l{layer}.mix.{n}"] * by
    tensors[f"l{layer}.mix.o"] = tensors[f"l{layer}.mix.o"] * out_by
    save(path, tensors)


def _sharp_attention_model(tmp_path, window, keep, name, heads=(2, 1), dim=16, page_conv=2):
    """One attention layer whose key 'keep - 1' (the last kept one), key 'keep' (the first not kept) and the keys at the
    window's edge decide rows far behind them: the queries are lengthened so that the softmax is sharp."""
    cfg = _one_layer(attn(heads[0], heads[1], dim, min(dim, 32), 4.0 / math.sqrt(dim), window=window, keep_first=keep, conv=page_conv, rot=rot(4, 50.0)))
    path = make_folder(str(tmp_path / name), cfg, window * 7 + keep)
    sharpen(path)
    return cfg, path


def test_window_edges_and_kept_first_keys_show_in_the_logits(tmp_path):
    """The comparison is sharp enough to see a window or a number of kept keys that is one off: the plain implementation
    with either one larger or smaller differs from the engine by far more than the engine does from the right one, at prompt
    rows and at decoded ones."""
    cfg, path = _sharp_attention_model(tmp_path, 21, 6, "edges")
    raw, tensors = read_folder(path)
    toks = tokens_for(cfg, 150, 9)
    runner = runner_for(path, "float32", max_tokens=256)
    got = replay_in_process(runner, trace_tail({"e": toks}, tail=60))["e"].double()
    ref = plain.forward(raw, tensors, toks)
    scale = ref.pow(2).mean().sqrt().item()
    assert (got - ref).abs().max().item() < 2e-5 * scale
    for key in ("size", "keep_first"):
        for d in (-1, 1):
            off = json.loads(json.dumps(raw))
            off["layers"][0]["mixer"]["mask"][key] += d
            wrong = plain.forward(off, tensors, toks)
            assert (got[40:90] - wrong[40:90]).abs().max().item() > 3e-4 * scale, f"{key} one off would not be noticed in a prompt"
            assert (got[90:] - wrong[90:]).abs().max().item() > 3e-4 * scale, f"{key} one off would not be noticed while decoding"
            assert (ref[:6] - wrong[:6]).abs().max().item() < 1e-9


def test_windows_and_kept_keys_at_and_around_page_borders(tmp_path):
    """Windows of 15, 16, 17, 32 and 33 keys and 15, 16, 17, 1 and 40 kept keys with pages of 16: the oldest key seen and the
    last kept one are the last of a page, the first of one, and one to either side; prompts and decoded tokens, portions
    that end inside a page; pages behind the window are given back on the way, the kept ones are not."""
    for window, keep, dim in ((15, 16, 16), (16, 17, 32), (17, 15, 32), (32, 1, 16), (33, 40, 64), (70, 65, 32)):
        # (heads of 32 and 64 numbers: the tensor-core kernels in bfloat16, whose tiles hold 64 and 16 keys)
        cfg, path = _sharp_attention_model(tmp_path, window, keep, f"w{window}", dim=dim)
        toks = tokens_for(cfg, 190, window)
        for dtype in DTYPES:
            runner = runner_for(path, dtype, max_tokens=256)
            steps = trace_portions({"w": toks[:150]}, sizes=(13, 16, 3, 17, 21, 70))
            steps[-1]["end"] = []
            steps += [{"step": 100 + i, "entries": [{"id": "w", "tokens": [t], "want": [0]}], "end": ["w"] if i == 39 else []}
                      for i, t in enumerate(toks[150:])]
            got = replay_in_process(runner, steps)["w"]
            compare(got, path, toks, dtype, f"window {window} keep {keep} {dtype}")
        raw, tensors = read_folder(path)
        ref = oracle(path, toks)
        for key in ("size", "keep_first"):
            off = json.loads(json.dumps(raw))
            off["layers"][0]["mixer"]["mask"][key] += 1
            assert (ref - plain.forward(off, tensors, toks)).abs().max().item() > 1e-3 * ref.pow(2).mean().sqrt().item()


def test_a_far_key_among_hundreds_and_old_state(tmp_path):
    """No window and a sharp softmax: a row's weight sits on the few keys that match it best, wherever they are among 300;
    a decay of one keeps the first token in the linear attention's state for ever. The engine follows the plain
    implementation while decoding, and one that sees only the last 200 keys, or forgets, does not."""
    for layer in (attn(4, 2, 16, 24, 1.2, conv=2, rot=rot(8, 10000.0)), latent(3, 16, 8, 12, 24, 1.2, base=10000.0)):
        cfg = _one_layer(layer)
        path = make_folder(str(tmp_path / layer["type"]), cfg, 11)
        sharpen(path, kinds=("q", "k", "v") if layer["type"] == "attention" else ("q", "uv"))
        raw, tensors = read_folder(path)
        toks = tokens_for(cfg, 300, 5)
        runner = runner_for(path, "float32", max_tokens=512)
        got = replay_in_process(runner, trace_tail({"f": toks}, tail=60))["f"].double()
        ref = plain.forward(raw, tensors, toks)
        scale = ref.pow(2).mean().sqrt().item()
        assert (got - ref).abs().max().item() < 1e-4 * scale
        if layer["type"] == "attention":
            near = json.loads(json.dumps(raw))
            near["layers"][0]["mixer"]["mask"] = {"size": 200}
            wrong = plain.forward(near, tensors, toks)
            assert (ref[240:] - wrong[240:]).abs().max().item() > 1e-2 * scale, "lost far keys would not be noticed"
        else:
            other = plain.forward(raw, tensors, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
            assert (ref[240:] - other[240:]).abs().max().item() > 100 * (got - ref).abs().max().item()
    cfg = _one_layer(lightning(2, 8, 8, (1.0, 0.999)))
    path = make_folder(str(tmp_path / "lin"), cfg, 12)
    raw, tensors = read_folder(path)
    toks = tokens_for(cfg, 400, 6)
    runner = runner_for(path, "float32", max_tokens=512)
    got = replay_in_process(runner, trace_tail({"f": toks}, tail=100))["f"].double()
    ref = plain.forward(raw, tensors, toks)
    other = plain.forward(raw, tensors, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert (ref[300:] - other[300:]).abs().max().item() > 100 * (got - ref).abs().max().item(), "the first token would not be missed"


def test_long_decoding(folders):
    """600 single-token steps behind a short prompt: matrix state, filter state, windows, kept keys and released pages over
    a long run."""
    name = "D"
    cfg = CASES[name][0]
    toks = tokens_for(cfg, 620, 77)
    runner = runner_for(folders[name], "float32", max_tokens=704)
    got = replay_in_process(runner, trace_tail({"l": toks}, tail=600))["l"]
    compare(got, folders[name], toks, "float32", "long decoding")


@pytest.mark.parametrize("name", ["A", "E"])
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
