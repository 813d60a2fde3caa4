"""Delunex in the engine against the plain implementation: every mechanism's kernel alone, whole prompts, decoding
through the cache, portions, mixed batches, pages and slots that are used again, window edges, greedy generation
through the scheduler, the command line and the trace program."""
import dataclasses
import json
import os
import random
import subprocess
import sys

import pytest
import torch

import plain_delunex as plain
from delunex_cases import CASES, assert_logits, make_folder, oracle, read_folder, tokens_for
from helpers import (ROOT, count_page_handouts, replay_in_process, replay_trace_run, round64, trace_mixed, trace_portions,
                     trace_tail, trace_whole)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(str(tmp_path_factory.mktemp(f"dlx{n}")), cfg, seed) for n, (cfg, seed) in CASES.items()}


def runner_for(path, dtype, max_tokens=2048, max_requests=4, page_size=16, graphs=True):
    from openinfer_b200.engine.runner import ModelRunner
    r = ModelRunner.from_folder(path, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, page_size=page_size)
    r.cuda_graph = graphs
    return r


def check_trace(runner, path, requests, steps, dtype, what):
    got = replay_in_process(runner, steps)
    for rid, toks in requests.items():
        assert_logits(got[rid], oracle(path, toks), dtype, f"{what}/{rid}")
    runner.cache.check()
    assert runner.cache.min_free_pages() == runner.cache.num_pages and runner.cache.slot_pool.used_count == 0


# ---------------------------------------------------------------------------------------------- kernels alone
def _dev(t, dtype=None):
    return t.to(device="cuda", dtype=dtype or t.dtype)


@pytest.mark.parametrize("taps,channels", [(1, 24), (2, 40), (3, 64), (5, 300), (3, 30), (9, 32), (4, 1030)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_short_conv_kernel_portions_and_state(taps, channels, out_dtype):
    """Three requests in three steps of unequal portions (one token, fewer than taps - 1, many): every step's output
    equals the convolution of the whole sequence, whatever the cutting, and slots are independent."""
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(taps * 100 + channels)
    lens = [11, 1 + 2 * taps, 7]
    seqs = [torch.randn(n, channels, generator=g, dtype=torch.float64) for n in lens]
    w = torch.randn(channels, taps, generator=g, dtype=torch.float64).to(torch.bfloat16)
    want = [s + plain.causal_conv(s, w.double()) for s in seqs]
    cuts = [[1, 2, 8], [taps, 1, taps], [3, 3, 1]]                 # per request: its portions, step by step
    slots = [2, 0, 3]
    state = torch.full((4, 2, max(taps - 1, 1), channels), 7.0, device="cuda")[:, :, : taps - 1].contiguous()
    state[slots] = 0                                               # an opened request's state is zero; slot 1 is someone else's
    at = [0, 0, 0]
    for step in range(3):
        rows = [seqs[b][at[b]: at[b] + cuts[b][step]] for b in range(3)]
        x = _dev(torch.cat(rows), torch.float32)
        cu = torch.tensor([0] + list(torch.tensor([r.shape[0] for r in rows]).cumsum(0)), dtype=torch.int32, device="cuda")
        req = torch.cat([torch.full((r.shape[0],), b, dtype=torch.int32) for b, r in enumerate(rows)]).cuda()
        out = torch.empty(x.shape, dtype=out_dtype, device="cuda")
        # the two copies of a request's state take turns: its second request sits the first step's phase out of step
        phase = torch.tensor([step & 1, (step + 1) & 1, step & 1], dtype=torch.int32, device="cuda")
        if step == 0 and taps > 1:
            state[0, 0].copy_(state[0, 1])                         # (request 1 starts in phase 1: its zeros are there already)
        ops.short_conv(out, x, _dev(w), state if taps > 1 else None, cu, req, torch.tensor(slots, dtype=torch.int32, device="cuda"),
                       phase if taps > 1 else None)
        ref = torch.cat([want[b][at[b]: at[b] + cuts[b][step]] for b in range(3)])
        tol = 1e-5 if out_dtype == torch.float32 else 2e-2
        assert (out.double().cpu() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
        at = [a + c[step] for a, c in zip(at, cuts)]
    if taps > 1:
        assert (state[1] == 7.0).all()                             # a slot no request of the steps held


@pytest.mark.parametrize("taps,channels,act", [(4, 64, "none"), (3, 1032, "silu"), (2, 40, "silu"), (5, 30, "none"), (9, 32, "silu")])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_short_conv_on_columns_of_wider_rows(taps, channels, act, dtype):
    """The filter alone (no input added) on a slice of columns of a wider buffer, into a slice of another, with and without
    the activation, in two steps of unequal portions: the columns beside the slices stay as they were."""
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(taps + channels)
    lens, cuts, slots = [9, 2 * taps + 20], [[2, 7], [taps + 17, taps + 3]], [1, 0]
    seqs = [torch.randn(n, channels, generator=g).to(dtype) for n in lens]
    w = torch.randn(channels, taps, generator=g).to(torch.bfloat16)
    want = [plain.causal_conv(s.double(), w.double()) for s in seqs]
    if act == "silu":
        want = [v * torch.sigmoid(v) for v in want]
    state = torch.zeros((2, 2, taps - 1, channels), device="cuda")
    at = [0, 0]
    for step in range(2):
        rows = [seqs[b][at[b]: at[b] + cuts[b][step]] for b in range(2)]
        n = sum(r.shape[0] for r in rows)
        wide_in = torch.full((n, channels + 24), 3.0, dtype=dtype, device="cuda")
        wide_in[:, 16: 16 + channels] = _dev(torch.cat(rows))
        wide_out = torch.full((n, channels + 12), 5.0, dtype=dtype, device="cuda")
        cu = torch.tensor([0, rows[0].shape[0], n], dtype=torch.int32, device="cuda")
        req = torch.cat([torch.full((r.shape[0],), b, dtype=torch.int32) for b, r in enumerate(rows)]).cuda()
        phase = torch.full((2,), step & 1, dtype=torch.int32, device="cuda")
        ops.short_conv_act(wide_out[:, 8: 8 + channels], wide_in[:, 16: 16 + channels], _dev(w), state, cu, req,
                           torch.tensor(slots, dtype=torch.int32, device="cuda"), phase, act=act, add_input=False)
        ref = torch.cat([want[b][at[b]: at[b] + cuts[b][step]] for b in range(2)])
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert (wide_out[:, 8: 8 + channels].double().cpu() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
        assert (wide_out[:, :8] == 5.0).all() and (wide_out[:, 8 + channels:] == 5.0).all() and (wide_in[:, :16] == 3.0).all()
        at = [a + c[step] for a, c in zip(at, cuts)]


@pytest.mark.parametrize("a_dtype", [torch.float32, torch.bfloat16])
def test_branch_norm_add_and_history_kernels(a_dtype):
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    rows, hidden, n_prev = 9, 72, 3
    h = torch.randn(rows, hidden, generator=g)
    a = torch.randn(rows, hidden, generator=g).to(a_dtype)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    coef = torch.randn(n_prev + 1, generator=g).to(torch.bfloat16)
    hist = torch.randn(n_prev + 2, rows, hidden, generator=g)
    v = h.double() + plain.rms(a.double(), w.double(), 1e-5)
    # plain
    hd = _dev(h.clone())
    ops.branch_norm_add(hd, _dev(a), _dev(w), 1e-5)
    assert (hd.double().cpu() - v).abs().max().item() < 1e-5
    # with the average and the rounded copy
    hd, histd = _dev(h.clone()), _dev(hist.clone())
    low = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
    ops.branch_norm_add(hd, _dev(a), _dev(w), 1e-5, history=histd, n_prev=n_prev, coef=_dev(coef), low=low)
    avg = sum(coef[j].double() * hist[j].double() for j in range(n_prev)) + coef[n_prev].double() * v
    assert (histd[n_prev].double().cpu() - v).abs().max().item() < 1e-5
    assert (hd.double().cpu() - avg).abs().max().item() < 2e-5
    assert torch.equal(low.cpu(), hd.cpu().to(torch.bfloat16))
    assert torch.equal(histd[n_prev + 1].cpu(), hist[n_prev + 1]) and torch.equal(histd[:n_prev].cpu(), hist[:n_prev])
    # the average alone
    hd, histd = _dev(h.clone()), _dev(hist.clone())
    ops.history_average(hd, histd, n_prev, _dev(coef))
    avg = sum(coef[j].double() * hist[j].double() for j in range(n_prev)) + coef[n_prev].double() * h.double()
    assert (hd.double().cpu() - avg).abs().max().item() < 2e-5 and torch.equal(histd[n_prev].cpu(), h)


def test_rmsnorm_cast_latent_store_head_gate_xielu_kernels():
    from openinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    # norm from a float32 stream into bfloat16 rows, gathered
    x = torch.randn(7, 100, generator=g) * 3
    w = (1 + 0.1 * torch.randn(100, generator=g)).to(torch.bfloat16)
    idx = torch.tensor([5, 0, 5, 2], dtype=torch.int32)
    out = torch.empty(4, 100, dtype=torch.bfloat16, device="cuda")
    ops.rmsnorm_cast(out, _dev(x), _dev(w), 1e-6, row_idx=_dev(idx))
    ref = plain.rms(x.double(), w.double(), 1e-6)[idx.long()]
    assert (out.double().cpu() - ref).abs().max().item() < 2e-2 and out.dtype == torch.bfloat16
    # latent: norm of a slice of wider rows, written to the rows' slots of pages whose rows are padded
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        rank, row, page, pages = 36, 40, 4, 6
        src = (torch.randn(5, 90, generator=g) * 2).to(dtype)
        wn = (1 + 0.1 * torch.randn(rank, generator=g)).to(torch.bfloat16)
        slots = torch.tensor([9, 2, -1, 23, 0], dtype=torch.int32)
        store = torch.full((pages, page, 1, row), 5.0, dtype=dtype, device="cuda")
        ops.latent_store(store, page * row, _dev(src)[:, 17: 17 + rank], _dev(wn), _dev(slots), rank, 1e-5)
        ref = plain.rms(src[:, 17: 17 + rank].double(), wn.double(), 1e-5)
        flat = store.view(pages * page, row).double().cpu()
        for t, s in enumerate(slots.tolist()):
            if s >= 0:
                assert (flat[s, :rank] - ref[t]).abs().max().item() < tol * max(1.0, ref.abs().max().item())
                assert (flat[s, rank:] == 0).all()
        untouched = [s for s in range(pages * page) if s not in slots.tolist()]
        assert (flat[untouched] == 5.0).all()
    # gate per head, read from wider rows
    o = torch.randn(6, 3 * 8, generator=g).to(torch.bfloat16)
    gl = torch.randn(6, 11, generator=g).to(torch.bfloat16)
    od = _dev(o.clone())
    ops.head_gate(od, _dev(gl)[:, 4:7], 3, 8)
    ref = (o.double().view(6, 3, 8) * torch.sigmoid(gl[:, 4:7].double())[:, :, None]).view(6, 24)
    assert (od.double().cpu() - ref).abs().max().item() < 2e-2
    # xIELU on both sides of zero, large arguments included
    z = torch.cat([torch.linspace(-30, 30, 999), torch.tensor([0.0, -1e-4, 1e-4])])
    pq = torch.tensor([0.3, -1.2])
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        zd = _dev(z, dtype)
        out = torch.empty_like(zd)
        ops.xielu(out, zd, _dev(pq))
        ref = plain.xielu(zd.double().cpu(), pq[0].double(), pq[1].double())
        assert ((out.double().cpu() - ref).abs() <= tol * (1 + ref.abs())).all()


# ---------------------------------------------------------------------------------------------- the model
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_whole_prompts_and_decoding_match_plain(folders, name, dtype):
    """Whole prompts in one step; then most of a prompt in one step and its last 70 tokens one by one (through
    recorded graphs), far enough for every window to pass over decoded tokens."""
    cfg = CASES[name][0]
    requests = {f"w{n}": tokens_for(cfg, n, 100 + n) for n in (1, 2, 37, 230)}
    runner = runner_for(folders[name], dtype)
    check_trace(runner, folders[name], requests, trace_whole(requests), dtype, f"{name}/whole")
    del requests["w1"], requests["w2"]
    check_trace(runner, folders[name], requests, trace_tail(requests, tail=70), dtype, f"{name}/decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_portions_down_to_two_tokens(folders, name, dtype):
    cfg = CASES[name][0]
    requests = {"p0": tokens_for(cfg, 190, 1), "p1": tokens_for(cfg, 45, 2)}
    runner = runner_for(folders[name], dtype, graphs=False)
    check_trace(runner, folders[name], requests, trace_portions(requests), dtype, f"{name}/portions")
    check_trace(runner, folders[name], requests, trace_portions(requests, sizes=(2, 3, 1, 2, 4)), dtype, f"{name}/small portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("A", 16), ("B", 8), ("C", 16), ("E", 32)])
def test_mixed_batches_with_pages_and_slots_used_again(folders, name, page, dtype):
    """Up to three live requests of unequal lengths, portions beside single tokens, in a pool that holds less than the
    sum of the requests and has three state slots: every request's logits are those of the request alone."""
    cfg = CASES[name][0]
    lens = [150, 3, 64, 97, 1, 33, 120, 18]
    requests = {f"m{i}": tokens_for(cfg, n, 50 + i) for i, n in enumerate(lens)}
    max_tokens = 384
    runner = runner_for(folders[name], dtype, max_tokens=max_tokens, max_requests=3, page_size=page)
    handed = count_page_handouts(runner.cache)
    steps = trace_mixed(requests, max_tokens, seed=3, max_live=3, tail=20)
    check_trace(runner, folders[name], requests, steps, dtype, f"{name}/mixed")
    assert max(handed.values()) >= 2, "no page was used a second time"


def test_window_edges_show_in_the_logits(folders):
    """The comparison is sharp enough to see a window that is one key off: the plain implementation with every window
    one longer or one shorter differs from the engine by far more than the bound, at prompt rows and at decoded ones."""
    name = "A"
    cfg, tensors = read_folder(folders[name])
    toks = tokens_for(cfg, 120, 9)
    requests = {"e": toks}
    runner = runner_for(folders[name], "float32")
    got = replay_in_process(runner, trace_tail(requests, tail=60))["e"].double()
    assert_logits(got, oracle(folders[name], toks), "float32", "edges")
    for delta in (-1, 1):
        off = json.loads(json.dumps(cfg))
        for layer in off["layers"]:
            if layer["mixer"].get("mask"):
                layer["mixer"]["mask"]["size"] += delta
        wrong = plain.forward(off, tensors, toks)
        assert (got - wrong).abs().max().item() > 1e-2, "a window one key off would not be noticed"
        assert (got[:15] - wrong[:15]).abs().max().item() < 1e-4     # before any window is full the two agree


def test_far_keys_reach_a_layer_without_a_window(folders):
    """A layer without a window sees the first tokens from far away, also while decoding: the engine agrees with the
    plain implementation, and a plain implementation that cuts that layer's view at 200 keys does not."""
    name = "C"
    cfg, tensors = read_folder(folders[name])
    toks = tokens_for(cfg, 400, 21)
    runner = runner_for(folders[name], "float32")
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:250], "want": []}], "end": []}]
    steps += [{"step": 1 + i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": ["x"] if i == 149 else []}
              for i, t in enumerate(toks[250:])]
    got = replay_in_process(runner, steps)["x"].double()
    assert_logits(got, oracle(folders[name], toks)[250:], "float32", "far keys")
    near = json.loads(json.dumps(cfg))
    near["layers"][1]["mixer"]["mask"] = {"size": 200}
    assert (got - plain.forward(near, tensors, toks)[250:]).abs().max().item() > 1e-2, "lost far keys would not be noticed"


@pytest.mark.parametrize("dtype", DTYPES)
def test_up_projections_applied_in_every_step_give_the_same_logits(folders, dtype):
    """The mixer's other mode (queries and outputs pass through the per-head up-projections in every step instead of
    the up-projections being multiplied into the weights at load time) computes the same function."""
    from openinfer_b200.cache.manager import CacheManager
    from openinfer_b200.config.base import load_config, resolve_architecture
    from openinfer_b200.engine.runner import ModelRunner, _dtype_of
    from openinfer_b200.parts.model import Model
    from openinfer_b200.weights.loader import load_tensors
    name = "A"
    config = load_config(folders[name])
    spec = resolve_architecture(config.to_dict()).build_spec(config)
    spec = dataclasses.replace(spec, blocks=tuple(
        dataclasses.replace(b, mixer=dataclasses.replace(b.mixer, absorb="runtime")) for b in spec.blocks))
    model = Model(spec, _dtype_of(dtype))
    model.load(load_tensors(folders[name], model.expected_tensors(), _dtype_of(dtype), "cuda:0"), "cuda:0")
    cache = CacheManager(page_size=16)
    model.bind_cache(cache)
    cache.allocate(64, 4, device=torch.device("cuda:0"), dtype=_dtype_of(dtype))
    runner = ModelRunner(model, cache, torch.device("cuda:0"))
    requests = {"r0": tokens_for(CASES[name][0], 90, 4), "r1": tokens_for(CASES[name][0], 31, 5)}
    check_trace(runner, folders[name], requests, trace_portions(requests, sizes=(40, 1, 1, 9, 2)), dtype, "runtime absorb")


def test_shared_latent_pages_outlive_the_owners_window(folders):
    """A layer that reads another layer's latent through a longer window (or none) keeps that layer's pages alive for
    as long as it needs them; layers that own their latent with a window give pages back while the request runs."""
    runner = runner_for(folders["A"], "float32", max_tokens=1024)
    windows = sorted((g.window is None, g.window) for g in runner.cache.groups)
    assert windows == [(False, 50), (True, None)]       # layer 0 (21) widened by its reader (50); layer 2 (17) by one with none
    from openinfer_b200.engine.runner import StepEntry
    runner.step([StepEntry("a", tokens_for(CASES["A"][0], 200, 1), [])])
    held = [sum(1 for p in runner.cache.block_table("a", g) if p >= 0) for g in range(len(runner.cache.groups))]
    by_window = {runner.cache.groups[g].window: held[g] for g in range(len(held))}
    assert by_window[None] == 13 and by_window[50] == 13 - (200 - 50 + 1) // 16
    runner.end("a")


@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation_through_the_scheduler(folders, name):
    from openinfer_b200 import LLM
    cfg, tensors = read_folder(folders[name])
    prompts = [tokens_for(cfg, n, 70 + n) for n in (1, 9, 33, 70)]
    n_new = 25

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
    # bfloat16 with sampling: runs, is reproducible under a seed, and leaves nothing behind
    from openinfer_b200 import SamplingParams
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
    requests = {f"t{i}": tokens_for(cfg, n, 30 + i) for i, n in enumerate([80, 5, 130, 41, 1])}
    max_tokens = round64(130) + round64(80) + 64
    steps = trace_mixed(requests, max_tokens, seed=1, max_live=4, tail=16)
    for dtype in DTYPES:
        got = replay_trace_run(folders[name], dtype, steps, str(tmp_path / dtype), max_tokens, cfg["vocab"])
        for rid, t in requests.items():
            assert_logits(got[rid], oracle(folders[name], t), dtype, f"trace_run/{dtype}/{rid}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_native_step_and_part_by_part_step_give_the_same_bits(folders, name, dtype):
    """All layers of a step launched by one native call, or the parts called one by one from Python: the same kernels
    with the same arguments, so the same bits, in prompt portions, mixed steps and recorded single-token steps."""
    cfg = CASES[name][0]
    requests = {f"n{i}": tokens_for(cfg, n, 80 + i) for i, n in enumerate([70, 9, 41])}
    steps = trace_mixed(requests, 512, seed=2, max_live=3, tail=12)
    out = []
    for native in (True, False):
        runner = runner_for(folders[name], dtype, max_tokens=512)
        runner.model.native_step = native
        out.append(replay_in_process(runner, steps))
        # (a bfloat16 model whose first layer has no filter in front of its mixer is always run part by part)
        assert (runner.model._native is not None) == (native and not (dtype == "bfloat16" and "canon" not in cfg))
    for rid in requests:
        assert torch.equal(out[0][rid], out[1][rid]), f"{name}/{dtype}/{rid}"


@pytest.mark.parametrize("rows", [1, 8, 32, 33, 100, 300, 2100])
def test_dense_feed_forward_with_the_activation_in_the_products_epilogue(rows):
    """bfloat16 at sizes the tensor-core products take: up to 32 rows the weight stream applies the activation where it
    adds up its K slices, beyond that the tcgen05 tiles in their epilogue (pairs of CTAs from 2,048 rows); the result is
    the plain feed-forward's. A size they refuse goes through the plain product and the activation kernel."""
    from openinfer_b200.parts.mlp import DenseMlp
    from openinfer_b200.parts.spec import DenseMlpSpec
    from openinfer_b200.kernels import gemm_tcgen05, linear
    g = torch.Generator().manual_seed(rows)
    for hidden, inter in ((256, 768), (72, 100)):
        part = DenseMlp(DenseMlpSpec(hidden_size=hidden, intermediate_size=inter))
        w = {"up": torch.randn(inter, hidden, generator=g) * hidden ** -0.5, "down": torch.randn(hidden, inter, generator=g) * inter ** -0.5,
             "act": torch.tensor([0.4, -0.8])}
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
        part.load({k: _dev(v) for k, v in w.items()})
        x = (torch.randn(rows, hidden, generator=g) * 1.5).to(torch.bfloat16)
        got = part.forward(_dev(x), None)
        assert got.dtype == torch.float32
        ref = plain.dense_ff(x.double(), w["up"].double(), w["down"].double(), w["act"].double())
        err = (got.double().cpu() - ref).abs().max().item() / ref.abs().max().item()
        assert err < 2e-2, f"rows {rows} hidden {hidden}: {err}"
    assert gemm_tcgen05.status() == 0 and linear.stream_status() == 0
