"""Python wrappers of the CUDA entry points: shape and dtype checks, pointers, error mapping.

Every function takes torch tensors that live on the CUDA device and launches on
the current stream. None of them has another implementation to fall back to.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import lib as _lib
from .lib import KernelError

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(
                "a kernel was given a tensor that is not on a CUDA device; "
                "this package has no CPU path"
            )


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _stream() -> int:
    return _lib.current_stream()


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{what} must be a contiguous int32 tensor")


def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[ids[t], :]"""
    _cuda(out, table, ids)
    _i32(ids, "embedding ids")
    tokens, hidden = out.shape
    if table.shape[1] != hidden or ids.numel() != tokens or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError(f"embedding: shapes out={tuple(out.shape)} table={tuple(table.shape)} ids={tuple(ids.shape)}")
    L = _lib.load()
    _lib.check(L.oi_embedding(out.data_ptr(), _code(out, "embedding"), table.data_ptr(), _code(table, "embedding"),
                              ids.data_ptr(), tokens, hidden, table.shape[0], _stream()), "embedding")
    return out


def gather_tokens(ids: torch.Tensor, src: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """ids[i] = tokens[src[i]] wherever src[i] >= 0 (all int32, on the device)."""
    _cuda(ids, src, tokens)
    _i32(ids, "gather_tokens ids")
    _i32(src, "gather_tokens src")
    _i32(tokens, "gather_tokens tokens")
    if ids.numel() != src.numel() or not (ids.is_contiguous() and src.is_contiguous() and tokens.is_contiguous()):
        raise KernelError("gather_tokens: ids and src must be contiguous and of one length")
    L = _lib.load()
    _lib.check(L.oi_gather_tokens(ids.data_ptr(), src.data_ptr(), tokens.data_ptr(), ids.numel(), tokens.numel(),
                                  _stream()), "gather_tokens")
    return ids


def copy_words(dst: torch.Tensor, src: torch.Tensor, n: int, *, ids_off: int = -1, src_off: int = 0, n_ids: int = 0,
               tokens: Optional[torch.Tensor] = None, fence: bool = False) -> None:
    """dst[:n] = src[:n] (int32) by a kernel; one of the two may be pinned host memory, which the device
    reads or writes directly. With ``ids_off >= 0`` the words [ids_off, ids_off + n_ids) are token ids:
    where the source index at ``src_off`` is >= 0 the id comes from ``tokens`` (int32, on the device).
    ``fence``: what is copied is read by later kernels before their own wait for their predecessor (a step's
    lengths, block tables, positions, work items): the kernel launched next then gets plain stream order."""
    for t, what in ((dst, "dst"), (src, "src")):
        if t.dtype != torch.int32 or not t.is_contiguous() or t.numel() < n or not (t.is_cuda or t.is_pinned()):
            raise KernelError(f"copy_words: {what} must be contiguous int32 of at least {n} words, on the device or pinned")
    if tokens is not None:
        _cuda(tokens)
        _i32(tokens, "copy_words tokens")
    L = _lib.load()
    _lib.check(L.oi_copy_words(dst.data_ptr(), src.data_ptr(), int(n), int(ids_off), int(src_off), int(n_ids),
                               _ptr(tokens), 0 if tokens is None else tokens.numel(), _stream()), "copy_words")
    if fence:
        L.oi_launch_fence()


class UploadRing:
    """Small host arrays of int32 to the device without a copy-engine operation and without making the host wait
    for the stream: a ring of pinned buffers that a kernel reads (``copy_words``), each guarded by the event of its
    last use."""

    def __init__(self, slots: int = 4) -> None:
        self.slots = slots
        self.buffers: list = []
        self.events: list = []
        self.turn = 0

    def upload(self, host, device) -> torch.Tensor:
        n = int(host.size)
        if not self.buffers or self.buffers[0].numel() < n:
            if self.buffers:
                torch.cuda.current_stream().synchronize()   # kernels in flight may still read the old buffers
            self.buffers = [torch.empty(max(4096, 2 * n), dtype=torch.int32, pin_memory=True) for _ in range(self.slots)]
            self.events = [None] * self.slots
        self.turn = (self.turn + 1) % self.slots
        if self.events[self.turn] is not None:
            self.events[self.turn].synchronize()
        buf = self.buffers[self.turn]
        buf[:n].numpy()[:] = host
        dev = torch.empty(max(n, 1), dtype=torch.int32, device=device)
        if n:
            copy_words(dev, buf, n, fence=True)
        event = torch.cuda.Event()
        event.record()
        self.events[self.turn] = event
        return dev[:n]


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float, *,
            delta: Optional[torch.Tensor] = None, row_idx: Optional[torch.Tensor] = None,
            weight_offset: float = 0.0) -> torch.Tensor:
    """out = x * rsqrt(mean(x^2) + eps) * (weight_offset + weight), row by row.

    ``delta``: x <- x + delta first (stored in x), the norm is of the sum.
    ``row_idx``: output row r reads x[row_idx[r]].
    """
    _cuda(out, x, weight, delta, row_idx)
    _i32(row_idx, "rmsnorm row_idx")
    hidden = x.shape[-1]
    rows = out.shape[0]
    if out.dtype != x.dtype or (delta is not None and (delta.dtype != x.dtype or delta.shape != x.shape)):
        raise KernelError("rmsnorm: out, x and delta must share a dtype and shape")
    if not (out.is_contiguous() and x.is_contiguous() and weight.is_contiguous()) or weight.numel() != hidden:
        raise KernelError(f"rmsnorm: shapes x={tuple(x.shape)} weight={tuple(weight.shape)}")
    if delta is not None and not delta.is_contiguous():
        raise KernelError("rmsnorm: delta must be contiguous")
    if out.shape[-1] != hidden or (row_idx is None and rows != x.shape[0]) or (row_idx is not None and row_idx.numel() != rows):
        raise KernelError("rmsnorm: row counts do not match")
    L = _lib.load()
    _lib.check(L.oi_rmsnorm(out.data_ptr(), x.data_ptr(), _ptr(delta), _code(x, "rmsnorm"), weight.data_ptr(),
                            _code(weight, "rmsnorm weight"), _ptr(row_idx), rows, hidden, float(eps),
                            float(weight_offset), _stream()), "rmsnorm")
    return out


def add_inplace(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    _cuda(x, delta)
    if x.dtype != delta.dtype or x.shape != delta.shape or not (x.is_contiguous() and delta.is_contiguous()):
        raise KernelError("add: operands must share dtype and shape and be contiguous")
    L = _lib.load()
    _lib.check(L.oi_add_inplace(x.data_ptr(), delta.data_ptr(), _code(x, "add"), x.numel(), _stream()), "add")
    return x


def scale_cap(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place: x = x * scale, then, with cap > 0, x = cap * tanh(x / cap)."""
    _cuda(x)
    if not x.is_contiguous():
        raise KernelError("scale_cap: the tensor must be contiguous")
    L = _lib.load()
    _lib.check(L.oi_scale_cap(x.data_ptr(), _code(x, "scale_cap"), x.numel(), float(scale), float(cap), _stream()), "scale_cap")
    return x


# gate activations of a gated feed-forward: name -> code of the C interface (common.cuh)
ACTIVATIONS = {"silu": 1, "gelu_tanh": 2}


def act_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation {name!r} has no kernel (known: {', '.join(sorted(ACTIVATIONS))})") from None


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor, block: Optional[int] = None, act: str = "silu") -> torch.Tensor:
    """out[r, i] = act(gate_i) * up_i for a fused gate|up buffer [rows, 2 * inter] laid out in
    blocks of ``block`` gate values followed by their up values (default: all gates, then all ups)."""
    _cuda(out, gate_up)
    rows, inter = out.shape
    block = inter if block is None else int(block)
    if gate_up.shape != (rows, 2 * inter) or out.dtype != gate_up.dtype or not (out.is_contiguous() and gate_up.is_contiguous()):
        raise KernelError(f"silu_mul: shapes out={tuple(out.shape)} gate_up={tuple(gate_up.shape)}")
    L = _lib.load()
    _lib.check(L.oi_silu_mul(out.data_ptr(), gate_up.data_ptr(), _code(out, "silu_mul"), rows, inter, block, act_code(act),
                             _stream()), "silu_mul")
    return out


def qk_norm_rope_kv(qkv: torch.Tensor, nq: int, nkv: int, hd: int, *, q_norm_w: Optional[torch.Tensor],
                    k_norm_w: Optional[torch.Tensor], eps: float, weight_offset: float,
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                    slots: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                    v_cache: Optional[torch.Tensor], page_stride: int, page_size: int,
                    write_kv: bool = True, interleaved: bool = False) -> None:
    """Per-head norm and rotation of q (in place) and k, and the write of k and v into
    their pages. ``qkv`` is [tokens, >= (nq + 2 nkv) * hd] (or [tokens, >= nq * hd] when
    write_kv is false); ``cos``/``sin`` are float32 [max_pos, rotary_dim / 2]; ``interleaved``: angle d turns the
    neighbours (2 d, 2 d + 1) instead of (d, d + rotary_dim / 2)."""
    _cuda(qkv, q_norm_w, k_norm_w, cos, sin, positions, slots, k_cache, v_cache)
    _i32(positions, "positions")
    _i32(slots, "slots")
    tokens = qkv.shape[0]
    width = (nq + 2 * nkv) * hd if write_kv else nq * hd
    if qkv.dim() != 2 or qkv.shape[1] < width or qkv.stride(1) != 1:
        raise KernelError(f"qk_norm_rope_kv: qkv shape {tuple(qkv.shape)} too narrow for {width}")
    if positions.numel() != tokens or (slots is not None and slots.numel() != tokens):
        raise KernelError("qk_norm_rope_kv: positions/slots length differs from the token count")
    norm_code = 0
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            if w.numel() != hd or not w.is_contiguous():
                raise KernelError("qk_norm_rope_kv: norm weight must have head_dim elements")
            norm_code = _code(w, "qk norm weight")
    if q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("qk_norm_rope_kv: q and k norm weights must share a dtype")
    rot_half, max_pos = 0, 0
    if cos is not None:
        if cos.dtype != torch.float32 or sin is None or sin.shape != cos.shape or not (cos.is_contiguous() and sin.is_contiguous()):
            raise KernelError("qk_norm_rope_kv: cos/sin must be contiguous float32 tables of one shape")
        max_pos, rot_half = cos.shape
    if write_kv:
        if k_cache is None or v_cache is None or slots is None or k_cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_kv: the cache must be given and share qkv's dtype")
    L = _lib.load()
    _lib.check(L.oi_qk_norm_rope_kv(
        qkv.data_ptr(), _code(qkv, "qk_norm_rope_kv"), qkv.stride(0), tokens, nq, nkv, hd, _ptr(q_norm_w),
        _ptr(k_norm_w), norm_code, float(eps), float(weight_offset), _ptr(cos), _ptr(sin), rot_half, max_pos,
        positions.data_ptr(), _ptr(slots), _ptr(k_cache), _ptr(v_cache), int(page_stride), int(page_size),
        1 if write_kv else 0, 1 if interleaved else 0, _stream()), "qk_norm_rope_kv")


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      page_stride: int, page_size: int, block_table: torch.Tensor, token_req: torch.Tensor,
                      positions: torch.Tensor, nq: int, nkv: int, hd: int, scale: float,
                      window: Optional[int] = None, mods=None) -> torch.Tensor:
    """Paged causal attention, one warp per (token, head). ``q`` is [tokens, >= nq*hd] with
    any row stride; ``out`` is [tokens, nq*hd]; ``block_table`` is int32 [requests, max_pages]; ``mods`` a
    ``native.ScoreMods`` (sink, slopes, cap, query temperature) or None."""
    import ctypes
    _cuda(q, out, k_cache, v_cache, block_table, token_req, positions)
    _i32(block_table, "block_table")
    _i32(token_req, "token_req")
    _i32(positions, "positions")
    tokens = out.shape[0]
    if q.shape[0] != tokens or q.stride(1) != 1 or out.stride(1) != 1 or out.shape[1] != nq * hd:
        raise KernelError(f"attention: shapes q={tuple(q.shape)} out={tuple(out.shape)}")
    if q.dtype != out.dtype or q.dtype != k_cache.dtype or q.dtype != v_cache.dtype:
        raise KernelError("attention: q, out and the cache must share a dtype")
    L = _lib.load()
    _lib.check(L.oi_attention_generic(
        q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), _code(q, "attention"), k_cache.data_ptr(),
        v_cache.data_ptr(), int(page_stride), int(page_size), block_table.data_ptr(), block_table.stride(0),
        token_req.data_ptr(), positions.data_ptr(), tokens, nq, nkv, hd, float(scale),
        int(window) if window else 0, ctypes.cast(ctypes.pointer(mods), ctypes.c_void_p) if mods is not None else None,
        _stream()), "attention")
    return out


def gemm_generic(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T, float32 accumulation on the ordinary pipes, k ascending."""
    _cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: shapes a={tuple(a.shape)} w={tuple(w.shape)} out={tuple(out.shape)}")
    L = _lib.load()
    _lib.check(L.oi_gemm_generic(out.data_ptr(), _code(out, "gemm out"), a.data_ptr(), _code(a, "gemm a"),
                                 w.data_ptr(), _code(w, "gemm w"), M, N, K, a.stride(0), w.stride(0),
                                 out.stride(0), _stream()), "gemm")
    return out


def argmax(out: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
    """out[r] = index of the largest logit of row r (lowest index on ties)."""
    _cuda(out, logits)
    _i32(out, "argmax out")
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.numel() != rows:
        raise KernelError("argmax: logits must be float32 rows")
    L = _lib.load()
    nchunks = -(-vocab // 4096)
    pv = pi = None
    if nchunks >= 4:  # a large vocabulary: many blocks per row, partial results in scratch
        pv = torch.empty(rows * nchunks, dtype=torch.float32, device=logits.device)
        pi = torch.empty(rows * nchunks, dtype=torch.int32, device=logits.device)
    _lib.check(L.oi_argmax(out.data_ptr(), logits.data_ptr(), rows, vocab, logits.stride(0), _ptr(pv), _ptr(pi),
                           _stream()), "argmax")
    return out


def token_logprobs(logits: torch.Tensor, rows: torch.Tensor, picked: torch.Tensor, ks: torch.Tensor, k_max: int):
    """For the listed rows of float32 ``logits``: (log-softmax of ``picked[i]``, the ``ks[i]`` largest
    log-probabilities [n, k_max], their ids [n, k_max]; unused places -inf / -1). All index tensors int32
    on the device."""
    _cuda(logits, rows, picked, ks)
    for t, what in ((rows, "rows"), (picked, "picked"), (ks, "ks")):
        _i32(t, f"token_logprobs {what}")
    n = rows.numel()
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or picked.numel() != n or ks.numel() != n:
        raise KernelError("token_logprobs: logits must be float32 rows; rows, picked and ks of one length")
    lp = torch.empty(n, dtype=torch.float32, device=logits.device)
    vals = torch.empty((n, max(k_max, 1)), dtype=torch.float32, device=logits.device)
    ids = torch.empty((n, max(k_max, 1)), dtype=torch.int32, device=logits.device)
    L = _lib.load()
    _lib.check(L.oi_token_logprobs(logits.data_ptr(), logits.stride(0), logits.shape[1], rows.data_ptr(), picked.data_ptr(),
                                   ks.data_ptr(), n, int(k_max), lp.data_ptr(), vals.data_ptr(), ids.data_ptr(), _stream()),
               "token_logprobs")
    return lp, vals[:, :k_max], ids[:, :k_max]


def sample_use_clusters(on: bool) -> None:
    """Whether rows that can be read 16 bytes at a time are sampled by a cluster of CTAs per row (the default) or
    every row by one block (what the clusters leave unanswered always is)."""
    _lib.check(_lib.load().oi_sample_use_clusters(1 if on else 0), "sample_use_clusters")


def sample(out: torch.Tensor, logits: torch.Tensor, probs_scratch: torch.Tensor, temperature: torch.Tensor,
           top_k: torch.Tensor, top_p: torch.Tensor, min_p: torch.Tensor, uniform: torch.Tensor) -> torch.Tensor:
    """One token per row from softmax(logits / temperature) after top-k, top-p and min-p,
    by inverse CDF at ``uniform[r]`` in [0, 1)."""
    _cuda(out, logits, probs_scratch, temperature, top_k, top_p, min_p, uniform)
    _i32(out, "sample out")
    _i32(top_k, "top_k")
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 rows")
    for t, name in ((temperature, "temperature"), (top_p, "top_p"), (min_p, "min_p"), (uniform, "uniform")):
        if t.dtype != torch.float32 or t.numel() != rows or not t.is_contiguous():
            raise KernelError(f"sample: {name} must be float32 with one entry per row")
    if top_k.numel() != rows or out.numel() != rows:
        raise KernelError("sample: top_k/out must have one entry per row")
    if probs_scratch.dtype != torch.float32 or probs_scratch.numel() < rows * vocab or not probs_scratch.is_contiguous():
        raise KernelError("sample: scratch must hold rows * vocab float32 values")
    L = _lib.load()
    _lib.check(L.oi_sample(out.data_ptr(), logits.data_ptr(), logits.stride(0), probs_scratch.data_ptr(), rows, vocab,
                           temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(),
                           uniform.data_ptr(), _stream()), "sample")
    return out


# ---------------------------------------------------------------------------
# layers with a 32-bit residual stream (csrc/branch_ops.cu)
# ---------------------------------------------------------------------------
def rmsnorm_cast(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float, *,
                 row_idx: Optional[torch.Tensor] = None, weight_offset: float = 0.0) -> torch.Tensor:
    """out = x * rsqrt(mean(x^2) + eps) * (weight_offset + weight) row by row, where x and out may differ in
    type (a float32 stream normed into the model's type). ``row_idx``: output row r reads x[row_idx[r]]."""
    _cuda(out, x, weight, row_idx)
    _i32(row_idx, "rmsnorm_cast row_idx")
    hidden, rows = x.shape[-1], out.shape[0]
    if not (out.is_contiguous() and x.is_contiguous() and weight.is_contiguous()) or weight.numel() != hidden \
            or out.shape[-1] != hidden:
        raise KernelError(f"rmsnorm_cast: shapes x={tuple(x.shape)} out={tuple(out.shape)} weight={tuple(weight.shape)}")
    if (row_idx is None and rows != x.shape[0]) or (row_idx is not None and row_idx.numel() != rows):
        raise KernelError("rmsnorm_cast: row counts do not match")
    _lib.check(_lib.load().oi_rmsnorm_cast(out.data_ptr(), _code(out, "rmsnorm_cast"), x.data_ptr(), _code(x, "rmsnorm_cast"),
                                           weight.data_ptr(), _code(weight, "rmsnorm_cast weight"), _ptr(row_idx), rows,
                                           hidden, float(eps), float(weight_offset), _stream()), "rmsnorm_cast")
    return out


def branch_norm_add(h: torch.Tensor, a: torch.Tensor, weight: torch.Tensor, eps: float, *, weight_offset: float = 0.0,
                    history: Optional[torch.Tensor] = None, n_prev: int = 0,
                    coef: Optional[torch.Tensor] = None, low: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h <- h + a * rsqrt(mean(a^2) + eps) * (weight_offset + weight) (h float32, in place; a float32 or bfloat16).
    With ``history`` [slots, rows, hidden] float32 and ``coef`` [n_prev + 1]: the sum v is stored as
    history[n_prev] and h becomes sum_{j < n_prev} coef[j] history[j] + coef[n_prev] v. ``low`` (bfloat16, h's
    shape) receives the new h rounded, for the product that reads the stream next."""
    _cuda(h, a, weight, history, coef, low)
    if low is not None and (low.dtype != torch.bfloat16 or low.shape != h.shape or not low.is_contiguous()):
        raise KernelError("branch_norm_add: low must be contiguous bfloat16 of h's shape")
    rows, hidden = h.shape
    if h.dtype != torch.float32 or a.shape != h.shape or not (h.is_contiguous() and a.is_contiguous() and weight.is_contiguous()) \
            or weight.numel() != hidden:
        raise KernelError(f"branch_norm_add: h must be contiguous float32 and a of its shape; h={tuple(h.shape)} a={tuple(a.shape)}")
    stride = 0
    if history is not None:
        if (history.dtype != torch.float32 or history.dim() != 3 or history.shape[1:] != h.shape or not history.is_contiguous()
                or not 0 <= n_prev < history.shape[0] or coef is None or coef.numel() < n_prev + 1 or not coef.is_contiguous()):
            raise KernelError("branch_norm_add: history must be contiguous float32 [slots, rows, hidden] with coef [n_prev + 1]")
        stride = history.stride(0)
    _lib.check(_lib.load().oi_branch_norm_add(h.data_ptr(), a.data_ptr(), _code(a, "branch_norm_add"), weight.data_ptr(),
                                              _code(weight, "branch_norm_add weight"), rows, hidden, float(eps),
                                              float(weight_offset), _ptr(history), stride, int(n_prev), _ptr(coef),
                                              0 if coef is None else _code(coef, "branch_norm_add coef"), _ptr(low), _stream()),
               "branch_norm_add")
    return h


def history_average(h: torch.Tensor, history: torch.Tensor, n_prev: int, coef: torch.Tensor) -> torch.Tensor:
    """history[n_prev] = h; h <- sum_{j <= n_prev} coef[j] history[j] (all float32, h in place)."""
    _cuda(h, history, coef)
    if (h.dtype != torch.float32 or history.dtype != torch.float32 or history.shape[1:] != h.shape or not h.is_contiguous()
            or not history.is_contiguous() or not 0 <= n_prev < history.shape[0] or coef.numel() < n_prev + 1):
        raise KernelError("history_average: h and history must be contiguous float32, history [slots, *h.shape]")
    _lib.check(_lib.load().oi_history_average(h.data_ptr(), history.data_ptr(), history.stride(0), int(n_prev), coef.data_ptr(),
                                              _code(coef, "history_average coef"), h.numel(), _stream()), "history_average")
    return h


def short_conv(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, state: Optional[torch.Tensor],
               cu_seqlens: torch.Tensor, token_req: torch.Tensor, state_slots: torch.Tensor,
               state_phase: Optional[torch.Tensor] = None, *, add_input: bool = True, update_state: bool = True) -> torch.Tensor:
    """Causal convolution over time on each channel, per request of a flattened step:
    out[t] = (x[t] if add_input) + sum_j weight[:, j] * x_(t - taps + 1 + j). ``state`` float32 [slots, 2, taps - 1,
    channels] holds every request's last taps - 1 inputs (zeros before its start) in two copies: the step reads copy
    ``state_phase[request]`` and, with ``update_state``, leaves the state moved on by its rows in the other copy (the
    caller turns the phase over afterwards). x float32 or the type of out."""
    _cuda(out, x, weight, state, cu_seqlens, token_req, state_slots, state_phase)
    for t, what in ((cu_seqlens, "cu_seqlens"), (token_req, "token_req"), (state_slots, "state_slots"), (state_phase, "state_phase")):
        _i32(t, f"short_conv {what}")
    tokens, channels = x.shape
    taps = weight.shape[1]
    if out.shape != x.shape or weight.shape[0] != channels or not (out.is_contiguous() and x.is_contiguous() and weight.is_contiguous()):
        raise KernelError(f"short_conv: shapes x={tuple(x.shape)} out={tuple(out.shape)} weight={tuple(weight.shape)}")
    stride = 0
    if taps > 1:
        if (state is None or state.dtype != torch.float32 or state.shape[1:] != (2, taps - 1, channels) or not state.is_contiguous()
                or state_phase is None):
            raise KernelError(f"short_conv: {taps} taps need a contiguous float32 state [slots, 2, {taps - 1}, {channels}] "
                              "and the requests' phases")
        stride = state.stride(0)
    requests = cu_seqlens.numel() - 1
    _lib.check(_lib.load().oi_short_conv(out.data_ptr(), _code(out, "short_conv"), x.data_ptr(), _code(x, "short_conv"),
                                         weight.data_ptr(), _code(weight, "short_conv weight"), _ptr(state), stride,
                                         cu_seqlens.data_ptr(), token_req.data_ptr(), state_slots.data_ptr(), _ptr(state_phase),
                                         tokens, requests,
                                         channels, taps, 1 if add_input else 0, 1 if update_state else 0, _stream()), "short_conv")
    return out


def latent_store(pages: torch.Tensor, page_stride: int, src: torch.Tensor, weight: torch.Tensor, slots: torch.Tensor,
                 rank: int, eps: float, weight_offset: float = 0.0) -> None:
    """RMS norm of src[t, :rank] (row stride free) with ``weight`` and the write of the result to the row's slot
    of ``pages`` [pages, page_size, 1, row_elems >= rank] (elements beyond rank are zeroed; slot < 0: no write)."""
    _cuda(pages, src, weight, slots)
    _i32(slots, "latent_store slots")
    if pages.dtype != src.dtype or src.stride(1) != 1 or src.shape[1] < rank or weight.numel() != rank or slots.numel() != src.shape[0]:
        raise KernelError(f"latent_store: src={tuple(src.shape)} pages={tuple(pages.shape)} rank={rank}")
    _lib.check(_lib.load().oi_latent_store(pages.data_ptr(), int(page_stride), pages.shape[1], pages.shape[-1], src.data_ptr(),
                                           src.stride(0), _code(src, "latent_store"), weight.data_ptr(),
                                           _code(weight, "latent_store weight"), slots.data_ptr(), src.shape[0], int(rank),
                                           float(eps), float(weight_offset), _stream()), "latent_store")


def head_gate(o: torch.Tensor, g: torch.Tensor, heads: int, head_elems: int) -> torch.Tensor:
    """o[t, h, :] *= sigmoid(g[t, h]) in place; o [tokens, >= heads * head_elems], g [tokens, >= heads], row strides free."""
    _cuda(o, g)
    if o.dtype != g.dtype or o.stride(1) != 1 or g.stride(1) != 1 or o.shape[0] != g.shape[0] or o.shape[1] < heads * head_elems \
            or g.shape[1] < heads:
        raise KernelError(f"head_gate: o={tuple(o.shape)} g={tuple(g.shape)} heads={heads} head_elems={head_elems}")
    _lib.check(_lib.load().oi_head_gate(o.data_ptr(), o.stride(0), g.data_ptr(), g.stride(0), _code(o, "head_gate"), o.shape[0],
                                        int(heads), int(head_elems), _stream()), "head_gate")
    return o


def xielu(out: torch.Tensor, x: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """out = a_p x^2 + x / 2 for x > 0, a_n (exp(x) - 1 - x) + x / 2 otherwise, with a_p = softplus(pq[0]) and
    a_n = 1/2 + softplus(pq[1]) formed on the device."""
    _cuda(out, x, pq)
    if out.dtype != x.dtype or out.shape != x.shape or not (out.is_contiguous() and x.is_contiguous()) or pq.numel() != 2:
        raise KernelError("xielu: out and x must be contiguous and alike, pq two numbers")
    _lib.check(_lib.load().oi_xielu(out.data_ptr(), x.data_ptr(), _code(x, "xielu"), pq.data_ptr(), _code(pq, "xielu pq"),
                                    x.numel(), _stream()), "xielu")
    return out


def glu_act(out: torch.Tensor, gate_up: torch.Tensor, block: Optional[int] = None, act: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """``silu_mul`` for every gated activation, the ones with a limit included ("swiglu_clamp": g' sigmoid(1.702 g')
    (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit))."""
    _cuda(out, gate_up)
    rows, inter = out.shape
    block = inter if block is None else int(block)
    if gate_up.shape != (rows, 2 * inter) or out.dtype != gate_up.dtype or not (out.is_contiguous() and gate_up.is_contiguous()):
        raise KernelError(f"glu_act: shapes out={tuple(out.shape)} gate_up={tuple(gate_up.shape)}")
    _lib.check(_lib.load().oi_glu_act(out.data_ptr(), gate_up.data_ptr(), _code(out, "glu_act"), rows, inter, block, glu_code(act),
                                      float(limit), _stream()), "glu_act")
    return out


# gated activations: the two of ACTIVATIONS and those that take a limit
GLU_ACTIVATIONS = dict(ACTIVATIONS, swiglu_clamp=4)


def glu_code(name: str) -> int:
    try:
        return GLU_ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"gated activation {name!r} has no kernel (known: {', '.join(sorted(GLU_ACTIVATIONS))})") from None


def short_conv_act(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, state: Optional[torch.Tensor], cu_seqlens: torch.Tensor,
                   token_req: torch.Tensor, state_slots: torch.Tensor, state_phase: Optional[torch.Tensor], *, act: str = "none",
                   add_input: bool = False) -> torch.Tensor:
    """``short_conv`` on a slice of columns of wider buffers (x and out [tokens, channels] with free row strides) and
    with an activation on the filter's result ("none" or "silu")."""
    _cuda(out, x, weight, state, cu_seqlens, token_req, state_slots, state_phase)
    tokens, channels = x.shape
    taps = weight.shape[1]
    if out.shape != x.shape or weight.shape[0] != channels or x.stride(1) != 1 or out.stride(1) != 1 or not weight.is_contiguous():
        raise KernelError(f"short_conv_act: shapes x={tuple(x.shape)} out={tuple(out.shape)} weight={tuple(weight.shape)}")
    stride = 0
    if taps > 1:
        if (state is None or state.dtype != torch.float32 or state.shape[1:] != (2, taps - 1, channels) or not state.is_contiguous()
                or state_phase is None):
            raise KernelError(f"short_conv_act: {taps} taps need a contiguous float32 state [slots, 2, {taps - 1}, {channels}]")
        stride = state.stride(0)
    _lib.check(_lib.load().oi_short_conv_strided(
        out.data_ptr(), _code(out, "short_conv"), out.stride(0), x.data_ptr(), _code(x, "short_conv"), x.stride(0), weight.data_ptr(),
        _code(weight, "short_conv weight"), _ptr(state), stride, cu_seqlens.data_ptr(), token_req.data_ptr(), state_slots.data_ptr(),
        _ptr(state_phase), tokens, cu_seqlens.numel() - 1, channels, taps, 1 if add_input else 0, 1,
        {"none": 0, "silu": 1}[act], _stream()), "short_conv_act")
    return out


# ---------------------------------------------------------------------------
# recurrent mixers with a matrix memory per head (csrc/recurrent.cu)
# ---------------------------------------------------------------------------
SCAN_MATRIX_MEMORY, SCAN_GATED_DELTA, SCAN_LINEAR_DECAY = 0, 1, 2


def recurrent_scan(mode: int, out: torch.Tensor, qkv: torch.Tensor, offsets, gates: torch.Tensor, gate_offsets, state: torch.Tensor,
                   ctx, heads: int, kv_heads: int, dim: int, vdim: int, *, p0: torch.Tensor, p1: Optional[torch.Tensor] = None,
                   decay: Optional[torch.Tensor] = None, cap: float = 0.0, q_scale: float = 1.0) -> torch.Tensor:
    """The rows of a step through a matrix memory, request by request (see csrc/recurrent.cu). ``qkv`` and ``gates`` are
    float32 [tokens, *] buffers read at the column ``offsets`` (q, k, v) and ``gate_offsets``; ``state`` float32
    [slots, 2, heads, elems]; ``out`` float32 [tokens, heads * vdim]. ``SCAN_LINEAR_DECAY``: ``p0`` holds the heads' fixed
    decays, q, k and v get their silu in the kernels (v in place in ``qkv``), gates and ``p1`` are not read."""
    if p1 is None:
        p1 = p0
    _cuda(out, qkv, gates, state, p0, p1, decay)
    for t in (out, qkv, gates, state, decay):
        if t is not None and (t.dtype != torch.float32 or t.stride(-1) != 1):
            raise KernelError("recurrent_scan: the buffers must be float32 rows")
    elems = dim * vdim + (dim + 1 if mode == SCAN_MATRIX_MEMORY else 0)
    if state.shape[1:] != (2, heads, elems) or not state.is_contiguous() or p0.dtype != p1.dtype:
        raise KernelError(f"recurrent_scan: state {tuple(state.shape)} is not [slots, 2, {heads}, {elems}]")
    L = _lib.load()
    tokens = out.shape[0]
    prep = torch.empty((tokens, heads, L.oi_recurrent_record(dim)), dtype=torch.float32, device=out.device)
    _lib.check(L.oi_recurrent_scan(
        mode, qkv.data_ptr(), qkv.stride(0), int(offsets[0]), int(offsets[1]), int(offsets[2]), gates.data_ptr(), gates.stride(0),
        int(gate_offsets[0]), int(gate_offsets[1]), _ptr(decay), 0 if decay is None else decay.stride(0), p0.data_ptr(), p1.data_ptr(),
        _code(p0, "recurrent_scan"), float(cap), float(q_scale), prep.data_ptr(), state.data_ptr(), state.stride(0),
        ctx.cu_seqlens.data_ptr(), ctx.token_req.data_ptr(), ctx.state_slots.data_ptr(), ctx.state_phase.data_ptr(), out.data_ptr(),
        out.stride(0), tokens, ctx.num_requests, heads, kv_heads, dim, vdim, _stream()), "recurrent_scan")
    return out


def head_norm_gate(out: torch.Tensor, o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, heads: int, vdim: int, eps: float,
                   *, weight_per_head: bool, scale: float = 1.0) -> torch.Tensor:
    """out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * sigmoid(gate[t, h, :]) * scale; o and gate float32 rows,
    ``weight`` [heads * vdim] (``weight_per_head``) or [vdim] shared by the heads."""
    _cuda(out, o, gate, weight)
    if o.dtype != torch.float32 or gate.dtype != torch.float32 or o.stride(1) != 1 or gate.stride(1) != 1 or out.stride(1) != 1 \
            or weight.numel() != (heads * vdim if weight_per_head else vdim) or not weight.is_contiguous():
        raise KernelError("head_norm_gate: o and gate must be float32 rows and the weight of the stated size")
    _lib.check(_lib.load().oi_head_norm_gate(out.data_ptr(), _code(out, "head_norm_gate"), out.stride(0), o.data_ptr(), o.stride(0),
                                             gate.data_ptr(), gate.stride(0), weight.data_ptr(), _code(weight, "head_norm_gate weight"),
                                             vdim if weight_per_head else 0, o.shape[0], heads, vdim, float(eps), float(scale),
                                             _stream()), "head_norm_gate")
    return out


# ---------------------------------------------------------------------------
# several residual streams (csrc/hyper.cu)
# ---------------------------------------------------------------------------
def hyper_fanout(X: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
    """X[t, s, :] = h[t, :] for every stream s; X float32 [tokens, streams, width]."""
    _cuda(X, h)
    if X.dtype != torch.float32 or X.dim() != 3 or not (X.is_contiguous() and h.is_contiguous()) or h.shape != (X.shape[0], X.shape[2]):
        raise KernelError(f"hyper_fanout: X={tuple(X.shape)} h={tuple(h.shape)}")
    _lib.check(_lib.load().oi_hyper_fanout(X.data_ptr(), h.data_ptr(), _code(h, "hyper_fanout"), X.shape[0], X.shape[1], X.shape[2],
                                           _stream()), "hyper_fanout")
    return X


def hyper_step(X: torch.Tensor, *, y: Optional[torch.Tensor] = None, y2: Optional[torch.Tensor] = None, c1: float = 1.0,
               c2: float = 0.0, mix: Optional[torch.Tensor] = None,
               b_out: Optional[torch.Tensor] = None, a_in: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
               eps: float = 0.0, weight_offset: float = 0.0, out: Optional[torch.Tensor] = None,
               row_idx: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """With ``y`` (float32 [tokens, width]): X[t, r] <- sum_s mix[s, r] X[t, s] + b_out[r] y[t] (in place; no coefficients:
    X + y); with ``y2`` the result that comes back is c1 y + c2 y2 (two branches that were computed side by side). With ``out``: out[t] = rms(sum_s a_in[s] X[t, s]) * (weight_offset + norm_w) from the new streams; ``row_idx``
    gathers the rows that are read (then nothing is written to X)."""
    _cuda(X, y, mix, b_out, a_in, norm_w, out, row_idx)
    _i32(row_idx, "hyper_step row_idx")
    T, S, W = X.shape
    if X.dtype != torch.float32 or not X.is_contiguous():
        raise KernelError("hyper_step: the streams must be contiguous float32 [tokens, streams, width]")
    for t in (y, y2):
        if t is not None and (t.dtype != torch.float32 or t.shape != (T, W) or not t.is_contiguous()):
            raise KernelError(f"hyper_step: y must be contiguous float32 [{T}, {W}], got {tuple(t.shape)} {t.dtype}")
    if y2 is not None and y is None:
        raise KernelError("hyper_step: a second result needs a first")
    coefs = [t for t in (mix, b_out, a_in) if t is not None]
    for t, n in ((mix, S * S), (b_out, S), (a_in, S)):
        if t is not None and (t.numel() != n or not t.is_contiguous() or t.dtype != coefs[0].dtype):
            raise KernelError("hyper_step: the coefficients must be contiguous, of one type, [S, S], [S] and [S]")
    rows = T if row_idx is None else row_idx.numel()
    if out is not None and (out.shape != (rows, W) or not out.is_contiguous() or norm_w is None or norm_w.numel() != W):
        raise KernelError("hyper_step: out must be contiguous [rows, width] and the norm weight [width]")
    _lib.check(_lib.load().oi_hyper_step(
        X.data_ptr(), rows, S, W, _ptr(y), _ptr(y2), float(c1), float(c2), _ptr(mix), _ptr(b_out), _ptr(a_in), _code(coefs[0], "hyper_step") if coefs else 0,
        _ptr(norm_w), 0 if norm_w is None else _code(norm_w, "hyper_step norm"), float(eps), float(weight_offset), _ptr(out),
        0 if out is None else _code(out, "hyper_step out"), _ptr(row_idx), _stream()), "hyper_step")
    return out


def scaled_sum(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, ca: float, cb: float) -> torch.Tensor:
    """out = ca * a + cb * b, float32."""
    _cuda(out, a, b)
    if not (out.dtype == a.dtype == b.dtype == torch.float32) or out.shape != a.shape or a.shape != b.shape \
            or not (out.is_contiguous() and a.is_contiguous() and b.is_contiguous()):
        raise KernelError("scaled_sum: three contiguous float32 tensors of one shape")
    _lib.check(_lib.load().oi_scaled_sum(out.data_ptr(), a.data_ptr(), b.data_ptr(), float(ca), float(cb), out.numel(), _stream()),
               "scaled_sum")
    return out


# ---------------------------------------------------------------------------
# routed experts (csrc/moe.cu)
# ---------------------------------------------------------------------------
def moe_route(x: torch.Tensor, w_router: torch.Tensor, top: int, *, scoring: str = "softmax_top",
              correction: Optional[torch.Tensor] = None, groups: int = 1, keep_groups: int = 1):
    """Router logits in float32, the ``top`` largest per row and their softmax, and the rows grouped by expert.
    ``scoring`` "sigmoid_groups": scores sigmoid(logit); the choice goes by score + ``correction`` (float32 [experts]) among
    the experts of the ``keep_groups`` best of ``groups`` equal groups of neighbours (a group's score: the sum of its two
    largest choice scores); the weights are the chosen scores divided by their sum.
    Returns (ids [rows, top] int32, weights [rows, top] float32, sorted pairs, tile list): the last two feed ``moe_experts``."""
    _cuda(x, w_router, correction)
    if scoring not in ("softmax_top", "sigmoid_groups"):
        raise KernelError(f"moe_route: unknown scoring {scoring!r}")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != w_router.shape[0] or not correction.is_contiguous()):
        raise KernelError("moe_route: the correction must be a contiguous float32 tensor of one number an expert")
    rows, K = x.shape
    E = w_router.shape[0]
    if x.stride(1) != 1 or not w_router.is_contiguous() or w_router.shape[1] != K:
        raise KernelError(f"moe_route: x={tuple(x.shape)} router={tuple(w_router.shape)}")
    L = _lib.load()
    ids = torch.empty((rows, top), dtype=torch.int32, device=x.device)
    wts = torch.empty((rows, top), dtype=torch.float32, device=x.device)
    order = torch.empty(rows * top, dtype=torch.int32, device=x.device)
    tiles = torch.empty(3 * L.oi_moe_max_tiles(rows * top, E) + 1, dtype=torch.int32, device=x.device)
    _lib.check(L.oi_moe_route_scored(x.data_ptr(), _code(x, "moe_route"), x.stride(0), w_router.data_ptr(),
                                     _code(w_router, "moe_route router"), rows, K, E, int(top), 1 if scoring == "sigmoid_groups" else 0,
                                     _ptr(correction), int(groups), int(keep_groups), ids.data_ptr(), wts.data_ptr(), order.data_ptr(),
                                     tiles.data_ptr(), _stream()), "moe_route")
    return ids, wts, order, tiles


def moe_route_table(token_ids: torch.Tensor, table: torch.Tensor, experts: int):
    """Routing by the token id: row t uses the experts ``table[token_ids[t], :]`` (int32 [vocab, top]), each weighted 1 / top.
    Returns what ``moe_route`` returns."""
    _cuda(token_ids, table)
    _i32(token_ids, "moe_route_table token ids")
    _i32(table, "moe_route_table table")
    rows, (vocab, top) = token_ids.numel(), table.shape
    L = _lib.load()
    ids = torch.empty((rows, top), dtype=torch.int32, device=table.device)
    wts = torch.empty((rows, top), dtype=torch.float32, device=table.device)
    order = torch.empty(rows * top, dtype=torch.int32, device=table.device)
    tiles = torch.empty(3 * L.oi_moe_max_tiles(rows * top, experts) + 1, dtype=torch.int32, device=table.device)
    _lib.check(L.oi_moe_route_table(token_ids.data_ptr(), table.data_ptr(), rows, vocab, int(experts), top, ids.data_ptr(), wts.data_ptr(),
                                    order.data_ptr(), tiles.data_ptr(), _stream()), "moe_route_table")
    return ids, wts, order, tiles


def moe_experts(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, routing, limit: float,
                act: str = "swiglu_clamp", add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sum_j weight_j * down_e(act(gate_e x, up_e x)) over a row's chosen experts (+ ``add``, float32 [rows, width], when
    given: an expert every row uses); float32 [rows, width].
    ``w_gate_up`` [E, 2 F, W] (F gate rows, then F up rows), ``w_down`` [E, W, F], in x's type."""
    ids, wts, order, tiles = routing
    _cuda(x, w_gate_up, w_down)
    rows, W = x.shape
    E, F2, _ = w_gate_up.shape
    top = ids.shape[1]
    if w_gate_up.dtype != x.dtype or w_down.dtype != x.dtype or w_down.shape != (E, W, F2 // 2) or x.stride(1) != 1 \
            or not (w_gate_up.is_contiguous() and w_down.is_contiguous()):
        raise KernelError("moe_experts: the experts' weights must be contiguous, in x's type, [E, 2F, W] and [E, W, F]")
    if add is not None and (add.dtype != torch.float32 or add.shape != (rows, W) or not add.is_contiguous()):
        raise KernelError("moe_experts: add must be a contiguous float32 [rows, width] tensor")
    _cuda(add)
    hidden = torch.empty((rows * top, F2 // 2), dtype=x.dtype, device=x.device)
    y = torch.empty((rows * top, W), dtype=torch.float32, device=x.device)
    out = torch.empty((rows, W), dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().oi_moe_experts(x.data_ptr(), _code(x, "moe_experts"), x.stride(0), w_gate_up.data_ptr(), w_down.data_ptr(), rows,
                                          W, F2 // 2, E, top, float(limit), glu_code(act), ids.data_ptr(), order.data_ptr(), tiles.data_ptr(),
                                          wts.data_ptr(), hidden.data_ptr(), y.data_ptr(), out.data_ptr(), _ptr(add), _stream()), "moe_experts")
    return out


# ---------------------------------------------------------------------------
# blocks whose sublayers share one norm; a latent with a rotated key part (csrc/parallel_ops.cu)
# ---------------------------------------------------------------------------
def latent_rope_store(pages: Optional[torch.Tensor], page_stride: int, proj: torch.Tensor, latent_off: int, rank: int,
                      weight: Optional[torch.Tensor], eps: float, weight_offset: float, cos: torch.Tensor, sin: torch.Tensor,
                      positions: torch.Tensor, slots: Optional[torch.Tensor], heads: int, q_head_stride: int, q_rot_off: int,
                      store: bool = True) -> None:
    """One pass over the fused input product ``proj`` [tokens, queries | latent, rotated key part | ...]: every head's rotated
    query part (``2 * cos.shape[1]`` numbers at ``h * q_head_stride + q_rot_off``) is turned in place by its row's position;
    with ``store`` the latent (``rank`` numbers at ``latent_off``) is RMS-normed with ``weight`` and written, followed by the
    turned key part that lies behind it, to the row's slot of ``pages`` [pages, page_size, 1, row_elems] (the rest zero)."""
    _cuda(pages, proj, weight, cos, sin, positions, slots)
    _i32(positions, "latent_rope_store positions")
    _i32(slots, "latent_rope_store slots")
    if cos.dtype != torch.float32 or sin.shape != cos.shape or not (cos.is_contiguous() and sin.is_contiguous()) or proj.stride(1) != 1:
        raise KernelError("latent_rope_store: cos/sin must be contiguous float32 tables of one shape, proj contiguous along a row")
    max_pos, rot_half = cos.shape
    if store and (pages is None or pages.dtype != proj.dtype or weight is None or weight.numel() != rank or slots is None):
        raise KernelError("latent_rope_store: the store needs pages of proj's type, the norm's weight and the rows' slots")
    tokens = proj.shape[0]
    _lib.check(_lib.load().oi_latent_rope_store(
        _ptr(pages), int(page_stride), pages.shape[1] if pages is not None else 1, pages.shape[-1] if pages is not None else rank + 2 * rot_half,
        proj.data_ptr(), proj.stride(0), _code(proj, "latent_rope_store"), tokens, int(latent_off), int(rank), _ptr(weight),
        _code(weight, "latent_rope_store weight") if weight is not None else 0, float(eps), float(weight_offset), rot_half,
        cos.data_ptr(), sin.data_ptr(), max_pos, positions.data_ptr(), _ptr(slots), int(heads), int(q_head_stride), int(q_rot_off),
        1 if store else 0, _stream()), "latent_rope_store")


def add2_cast(x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor] = None, low: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x <- x + a (+ b) on contiguous float32 tensors of one shape; ``low`` (same shape, float32 or bfloat16) gets the new x rounded."""
    _cuda(x, a, b, low)
    for t in (x, a, b):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.shape != x.shape):
            raise KernelError("add2_cast: x, a and b must be contiguous float32 tensors of one shape")
    if low is not None and (low.shape != x.shape or not low.is_contiguous()):
        raise KernelError("add2_cast: low must be contiguous and shaped like x")
    _lib.check(_lib.load().oi_add2_cast(x.data_ptr(), a.data_ptr(), _ptr(b), _ptr(low), _code(low, "add2_cast low") if low is not None else 0,
                                        x.numel(), _stream()), "add2_cast")
    return x


def token_gate(g: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, off: int) -> torch.Tensor:
    """g [tokens, dim] <- gelu_tanh(g) * table[token_ids[t], off : off + dim] in place (table [vocab, >= off + dim])."""
    _cuda(g, token_ids, table)
    _i32(token_ids, "token_gate token ids")
    tokens, dim = g.shape
    if g.stride(1) != 1 or table.dim() != 2 or table.stride(1) != 1 or table.shape[1] < off + dim or token_ids.numel() != tokens:
        raise KernelError(f"token_gate: g={tuple(g.shape)} table={tuple(table.shape)} off={off}")
    _lib.check(_lib.load().oi_token_gate(g.data_ptr(), g.stride(0), _code(g, "token_gate"), token_ids.data_ptr(), table.data_ptr(),
                                         _code(table, "token_gate table"), table.stride(0), table.shape[0], int(off), dim, tokens,
                                         _stream()), "token_gate")
    return g


# ---------------------------------------------------------------------------
# blocks with a norm on both sides of a sublayer; rotation before the norm (csrc/sandwich_ops.cu)
# ---------------------------------------------------------------------------
def dyt_step(h: torch.Tensor, *, branch: Optional[torch.Tensor] = None, post=None, pre=None, out: Optional[torch.Tensor] = None,
             row_idx: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One pass over the float32 stream ``h`` [rows, width] with the norm dyt(v) = tanh(alpha v) w + b:
    h += dyt(branch; post) when ``branch`` (float32) is given, and out = dyt(h; pre) when ``out`` is. ``post`` and ``pre``
    are (alpha, w, b) tensor triples of one dtype each. ``row_idx``: out row r is formed from row row_idx[r] (h is then
    left unchanged). ``out`` may be ``h`` itself (the norm in place)."""
    _cuda(h, branch, out, row_idx, *(post or ()), *(pre or ()))
    _i32(row_idx, "dyt_step row_idx")
    if h.dtype != torch.float32 or not h.is_contiguous() or h.dim() != 2:
        raise KernelError("dyt_step: the stream must be contiguous float32 rows")
    width = h.shape[1]
    rows = h.shape[0] if row_idx is None else row_idx.numel()
    if branch is not None and (branch.dtype != torch.float32 or branch.shape != h.shape or not branch.is_contiguous() or post is None):
        raise KernelError("dyt_step: the branch must be float32 of the stream's shape, with the norm of its output")
    if out is not None and (pre is None or out.shape != (rows, width) or not out.is_contiguous()):
        raise KernelError("dyt_step: the output must be contiguous [rows, width], with its norm")
    for trio in (post, pre):
        if trio is not None:
            a, w, b = trio
            if not (a.dtype == w.dtype == b.dtype) or a.numel() != 1 or w.numel() != width or b.numel() != width \
                    or not (w.is_contiguous() and b.is_contiguous()):
                raise KernelError("dyt_step: a norm is one number, a weight and a bias of the stream's width, of one dtype")
    pa, pw, pb = post if post is not None else (None, None, None)
    ra, rw, rb = pre if pre is not None else (None, None, None)
    _lib.check(_lib.load().oi_dyt_step(h.data_ptr(), _ptr(branch), _ptr(pa), _ptr(pw), _ptr(pb), _code(pw, "dyt_step") if pw is not None else 0,
                                       _ptr(ra), _ptr(rw), _ptr(rb), _code(rw, "dyt_step") if rw is not None else 0, _ptr(out),
                                       _code(out, "dyt_step") if out is not None else 0, _ptr(row_idx), rows, width, _stream()), "dyt_step")
    return out


def rope_norm_store(qkv: torch.Tensor, nq: int, nkv: int, hd: int, qk_dim: int, *, bias_tab: Optional[torch.Tensor],
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], unit_norm: bool, eps: float, positions: torch.Tensor,
                    slots: Optional[torch.Tensor], k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], page_stride: int,
                    page_size: int, write_kv: bool) -> None:
    """The fused q | k | v rows (heads of ``hd`` numbers) of a step: add ``bias_tab[min(position, last)]`` (float32
    [n, >= columns]), turn the first 2 * cos.shape[1] numbers of q and k heads (pairs (d, d + half)), then, with
    ``unit_norm``, divide q and k heads by their root mean square over ``qk_dim`` numbers; q is written back in place, k and
    v (``write_kv``) go to the rows' page slots."""
    _cuda(qkv, bias_tab, cos, sin, positions, slots, k_cache, v_cache)
    _i32(positions, "rope_norm_store positions")
    _i32(slots, "rope_norm_store slots")
    cols = (nq + (2 * nkv if write_kv else 0)) * hd
    if qkv.stride(1) != 1 or qkv.shape[1] < cols:
        raise KernelError(f"rope_norm_store: rows of {qkv.shape[1]} numbers for {cols} columns")
    if bias_tab is not None and (bias_tab.dtype != torch.float32 or bias_tab.dim() != 2 or bias_tab.shape[1] < cols or bias_tab.stride(1) != 1):
        raise KernelError("rope_norm_store: the bias table must be float32 [n, columns]")
    if cos is not None and (cos.dtype != torch.float32 or sin is None or sin.shape != cos.shape or not (cos.is_contiguous() and sin.is_contiguous())):
        raise KernelError("rope_norm_store: cos / sin must be contiguous float32 tables of one shape")
    if write_kv and (k_cache is None or v_cache is None or k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype):
        raise KernelError("rope_norm_store: the cache must have the rows' dtype")
    _lib.check(_lib.load().oi_rope_norm_store(
        qkv.data_ptr(), _code(qkv, "rope_norm_store"), qkv.stride(0), qkv.shape[0], nq, nkv, hd, qk_dim, _ptr(bias_tab),
        0 if bias_tab is None else bias_tab.shape[0], 0 if bias_tab is None else bias_tab.stride(0), _ptr(cos), _ptr(sin),
        0 if cos is None else cos.shape[1], 0 if cos is None else cos.shape[0], 1 if unit_norm else 0, float(eps), positions.data_ptr(),
        _ptr(slots), _ptr(k_cache), _ptr(v_cache), int(page_stride), int(page_size), 1 if write_kv else 0, _stream()), "rope_norm_store")
