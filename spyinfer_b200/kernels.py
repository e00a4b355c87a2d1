"""Python faces of the CUDA kernels: argument checks, then one C call on the current stream.

Every function takes CUDA tensors, checks device, dtype, shape and contiguity (a kernel
never sees a tensor it cannot index), and raises ``KernelError`` with the module's message
if the C side refuses the sizes.  Nothing here falls back to a library or to the CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_MESSAGES = {
    1: "a token id outside the vocabulary (batch token index {detail})",
    2: "a position beyond the position table (batch token index {detail})",
    3: "a block-table entry that is no page of the pool (batch token index {detail})",
    4: "a wait inside it ran out of its time limit (code {detail})",
}
STATUS_WAIT_TIMEOUT = 4


class KernelError(RuntimeError):
    pass


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is visible: this engine runs its kernels on the GPU only and has no CPU path")


def _code(t: torch.Tensor, what: str) -> int:
    if t.dtype not in _CODES:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)")
    return _CODES[t.dtype]


def _check(t: torch.Tensor, what: str, dtype=None, ndim=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what}: expected a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, found {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{what}: expected {ndim} dimensions, found shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise KernelError(f"{what}: expected a contiguous tensor, found strides {t.stride()} for shape {tuple(t.shape)}")


def _check_weight(w: torch.Tensor, what: str, dtype=None) -> int:
    """A weight ``[N, K]`` whose rows are contiguous; the rows themselves may lie apart (a view of some columns of a wider
    matrix).  Returns the distance between rows in elements."""
    if not isinstance(w, torch.Tensor) or not w.is_cuda or w.dim() != 2:
        raise KernelError(f"{what}: expected a CUDA matrix")
    if dtype is not None and w.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, found {w.dtype}")
    if w.shape[1] > 1 and w.stride(1) != 1:
        raise KernelError(f"{what}: rows must be contiguous, found strides {w.stride()}")
    return int(w.stride(0)) if w.shape[0] > 1 else max(int(w.stride(0)), int(w.shape[1]))


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_launches = 0


def launch_count() -> int:
    """How many kernel launches this process has made through this module (a replayed CUDA
    graph counts the launches it holds)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


_timed_calls = None


def time_calls(sink) -> None:
    """``sink`` a list: from now on every kernel call made through this module (outside stream capture) is put between
    two CUDA events, and ``(module.function, start, end)`` is appended to the list; None turns it off.  For
    measurements: the events keep a kernel from starting while the one before it drains, so a step runs a little
    slower than without them."""
    global _timed_calls
    _timed_calls = sink


def _call(module: str, fn: str, *args) -> None:
    global _launches
    _launches += 1
    lib = build.load(module)
    f = getattr(lib, fn)
    f.restype = ctypes.c_int
    if _timed_calls is not None and not torch.cuda.is_current_stream_capturing():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = f(*args)
        e1.record()
        _timed_calls.append((f"{module}.{fn}", e0, e1))
        if rc != 0:
            raise KernelError(build.last_error(module))
        return
    if f(*args) != 0:
        raise KernelError(build.last_error(module))


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` widened to float32.  table [V, H]; ids [T] int32; out [T, H] float32."""
    _check(table, "embedding table", ndim=2)
    _check(ids, "token ids", torch.int32, 1)
    _check(out, "embedding output", torch.float32, 2)
    T, (V, H) = ids.shape[0], table.shape
    if tuple(out.shape) != (T, H):
        raise KernelError(f"embedding output: expected shape {(T, H)}, found {tuple(out.shape)}")
    _call("embedding", "spy_embedding", _ptr(table), _code(table, "embedding table"), _ptr(ids), _ptr(out), T, H, V, _ptr(status), _stream())
    return out


def embedding_scaled(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float, status: Optional[torch.Tensor] = None,
                     pairs: Optional[torch.Tensor] = None, mul_prev: int = 0, mul_cur: int = 0, positions: Optional[torch.Tensor] = None,
                     seq_of_token: Optional[torch.Tensor] = None, q_start: Optional[torch.Tensor] = None, state_slot: Optional[torch.Tensor] = None,
                     prev_state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]] * scale`` and, with ``pairs [buckets + 1, H]``, ``+ pairs[row]`` where ``row`` is
    ``(previous token * mul_prev + ids[t] * mul_cur) mod buckets``, or ``buckets`` at position 0.  The token before a
    portion's first one is read from ``prev_state [slots]`` (int32, row ``state_slot[seq]``), which then takes the
    portion's last token."""
    _check(table, "embedding table", ndim=2)
    _check(ids, "token ids", torch.int32, 1)
    _check(out, "embedding output", torch.float32, 2)
    T, (V, H) = ids.shape[0], table.shape
    if tuple(out.shape) != (T, H):
        raise KernelError(f"embedding output: expected shape {(T, H)}, found {tuple(out.shape)}")
    buckets = slots = 0
    if pairs is not None:
        _check(pairs, "pair table", ndim=2)
        if pairs.shape[1] != H or pairs.shape[0] < 2:
            raise KernelError(f"pair table: expected [buckets + 1, {H}], found {tuple(pairs.shape)}")
        buckets = pairs.shape[0] - 1
        for t, what in ((positions, "positions"), (seq_of_token, "seq_of_token"), (q_start, "q_start"), (state_slot, "state_slot")):
            _check(t, what, torch.int32, 1)
        _check(prev_state, "previous-token state", torch.int32)
        slots = prev_state.numel()
        if positions.shape[0] != T or seq_of_token.shape[0] != T:
            raise KernelError("embedding: positions and seq_of_token must have one entry per token")
    _call("embedding", "spy_embedding_scaled", _ptr(table), _code(table, "embedding table"), _ptr(ids), _ptr(out), T, H, V, ctypes.c_float(scale),
          _ptr(pairs), _code(pairs, "pair table") if pairs is not None else 0, ctypes.c_longlong(buckets), ctypes.c_longlong(int(mul_prev)),
          ctypes.c_longlong(int(mul_cur)), _ptr(positions), _ptr(seq_of_token), _ptr(q_start), _ptr(state_slot), _ptr(prev_state), slots,
          _ptr(status), _stream())
    return out


def _stack_of(delta: Optional[torch.Tensor], like: torch.Tensor, what: str):
    """(pointer argument, parts, elements between parts) of a delta that is None, ``like``'s shape, or a stack of it."""
    if delta is None:
        return None, 0, 0
    if delta.dim() == 3:
        _check(delta, what, ndim=3)
        if tuple(delta.shape[1:]) != tuple(like.shape):
            raise KernelError(f"{what}: stacked shape {tuple(delta.shape)} does not fit {tuple(like.shape)}")
        return delta, delta.shape[0], delta.shape[1] * delta.shape[2]
    _check(delta, what, ndim=2)
    if tuple(delta.shape) != tuple(like.shape):
        raise KernelError(f"{what}: shape {tuple(delta.shape)} differs from {tuple(like.shape)}")
    return delta, 1, 0


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, delta: Optional[torch.Tensor] = None, delta_scale: float = 1.0,
              delta2: Optional[torch.Tensor] = None, delta2_scale: float = 1.0, rows: Optional[torch.Tensor] = None, write_back: bool = False,
              center: bool = True, bias: Optional[torch.Tensor] = None, delta_weight: Optional[torch.Tensor] = None,
              delta_bias: Optional[torch.Tensor] = None, delta_rows: Optional[tuple] = None) -> torch.Tensor:
    """``out = layer_norm(x + delta_scale * delta_weight * (delta + delta_bias) + delta2_scale * delta2) * weight (+ bias)`` row by row (mean
    removed; ``center=False``: the mean stays, an RMS norm); with ``write_back`` the sum is stored into ``x``; ``rows`` gathers
    rows.  Each delta has x's shape or is a stack ``[splits, rows, len]`` of partial sums that are added in order; both have
    one dtype.  ``bias`` and ``delta_weight`` (a multiplier along the row for ``delta``) are ``[len]`` of the weight's dtype,
    ``delta_bias`` (the bias of the projection that made ``delta``) ``[len]`` float32.  ``delta_rows = (rows [*, len] of the output's
    dtype, weights [*] float32)`` adds ``weights[t] * rows[t]`` to ``delta`` (ahead of ``delta_weight``)."""
    _check(x, "layernorm input", ndim=2)
    _check(weight, "layernorm weight", ndim=1)
    _check(out, "layernorm output", ndim=2)
    H = x.shape[1]
    if weight.shape[0] != H or out.shape[1] != H:
        raise KernelError(f"layernorm: row lengths differ: input {H}, weight {weight.shape[0]}, output {out.shape[1]}")
    if delta is None and delta2 is not None:
        delta, delta_scale, delta2, delta2_scale = delta2, delta2_scale, None, 1.0
    for extra, what in ((bias, "layernorm bias"), (delta_weight, "layernorm delta weight")):
        if extra is not None:
            _check(extra, what, weight.dtype, 1)
            if extra.shape[0] != H:
                raise KernelError(f"{what}: {extra.shape[0]} elements for rows of {H}")
    if delta_bias is not None:
        _check(delta_bias, "layernorm delta bias", torch.float32, 1)
        if delta_bias.shape[0] != H:
            raise KernelError(f"layernorm delta bias: {delta_bias.shape[0]} elements for rows of {H}")
    if delta_rows is not None:
        _check(delta_rows[0], "layernorm delta rows", out.dtype, 2)
        _check(delta_rows[1], "layernorm delta row weights", torch.float32, 1)
        if tuple(delta_rows[0].shape) != tuple(x.shape) or delta_rows[1].shape[0] != x.shape[0]:
            raise KernelError("layernorm: the delta's row term has the input's shape and one weight a row")
    if (delta_weight is not None or delta_bias is not None or delta_rows is not None) and delta is None:
        raise KernelError("layernorm: a delta weight, bias or row term without a delta")
    a, a_splits, a_stride = _stack_of(delta, x, "layernorm delta")
    b, b_splits, b_stride = _stack_of(delta2, x, "layernorm second delta")
    if a is not None and b is not None and a.dtype != b.dtype:
        raise KernelError(f"layernorm: the two deltas differ in dtype ({a.dtype}, {b.dtype})")
    if rows is not None:
        _check(rows, "layernorm rows", torch.int32, 1)
        n = rows.shape[0]
    else:
        n = x.shape[0]
    if out.shape[0] != n:
        raise KernelError(f"layernorm: output has {out.shape[0]} rows, expected {n}")
    if bias is not None or delta_weight is not None or delta_bias is not None or delta_rows is not None:
        _call("layernorm", "spy_layernorm_affine", _ptr(x), _code(x, "layernorm input"), _ptr(a), a_splits, ctypes.c_longlong(a_stride),
              ctypes.c_float(delta_scale), _ptr(delta_weight), _ptr(delta_bias), _ptr(delta_rows[0] if delta_rows is not None else None),
              _ptr(delta_rows[1] if delta_rows is not None else None), _ptr(b), b_splits, ctypes.c_longlong(b_stride), ctypes.c_float(delta2_scale),
              _code(a, "layernorm delta") if a is not None else 0, _ptr(rows), _ptr(weight), _ptr(bias), _code(weight, "layernorm weight"), _ptr(out),
              _code(out, "layernorm output"), n, H, ctypes.c_float(eps), int(bool(write_back)), int(bool(center)), _stream())
        return out
    _call("layernorm", "spy_layernorm", _ptr(x), _code(x, "layernorm input"), _ptr(a), a_splits, ctypes.c_longlong(a_stride), ctypes.c_float(delta_scale),
          _ptr(b), b_splits, ctypes.c_longlong(b_stride), ctypes.c_float(delta2_scale), _code(a, "layernorm delta") if a is not None else 0,
          _ptr(rows), _ptr(weight), _code(weight, "layernorm weight"), _ptr(out), _code(out, "layernorm output"), n, H, ctypes.c_float(eps),
          int(bool(write_back)), int(bool(center)), _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None, write_back: bool = False) -> torch.Tensor:
    """``out = rmsnorm(x [+ delta]) * weight`` row by row; with ``write_back`` the sum is stored
    into ``x`` (the residual stream); ``rows`` gathers rows of x (and delta) into out.
    ``delta`` has x's shape, or is a stack ``[splits, rows, len]`` of partial sums (the
    unreduced output of a split-K product) that are added in order."""
    _check(x, "rmsnorm input", ndim=2)
    _check(weight, "rmsnorm weight", ndim=1)
    _check(out, "rmsnorm output", ndim=2)
    H = x.shape[1]
    if weight.shape[0] != H or out.shape[1] != H:
        raise KernelError(f"rmsnorm: row lengths differ: input {H}, weight {weight.shape[0]}, output {out.shape[1]}")
    splits, split_stride = 0, 0
    if delta is not None:
        if delta.dim() == 3:
            _check(delta, "rmsnorm delta", ndim=3)
            splits, split_stride = delta.shape[0], delta.shape[1] * delta.shape[2]
            if tuple(delta.shape[1:]) != tuple(x.shape):
                raise KernelError(f"rmsnorm: stacked delta shape {tuple(delta.shape)} does not fit input shape {tuple(x.shape)}")
        else:
            _check(delta, "rmsnorm delta", ndim=2)
            splits = 1
            if tuple(delta.shape) != tuple(x.shape):
                raise KernelError(f"rmsnorm: delta shape {tuple(delta.shape)} differs from input shape {tuple(x.shape)}")
    if rows is not None:
        _check(rows, "rmsnorm rows", torch.int32, 1)
        n = rows.shape[0]
    else:
        n = x.shape[0]
    if out.shape[0] != n:
        raise KernelError(f"rmsnorm: output has {out.shape[0]} rows, expected {n}")
    _call("rmsnorm", "spy_rmsnorm", _ptr(x), _code(x, "rmsnorm input"), _ptr(delta), _code(delta, "rmsnorm delta") if delta is not None else 0,
          splits, ctypes.c_longlong(split_stride), _ptr(rows), _ptr(weight), _code(weight, "rmsnorm weight"), _ptr(out),
          _code(out, "rmsnorm output"), n, H, ctypes.c_float(eps), int(bool(write_back)), _stream())
    return out


def build_rope_table(inv_freq: torch.Tensor, rows: int) -> torch.Tensor:
    """(cos, sin) of ``position * inv_freq[j]`` as float32 ``[rows, len(inv_freq), 2]``."""
    _check(inv_freq, "inverse frequencies", torch.float32, 1)
    table = torch.empty((rows, inv_freq.shape[0], 2), dtype=torch.float32, device=inv_freq.device)
    _call("qk_rope_store", "spy_build_rope_table", _ptr(table), _ptr(inv_freq), rows, inv_freq.shape[0], _stream())
    return table


def qk_rope_store(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, q_weight: Optional[torch.Tensor],
                  k_weight: Optional[torch.Tensor], eps: float, rope_table: Optional[torch.Tensor], positions: torch.Tensor,
                  seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor], pages: Optional[torch.Tensor], store: bool = True,
                  status: Optional[torch.Tensor] = None, q_out: Optional[torch.Tensor] = None, pairing: str = "half") -> torch.Tensor:
    """Per-head RMSNorm (if weights are given) and rotation (if a table is given) of the q and k
    heads of ``qkv [T, (nh + 2 nkv) hd]``, or of a stack ``[splits, T, ...]`` of float32 partial
    products that is summed on the way.  q goes to ``q_out [T, nh hd]`` (default: in place,
    which a stack does not allow).  With ``store`` the k heads (normed, rotated) and the v heads
    go to ``pages [num_pages, 2, nkv, page_size, hd]`` through ``block_table [S, width]``.
    ``pairing``: which elements the angle ``j`` of the table rotates: ``"half"`` ``(j, j + r)``,
    ``"interleaved"`` ``(2j, 2j + 1)``.
    Returns the tensor that holds q (rows may be wider than ``nh hd``)."""
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"qk_rope_store: unknown pairing rule {pairing!r}")
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.dim() == 3:
        _check(qkv, "qkv partial products", torch.float32, 3)
        splits, T = qkv.shape[0], qkv.shape[1]
        split_stride = qkv.shape[1] * qkv.shape[2]
        if q_out is None:
            raise KernelError("qk_rope_store: a stack of partial products needs q_out")
    else:
        _check(qkv, "qkv", ndim=2)
        splits, T, split_stride = 1, qkv.shape[0], 0
    if qkv.shape[-1] != width:
        raise KernelError(f"qkv: expected {width} columns, found {qkv.shape[-1]}")
    if q_out is None:
        q_out = qkv
    else:
        _check(q_out, "q output", ndim=2)
        if q_out.shape[0] != T or q_out.shape[1] < num_heads * head_dim:
            raise KernelError(f"q output: expected [{T}, >= {num_heads * head_dim}], found {tuple(q_out.shape)}")
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    if positions.shape[0] != T or seq_of_token.shape[0] != T:
        raise KernelError("qk_rope_store: positions and seq_of_token must have one entry per token")
    w_code = 0
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_rope_store: q and k norm weights must both be given or both be None")
    if q_weight is not None:
        _check(q_weight, "q norm weight", ndim=1)
        _check(k_weight, "k norm weight", q_weight.dtype, 1)
        if q_weight.shape[0] != head_dim or k_weight.shape[0] != head_dim:
            raise KernelError(f"qk_rope_store: norm weights must have head_dim={head_dim} elements")
        w_code = _code(q_weight, "q norm weight")
    rot_half = table_rows = 0
    if rope_table is not None:
        _check(rope_table, "rope table", torch.float32, 3)
        table_rows, rot_half = rope_table.shape[0], rope_table.shape[1]
    page_size = num_pages = table_width = cache_code = 0
    if store:
        if pages is None or block_table is None:
            raise KernelError("qk_rope_store: storing needs pages and a block table")
        _check(pages, "cache pages", ndim=5)
        _check(block_table, "block table", torch.int32, 2)
        num_pages, two, nkv, page_size, hd = pages.shape
        if two != 2 or nkv != num_kv_heads or hd != head_dim:
            raise KernelError(f"cache pages: expected [pages, 2, {num_kv_heads}, page_size, {head_dim}], found {tuple(pages.shape)}")
        table_width = block_table.shape[1]
        cache_code = _code(pages, "cache pages")
    _call("qk_rope_store", "spy_qk_rope_store", _ptr(qkv), _code(qkv, "qkv"), splits, ctypes.c_longlong(split_stride), _ptr(q_out),
          _code(q_out, "q output"), ctypes.c_longlong(q_out.shape[1]), T, num_heads, num_kv_heads, head_dim, _ptr(q_weight), _ptr(k_weight),
          w_code, ctypes.c_float(eps), _ptr(rope_table), rot_half, table_rows, _ptr(positions), _ptr(seq_of_token),
          _ptr(block_table if store else None), table_width, _ptr(pages if store else None), cache_code, page_size, num_pages,
          int(bool(store)), 0 if pairing == "half" else 1, _ptr(status), _stream())
    return q_out


def attention_generic(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                      positions: torch.Tensor, seq_of_token: torch.Tensor, scale: float, window: Optional[int] = None,
                      status: Optional[torch.Tensor] = None, keep_first: int = 0, sink: bool = False) -> torch.Tensor:
    """Attention of every token of the batch over its sequence's pages (any mix of prompt
    portions and single tokens).  ``q [T, >= nh*hd]`` (only the first nh*hd columns are read),
    ``out [T, nh*hd]``.  ``keep_first`` (with a window): the sequence's first so many keys stay visible;
    ``sink``: one is added to the softmax's denominator."""
    _check(q, "attention queries", ndim=2)
    _check(out, "attention output", q.dtype, 2)
    _check(pages, "cache pages", ndim=5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    T = q.shape[0]
    num_pages, planes, nkv, page_size, hd = pages.shape
    if planes not in (1, 2) or hd != head_dim:
        raise KernelError(f"cache pages: expected [pages, 2 (or 1: the values are the keys), nkv, page_size, {head_dim}], found {tuple(pages.shape)}")
    if q.shape[1] < num_heads * head_dim or tuple(out.shape) != (T, num_heads * head_dim):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {num_heads} heads of {head_dim}")
    if positions.shape[0] != T or seq_of_token.shape[0] != T:
        raise KernelError("attention: positions and seq_of_token must have one entry per token")
    _call("attention_generic", "spy_attention_generic", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _code(q, "attention queries"),
          _ptr(pages), _code(pages, "cache pages"), _ptr(block_table), block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim,
          _ptr(positions), _ptr(seq_of_token), T, int(window or 0), ctypes.c_float(scale), _ptr(status), _stream(), planes, int(keep_first),
          int(bool(sink)))
    return out


def scaled_sum(out: torch.Tensor, a: torch.Tensor, a_scale: float, b: torch.Tensor, b_scale: float) -> torch.Tensor:
    """``out = a_scale * a + b_scale * b`` in 32-bit; ``a`` and ``b`` have out's shape or are stacks of partial sums (one dtype)."""
    _check(out, "weighted sum", torch.float32, 2)
    if a.dtype != b.dtype:
        a, b = (t.float() if t.dim() == 2 else t for t in (a, b))
    pa, sa, stride_a = _stack_of(a, out, "first result")
    pb, sb, stride_b = _stack_of(b, out, "second result")
    if pa.dtype != pb.dtype:
        raise KernelError(f"scaled_sum: the two results differ in dtype ({pa.dtype}, {pb.dtype})")
    _call("layernorm", "spy_scaled_sum", _ptr(out), _ptr(pa), sa, ctypes.c_longlong(stride_a), ctypes.c_float(a_scale), _ptr(pb), sb,
          ctypes.c_longlong(stride_b), ctypes.c_float(b_scale), _code(pa, "first result"), ctypes.c_longlong(out.numel()), _stream())
    return out


def _paged(pages: torch.Tensor, what: str, head_dim: int):
    _check(pages, what, ndim=5)
    num_pages, two, nkv, page_size, hd = pages.shape
    if two != 2 or hd != head_dim:
        raise KernelError(f"{what}: expected [pages, 2, nkv, page_size, {head_dim}], found {tuple(pages.shape)}")
    return num_pages, nkv, page_size


def pool_store(pages: torch.Tensor, block_table: torch.Tensor, pooled: torch.Tensor, pool_table: torch.Tensor, pool: int, positions: torch.Tensor,
               seq_of_token: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """For every token of the batch whose position ends a block of ``pool`` tokens: the means of the block's keys and of its
    values, read from ``pages`` through ``block_table``, go to entry ``position // pool`` of ``pooled`` through ``pool_table``."""
    hd = pages.shape[-1]
    num_pages, nkv, page_size = _paged(pages, "cache pages", hd)
    num_pooled, nkv2, page_size2 = _paged(pooled, "pooled pages", hd)
    if (nkv2, page_size2) != (nkv, page_size) or pooled.dtype != pages.dtype:
        raise KernelError("pool_store: the pooled cache must have the token cache's heads, page size and dtype")
    _check(block_table, "block table", torch.int32, 2)
    _check(pool_table, "pooled block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    if block_table.shape != pool_table.shape:
        raise KernelError("pool_store: the two block tables must have one shape")
    _call("attention_pool", "spy_pool_store", _ptr(pages), num_pages, _ptr(block_table), _ptr(pooled), num_pooled, _ptr(pool_table), block_table.shape[1],
          page_size, nkv, hd, _code(pages, "cache pages"), int(pool), _ptr(positions), _ptr(seq_of_token), positions.shape[0], _ptr(status), _stream())


def attention_pool(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                   pooled: Optional[torch.Tensor], pool_table: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor, scale: float,
                   window: int, pool: int, status: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of every token of the batch over the last ``window`` keys of its sequence and one pooled entry for every
    block of ``pool`` tokens that ends at least ``window`` positions before it (``pool`` 0: none), under one softmax.
    ``q [T, >= nh*hd]``, ``out [T, nh*hd]``.  With ``lse [T, nh]`` the window's keys have been done already (``out`` holds
    their normalised result, ``lse`` the logarithm of each row's sum of exponentials, as ``attention_tc`` leaves them) and
    only the pooled entries are added to that softmax."""
    _check(q, "attention queries", ndim=2)
    _check(out, "attention output", q.dtype, 2)
    num_pages, nkv, page_size = _paged(pages, "cache pages", head_dim)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    T = q.shape[0]
    if q.shape[1] < num_heads * head_dim or tuple(out.shape) != (T, num_heads * head_dim):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {num_heads} heads of {head_dim}")
    if positions.shape[0] != T or seq_of_token.shape[0] != T:
        raise KernelError("attention: positions and seq_of_token must have one entry per token")
    num_pooled = 0
    if pool:
        num_pooled, nkv2, page_size2 = _paged(pooled, "pooled pages", head_dim)
        _check(pool_table, "pooled block table", torch.int32, 2)
        if (nkv2, page_size2) != (nkv, page_size) or pooled.dtype != pages.dtype or pool_table.shape != block_table.shape:
            raise KernelError("attention: the pooled cache must have the token cache's heads, page size, dtype and table shape")
    if lse is not None:
        _check(lse, "logarithms of the sums", torch.float32, 2)
        if tuple(lse.shape) != (T, num_heads):
            raise KernelError(f"attention: lse {tuple(lse.shape)} does not fit {T} tokens of {num_heads} heads")
    _call("attention_pool", "spy_attention_pool", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _code(q, "attention queries"), _ptr(pages), num_pages,
          _ptr(block_table), _ptr(pooled if pool else None), num_pooled, _ptr(pool_table if pool else None), _code(pages, "cache pages"),
          block_table.shape[1], page_size, num_heads, nkv, head_dim, _ptr(positions), _ptr(seq_of_token), T, int(window), int(pool or 0),
          ctypes.c_float(scale), _ptr(lse), _ptr(status), _stream())
    return out


def mlstm_record(dk: int, dv: int) -> int:
    """Floats of one head's state of the gated matrix memory (the matrix, and the normaliser vector and running maximum once per column tile)."""
    lib = build.load("recurrence")
    lib.spy_mlstm_record.restype = ctypes.c_longlong
    return int(lib.spy_mlstm_record(int(dk), int(dv)))


def _scan_common(proj, state, q_start, state_slot, out, heads, dv):
    _check(proj, "fused projection", torch.float32, 2)
    _check(state, "recurrent state", torch.float32)
    _check(q_start, "q_start", torch.int32, 1)
    _check(state_slot, "state_slot", torch.int32, 1)
    _check(out, "recurrence output", torch.float32, 2)
    if tuple(out.shape) != (proj.shape[0], heads * dv):
        raise KernelError(f"recurrence output: expected {(proj.shape[0], heads * dv)}, found {tuple(out.shape)}")


def mlstm_scan(proj: torch.Tensor, offsets, bias_i: torch.Tensor, bias_f: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor,
               state_slot: torch.Tensor, num_seqs: int, out: torch.Tensor, heads: int, dk: int, dv: int, q_scale: float, cap: float,
               status: Optional[torch.Tensor] = None, longest: Optional[int] = None) -> torch.Tensor:
    """The gated matrix memory over every request's tokens of this step, in order, from and into ``state [slots, heads * record]``.
    ``proj [T, ld]`` float32 holds q, k, v and the two gates' pre-activations at the columns ``offsets = (q, k, v, i, f)``.
    ``longest``: the most tokens a request brings, or more (default: all the batch's tokens): it sizes the kernel's staging, and 1
    says that every request brings exactly one token (the kernel made for decoding then runs; ``delta_scan`` likewise)."""
    _scan_common(proj, state, q_start, state_slot, out, heads, dv)
    if state.dim() != 2 or state.shape[1] != heads * mlstm_record(dk, dv):
        raise KernelError(f"mlstm: state {tuple(state.shape)} does not fit {heads} heads of {dk} x {dv}")
    _check(bias_i, "input gate bias", torch.float32, 1)
    _check(bias_f, "forget gate bias", torch.float32, 1)
    oq, ok, ov, oi, of = (int(o) for o in offsets)
    if max(oq + heads * dk, ok + heads * dk, ov + heads * dv, oi + heads, of + heads) > proj.shape[1] or bias_i.shape[0] != heads or bias_f.shape[0] != heads:
        raise KernelError("mlstm: the column offsets or the biases do not fit the projection")
    _call("recurrence", "spy_mlstm_scan", _ptr(proj), ctypes.c_longlong(proj.shape[1]), oq, ok, ov, oi, of, _ptr(bias_i), _ptr(bias_f), _ptr(state),
          state.shape[0], _ptr(q_start), _ptr(state_slot), int(num_seqs), int(longest or proj.shape[0]), _ptr(out), heads, dk, dv,
          ctypes.c_float(q_scale), ctypes.c_float(cap), _ptr(status), _stream())
    return out


def delta_scan(proj: torch.Tensor, offsets, decay_pre: torch.Tensor, bias_a: torch.Tensor, decay_offset: torch.Tensor, state: torch.Tensor,
               q_start: torch.Tensor, state_slot: torch.Tensor, num_seqs: int, out: torch.Tensor, heads: int, dk: int,
               status: Optional[torch.Tensor] = None, longest: Optional[int] = None) -> torch.Tensor:
    """The generalised delta rule over every request's tokens of this step, from and into ``state [slots, heads * dk * dk]``.
    ``proj [T, ld]`` float32 holds r, k, v and the removal rate's pre-activation at ``offsets = (r, k, v, a)``;
    ``decay_pre [T, heads * dk]`` the decay's pre-activation."""
    _scan_common(proj, state, q_start, state_slot, out, heads, dk)
    if state.dim() != 2 or state.shape[1] != heads * dk * dk:
        raise KernelError(f"delta rule: state {tuple(state.shape)} does not fit {heads} heads of {dk} x {dk}")
    _check(decay_pre, "decay pre-activation", torch.float32, 2)
    _check(bias_a, "removal rate bias", torch.float32, 1)
    _check(decay_offset, "decay offset", torch.float32, 1)
    o_r, ok, ov, oa = (int(o) for o in offsets)
    n = heads * dk
    if max(o_r, ok, ov, oa) + n > proj.shape[1] or tuple(decay_pre.shape) != (proj.shape[0], n) or bias_a.shape[0] != n or decay_offset.shape[0] != n:
        raise KernelError("delta rule: the column offsets, the decay or the biases do not fit the projection")
    _call("recurrence", "spy_delta_scan", _ptr(proj), ctypes.c_longlong(proj.shape[1]), o_r, ok, ov, oa, _ptr(decay_pre), _ptr(bias_a), _ptr(decay_offset),
          _ptr(state), state.shape[0], _ptr(q_start), _ptr(state_slot), int(num_seqs), int(longest or proj.shape[0]), _ptr(out), heads, dk,
          _ptr(status), _stream())
    return out


def gla_scan(proj: torch.Tensor, offsets, decay_pre: torch.Tensor, decay_bias: torch.Tensor, tau: float, state: torch.Tensor, q_start: torch.Tensor,
             state_slot: torch.Tensor, num_seqs: int, out: torch.Tensor, heads: int, dk: int, dv: int, q_scale: float,
             status: Optional[torch.Tensor] = None, longest: Optional[int] = None) -> torch.Tensor:
    """Gated linear attention with a decay per key channel over every request's tokens of this step, from and into
    ``state [slots, heads * dk * dv]``: ``S = diag(a) S + k v^T``, ``o = S^T (q_scale q)``, ``a = sigmoid(z + bias)^(1 / tau)``.
    ``proj [T, ld]`` float32 holds q, k, v at ``offsets = (q, k, v)``; ``decay_pre [T, heads * dk]`` is ``z``."""
    _scan_common(proj, state, q_start, state_slot, out, heads, dv)
    if state.dim() != 2 or state.shape[1] != heads * dk * dv:
        raise KernelError(f"gated linear attention: state {tuple(state.shape)} does not fit {heads} heads of {dk} x {dv}")
    _check(decay_pre, "decay pre-activation", torch.float32, 2)
    _check(decay_bias, "decay bias", torch.float32, 1)
    oq, ok, ov = (int(o) for o in offsets)
    n = heads * dk
    if max(oq + n, ok + n, ov + heads * dv) > proj.shape[1] or tuple(decay_pre.shape) != (proj.shape[0], n) or decay_bias.shape[0] != n or not tau > 0:
        raise KernelError("gated linear attention: the column offsets, the decay or its bias do not fit the projection, or tau is not positive")
    _call("recurrence", "spy_gla_scan", _ptr(proj), ctypes.c_longlong(proj.shape[1]), oq, ok, ov, _ptr(decay_pre), _ptr(decay_bias), ctypes.c_float(1.0 / tau),
          _ptr(state), state.shape[0], _ptr(q_start), _ptr(state_slot), int(num_seqs), int(longest or proj.shape[0]), _ptr(out), heads, dk, dv,
          ctypes.c_float(q_scale), _ptr(status), _stream())
    return out


def gated_head_norm(o: torch.Tensor, proj: torch.Tensor, gate_offset: int, weight: torch.Tensor, out: torch.Tensor, heads: int, dv: int, eps: float,
                    gate: str = "sigmoid") -> torch.Tensor:
    """``out = o / rms(o per head) * weight * gate(proj[:, gate_offset : gate_offset + heads * dv])``; ``o`` float32 ``[T, heads * dv]``;
    ``gate``: ``"sigmoid"`` or ``"silu"``."""
    if gate not in ("sigmoid", "silu"):
        raise KernelError(f"gated_head_norm: unknown gate {gate!r}")
    _check(o, "recurrence output", torch.float32, 2)
    _check(proj, "fused projection", torch.float32, 2)
    _check(weight, "head norm weight", torch.float32, 1)
    _check(out, "gated output", ndim=2)
    n = heads * dv
    if o.shape[1] != n or tuple(out.shape) != tuple(o.shape) or weight.shape[0] != n or gate_offset + n > proj.shape[1] or proj.shape[0] != o.shape[0]:
        raise KernelError("gated_head_norm: shapes do not fit")
    _call("recurrence", "spy_gated_head_norm", _ptr(o), _ptr(proj), ctypes.c_longlong(proj.shape[1]), int(gate_offset), _ptr(weight), _ptr(out),
          _code(out, "gated output"), o.shape[0], heads, dv, ctypes.c_float(eps), _stream(), ("sigmoid", "silu").index(gate))
    return out


def tanh_cols(proj: torch.Tensor, offset: int, n: int, out: torch.Tensor, activation: str = "tanh") -> torch.Tensor:
    """``out[t, j] = tanh(proj[t, offset + j])`` for ``j < n``; proj float32.  ``activation="none"``: the columns as they are
    (in ``out``'s type)."""
    if activation not in ("tanh", "none"):
        raise KernelError(f"tanh_cols: unknown activation {activation!r}")
    _check(proj, "fused projection", torch.float32, 2)
    _check(out, "tanh output", ndim=2)
    if offset + n > proj.shape[1] or tuple(out.shape) != (proj.shape[0], n):
        raise KernelError("tanh_cols: shapes do not fit")
    _call("recurrence", "spy_tanh_cols", _ptr(proj), ctypes.c_longlong(proj.shape[1]), int(offset), int(n), _ptr(out), _code(out, "tanh output"),
          proj.shape[0], _stream(), ("tanh", "none").index(activation))
    return out


_attn_scratch = {}


def attention_scratch(device, floats: int) -> torch.Tensor:
    """A float32 buffer of at least ``floats`` for the split attention kernel's partial
    results.  Buffers are kept for the life of the process (captured graphs point at them);
    a larger request makes a new one."""
    key = str(torch.device(device))
    buf = _attn_scratch.get(key)
    if buf is None or buf[-1].numel() < floats:
        size = max(floats, 1 << 20)
        _attn_scratch.setdefault(key, []).append(torch.empty(size, dtype=torch.float32, device=device))
        buf = _attn_scratch[key]
    return buf[-1]


def attention_mma_takes(num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core attention kernel takes these sizes: bfloat16, head size 64 or
    128, at most 16 query heads per key/value head."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16


def attention_mma(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                  positions: torch.Tensor, q_start: torch.Tensor, num_seqs: int, scale: float, window: Optional[int] = None,
                  split_keys: int = 0, max_splits: int = 0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-core attention of a batch over its pages.  ``split_keys == 0``: tiles mode, any
    mix of portions and single tokens.  ``split_keys > 0``: every sequence brings one token
    and its keys are cut into splits of ``split_keys`` (a multiple of 64), at most
    ``max_splits`` of them, merged through scratch memory."""
    _check(q, "attention queries", torch.bfloat16, 2)
    _check(out, "attention output", torch.bfloat16, 2)
    _check(pages, "cache pages", torch.bfloat16, 5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(q_start, "q_start", torch.int32, 1)
    T = q.shape[0]
    num_pages, two, nkv, page_size, hd = pages.shape
    if two != 2 or hd != head_dim:
        raise KernelError(f"cache pages: expected [pages, 2, nkv, page_size, {head_dim}], found {tuple(pages.shape)}")
    if q.shape[1] < num_heads * head_dim or tuple(out.shape) != (T, num_heads * head_dim):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {num_heads} heads of {head_dim}")
    if positions.shape[0] != T or q_start.shape[0] != num_seqs + 1 or block_table.shape[0] < num_seqs:
        raise KernelError("attention: positions need one entry per token, q_start one per sequence plus one, the block table a row per sequence")
    mode = 1 if split_keys > 0 else 0
    scratch, floats = None, 0
    if mode == 1 and max_splits > 1:
        floats = num_seqs * num_heads * max_splits * (head_dim + 2)
        scratch = attention_scratch(q.device, floats)
        floats = scratch.numel()
    if status is None:
        status = status_word(q.device)
    _call("attention_mma", "spy_attention_mma", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _ptr(pages), _ptr(block_table),
          block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim, _ptr(positions), _ptr(q_start), T, num_seqs,
          int(window or 0), ctypes.c_float(scale), mode, int(split_keys), int(max_splits), _ptr(scratch), ctypes.c_longlong(floats),
          _ptr(status), _stream())
    return out


def attention_tc(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                 positions: torch.Tensor, q_start: torch.Tensor, num_seqs: int, scale: float, window: Optional[int] = None,
                 status: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of a batch over its pages on tcgen05 (blocks of two 128-row query tiles that share
    every key and value tile, scores and output in tensor memory, pages brought in by TMA): prompt
    portions, any mix.  Page sizes 8 .. 128.  ``lse [T, nh]`` (float32, optional) receives the natural
    logarithm of every row's sum of ``exp(score * scale)``, with which further keys can be merged in."""
    _check(q, "attention queries", torch.bfloat16, 2)
    _check(out, "attention output", torch.bfloat16, 2)
    _check(pages, "cache pages", torch.bfloat16, 5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(q_start, "q_start", torch.int32, 1)
    T = q.shape[0]
    num_pages, planes, nkv, page_size, hd = pages.shape
    if planes not in (1, 2) or hd != head_dim:
        raise KernelError(f"cache pages: expected [pages, 2 (or 1: the values are the keys), nkv, page_size, {head_dim}], found {tuple(pages.shape)}")
    if q.shape[1] < num_heads * head_dim or tuple(out.shape) != (T, num_heads * head_dim):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {num_heads} heads of {head_dim}")
    if positions.shape[0] != T or q_start.shape[0] != num_seqs + 1 or block_table.shape[0] < num_seqs:
        raise KernelError("attention: positions need one entry per token, q_start one per sequence plus one, the block table a row per sequence")
    if status is None:
        status = status_word(q.device)
    if lse is not None:
        _check(lse, "logarithms of the sums", torch.float32, 2)
        if tuple(lse.shape) != (T, num_heads):
            raise KernelError(f"attention: lse {tuple(lse.shape)} does not fit {T} tokens of {num_heads} heads")
        _call("attention_tc", "spy_attention_tc_lse", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _ptr(lse), _ptr(pages), _ptr(block_table),
              block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim, _ptr(positions), _ptr(q_start), T, num_seqs,
              int(window or 0), ctypes.c_float(scale), _ptr(status), _stream(), planes)
        return out
    _call("attention_tc", "spy_attention_tc", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _ptr(pages), _ptr(block_table),
          block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim, _ptr(positions), _ptr(q_start), T, num_seqs,
          int(window or 0), ctypes.c_float(scale), _ptr(status), _stream(), planes)
    return out


ATTENTION_DECODE_MAX_SEQS = 1024
ATTENTION_DECODE_MAX_PAIRS = 65536   # sequences x key/value heads


ATTENTION_TMA_PAGE_SIZES = (8, 16, 32, 64, 128)   # a page of the cache is one TMA box


def attention_tc_takes(num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tcgen05 attention kernels (prompt portions and decoding) take these sizes: bfloat16, a
    head size that is a multiple of 8 up to 128 (their tiles are 64 or 128 wide; the TMA boxes fill what
    lies beyond the head size with zeros), at most 16 query heads per key/value head.  The page size must
    be one of ``ATTENTION_TMA_PAGE_SIZES`` besides."""
    return (dtype == torch.bfloat16 and 8 <= head_dim <= 128 and head_dim % 8 == 0 and num_kv_heads > 0 and num_heads % num_kv_heads == 0
            and num_heads // num_kv_heads <= 16)


def attention_decode_takes(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether the persistent tcgen05 decode-attention kernel takes these sizes: those of
    ``attention_tc_takes`` and pages of 8 .. 128 tokens (a power of two)."""
    return attention_tc_takes(num_heads, num_kv_heads, head_dim, dtype) and page_size in ATTENTION_TMA_PAGE_SIZES


def attention_decode(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                     positions: torch.Tensor, q_start: torch.Tensor, num_seqs: int, scale: float, window: Optional[int] = None,
                     status: Optional[torch.Tensor] = None, share: str = "auto", lse: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of a decoding batch (one token per sequence) over its pages: one persistent block
    per SM, keys in the rows of tcgen05 tiles, pages brought in by TMA, the batch's tiles shared out
    evenly over the blocks and merged through scratch memory.  At most 1024 sequences.  ``positions``,
    ``q_start`` and ``block_table`` are read while kernels launched earlier may still be running: they
    must be complete before those start (the engine copies them at the start of a step).  Launches
    on different streams must not overlap (they share the counters of the merge).  ``share``: how
    the work is dealt out, "auto" (the kernel decides), "split" (tiles split evenly, merged) or
    "whole" ((sequence, kv head) pairs whole).  ``lse [T, nh]`` (float32, optional) receives, at every sequence's token, the
    natural logarithm of each head's sum of ``exp(score * scale)``, with which further keys can be merged in."""
    if share not in ("auto", "split", "whole"):
        raise KernelError(f"attention_decode: share {share!r} is not 'auto', 'split' or 'whole'")
    _check(q, "attention queries", torch.bfloat16, 2)
    _check(out, "attention output", torch.bfloat16, 2)
    _check(pages, "cache pages", torch.bfloat16, 5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(q_start, "q_start", torch.int32, 1)
    T = q.shape[0]
    num_pages, planes, nkv, page_size, hd = pages.shape
    if planes not in (1, 2) or hd != head_dim:
        raise KernelError(f"cache pages: expected [pages, 2 (or 1: the values are the keys), nkv, page_size, {head_dim}], found {tuple(pages.shape)}")
    if q.shape[1] < num_heads * head_dim or tuple(out.shape) != (T, num_heads * head_dim):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {num_heads} heads of {head_dim}")
    if positions.shape[0] != T or q_start.shape[0] != num_seqs + 1 or block_table.shape[0] < num_seqs or T < num_seqs:
        raise KernelError("attention: positions need one entry per token, q_start one per sequence plus one, the block table a row per sequence")
    lib = build.load("attention_decode")
    lib.spy_attention_decode_scratch_floats.restype = ctypes.c_longlong
    floats = int(lib.spy_attention_decode_scratch_floats(num_seqs, num_heads, nkv, head_dim))
    scratch = attention_scratch(q.device, floats)
    if status is None:
        status = status_word(q.device)
    if lse is not None:
        _check(lse, "logarithms of the sums", torch.float32, 2)
        if tuple(lse.shape) != (T, num_heads):
            raise KernelError(f"attention: lse {tuple(lse.shape)} does not fit {T} tokens of {num_heads} heads")
        _call("attention_decode", "spy_attention_decode_lse", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _ptr(lse), _ptr(pages), _ptr(block_table),
              block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim, _ptr(positions), _ptr(q_start), T, num_seqs,
              int(window or 0), ctypes.c_float(scale), ("auto", "split", "whole").index(share), _ptr(scratch), ctypes.c_longlong(scratch.numel()),
              _ptr(status), _stream(), planes)
        return out
    _call("attention_decode", "spy_attention_decode", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _ptr(pages), _ptr(block_table),
          block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim, _ptr(positions), _ptr(q_start), T, num_seqs,
          int(window or 0), ctypes.c_float(scale), ("auto", "split", "whole").index(share), _ptr(scratch), ctypes.c_longlong(scratch.numel()),
          _ptr(status), _stream(), planes)
    return out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[M, N] = a[M, K] @ w[N, K]^T`` on the CUDA cores in 32-bit, any sizes and dtypes."""
    _check(a, "gemm input", ndim=2)
    ldw = _check_weight(w, "gemm weight")
    _check(out, "gemm output", ndim=2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes do not fit: input {tuple(a.shape)}, weight {tuple(w.shape)}, output {tuple(out.shape)}")
    _call("gemm_simt", "spy_gemm_simt", _ptr(a), _code(a, "gemm input"), ctypes.c_longlong(K), _ptr(w), _code(w, "gemm weight"),
          ctypes.c_longlong(ldw), _ptr(out), _code(out, "gemm output"), ctypes.c_longlong(N), M, N, K, _stream())
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]``; gate_up [T, 2I], out [T, I]."""
    _check(gate_up, "swiglu input", ndim=2)
    _check(out, "swiglu output", gate_up.dtype, 2)
    T, two_i = gate_up.shape
    if two_i % 2 != 0 or tuple(out.shape) != (T, two_i // 2):
        raise KernelError(f"swiglu: input {tuple(gate_up.shape)} and output {tuple(out.shape)} do not fit")
    _call("swiglu", "spy_swiglu", _ptr(gate_up), _ptr(out), _code(gate_up, "swiglu input"), T, two_i // 2, _stream())
    return out


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``out[t, c] += bias[c]`` in place (32-bit sum); out [T, C] float32 or bfloat16, bias [C]."""
    _check(out, "bias target", ndim=2)
    _check(bias, "bias", ndim=1)
    if bias.shape[0] != out.shape[1]:
        raise KernelError(f"add_bias: a bias of {bias.shape[0]} does not fit rows of {out.shape[1]}")
    _call("swiglu", "spy_add_bias", _ptr(out), _code(out, "bias target"), _ptr(bias), _code(bias, "bias"), out.shape[0], out.shape[1], _stream())
    return out


_ACTIVATIONS = ("relu2", "gelu_tanh", "silu", "relu")


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """``out = act(x)`` element by element in 32-bit; ``kind``: ``relu2`` (the square of relu), ``gelu_tanh``, ``silu``, ``relu``."""
    if kind not in _ACTIVATIONS:
        raise KernelError(f"activation: unknown kind {kind!r} (known: {', '.join(_ACTIVATIONS)})")
    _check(x, "activation input")
    _check(out, "activation output", x.dtype)
    if out.shape != x.shape:
        raise KernelError("activation: input and output differ in shape")
    _call("swiglu", "spy_activation", _ptr(x), _ptr(out), _code(x, "activation input"), ctypes.c_longlong(x.numel()), _ACTIVATIONS.index(kind), _stream())
    return out


def scale_(x: torch.Tensor, scale: float) -> torch.Tensor:
    """``x *= scale`` in place; x float32."""
    _check(x, "scaled tensor", torch.float32)
    _call("swiglu", "spy_scale", _ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(scale), _stream())
    return x


def residual_norm(hidden: torch.Tensor, y: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float, weight_offset: float = 0.0,
                  copy: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``hidden += rms_norm(y) * (weight_offset + weight)`` row by row in 32-bit (``hidden`` float32, in place); ``y`` has hidden's
    shape or is a stack ``[splits, rows, len]`` of partial sums that are added in order.  ``copy`` (optional, any dtype) receives
    the new ``hidden``.  With ``y`` None only the copy is made."""
    _check(hidden, "residual stream", torch.float32, 2)
    rows, H = hidden.shape
    yp, splits, stride = _stack_of(y, hidden, "residual_norm input")
    if y is not None:
        _check(weight, "residual_norm weight", ndim=1)
        if weight.shape[0] != H:
            raise KernelError(f"residual_norm: a weight of {weight.shape[0]} does not fit rows of {H}")
    if copy is not None:
        _check(copy, "residual_norm copy", ndim=2)
        if tuple(copy.shape) != (rows, H):
            raise KernelError(f"residual_norm: the copy {tuple(copy.shape)} differs from the stream {tuple(hidden.shape)}")
    _call("residual_norm", "spy_residual_norm", _ptr(hidden), _ptr(yp), _code(yp, "residual_norm input") if yp is not None else 0, splits,
          ctypes.c_longlong(stride if splits > 1 else 0), _ptr(weight if y is not None else None), _code(weight, "residual_norm weight") if y is not None else 0,
          ctypes.c_float(weight_offset), _ptr(copy), _code(copy, "residual_norm copy") if copy is not None else 0, rows, H, ctypes.c_float(eps), _stream())
    return copy


def latent_prep(fused: torch.Tensor, q_offset: int, q_rank: int, q_weight: Optional[torch.Tensor], cq_out: Optional[torch.Tensor], c_offset: int, kv_rank: int,
                c_weight: Optional[torch.Tensor], rot_dim: int, rope_table: Optional[torch.Tensor], interleaved: bool, positions: torch.Tensor,
                seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor], pages: Optional[torch.Tensor], eps: float,
                status: Optional[torch.Tensor] = None) -> None:
    """The norms and the cache store of attention through a latent.  ``fused [T, ld]`` float32 holds, from column ``q_offset``,
    the query latent (``q_rank`` columns; RMS-normed with ``q_weight`` into ``cq_out [T, q_rank]``) and, from ``c_offset``
    (negative: nothing is stored), the key/value latent (``kv_rank`` columns, RMS-normed with ``c_weight``) followed by the
    shared key part (``rot_dim`` columns, rotated by ``rope_table [positions, r, 2]``: pairs ``(j, j + r)`` or, ``interleaved``,
    ``(2j, 2j + 1)``).  The row ``[latent | rotated part]`` goes to plane 0 of ``pages [num_pages, planes, 1, page_size,
    kv_rank + rot_dim]`` through ``block_table``."""
    _check(fused, "fused projection", torch.float32, 2)
    T, ld = fused.shape
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    if positions.shape[0] != T or seq_of_token.shape[0] != T:
        raise KernelError("latent_prep: positions and seq_of_token must have one entry per token")
    out_code = 0
    if q_rank > 0:
        _check(q_weight, "query latent norm weight", torch.float32, 1)
        _check(cq_out, "query latent", ndim=2)
        if q_offset < 0 or q_offset + q_rank > ld or q_weight.shape[0] != q_rank or tuple(cq_out.shape) != (T, q_rank):
            raise KernelError("latent_prep: the query latent's columns, weight or output do not fit")
        out_code = _code(cq_out, "query latent")
    rot_half = table_rows = page_size = num_pages = planes = width = cache_code = 0
    if c_offset >= 0:
        _check(c_weight, "latent norm weight", torch.float32, 1)
        _check(pages, "cache pages", ndim=5)
        _check(block_table, "block table", torch.int32, 2)
        num_pages, planes, nkv, page_size, hd = pages.shape
        if planes not in (1, 2) or nkv != 1 or hd != kv_rank + rot_dim or c_offset + hd > ld or c_weight.shape[0] != kv_rank:
            raise KernelError(f"latent_prep: cache pages {tuple(pages.shape)} do not fit one head of {kv_rank} + {rot_dim}, or the columns do not fit")
        width, cache_code = block_table.shape[1], _code(pages, "cache pages")
        if rope_table is not None:
            _check(rope_table, "rope table", torch.float32, 3)
            table_rows, rot_half = rope_table.shape[0], rope_table.shape[1]
            if 2 * rot_half > rot_dim:
                raise KernelError(f"latent_prep: {rot_half} rotated pairs do not fit a rotated part of {rot_dim}")
    _call("latent", "spy_latent_prep", _ptr(fused), ctypes.c_longlong(ld), int(q_offset), int(q_rank), _ptr(q_weight), _ptr(cq_out), out_code, int(c_offset),
          int(kv_rank), _ptr(c_weight), int(rot_dim), _ptr(rope_table), rot_half, table_rows, int(bool(interleaved)), _ptr(positions), _ptr(seq_of_token),
          _ptr(block_table if c_offset >= 0 else None), width, _ptr(pages if c_offset >= 0 else None), cache_code, page_size, num_pages, planes,
          ctypes.c_float(eps), T, _ptr(status), _stream())


def head_product(x: torch.Tensor, in_head_stride: int, weight: torch.Tensor, out: torch.Tensor, out_head_stride: int, tail: int = 0,
                 rope_table: Optional[torch.Tensor] = None, interleaved: bool = False, positions: Optional[torch.Tensor] = None,
                 gate: Optional[torch.Tensor] = None, gate_offset: int = 0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t, h * out_head_stride + n] = sum_k weight[h, k, n] * x[t, h * in_head_stride + k]`` (32-bit sums) for a weight
    ``[heads, K, N]``; x and out ``[T, >= heads * stride]`` of one dtype.  ``tail`` elements that follow each head's K inputs go,
    rotated by ``rope_table`` at the token's position (pairs as in ``latent_prep``), to the columns after its N results.
    ``gate`` (float32 ``[T, ld]``): the results are multiplied by ``sigmoid(gate[t, gate_offset + h * N + n])``."""
    _check(x, "head_product input", ndim=2)
    _check(out, "head_product output", x.dtype, 2)
    _check(weight, "head_product weight", ndim=3)
    H, K, N = weight.shape
    T = x.shape[0]
    if (out.shape[0] != T or in_head_stride < K + tail or out_head_stride < N + tail or (H - 1) * in_head_stride + K + tail > x.shape[1]
            or (H - 1) * out_head_stride + N + tail > out.shape[1]):
        raise KernelError(f"head_product: input {tuple(x.shape)}, weight {tuple(weight.shape)}, output {tuple(out.shape)} and the strides do not fit")
    rot_half = table_rows = 0
    if tail > 0:
        _check(positions, "positions", torch.int32, 1)
        if positions.shape[0] != T:
            raise KernelError("head_product: positions must have one entry per token")
        if rope_table is not None:
            _check(rope_table, "rope table", torch.float32, 3)
            table_rows, rot_half = rope_table.shape[0], rope_table.shape[1]
            if 2 * rot_half > tail:
                raise KernelError(f"head_product: {rot_half} rotated pairs do not fit a tail of {tail}")
    gate_ld = 0
    if gate is not None:
        _check(gate, "gate", torch.float32, 2)
        gate_ld = gate.shape[1]
        if gate.shape[0] != T or gate_offset < 0 or gate_offset + H * N > gate_ld:
            raise KernelError("head_product: the gate's columns do not fit")
    _call("latent", "spy_head_product", _ptr(x), ctypes.c_longlong(x.shape[1]), int(in_head_stride), K, _ptr(weight), _code(weight, "head_product weight"), N,
          _ptr(out), ctypes.c_longlong(out.shape[1]), int(out_head_stride), _code(x, "head_product input"), int(tail), _ptr(rope_table), rot_half, table_rows,
          int(bool(interleaved)), _ptr(positions), _ptr(gate), ctypes.c_longlong(gate_ld), int(gate_offset), T, H, _ptr(status), _stream())
    return out


def sample(logits: torch.Tensor, tokens: torch.Tensor, temperature: Optional[torch.Tensor] = None, seed: Optional[torch.Tensor] = None,
           draw: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of ``logits [R, V]`` float32 into ``tokens [R]`` int32: argmax where the
    row's temperature is 0 (or no temperatures are given), else a seeded draw from
    ``softmax(logits / temperature)``, among the row's ``top_k[r]`` largest logits only where
    that is positive (logits equal to the k-th largest all stay)."""
    _check(logits, "logits", torch.float32, 2)
    _check(tokens, "sampled tokens", torch.int32, 1)
    R, V = logits.shape
    if tokens.shape[0] != R:
        raise KernelError("sample: one output token per row of logits is needed")
    if temperature is not None:
        _check(temperature, "temperatures", torch.float32, 1)
        _check(seed, "seeds", torch.int64, 1)
        _check(draw, "draw counters", torch.int64, 1)
        if not (temperature.shape[0] == seed.shape[0] == draw.shape[0] == R):
            raise KernelError("sample: temperature, seed and draw need one entry per row")
    floor_v = None
    if top_k is not None:
        if temperature is None:
            raise KernelError("sample: top_k is for rows with a temperature; give the temperatures too")
        _check(top_k, "top_k", torch.int32, 1)
        if top_k.shape[0] != R:
            raise KernelError("sample: top_k needs one entry per row")
        floor_v = torch.empty(R, dtype=torch.float32, device=logits.device)
    lib = build.load("sampling")
    slices = lib.spy_sample_slices(V)
    slice_v = torch.empty(R * slices, dtype=torch.float32, device=logits.device)
    slice_i = torch.empty(R * slices, dtype=torch.int32, device=logits.device)
    _call("sampling", "spy_sample", _ptr(logits), ctypes.c_longlong(V), R, V, _ptr(temperature), _ptr(seed), _ptr(draw), _ptr(top_k),
          _ptr(floor_v), _ptr(tokens), _ptr(slice_v), _ptr(slice_i), _stream())
    return tokens


def tensor_core_gemm_takes(out_features: int, in_features: int) -> bool:
    """Whether the tcgen05 kernel takes a weight of this shape: its rows must be 16 bytes
    aligned for TMA, so ``in_features`` must be a multiple of 8.  Any ``out_features``."""
    return in_features % 8 == 0 and in_features > 0


_status_words = {}


def status_word(device) -> torch.Tensor:
    """The device's status word: two int32 (code, detail), zero while all is well.  Kernels
    that meet an index outside their buffers, or whose bounded waits run out, store a code
    here and skip the access; the engine reads it after a step."""
    key = str(torch.device(device))
    if key not in _status_words:
        _status_words[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return _status_words[key]


GEMM_SCRATCH_FLOATS = 16 * 1024 * 1024
_gemm_scratch = {}


def _scratch(device) -> torch.Tensor:
    """The split-K scratch of a device: one fixed buffer (64 MB), made at first use, so that
    captured graphs keep pointing at live memory.  Products on one stream use it in turn."""
    key = str(device)
    if key not in _gemm_scratch:
        _gemm_scratch[key] = torch.empty(GEMM_SCRATCH_FLOATS, dtype=torch.float32, device=device)
    return _gemm_scratch[key]


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, epilogue: Optional[str] = None, defer: bool = False,
                 prefetch: Optional[torch.Tensor] = None, prefetch_bytes: int = 0, glu: Optional[tuple] = None) -> torch.Tensor:
    """``a[M, K] @ w[N, K]^T`` on the tensor cores: bfloat16 operands, 32-bit accumulation,
    bfloat16 or float32 output.  K must be a multiple of 8.

    ``epilogue="swiglu"``: ``w``'s rows alternate gate and up rows and the result is
    ``silu(gate) * up``, ``[M, N / 2]``; ``epilogue="geglu_tanh"``: the same with the tanh form of gelu on the gate.  ``epilogue="relu2"``: the result is ``relu(a @ w^T)^2`` (bfloat16 output).  ``defer=True``: when the kernel splits K, the float32
    partial products are returned unsummed as ``[splits, M, N]`` for a consumer that adds them
    (``rmsnorm``'s delta, ``qk_rope_store``'s input); otherwise the result is ``[M, N]``.
    ``prefetch``: a tensor that a later kernel will read (the next product's weights); with up to 256
    rows in ``a`` the blocks ask for its first ``prefetch_bytes`` bytes (0: all) to be brought into L2
    once their own loads are on their way."""
    _check(a, "gemm input", torch.bfloat16, 2)
    ldw = _check_weight(w, "gemm weight", torch.bfloat16)
    M, K = a.shape
    N = w.shape[0]
    if ldw % 8 != 0 or w.data_ptr() % 16 != 0:
        raise KernelError(f"gemm: the weight's rows must start on 16-byte borders (row distance {ldw}, address {w.data_ptr():#x})")
    if w.shape[1] != K:
        raise KernelError(f"gemm: shapes do not fit: input {tuple(a.shape)}, weight {tuple(w.shape)}")
    if epilogue not in (None, "swiglu", "relu2", "geglu_tanh", "clamped_swish"):
        raise KernelError(f"gemm: unknown epilogue {epilogue!r}")
    if epilogue == "clamped_swish":
        # glu = (bias or None, limit, slope): the bias [N] float32 lies in the order of the weight's rows (gate and up in turns)
        if glu is None or (out_dtype or torch.bfloat16) != torch.bfloat16:
            raise KernelError("gemm: the clamped epilogue needs its (bias, limit, slope) and writes bfloat16")
        if glu[0] is not None:
            _check(glu[0], "gate|up bias", torch.float32, 1)
            if glu[0].shape[0] != N:
                raise KernelError("gemm: the clamped epilogue's bias has one entry per weight row")
    if epilogue == "relu2" and (out_dtype or torch.bfloat16) != torch.bfloat16:
        raise KernelError("gemm: the relu2 epilogue writes bfloat16")
    n_out = N // 2 if epilogue in ("swiglu", "geglu_tanh", "clamped_swish") else N
    if status is None:
        status = status_word(a.device)
    lib = build.load("gemm_tcgen05")
    pf_ptr, pf_bytes = None, 0
    if prefetch is not None and M <= 256:
        total = prefetch.numel() * prefetch.element_size()
        pf_ptr, pf_bytes = _ptr(prefetch), min(total, prefetch_bytes) if prefetch_bytes > 0 else total
    if defer and epilogue is None and out is None:
        splits, need = ctypes.c_int(1), ctypes.c_longlong(0)
        lib.spy_gemm_tcgen05_plan(M, N, K, ctypes.c_longlong(1 << 40), ctypes.byref(splits), ctypes.byref(need))
        if splits.value > 1:
            stack = torch.empty((splits.value, M, N), dtype=torch.float32, device=a.device)
            used = ctypes.c_int(0)
            _call("gemm_tcgen05", "spy_gemm_tcgen05_ex", _ptr(a), ctypes.c_longlong(K), _ptr(w), ctypes.c_longlong(ldw), None, BF16,
                  ctypes.c_longlong(N), M, N, K, _ptr(stack), ctypes.c_longlong(stack.numel()), 0, 1, ctypes.byref(used), _ptr(status),
                  _stream(), pf_ptr, ctypes.c_longlong(pf_bytes))
            if used.value != splits.value:
                raise KernelError(f"gemm: planned {splits.value} splits, the kernel used {used.value}")
            return stack
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype or torch.bfloat16, device=a.device)
    else:
        _check(out, "gemm output", ndim=2)
        if tuple(out.shape) != (M, n_out):
            raise KernelError(f"gemm: output {tuple(out.shape)} does not fit [{M}, {n_out}]")
    scratch = _scratch(a.device)
    if epilogue == "clamped_swish":
        _call("gemm_tcgen05", "spy_gemm_tcgen05_clamped", _ptr(a), ctypes.c_longlong(K), _ptr(w), ctypes.c_longlong(ldw), _ptr(out), ctypes.c_longlong(n_out),
              M, N, K, _ptr(scratch), ctypes.c_longlong(scratch.numel()), _ptr(glu[0]), ctypes.c_float(glu[1]), ctypes.c_float(glu[2]), _ptr(status),
              _stream(), pf_ptr, ctypes.c_longlong(pf_bytes))
        return out
    _call("gemm_tcgen05", "spy_gemm_tcgen05_ex", _ptr(a), ctypes.c_longlong(K), _ptr(w), ctypes.c_longlong(ldw), _ptr(out),
          _code(out, "gemm output"), ctypes.c_longlong(n_out), M, N, K, _ptr(scratch), ctypes.c_longlong(scratch.numel()),
          {None: 0, "swiglu": 1, "relu2": 2, "geglu_tanh": 3}[epilogue], 0, None, _ptr(status), _stream(), pf_ptr, ctypes.c_longlong(pf_bytes))
    return out


def gemm_tcgen05_reset() -> None:
    """Lowers the flags that the blocks of a product with shared K blocks signal one another by.
    To be called after a status word of 4 (a wait ran out): the product that gave up may have left
    flags raised, which the next such product would take for partial tiles that are ready."""
    _call("gemm_tcgen05", "spy_gemm_tcgen05_reset", _stream())


def wait_selftest(limit_ns: int, status: Optional[torch.Tensor] = None) -> int:
    """Runs the kernels' bounded wait on a barrier that nothing arrives at, with ``limit_ns`` as its
    limit (at most 100 ms).  The kernel returns by itself and leaves code 4 in the status word; the
    nanoseconds its first thread waited are returned.  A health check of the mechanism that keeps a
    lost signal inside a tensor-core kernel from holding the GPU."""
    dev = torch.device("cuda", torch.cuda.current_device()) if status is None else status.device
    if status is None:
        status = status_word(dev)
    waited = torch.zeros(1, dtype=torch.int64, device=dev)
    _call("gemm_tcgen05", "spy_tcgen05_wait_selftest", ctypes.c_ulonglong(int(limit_ns)), _ptr(status), _ptr(waited), _stream())
    return int(waited.item())



def group_norm(hidden: torch.Tensor, groups: int, eps: float, y: Optional[torch.Tensor] = None, y_weight: Optional[torch.Tensor] = None,
               y_scale: float = 1.0, weight: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
               write_back: bool = True) -> Optional[torch.Tensor]:
    """RMS norm in ``groups`` equal consecutive parts of a row, around the 32-bit stream ``hidden [T, len]``.  With ``y`` (a
    sublayer's output of hidden's shape, or a stack ``[splits, T, len]`` of partial sums) first
    ``hidden += y_scale * group_norm(y) * y_weight`` (stored unless ``write_back`` is false or ``rows`` is given); with
    ``weight`` and ``out [n, len]`` then ``out = group_norm(hidden) * weight``, of all rows or of the gathered ``rows``."""
    _check(hidden, "residual stream", torch.float32, 2)
    T, H = hidden.shape
    yp, splits, stride = _stack_of(y, hidden, "group_norm sublayer output")
    w_code = None
    for w, what in ((y_weight if y is not None else None, "group_norm output weight"), (weight, "group_norm weight")):
        if w is not None:
            _check(w, what, ndim=1)
            if w.shape[0] != H:
                raise KernelError(f"{what}: {w.shape[0]} elements do not fit rows of {H}")
            if w_code is not None and _code(w, what) != w_code:
                raise KernelError("group_norm: the two weights differ in dtype")
            w_code = _code(w, what)
    if y is not None and y_weight is None:
        raise KernelError("group_norm: a sublayer output needs its norm weight")
    n = T
    if rows is not None:
        _check(rows, "group_norm rows", torch.int32, 1)
        n = rows.shape[0]
    if weight is not None:
        _check(out, "group_norm output", ndim=2)
        if tuple(out.shape) != (n, H):
            raise KernelError(f"group_norm output: expected {(n, H)}, found {tuple(out.shape)}")
    elif rows is not None:
        raise KernelError("group_norm: gathered rows need a norm to go through")
    if H % groups:
        raise KernelError(f"group_norm: rows of {H} cannot be cut into {groups} equal groups")
    _call("group_norm", "spy_group_norm", _ptr(hidden), _ptr(yp), _code(yp, "group_norm sublayer output") if yp is not None else 0, max(splits, 1),
          ctypes.c_longlong(stride if splits > 1 else 0), _ptr(y_weight if y is not None else None), ctypes.c_float(y_scale), _ptr(rows),
          _ptr(weight), w_code or 0, _ptr(out if weight is not None else None), _code(out, "group_norm output") if weight is not None else 0,
          n, H, int(groups), ctypes.c_float(eps), int(bool(write_back and rows is None)), _stream())
    return out


def time_conv(x: torch.Tensor, channels: int, kernel: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor], q_start: torch.Tensor,
              state_slot: torch.Tensor, num_seqs: int, longest: int, out: torch.Tensor, residual: bool = False, activation: Optional[str] = None) -> torch.Tensor:
    """Causal convolution over time on the first ``channels`` columns of ``x [T, ld]``: ``kernel [channels, taps]`` (its last
    column meets the current token), optional ``bias``, ``out = act(conv + bias (+ x))``.  The inputs before a request's run
    of this step come from ``state [slots, (taps - 1) * channels]`` (float32) and the run's last ones go there.  ``longest``:
    no request brings more tokens than this."""
    if activation not in (None, "silu"):
        raise KernelError(f"time_conv: unknown activation {activation!r}")
    _check(x, "time_conv input", ndim=2)
    _check(kernel, "time_conv kernel", ndim=2)
    _check(out, "time_conv output", ndim=2)
    _check(q_start, "q_start", torch.int32, 1)
    _check(state_slot, "state_slot", torch.int32, 1)
    taps = kernel.shape[1]
    if kernel.shape[0] != channels or x.shape[1] < channels or out.shape[1] < channels or out.shape[0] != x.shape[0]:
        raise KernelError(f"time_conv: input {tuple(x.shape)}, kernel {tuple(kernel.shape)}, output {tuple(out.shape)} do not fit {channels} channels")
    if bias is not None:
        _check(bias, "time_conv bias", kernel.dtype, 1)
        if bias.shape[0] != channels:
            raise KernelError("time_conv: the bias does not fit the channels")
    if taps > 1:
        _check(state, "time_conv state", torch.float32)
        if state.dim() != 2 or state.shape[1] != (taps - 1) * channels:
            raise KernelError(f"time_conv: state {tuple(state.shape)} does not fit {taps - 1} inputs of {channels} channels")
    if q_start.shape[0] < num_seqs + 1 or state_slot.shape[0] < num_seqs:
        raise KernelError("time_conv: q_start needs one entry per request plus one, state_slot one per request")
    _call("time_conv", "spy_time_conv", _ptr(x), _code(x, "time_conv input"), ctypes.c_longlong(x.shape[1]), _ptr(kernel), _ptr(bias),
          _code(kernel, "time_conv kernel"), _ptr(state if taps > 1 else None), _ptr(q_start), _ptr(state_slot), int(num_seqs), int(longest), _ptr(out),
          _code(out, "time_conv output"), ctypes.c_longlong(out.shape[1]), int(channels), int(taps), int(bool(residual)), 1 if activation == "silu" else 0,
          _stream())
    return out


def diff_qkv_store(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, bias: Optional[torch.Tensor], q_weight: torch.Tensor, k_weight: torch.Tensor,
                   eps: float, rope_table: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor, q_out: torch.Tensor,
                   block_table: torch.Tensor, pages: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                   status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differential attention, the step ahead of the attention kernel.  ``proj [T, ld]`` holds, from the given columns, the
    queries (``heads`` x two maps x ``dim``), the keys (``kv_heads`` x two maps x ``dim``) and the values (``kv_heads`` x
    ``vdim``); ``bias [ld]`` is added.  Every map of a query or key is brought to unit root mean square over ``dim`` and
    multiplied by ``q_weight`` / ``k_weight [dim]``, its pairs ``(2i, 2i + 1)`` rotated by ``rope_table [positions, r, 2]``.
    ``q_out [T, 2 heads, hd]`` gets each map as a query head with zeros in the other map's columns;
    ``pages [num_pages, 2, kv_heads, page_size, hd]`` get the key rows ``[map 1 | map 2]`` and the values."""
    _check(proj, "projection", ndim=2)
    _check(q_out, "queries", ndim=2)
    _check(pages, "cache pages", q_out.dtype, 5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    _check(q_weight, "q norm weight", ndim=1)
    _check(k_weight, "k norm weight", q_weight.dtype, 1)
    T, ld = proj.shape
    num_pages, two, nkv, page_size, hd = pages.shape
    if two != 2 or nkv != kv_heads or tuple(q_out.shape) != (T, 2 * heads * hd) or positions.shape[0] != T or seq_of_token.shape[0] != T:
        raise KernelError(f"diff_qkv_store: pages {tuple(pages.shape)} / queries {tuple(q_out.shape)} do not fit {heads} heads over {kv_heads} of rows {hd}")
    if max(q_col + 2 * heads * dim, k_col + 2 * kv_heads * dim, v_col + kv_heads * vdim) > ld or q_weight.shape[0] != dim or k_weight.shape[0] != dim:
        raise KernelError("diff_qkv_store: the columns or the norm weights do not fit the projection")
    if bias is not None:
        _check(bias, "projection bias", ndim=1)
        if bias.shape[0] != ld:
            raise KernelError("diff_qkv_store: the bias has one entry per column of the projection")
    rot_half = table_rows = 0
    if rope_table is not None:
        _check(rope_table, "rope table", torch.float32, 3)
        table_rows, rot_half = rope_table.shape[0], rope_table.shape[1]
    _call("diff_attention", "spy_diff_qkv_store", _ptr(proj), _code(proj, "projection"), ctypes.c_longlong(ld), int(q_col), int(k_col), int(v_col), _ptr(bias),
          _code(bias, "projection bias") if bias is not None else 0, _ptr(q_weight), _ptr(k_weight), _code(q_weight, "q norm weight"), ctypes.c_float(eps),
          _ptr(rope_table), rot_half, table_rows, _ptr(positions), _ptr(seq_of_token), _ptr(q_out), _code(q_out, "queries"), _ptr(block_table),
          block_table.shape[1], _ptr(pages), _code(pages, "cache pages"), page_size, num_pages, T, int(heads), int(kv_heads), int(dim), int(vdim), hd,
          _ptr(status), _stream())
    return q_out


def sink_qkv_store(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, q_weight: torch.Tensor, k_weight: Optional[torch.Tensor],
                   temp: Optional[torch.Tensor], eps: float, rope_table: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
                   q_out: torch.Tensor, block_table: Optional[torch.Tensor], pages: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int, vdim: int,
                   hd: int, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The step ahead of the attention kernel for queries and keys that are normed over the whole projection.  ``proj [T, ld]``
    holds, from the given columns, the queries (``heads`` x ``dim``), the keys (``kv_heads`` x ``dim``) and the values (``kv_heads``
    x ``vdim``).  All of a token's queries together are brought to unit root mean square and multiplied by ``q_weight [heads dim]``,
    the keys likewise with ``k_weight [kv_heads dim]``; the pairs ``(2i, 2i + 1)`` of every head are rotated by ``rope_table
    [positions, r, 2]``; a query head is multiplied by ``temp[head]``; every value head is brought to unit root mean square over
    ``vdim``.  ``q_out [T, heads hd]`` and ``pages [num_pages, 2, kv_heads, page_size, hd]`` get rows of ``hd`` with zeros behind their
    content.  ``pages`` None: the layer reads another layer's keys and values, and only the queries are made."""
    _check(proj, "projection", ndim=2)
    _check(q_out, "queries", ndim=2)
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    _check(q_weight, "q norm weight", ndim=1)
    T, ld = proj.shape
    if tuple(q_out.shape) != (T, heads * hd) or positions.shape[0] != T or seq_of_token.shape[0] != T or q_weight.shape[0] != heads * dim:
        raise KernelError(f"sink_qkv_store: queries {tuple(q_out.shape)} do not fit {heads} heads of rows {hd}, or the norm weight their {heads * dim} elements")
    if q_col + heads * dim > ld:
        raise KernelError("sink_qkv_store: the query columns do not fit the projection")
    num_pages = page_size = table_width = 0
    if pages is not None:
        _check(pages, "cache pages", q_out.dtype, 5)
        _check(block_table, "block table", torch.int32, 2)
        _check(k_weight, "k norm weight", q_weight.dtype, 1)
        num_pages, two, nkv, page_size, row = pages.shape
        table_width = block_table.shape[1]
        if two != 2 or nkv != kv_heads or row != hd or k_weight.shape[0] != kv_heads * dim or max(k_col + kv_heads * dim, v_col + kv_heads * vdim) > ld:
            raise KernelError(f"sink_qkv_store: pages {tuple(pages.shape)} do not fit {kv_heads} key/value heads of rows {hd}, or the columns the projection")
    if temp is not None:
        _check(temp, "head temperatures", q_weight.dtype, 1)
        if temp.shape[0] != heads:
            raise KernelError("sink_qkv_store: one temperature a head")
    rot_half = table_rows = 0
    if rope_table is not None:
        _check(rope_table, "rope table", torch.float32, 3)
        table_rows, rot_half = rope_table.shape[0], rope_table.shape[1]
    _call("sink_attention", "spy_sink_qkv_store", _ptr(proj), _code(proj, "projection"), ctypes.c_longlong(ld), int(q_col), int(k_col), int(v_col),
          _ptr(q_weight), _ptr(k_weight if pages is not None else None), _ptr(temp), _code(q_weight, "q norm weight"), ctypes.c_float(eps), _ptr(rope_table),
          rot_half, table_rows, _ptr(positions), _ptr(seq_of_token), _ptr(q_out), _code(q_out, "queries"), _ptr(block_table if pages is not None else None),
          table_width, _ptr(pages), page_size, num_pages, T, int(heads), int(kv_heads), int(dim), int(vdim), int(hd), _ptr(status), _stream())
    return q_out


def sink_merge(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, lse: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
               positions: torch.Tensor, seq_of_token: torch.Tensor, scale: float, window: Optional[int], keep_first: int, sink: bool,
               status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Completes a window attention whose normalised result is in ``out [T, nh hd]`` and whose logarithms of the sums of
    exponentials are in ``lse [T, nh]``: the keys of a sequence's first ``keep_first`` positions that lie before the window
    join the softmax, and with ``sink`` one is added to its denominator.  ``out`` is rewritten in place."""
    _check(q, "attention queries", ndim=2)
    _check(out, "attention output", q.dtype, 2)
    _check(lse, "logarithms of the sums", torch.float32, 2)
    _check(pages, "cache pages", q.dtype, 5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    T = q.shape[0]
    num_pages, planes, nkv, page_size, hd = pages.shape
    if planes != 2 or hd != head_dim or q.shape[1] < num_heads * hd or tuple(out.shape) != (T, num_heads * hd) or tuple(lse.shape) != (T, num_heads):
        raise KernelError(f"sink_merge: q {tuple(q.shape)}, out {tuple(out.shape)}, lse {tuple(lse.shape)}, pages {tuple(pages.shape)} do not fit")
    _call("sink_attention", "spy_sink_merge", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _code(q, "attention queries"), _ptr(lse), _ptr(pages),
          _ptr(block_table), block_table.shape[1], page_size, num_pages, int(num_heads), nkv, hd, _ptr(positions), _ptr(seq_of_token), T, int(window or 0),
          int(keep_first), int(bool(sink)), ctypes.c_float(scale), _ptr(status), _stream())
    return out


def diff_combine(attn: torch.Tensor, hd: int, gate: Optional[torch.Tensor], gate_col: int, out: torch.Tensor, heads: int, vdim: int, lam: float,
                 post: float, eps: float) -> torch.Tensor:
    """``out[t, h] = unit_rms(a1 - lam * a2) * post * sigmoid(gate[t, gate_col + h vdim ...])`` with ``a1``, ``a2`` the first
    ``vdim`` elements of the rows ``2h`` and ``2h + 1`` of ``attn [T, 2 heads * hd]``; ``out [T, heads * vdim]``."""
    _check(attn, "attention result", ndim=2)
    _check(out, "combined heads", ndim=2)
    T = attn.shape[0]
    if attn.shape[1] != 2 * heads * hd or tuple(out.shape) != (T, heads * vdim):
        raise KernelError(f"diff_combine: result {tuple(attn.shape)} / output {tuple(out.shape)} do not fit {heads} heads of {vdim} in rows of {hd}")
    gate_ld = 0
    if gate is not None:
        _check(gate, "gate", ndim=2)
        gate_ld = gate.shape[1]
        if gate.shape[0] != T or gate_col < 0 or gate_col + heads * vdim > gate_ld:
            raise KernelError("diff_combine: the gate's columns do not fit")
    _call("diff_attention", "spy_diff_combine", _ptr(attn), _code(attn, "attention result"), int(hd), _ptr(gate), _code(gate, "gate") if gate is not None else 0,
          ctypes.c_longlong(gate_ld), int(gate_col), _ptr(out), _code(out, "combined heads"), T, int(heads), int(vdim), ctypes.c_float(lam),
          ctypes.c_float(post), ctypes.c_float(eps), _stream())
    return out


def mingru_scan(proj: torch.Tensor, z_col: int, x_col: int, g_col: int, z_bias: Optional[torch.Tensor], x_bias: Optional[torch.Tensor], state: torch.Tensor,
                q_start: torch.Tensor, state_slot: torch.Tensor, num_seqs: int, out: torch.Tensor, width: int, longest: Optional[int] = None) -> torch.Tensor:
    """``S <- (1 - z) S + z c`` element by element over every request's tokens of this step, from and into ``state [slots, width]``;
    ``z = sigmoid(proj[:, z_col..] + z_bias)``, ``u = proj[:, x_col..] + x_bias``, ``c = u + 1/2`` where ``u >= 0`` else
    ``sigmoid(u)``; ``out = S * silu(proj[:, g_col..])``.  ``proj`` float32.  ``longest``: no request brings more tokens than this
    (default: the step's token count); long runs are scanned in slices that run side by side."""
    _check(proj, "fused projection", torch.float32, 2)
    _check(state, "recurrent state", torch.float32, 2)
    _check(out, "recurrence output", ndim=2)
    _check(q_start, "q_start", torch.int32, 1)
    _check(state_slot, "state_slot", torch.int32, 1)
    if max(z_col, x_col, g_col) + width > proj.shape[1] or state.shape[1] != width or tuple(out.shape) != (proj.shape[0], width):
        raise KernelError("mingru_scan: the columns, the state or the output do not fit")
    for b in (z_bias, x_bias):
        if b is not None:
            _check(b, "gate bias", ndim=1)
            if b.shape[0] != width or (z_bias is not None and b.dtype != z_bias.dtype):
                raise KernelError("mingru_scan: the biases have one entry per channel and one dtype")
    some = z_bias if z_bias is not None else x_bias
    _call("gated_scan", "spy_mingru_scan", _ptr(proj), ctypes.c_longlong(proj.shape[1]), int(z_col), int(x_col), int(g_col), _ptr(z_bias), _ptr(x_bias),
          _code(some, "gate bias") if some is not None else 0, _ptr(state), _ptr(q_start), _ptr(state_slot), int(num_seqs),
          int(longest if longest is not None else proj.shape[0]), _ptr(out),
          _code(out, "recurrence output"), int(width), _stream())
    return out


def selective_scan(x: torch.Tensor, dt_pre: torch.Tensor, dt_bias: torch.Tensor, proj: torch.Tensor, b_col: int, c_col: int, z: torch.Tensor, z_col: int,
                   a_log: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor, num_seqs: int,
                   out: torch.Tensor, longest: Optional[int] = None) -> torch.Tensor:
    """The selective scan over every request's tokens of this step, from and into ``state [slots, inner * n]``:
    ``dt = softplus(dt_pre + dt_bias)``, ``S[c, n] <- exp(-dt_c exp(a_log[c, n])) S[c, n] + dt_c x_c B_n``,
    ``y_c = sum_n S[c, n] C_n + d_skip_c x_c``, ``out = y * silu(z)``.  ``x [T, inner]``; ``dt_pre [T, inner]`` float32;
    ``proj`` float32 holds ``B`` and ``C`` (``n`` columns each) at ``b_col`` and ``c_col``; ``z`` float32 holds the gate's
    ``inner`` columns from ``z_col``.  ``longest`` as for ``mingru_scan``."""
    _check(x, "scan input", ndim=2)
    T, inner = x.shape
    _check(dt_pre, "step size pre-activation", torch.float32, 2)
    _check(proj, "B and C", torch.float32, 2)
    _check(z, "gate", torch.float32, 2)
    _check(a_log, "A_log", ndim=2)
    _check(dt_bias, "step size bias", a_log.dtype, 1)
    _check(d_skip, "D", a_log.dtype, 1)
    _check(state, "recurrent state", torch.float32, 2)
    _check(out, "scan output", ndim=2)
    n = a_log.shape[1]
    if (tuple(dt_pre.shape) != (T, inner) or a_log.shape[0] != inner or dt_bias.shape[0] != inner or d_skip.shape[0] != inner or state.shape[1] != inner * n
            or tuple(out.shape) != (T, inner) or max(b_col, c_col) + n > proj.shape[1] or proj.shape[0] != T or z.shape[0] != T or z_col + inner > z.shape[1]):
        raise KernelError("selective_scan: shapes do not fit")
    z_view_ptr = ctypes.c_void_p(z.data_ptr() + 4 * z_col)
    _call("gated_scan", "spy_selective_scan", _ptr(x), _code(x, "scan input"), _ptr(dt_pre), _ptr(dt_bias), _ptr(proj), ctypes.c_longlong(proj.shape[1]),
          int(b_col), int(c_col), z_view_ptr, ctypes.c_longlong(z.shape[1]), _ptr(a_log), _ptr(d_skip), _code(a_log, "A_log"), _ptr(state), _ptr(q_start),
          _ptr(state_slot), int(num_seqs), int(longest if longest is not None else T), _ptr(out), _code(out, "scan output"), inner, n, _stream())
    return out


def moe_activation(gate_up: torch.Tensor, logits: torch.Tensor, out: torch.Tensor, experts: int, top: int, ff: int, limit: float, shared_ff: int = 0,
                   shared_limit: float = 0.0, alpha: float = 1.702, weights_out: Optional[torch.Tensor] = None, identity: int = 0,
                   correction: Optional[torch.Tensor] = None, groups: Optional[tuple] = None, activation: str = "clamped_swish",
                   id_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Routing weights and expert activations of a mixture of experts in one pass.  ``logits [T, >= experts + identity (+ 1)]``
    float32: the router's logits and, with a shared expert, its gate's logit behind them.  ``gate_up [T, 2 (experts ff +
    shared_ff)]``: per expert ``[gate | up]``, the shared expert last.  ``out [T, experts ff + shared_ff]`` gets, per expert,
    ``weight * g * sigmoid(alpha g) * (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)`` (``activation``
    ``"silu"``: ``weight * silu(gate) * up``, no clamps); the weight is the expert's softmax score if it is among the token's
    ``top`` chosen, else 0, and ``sigmoid`` of its logit for the shared expert.

    The choice: the softmax runs over ``experts + identity`` router outputs, the last ``identity`` of which are experts that
    return their input (``id_weight [T]`` float32 receives the sum of the chosen ones' weights); ``correction [experts +
    identity]`` float32 is added to the scores for the choice only; ``groups = (count, keep)``: the outputs form ``count`` equal
    groups of neighbours and only those of the ``keep`` groups with the largest best choice score can be chosen."""
    _check(gate_up, "expert gate|up", ndim=2)
    _check(logits, "router logits", torch.float32, 2)
    _check(out, "expert activations", ndim=2)
    if activation not in ("clamped_swish", "silu"):
        raise KernelError(f"moe_activation: unknown activation {activation!r}")
    T = gate_up.shape[0]
    cols, total = experts * ff + shared_ff, experts + int(identity)
    if gate_up.shape[1] != 2 * cols or tuple(out.shape) != (T, cols) or logits.shape[0] != T or logits.shape[1] < total + (1 if shared_ff else 0):
        raise KernelError(f"moe_activation: gate|up {tuple(gate_up.shape)}, logits {tuple(logits.shape)}, output {tuple(out.shape)} do not fit")
    if weights_out is not None:
        _check(weights_out, "routing weights", torch.float32, 2)
        if tuple(weights_out.shape) != (T, total + 1):
            raise KernelError("moe_activation: the routing weights are [T, router outputs + 1]")
    if correction is not None:
        _check(correction, "choice correction", torch.float32, 1)
        if correction.shape[0] != total:
            raise KernelError("moe_activation: the correction has one entry per router output")
    if id_weight is not None:
        _check(id_weight, "identity weights", torch.float32, 1)
        if id_weight.shape[0] != T:
            raise KernelError("moe_activation: one identity weight a token")
    if identity and id_weight is None:
        raise KernelError("moe_activation: identity experts need a place for their weights")
    plain = not identity and correction is None and not groups and activation == "clamped_swish"
    args = (_ptr(gate_up), _code(gate_up, "expert gate|up"), ctypes.c_longlong(gate_up.shape[1]), _ptr(logits),
            ctypes.c_longlong(logits.shape[1]), _ptr(out), _code(out, "expert activations"), ctypes.c_longlong(out.shape[1]), T, int(experts), int(top),
            int(ff), ctypes.c_float(limit), int(shared_ff), ctypes.c_float(shared_limit), ctypes.c_float(alpha), _ptr(weights_out))
    if plain:
        _call("moe", "spy_moe_activation", *args, _stream())
    else:
        count, keep = (int(groups[0]), int(groups[1])) if groups else (0, 0)
        _call("moe", "spy_moe_activation_routed", *args, int(identity), _ptr(correction), count, keep, 1 if activation == "silu" else 0, _ptr(id_weight),
              None, _stream())
    return out


def moe_route_general(logits: torch.Tensor, experts: int, top: int, identity: int = 0, correction: Optional[torch.Tensor] = None,
                      groups: Optional[tuple] = None, has_shared: bool = False):
    """As ``moe_route`` for a choice with the options of ``moe_activation`` (identity experts, correction, groups): the (token,
    chosen real expert) pairs of a step sorted by expert.  Returns ``offsets [experts + 1]``, ``slot [T, top]`` (the row of each
    pair, -1 where a token chose fewer real experts than ``top``), ``row_token``, ``row_w`` (``[T top]``, the first ``offsets[-1]``
    rows count), ``shared_w [T]`` or None, and ``id_weight [T]`` (the chosen identity experts' summed weights) or None."""
    _check(logits, "router logits", torch.float32, 2)
    T, total, dev = logits.shape[0], experts + int(identity), logits.device
    if logits.shape[1] < total + (1 if has_shared else 0):
        raise KernelError("moe_route_general: the logits lack columns")
    weights = torch.empty((T, total + 1), dtype=torch.float32, device=dev)
    floats = torch.empty((2 * T * top + 2 * T,), dtype=torch.float32, device=dev)
    choice_w, row_w, shared_w, idw = floats[:T * top], floats[T * top:2 * T * top], floats[2 * T * top:2 * T * top + T], floats[2 * T * top + T:]
    count, keep = (int(groups[0]), int(groups[1])) if groups else (0, 0)
    _call("moe", "spy_moe_activation_routed", None, BF16, ctypes.c_longlong(0), _ptr(logits), ctypes.c_longlong(logits.shape[1]), None, BF16,
          ctypes.c_longlong(0), T, int(experts), int(top), 1, ctypes.c_float(0.0), 1 if has_shared else 0, ctypes.c_float(0.0), ctypes.c_float(0.0),
          _ptr(weights), int(identity), _ptr(correction), count, keep, 1, _ptr(idw if identity else None), _ptr(shared_w if has_shared else None), _stream())
    ints = torch.empty((3 * T * top + 2 * experts + 1,), dtype=torch.int32, device=dev)
    choice, slot, row_token = ints[:T * top], ints[T * top:2 * T * top], ints[2 * T * top:3 * T * top]
    counts, offsets = ints[3 * T * top:3 * T * top + experts], ints[3 * T * top + experts:]
    _call("moe", "spy_moe_route_weights", _ptr(weights), ctypes.c_longlong(total + 1), T, int(experts), int(top), _ptr(choice), _ptr(choice_w), _ptr(counts),
          _ptr(offsets), _ptr(slot), _ptr(row_token), _ptr(row_w), _stream())
    return offsets, slot.view(T, top), row_token, row_w, (shared_w if has_shared else None), (idw if identity else None)


def add_scaled_rows(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``out[t] += w[t] * x[t]`` in place; out float32 ``[T, H]``, x ``[T, H]``, w float32 ``[T]``."""
    _check(out, "row sum target", torch.float32, 2)
    _check(x, "rows", ndim=2)
    _check(w, "row weights", torch.float32, 1)
    if tuple(x.shape) != tuple(out.shape) or w.shape[0] != out.shape[0]:
        raise KernelError("add_scaled_rows: shapes do not fit")
    _call("moe", "spy_add_scaled_rows", _ptr(out), _ptr(x), _code(x, "rows"), _ptr(w), out.shape[0], out.shape[1], _stream())
    return out


_GATED_ACTIVATIONS = ("silu", "gelu_tanh")      # and "clamped_swish" through ``clamped_glu``


def gated_activation(gate_up: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """``out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i]``; ``kind``: ``silu`` or ``gelu_tanh``."""
    if kind not in _GATED_ACTIVATIONS:
        raise KernelError(f"gated_activation: unknown kind {kind!r}")
    _check(gate_up, "gated activation input", ndim=2)
    _check(out, "gated activation output", gate_up.dtype, 2)
    T, two_i = gate_up.shape
    if two_i % 2 != 0 or tuple(out.shape) != (T, two_i // 2):
        raise KernelError(f"gated_activation: input {tuple(gate_up.shape)} and output {tuple(out.shape)} do not fit")
    _call("swiglu", "spy_gated_activation", _ptr(gate_up), _ptr(out), _code(gate_up, "gated activation input"), T, two_i // 2,
          _GATED_ACTIVATIONS.index(kind), _stream())
    return out


def clamped_glu(gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, limit: float, alpha: float = 1.702) -> torch.Tensor:
    """``out[t, i] = g * sigmoid(alpha g) * (u + 1)`` with ``g = min(gate_up[t, i] + bias[i], limit)`` and ``u = clamp(gate_up[t, I + i]
    + bias[I + i], -limit, limit)``; ``bias [2 I]`` float32 or None; input and output may differ in type."""
    _check(gate_up, "gated activation input", ndim=2)
    _check(out, "gated activation output", ndim=2)
    T, two_i = gate_up.shape
    if two_i % 2 != 0 or tuple(out.shape) != (T, two_i // 2):
        raise KernelError(f"clamped_glu: input {tuple(gate_up.shape)} and output {tuple(out.shape)} do not fit")
    if bias is not None:
        _check(bias, "gate|up bias", torch.float32, 1)
        if bias.shape[0] != two_i:
            raise KernelError("clamped_glu: the bias has one entry per column of the input")
    _call("swiglu", "spy_clamped_glu", _ptr(gate_up), _code(gate_up, "gated activation input"), _ptr(bias), _ptr(out), _code(out, "gated activation output"),
          T, two_i // 2, ctypes.c_float(limit), ctypes.c_float(alpha), _stream())
    return out


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """``x = cap * tanh(x / cap)`` in place; x float32."""
    _check(x, "capped tensor", torch.float32)
    _call("swiglu", "spy_softcap", _ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), _stream())
    return x


def stream_add(stream: torch.Tensor, table: Optional[torch.Tensor], ids: Optional[torch.Tensor], row: Optional[torch.Tensor],
               status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``stream[t] += table[ids[t]] + row`` in place (either term optional); stream float32 ``[T, H]``."""
    _check(stream, "residual stream", torch.float32, 2)
    T, H = stream.shape
    V = 0
    if table is not None:
        _check(table, "embedding table", ndim=2)
        _check(ids, "token ids", torch.int32, 1)
        V = table.shape[0]
        if table.shape[1] != H or ids.shape[0] != T:
            raise KernelError("stream_add: the table's rows and the token ids must fit the stream")
    if row is not None:
        _check(row, "offset row", ndim=1)
        if row.shape[0] != H:
            raise KernelError("stream_add: the offset row must have the stream's width")
    _call("embedding", "spy_stream_add", _ptr(stream), _ptr(table), _code(table, "embedding table") if table is not None else 0, _ptr(ids), _ptr(row),
          _code(row, "offset row") if row is not None else 0, T, H, V, _ptr(status), _stream())
    return stream


def moe_route(logits: torch.Tensor, experts: int, top: int, has_shared: bool):
    """Sorts the (token, chosen expert) pairs of a step by expert.  ``logits [T, >= experts (+ 1)]`` float32 as for
    ``moe_activation``.  Returns ``offsets [experts + 1]`` (where each expert's run of rows starts), ``slot [T, top]`` (the row
    of each pair, the chosen experts in ascending order), ``row_token [T top]``, ``row_w [T top]`` (each row's token and its
    softmax score over all experts) and ``shared_w [T]`` (sigmoid of the shared gate's logit) or None."""
    _check(logits, "router logits", torch.float32, 2)
    T = logits.shape[0]
    if logits.shape[1] < experts + (1 if has_shared else 0):
        raise KernelError("moe_route: the logits lack columns")
    dev = logits.device
    ints = torch.empty((2 * T * top + T * top + experts + experts + 1,), dtype=torch.int32, device=dev)
    choice, slot, row_token = ints[:T * top], ints[T * top:2 * T * top], ints[2 * T * top:3 * T * top]
    counts, offsets = ints[3 * T * top:3 * T * top + experts], ints[3 * T * top + experts:]
    floats = torch.empty((2 * T * top + T,), dtype=torch.float32, device=dev)
    choice_w, row_w, shared_w = floats[:T * top], floats[T * top:2 * T * top], floats[2 * T * top:]
    _call("moe", "spy_moe_route", _ptr(logits), ctypes.c_longlong(logits.shape[1]), T, int(experts), int(top), int(bool(has_shared)), _ptr(choice),
          _ptr(choice_w), _ptr(shared_w), _ptr(counts), _ptr(offsets), _ptr(slot), _ptr(row_token), _ptr(row_w), _stream())
    return offsets, slot.view(T, top), row_token, row_w, (shared_w if has_shared else None)


def gather_rows(x: torch.Tensor, row_token: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[r] = x[row_token[r]]``."""
    _check(x, "gathered tensor", ndim=2)
    _check(out, "gather output", x.dtype, 2)
    _check(row_token, "row tokens", torch.int32, 1)
    if out.shape[1] != x.shape[1] or out.shape[0] != row_token.shape[0]:
        raise KernelError("gather_rows: shapes do not fit")
    _call("moe", "spy_gather_rows", _ptr(x), _ptr(row_token), _ptr(out), out.shape[0], ctypes.c_longlong(x.shape[1] * x.element_size()), _stream())
    return out


def expert_activation(gate_up: torch.Tensor, row_w: torch.Tensor, out: torch.Tensor, limit: float, alpha: float = 1.702,
                      activation: str = "clamped_swish") -> torch.Tensor:
    """``out[r] = row_w[r] * g * sigmoid(alpha g) * (u + 1)`` over rows ``[gate | up]`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``;
    ``activation="silu"``: ``row_w[r] * silu(gate) * up`` without clamps."""
    _check(gate_up, "expert gate|up", ndim=2)
    _check(out, "expert activations", ndim=2)
    _check(row_w, "row weights", torch.float32, 1)
    R, two = gate_up.shape
    if two % 2 or tuple(out.shape) != (R, two // 2) or row_w.shape[0] < R:
        raise KernelError("expert_activation: shapes do not fit")
    _call("moe", "spy_expert_activation", _ptr(gate_up), _code(gate_up, "expert gate|up"), ctypes.c_longlong(two), _ptr(row_w), _ptr(out),
          _code(out, "expert activations"), ctypes.c_longlong(two // 2), R, two // 2, ctypes.c_float(limit), ctypes.c_float(alpha), _stream(),
          1 if activation == "silu" else 0)
    return out


def moe_combine(rows: torch.Tensor, slot: torch.Tensor, shared: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_k rows[slot[t, k]] (+ shared[t])`` in 32-bit, the sum in the order of ``k``."""
    _check(rows, "expert results", ndim=2)
    _check(slot, "slots", torch.int32, 2)
    _check(out, "mixture output", torch.float32, 2)
    T, top = slot.shape
    if tuple(out.shape) != (T, rows.shape[1]) or rows.shape[0] != T * top:
        raise KernelError("moe_combine: shapes do not fit")
    if shared is not None:
        _check(shared, "shared expert result", rows.dtype, 2)
        if tuple(shared.shape) != tuple(out.shape):
            raise KernelError("moe_combine: the shared expert's result does not fit")
    _call("moe", "spy_moe_combine", _ptr(rows), _code(rows, "expert results"), _ptr(slot), top, _ptr(shared), _ptr(out), T, rows.shape[1], _stream())
    return out

