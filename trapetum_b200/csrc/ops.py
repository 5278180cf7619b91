"""Python faces of the CUDA kernels.

Every function takes CUDA tensors, checks what the kernel relies on (device,
dtype, contiguity, sizes) and launches on torch's current stream.  There is no
CPU path and no torch implementation behind these names: a tensor on the CPU,
or a kernel library that cannot be built, is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Tuple, Optional

import torch

from . import build


class KernelError(RuntimeError):
    """A kernel refused its arguments or the launch failed."""


_CODES = {torch.float32: 0, torch.bfloat16: 1}

PAGE_ROWS = 64          # rows of one cache page


def code(dt: torch.dtype) -> int:
    try:
        return _CODES[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {dt}") from None


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    """The current stream's handle.  Every launch asks for it, so it is read through torch's raw accessors where
    this torch has them (a Stream object costs several microseconds to make)."""
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return c_void_p(_RAW_STREAM(_RAW_DEVICE()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("this library computes on the GPU only: got a tensor on " + str(t.device))


_launches = 0


def launches() -> int:
    """How many kernel launches this process has made through this module (graph replays count their kernels)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(lib, status: int, what: str, kernels: int = 1) -> None:
    global _launches
    if status == 0:
        _launches += kernels
        return
    if status < 0:
        raise KernelError(f"{what}: {lib.tb_error().decode()}")
    raise KernelError(f"{what}: CUDA error {status} at launch "
                      f"({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


def _rows_contig(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be 2-D with contiguous rows, got shape {tuple(t.shape)} strides {t.stride()}")


# ---------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = float32(table[ids[t]]) * scale."""
    _cuda(ids, table, out)
    if ids.dtype != torch.int32 or ids.dim() != 1 or not ids.is_contiguous():
        raise KernelError("embed: ids must be a contiguous 1-D int32 tensor")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embed: table must be contiguous [vocab, hidden]")
    V, H = table.shape
    if out is None:
        out = torch.empty((ids.numel(), H), dtype=torch.float32, device=ids.device)
    lib = build.load("embed")
    _check(lib, lib.tb_embed(_ptr(ids), _ptr(table), c_int(code(table.dtype)), _ptr(out), c_int(ids.numel()),
                             c_int(H), c_int(V), c_float(scale), _stream()), "embed")
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """out[i] = x[rows[i]] for a float32 matrix."""
    _cuda(x, rows)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("gather_rows: x must be contiguous float32 [rows, width]")
    if rows.dtype != torch.int32 or not rows.is_contiguous():
        raise KernelError("gather_rows: rows must be contiguous int32")
    out = torch.empty((rows.numel(), x.shape[1]), dtype=torch.float32, device=x.device)
    lib = build.load("embed")
    _check(lib, lib.tb_gather_rows(_ptr(x), _ptr(rows), _ptr(out), c_int(rows.numel()), c_int(x.shape[1]),
                                   c_int(x.shape[0]), _stream()), "gather_rows")
    return out


def random_normal(out: torch.Tensor, key, std: float) -> None:
    """Fill ``out`` (bfloat16 or float32) with the counter-based normal numbers of ``key`` = (k0, k1), times
    ``std``, rounded to bfloat16 (see random_init.cu; ``weights.random_init`` makes the key from seed and name)."""
    _cuda(out)
    if not out.is_contiguous():
        raise KernelError("random_normal: the tensor must be contiguous")
    lib = build.load("random_init")
    _check(lib, lib.tb_random_normal(_ptr(out), c_int(code(out.dtype)), c_longlong(out.numel()),
                                     ctypes.c_uint(key[0]), ctypes.c_uint(key[1]), c_float(std), _stream()),
           "random_normal")


# ---------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, offset: float, out_dtype: torch.dtype) -> torch.Tensor:
    """norm(x) * (offset + w), statistics in 32-bit."""
    _cuda(x, w)
    if x.dim() != 2 or not x.is_contiguous() or w.dim() != 1 or w.numel() != x.shape[1] or not w.is_contiguous():
        raise KernelError(f"rmsnorm: x {tuple(x.shape)} / w {tuple(w.shape)} do not fit")
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    lib = build.load("norm")
    _check(lib, lib.tb_rmsnorm(_ptr(x), c_int(code(x.dtype)), _ptr(w), c_int(code(w.dtype)), _ptr(out),
                               c_int(code(out_dtype)), c_int(x.shape[0]), c_int(x.shape[1]), c_float(eps),
                               c_float(offset), _stream()), "rmsnorm")
    return out


def add_rmsnorm(h: torch.Tensor, a: torch.Tensor, wa: torch.Tensor, eps_a: float, off_a: float,
                wb: Optional[torch.Tensor] = None, eps_b: float = 0.0, off_b: float = 0.0,
                out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """h += norm_a(a) in place (h float32); with wb also returns norm_b(h).  ``a`` is [rows, width], or
    [splits, rows, width] partial sums (float32) that are added in split order on the way."""
    _cuda(h, a, wa, wb)
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("add_rmsnorm: the residual stream must be contiguous float32 [rows, width]")
    n_splits, split_stride = 1, 0
    if a.dim() == 3:
        if a.dtype != torch.float32:
            raise KernelError("add_rmsnorm: partial sums must be float32")
        n_splits, split_stride = a.shape[0], a.stride(0)
        if tuple(a.shape[1:]) != tuple(h.shape) or a.stride(1) != h.shape[1] or a.stride(2) != 1:
            raise KernelError(f"add_rmsnorm: partial sums {tuple(a.shape)} do not fit the stream {tuple(h.shape)}")
    elif a.shape != h.shape or not a.is_contiguous():
        raise KernelError(f"add_rmsnorm: branch {tuple(a.shape)} does not fit the stream {tuple(h.shape)}")
    if wa.numel() != h.shape[1] or (wb is not None and (wb.numel() != h.shape[1] or wb.dtype != wa.dtype)):
        raise KernelError("add_rmsnorm: norm weights do not fit (both must have the row width and one dtype)")
    out = None
    if wb is not None:
        out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
    lib = build.load("norm")
    _check(lib, lib.tb_add_rmsnorm(_ptr(h), _ptr(a), c_int(code(a.dtype)), c_int(n_splits), c_longlong(split_stride),
                                   _ptr(wa), c_float(eps_a), c_float(off_a),
                                   _ptr(wb), c_float(eps_b), c_float(off_b), c_int(code(wa.dtype)),
                                   _ptr(out), c_int(code(out_dtype) if out is not None else 0),
                                   c_int(h.shape[0]), c_int(h.shape[1]), _stream()), "add_rmsnorm")
    return out


def residual_add(h: torch.Tensor, a: torch.Tensor) -> None:
    """h += a (a may be [splits, rows, width] partial sums: they are added one after the other)."""
    _cuda(h, a)
    if a.dim() == 3:
        a = sum_partials(a.contiguous())
    if h.dtype != torch.float32 or not h.is_contiguous() or not a.is_contiguous() or a.shape != h.shape:
        raise KernelError("residual_add: h must be contiguous float32 and a of the same shape")
    lib = build.load("norm")
    _check(lib, lib.tb_residual_add(_ptr(h), _ptr(a), c_int(code(a.dtype)), c_longlong(h.numel()), _stream()),
           "residual_add")


# ---------------------------------------------------------------------------
ACTIVATIONS = {"gelu_tanh": 0, "silu": 1}


def gated_act(gu: torch.Tensor, activation: str, out_dtype: torch.dtype) -> torch.Tensor:
    """act(gu[:, :I]) * gu[:, I:]."""
    _cuda(gu)
    if gu.dim() != 2 or not gu.is_contiguous() or gu.shape[1] % 2:
        raise KernelError("gated_act: input must be contiguous [rows, 2*intermediate]")
    if activation not in ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation '{activation}' (known: {sorted(ACTIVATIONS)})")
    inter = gu.shape[1] // 2
    out = torch.empty((gu.shape[0], inter), dtype=out_dtype, device=gu.device)
    lib = build.load("activation")
    _check(lib, lib.tb_gated_act(_ptr(gu), c_int(code(gu.dtype)), _ptr(out), c_int(code(out_dtype)),
                                 c_int(gu.shape[0]), c_int(inter), c_int(ACTIVATIONS[activation]), _stream()),
           "gated_act")
    return out


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[r, :] += bias in place (x 2-D with contiguous rows, possibly a column slice of a wider matrix)."""
    _cuda(x, bias)
    _rows_contig(x, "add_bias: x")
    if bias.dim() != 1 or bias.numel() != x.shape[1] or not bias.is_contiguous():
        raise KernelError(f"add_bias: bias {tuple(bias.shape)} does not fit rows of width {x.shape[1]}")
    lib = build.load("activation")
    _check(lib, lib.tb_add_bias(_ptr(x), c_int(code(x.dtype)), c_longlong(x.stride(0)), _ptr(bias), c_int(code(bias.dtype)),
                                c_int(x.shape[0]), c_int(x.shape[1]), _stream()), "add_bias")
    return x


# ---------------------------------------------------------------------------
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, softcap: float = 0.0,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a[M,K] @ w[N,K]^T with 32-bit FMA (no tensor cores)."""
    _cuda(a, w, out)
    _rows_contig(a, "gemm: a")
    _rows_contig(w, "gemm: w")
    if a.shape[1] != w.shape[1]:
        raise KernelError(f"gemm: a is {tuple(a.shape)}, w is {tuple(w.shape)}: inner sizes differ")
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        _rows_contig(out, "gemm: out")
    lib = build.load("gemm_simt")
    _check(lib, lib.tb_gemm_simt(_ptr(a), c_int(code(a.dtype)), _ptr(w), c_int(code(w.dtype)), _ptr(out),
                                 c_int(code(out.dtype)), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)),
                                 c_longlong(w.stride(0)), c_longlong(out.stride(0)), c_float(softcap or 0.0),
                                 _stream()), "gemm_simt")
    return out


# ---------------------------------------------------------------------------
class _RopeKvArgs(ctypes.Structure):
    _fields_ = [("qkv", c_void_p), ("row_stride", c_longlong),
                ("q_off", c_int), ("k_off", c_int), ("v_off", c_int),
                ("n_heads", c_int), ("n_kv_heads", c_int), ("head_dim", c_int), ("rotary_dim", c_int),
                ("inv_freq", c_void_p), ("positions", c_void_p), ("token_seq", c_void_p), ("len_after", c_void_p),
                ("k_pool", c_void_p), ("v_pool", c_void_p), ("page_table", c_void_p), ("pt_stride", c_int),
                ("page_rows", c_int), ("ring_rows", c_int),
                ("partial", c_void_p), ("n_splits", c_int), ("split_stride", c_longlong),
                ("partial_row_stride", c_longlong)]


def rope_kv(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
            inv_freq: Optional[torch.Tensor], positions: torch.Tensor, token_seq: torch.Tensor,
            len_after: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
            page_table: Optional[torch.Tensor], ring_rows: int, partial: Optional[torch.Tensor] = None) -> None:
    """Rotate q and k of ``qkv`` [T, (n_heads + 2 n_kv_heads) * head_dim] in place and store k, v
    in the cache line (``k_pool``/``v_pool`` [pages, n_kv_heads, PAGE_ROWS, head_dim]).  With ``partial``
    ([splits, T, width] float32 partial sums of the q/k/v product) the values are taken from their sum
    and ``qkv`` is only written."""
    _cuda(qkv, inv_freq, positions, token_seq, len_after, k_pool, v_pool, page_table, partial)
    if partial is not None and (partial.dtype != torch.float32 or partial.dim() != 3 or partial.shape[1:] != qkv.shape
                                or partial.stride(2) != 1):
        raise KernelError("rope_kv: partial sums must be float32 [splits, tokens, width] matching qkv")
    _rows_contig(qkv, "rope_kv: qkv")
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("rope_kv: qkv width does not fit the head counts")
    for name, t in (("positions", positions), ("token_seq", token_seq)):
        if t.dtype != torch.int32 or t.numel() != T or not t.is_contiguous():
            raise KernelError(f"rope_kv: {name} must be contiguous int32 [{T}]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_kv: inv_freq must be float32 [rotary_dim/2]")
    if k_pool is not None:
        for p in (k_pool, v_pool):
            if p is None or p.dtype != qkv.dtype or not p.is_contiguous() or tuple(p.shape[1:]) != (n_kv_heads, PAGE_ROWS, head_dim):
                raise KernelError("rope_kv: cache pools must be contiguous [pages, n_kv_heads, PAGE_ROWS, head_dim] "
                                  "of the activations' dtype")
        if page_table is None or page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1:
            raise KernelError("rope_kv: page_table must be int32 [batch, pages]")
    a = _RopeKvArgs()
    a.qkv = qkv.data_ptr(); a.row_stride = qkv.stride(0)
    a.q_off = 0; a.k_off = n_heads * head_dim; a.v_off = (n_heads + n_kv_heads) * head_dim
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.rotary_dim = rotary_dim
    a.inv_freq = inv_freq.data_ptr() if inv_freq is not None else None
    a.positions = positions.data_ptr(); a.token_seq = token_seq.data_ptr(); a.len_after = len_after.data_ptr()
    a.k_pool = k_pool.data_ptr() if k_pool is not None else None
    a.v_pool = v_pool.data_ptr() if v_pool is not None else None
    a.page_table = page_table.data_ptr() if page_table is not None else None
    a.pt_stride = page_table.stride(0) if page_table is not None else 0
    a.page_rows = PAGE_ROWS; a.ring_rows = ring_rows
    a.partial = partial.data_ptr() if partial is not None else None
    a.n_splits = partial.shape[0] if partial is not None else 0
    a.split_stride = partial.stride(0) if partial is not None else 0
    a.partial_row_stride = partial.stride(1) if partial is not None else 0
    lib = build.load("rope_kv")
    _check(lib, lib.tb_rope_kv(ctypes.byref(a), c_int(code(qkv.dtype)), c_int(T), _stream()), "rope_kv")


# ---------------------------------------------------------------------------
def attn_prefill_simt(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_start: torch.Tensor,
                      token_seq: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      scale: float, softcap: float, window: int) -> torch.Tensor:
    """Causal attention of packed sequences over their own tokens.  q [T, n_heads*hd] and
    k, v [T, n_kv_heads*hd] may be column slices of one wider matrix."""
    _cuda(q, k, v, seq_start, token_seq)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _rows_contig(t, "attention: " + name)
    if k.stride(0) != v.stride(0) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("attention: k and v must share row stride and dtype with q")
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    lib = build.load("attention_simt")
    _check(lib, lib.tb_attn_prefill_simt(_ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                         _ptr(seq_start), _ptr(token_seq), _ptr(out), c_int(code(q.dtype)), c_int(T),
                                         c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale),
                                         c_float(softcap or 0.0), c_int(window or 0), _stream()), "attn_prefill_simt")
    return out


class _DecodeArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("q_stride", c_longlong), ("k_pool", c_void_p), ("v_pool", c_void_p),
                ("page_table", c_void_p), ("pt_stride", c_int), ("len_after", c_void_p), ("out", c_void_p),
                ("partial", c_void_p),
                ("n_heads", c_int), ("n_kv_heads", c_int), ("hd", c_int), ("page_rows", c_int),
                ("ring_rows", c_int), ("window", c_int), ("n_splits", c_int),
                ("scale", c_float), ("cap", c_float), ("tickets", c_void_p),
                ("qkv_part", c_void_p), ("qkv_splits", c_int), ("qkv_split_stride", c_longlong),
                ("qkv_row_stride", c_longlong), ("inv_freq", c_void_p), ("rotary_dim", c_int)]


def attn_decode_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                     len_after: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                     softcap: float, window: int, ring_rows: int, n_splits: int = 1,
                     scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query per sequence against the paged cache (the new token's k, v already stored)."""
    _cuda(q, k_pool, v_pool, page_table, len_after, scratch)
    _rows_contig(q, "attention: q")
    B = q.shape[0]
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1 or page_table.shape[0] < B:
        raise KernelError("attention: page_table must be int32 [batch, pages]")
    if len_after.dtype != torch.int32 or len_after.numel() < B:
        raise KernelError("attention: len_after must be int32 [batch]")
    out = torch.empty((B, n_heads * head_dim), dtype=q.dtype, device=q.device)
    need = B * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    a = _DecodeArgs()
    a.q = q.data_ptr(); a.q_stride = q.stride(0)
    a.k_pool = k_pool.data_ptr(); a.v_pool = v_pool.data_ptr()
    a.page_table = page_table.data_ptr(); a.pt_stride = page_table.stride(0)
    a.len_after = len_after.data_ptr(); a.out = out.data_ptr()
    a.partial = scratch.data_ptr() if need else None
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = head_dim; a.page_rows = PAGE_ROWS
    a.ring_rows = ring_rows; a.window = window or 0; a.n_splits = n_splits
    a.scale = scale; a.cap = softcap or 0.0
    lib = build.load("attention_simt")
    _check(lib, lib.tb_attn_decode_simt(ctypes.byref(a), c_int(code(q.dtype)), c_int(B), _stream()), "attn_decode_simt")
    return out


# ---------------------------------------------------------------------------
def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Greedy choice per row of float32 logits: int32 ids, the smallest index on a tie."""
    _cuda(logits)
    if logits.dtype != torch.float32:
        raise KernelError("argmax: logits must be float32")
    _rows_contig(logits, "argmax: logits")
    rows, V = logits.shape
    lib = build.load("sampling")
    lib.tb_argmax_scratch_bytes.restype = c_longlong
    nbytes = lib.tb_argmax_scratch_bytes(c_int(rows), c_int(V))
    scratch = torch.empty(max(int(nbytes), 8), dtype=torch.uint8, device=logits.device)
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(lib, lib.tb_argmax(_ptr(logits), c_longlong(logits.stride(0)), c_int(rows), c_int(V), _ptr(out),
                              _ptr(scratch), _stream()), "argmax")
    return out


class _SampleArgs(ctypes.Structure):
    _fields_ = [("logits", c_void_p), ("row_stride", c_longlong), ("vocab", c_int),
                ("temperature", c_void_p), ("top_p", c_void_p), ("penalty", c_void_p), ("draw", c_void_p),
                ("recent", c_void_p), ("n_recent", c_int), ("out", c_void_p)]


WIDE_SAMPLING_FROM = 16384          # vocabularies from this size on are sampled by many CTAs per row


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, penalty: torch.Tensor,
           draw: torch.Tensor, recent: Optional[torch.Tensor], nucleus: bool = True) -> torch.Tensor:
    """Per row: repetition penalty over ``recent`` ids (changes ``logits`` in place), then argmax if
    the row's temperature is <= 0, else a nucleus draw with the row's ``draw`` in [0,1).  ``nucleus=False``:
    the caller knows that every row's top_p is >= 1 (saves the launches that search the threshold)."""
    _cuda(logits, temperature, top_p, penalty, draw, recent)
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    _rows_contig(logits, "sample: logits")
    rows, V = logits.shape
    for name, t in (("temperature", temperature), ("top_p", top_p), ("penalty", penalty), ("draw", draw)):
        if t.dtype != torch.float32 or t.numel() != rows or not t.is_contiguous():
            raise KernelError(f"sample: {name} must be contiguous float32 [{rows}]")
    if recent is not None and (recent.dtype != torch.int32 or recent.dim() != 2 or recent.shape[0] != rows
                               or not recent.is_contiguous()):
        raise KernelError("sample: recent must be contiguous int32 [rows, n]")
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    a = _SampleArgs()
    a.logits = logits.data_ptr(); a.row_stride = logits.stride(0); a.vocab = V
    a.temperature = temperature.data_ptr(); a.top_p = top_p.data_ptr(); a.penalty = penalty.data_ptr()
    a.draw = draw.data_ptr()
    a.recent = recent.data_ptr() if recent is not None else None
    a.n_recent = recent.shape[1] if recent is not None else 0
    a.out = out.data_ptr()
    lib = build.load("sampling")
    if V >= WIDE_SAMPLING_FROM:
        lib.tb_sample_wide_scratch_bytes.restype = c_longlong
        need = int(lib.tb_sample_wide_scratch_bytes(c_int(rows), c_int(V)))
        scratch = torch.empty(need, dtype=torch.uint8, device=logits.device)
        _check(lib, lib.tb_sample_wide(ctypes.byref(a), c_int(rows), _ptr(scratch), c_int(1 if nucleus else 0), _stream()),
               "sample", 10 if nucleus else 4)
        return out
    _check(lib, lib.tb_sample(ctypes.byref(a), c_int(rows), _stream()), "sample")
    return out


# ---------------------------------------------------------------------------
# Choice of kernel per call
# ---------------------------------------------------------------------------
_SMS = {}


def sm_count(device=None) -> int:
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if idx not in _SMS:
        _SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SMS[idx]


def gemm_tc_takes(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core GEMM takes these operands (bfloat16, K and row strides multiples
    of 8 elements, 16-byte aligned); otherwise the FMA kernel computes the product."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        return False
    if a.stride(1) != 1 or w.stride(1) != 1 or a.shape[1] != w.shape[1]:
        return False
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, softcap: float = 0.0,
            splits: Optional[int] = None, out: Optional[torch.Tensor] = None, partials: bool = False,
            gated_act: Optional[str] = None) -> torch.Tensor:
    """a[M,K] @ w[N,K]^T in bfloat16 on tcgen05 tensor cores with 32-bit accumulation.
    ``splits`` None: the library picks the K split (more than 1 only for few tokens and few weight rows).
    ``partials=True`` returns float32 [splits, M, N] whose sum over the first axis, taken in order, is the
    product: a consumer that reads the product once anyway adds them on the way and saves a pass.
    ``gated_act`` ("gelu_tanh" or "silu"): ``w`` holds gate and up rows interleaved in blocks of 16
    (see :func:`interleave_gate_up`); the result is bfloat16 [M, N/2] = act(gate) * up, taken on the
    32-bit accumulators in the epilogue."""
    _cuda(a, w, out)
    if not gemm_tc_takes(a, w):
        raise KernelError(f"gemm_tc does not take a {tuple(a.shape)}/{a.stride()} {a.dtype}, "
                          f"w {tuple(w.shape)}/{w.stride()} {w.dtype}")
    M, K = a.shape
    N = w.shape[0]
    lib = build.load("gemm_tc")
    if splits is None:
        splits = lib.tb_gemm_tc_splits(c_int(M), c_int(N), c_int(K), c_int(sm_count(a.device)))
    splits = int(lib.tb_gemm_tc_effective_splits(c_int(K), c_int(splits)))
    if gated_act is not None:
        if gated_act not in ACTIVATIONS:
            raise KernelError(f"gemm_tc: unknown activation '{gated_act}' (known: {sorted(ACTIVATIONS)})")
        if N % 32 or partials or softcap:
            raise KernelError("gemm_tc: the gated epilogue needs a multiple of 32 weight rows, no partials, no cap")
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
        _check(lib, lib.tb_gemm_tc(_ptr(a), _ptr(w), _ptr(out), c_int(1), c_int(M), c_int(N), c_int(K),
                                   c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                   c_float(0.0), c_int(1), _ptr(None), c_int(1), c_int(ACTIVATIONS[gated_act]),
                                   _stream()), "gemm_tc")
        return out
    if partials:
        if softcap:
            raise KernelError("gemm_tc: a soft cap cannot be applied to partial sums")
        part = torch.empty((splits, M, N), dtype=torch.float32, device=a.device)
        if splits == 1:
            _check(lib, lib.tb_gemm_tc(_ptr(a), _ptr(w), _ptr(part), c_int(0), c_int(M), c_int(N), c_int(K),
                                       c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(N),
                                       c_float(0.0), c_int(1), _ptr(None), c_int(1), c_int(-1), _stream()), "gemm_tc")
        else:
            _check(lib, lib.tb_gemm_tc(_ptr(a), _ptr(w), _ptr(None), c_int(0), c_int(M), c_int(N), c_int(K),
                                       c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(N),
                                       c_float(0.0), c_int(splits), _ptr(part), c_int(0), c_int(-1), _stream()), "gemm_tc")
        return part
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        _rows_contig(out, "gemm: out")
    scratch = None
    if splits > 1:
        scratch = torch.empty(splits * M * N, dtype=torch.float32, device=a.device)
    _check(lib, lib.tb_gemm_tc(_ptr(a), _ptr(w), _ptr(out), c_int(code(out.dtype)), c_int(M), c_int(N), c_int(K),
                               c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                               c_float(softcap or 0.0), c_int(splits), _ptr(scratch), c_int(1), c_int(-1), _stream()), "gemm_tc",
           2 if splits > 1 else 1)
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up matrices -> [2I, K] with rows in blocks of 16: gate 0..15, up 0..15, gate 16..31, ...
    (the layout the gated epilogue of :func:`gemm_tc` expects; I must be a multiple of 16).  Run once, when
    the weights are bound."""
    I, K = gate.shape
    if up.shape != gate.shape or I % 16:
        raise KernelError("interleave_gate_up: gate and up must be [I, K] with I a multiple of 16")
    return torch.stack([gate.view(I // 16, 16, K), up.view(I // 16, 16, K)], dim=1).reshape(2 * I, K).contiguous()


def sum_partials(part: torch.Tensor) -> torch.Tensor:
    """[splits, rows, cols] float32 partial sums -> their sum, added in split order."""
    _cuda(part)
    if part.dtype != torch.float32 or part.dim() != 3 or not part.is_contiguous():
        raise KernelError("sum_partials: wants contiguous float32 [splits, rows, cols]")
    S, R, Cc = part.shape
    if S == 1:
        return part[0]
    out = torch.empty((R, Cc), dtype=torch.float32, device=part.device)
    lib = build.load("gemm_tc")
    _check(lib, lib.tb_sum_partials(_ptr(part), _ptr(out), c_int(R), c_int(Cc), c_int(S), _stream()), "sum_partials")
    return out


def kernel_errors() -> dict:
    """Error words of the kernels with bounded waits that this process has loaded: {} when no wait ever ran
    out.  Synchronises the device and clears the words."""
    out = {}
    loaded = build.loaded()
    if "gemm_tc" in loaded and gemm_tc_error():
        out["gemm_tc"] = "a bounded wait ran out"
    if "attention_decode" in loaded and attn_decode_error():
        out["attention_decode"] = "a bounded wait ran out"
    for name in loaded:
        if name.startswith("attention_prefill_tc@"):
            v = int(build.load(name).tb_attn_prefill_tc_error())
            if v:
                out[name] = f"error word {v}"
    return out


def gemm_tc_set_pair(mode: int) -> int:
    """Many-token products on pairs of SMs: 0 never, 1 whenever the shape allows, 2 where it pays (the default);
    returns the previous setting."""
    return int(build.load("gemm_tc").tb_gemm_tc_set_pair(c_int(int(mode))))


def gemm_tc_error() -> int:
    """Reads and clears the tensor-core GEMM's error word (synchronises): 0, or the role whose
    bounded wait ran out (1 loader, 2 MMA issuer, 3 epilogue; 4 to 6 the same roles of the kernel on pairs of SMs)."""
    return int(build.load("gemm_tc").tb_gemm_tc_error())


def attn_prefill_takes(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether the tensor-core prefill kernel takes this shape (bfloat16, head_dim a multiple of 16 up to 256)."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256


def attn_prefill_lib(head_dim: int) -> str:
    return f"attention_prefill@TB_HD={head_dim}"


def attn_prefill_mma(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_start: torch.Tensor, n_heads: int,
                     n_kv_heads: int, head_dim: int, scale: float, softcap: float, window: int,
                     max_seq_len: int) -> torch.Tensor:
    """Causal attention of packed sequences on tensor cores (see attention_prefill.cu); ``max_seq_len`` is the
    longest sequence of the batch (it sizes the grid)."""
    _cuda(q, k, v, seq_start)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _rows_contig(t, "attention: " + name)
    if not attn_prefill_takes(q.dtype, head_dim) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError(f"attn_prefill_mma does not take {q.dtype} with head_dim {head_dim}")
    if k.stride(0) != v.stride(0):
        raise KernelError("attention: k and v must share their row stride")
    if seq_start.dtype != torch.int32 or not seq_start.is_contiguous() or seq_start.numel() < 2:
        raise KernelError("attention: seq_start must be contiguous int32 [batch + 1]")
    T = q.shape[0]
    B = seq_start.numel() - 1
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    lib = build.load(attn_prefill_lib(head_dim))
    _check(lib, lib.tb_attn_prefill_mma(_ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                        _ptr(seq_start), _ptr(out), c_int(B), c_int(max_seq_len), c_int(n_heads),
                                        c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_float(softcap or 0.0),
                                        c_int(window or 0), _stream()), "attn_prefill_mma")
    return out


def attn_prefill_tc_takes(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether the tcgen05 prefill kernel takes this shape (bfloat16, head_dim 64, 128 or 256)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128, 256)


def attn_prefill_tc_lib(head_dim: int) -> str:
    return f"attention_prefill_tc@TB_HD={head_dim}"


def attn_prefill_tc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_start: torch.Tensor, seq_lens,
                    n_heads: int, n_kv_heads: int, head_dim: int, scale: float, softcap: float, window: int) -> torch.Tensor:
    """Causal attention of packed sequences on tcgen05 tensor cores (see attention_prefill_tc.cu).
    ``seq_lens``: the sequences' lengths on the host."""
    _cuda(q, k, v, seq_start)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _rows_contig(t, "attention: " + name)
    if not attn_prefill_tc_takes(q.dtype, head_dim) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError(f"attn_prefill_tc does not take {q.dtype} with head_dim {head_dim}")
    if k.stride(0) != v.stride(0):
        raise KernelError("attention: k and v must share their row stride")
    B = len(seq_lens)
    if seq_start.dtype != torch.int32 or not seq_start.is_contiguous() or seq_start.numel() != B + 1:
        raise KernelError("attention: seq_start must be contiguous int32 [batch + 1]")
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    lib = build.load(attn_prefill_tc_lib(head_dim))
    _check(lib, lib.tb_attn_prefill_tc(_ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
                                       _ptr(seq_start), _ptr(out), c_int(T), c_int(B), c_int(max(seq_lens)),
                                       c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale),
                                       c_float(softcap or 0.0), c_int(window or 0), _stream()), "attn_prefill_tc", 2)
    return out


def attn_prefill_tc_error(head_dim: int) -> int:
    """Reads and clears the tcgen05 prefill attention's error word (synchronises); 0 = no wait ran out."""
    return int(build.load(attn_prefill_tc_lib(head_dim)).tb_attn_prefill_tc_error())


def attn_prefill(q, k, v, seq_start, token_seq, n_heads, n_kv_heads, head_dim, scale, softcap, window,
                 max_seq_len: int, seq_lens=None, memo: Optional[dict] = None) -> torch.Tensor:
    """Prefill attention, kernel chosen here: tcgen05 for head sizes 64/128/256, mma.sync for other multiples
    of 16, the generic kernel for the rest and for float32.  ``memo``: a per-step dict for what a kernel wants
    uploaded once per step and not once per layer (none does at present)."""
    if attn_prefill_tc_takes(q.dtype, head_dim) and seq_lens is not None:
        return attn_prefill_tc(q, k, v, seq_start, seq_lens, n_heads, n_kv_heads, head_dim, scale, softcap, window)
    if attn_prefill_takes(q.dtype, head_dim):
        return attn_prefill_mma(q, k, v, seq_start, n_heads, n_kv_heads, head_dim, scale, softcap, window, max_seq_len)
    return attn_prefill_simt(q, k, v, seq_start, token_seq, n_heads, n_kv_heads, head_dim, scale, softcap, window)


def attn_decode_takes(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether the bulk-copy decode kernel takes this shape (bfloat16, head_dim 32/64/128/256, up to 8
    query heads per kv head); other shapes run on the generic kernel."""
    if dtype != torch.bfloat16 or n_kv_heads <= 0 or n_heads % n_kv_heads:
        return False
    g = n_heads // n_kv_heads
    return (head_dim in (64, 128, 256) and 1 <= g <= 8) or (head_dim == 32 and g in (1, 2, 4, 8))


_TICKETS: dict = {}
_TICKET_SLOTS = 1 << 16


def _tickets(device: torch.device) -> torch.Tensor:
    """Zeroed counters with which the split pieces of a decode attention launch find out which of them
    finishes last; every launch leaves them at zero.  One array per device: launches that may overlap on
    the GPU (different streams with no order between them) must not both use split pieces."""
    t = _TICKETS.get(device.index)
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("attn_decode: the first launch on a device must not be inside a graph capture")
        t = _TICKETS[device.index] = torch.zeros(_TICKET_SLOTS, dtype=torch.int32, device=device)
    return t


def _decode_partials(part: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, variant: str, rotate):
    """Checks the partial sums handed to a decode kernel that rotates by itself; returns them and a stand-in for q."""
    inv_freq, rotary_dim = rotate
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if variant != "mma" or head_dim < 64:
        raise KernelError("attention: only the tensor-core decode kernel (head_dim >= 64) rotates by itself")
    if part.dtype != torch.float32 or part.dim() != 3 or part.shape[2] != width or part.stride(2) != 1:
        raise KernelError(f"attention: the q/k/v partial sums must be float32 [splits, batch, {width}]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2
                                 or rotary_dim % 2 or not 0 < rotary_dim <= head_dim):
        raise KernelError("attention: inv_freq must be float32 [rotary_dim/2], rotary_dim even and within head_dim")
    _cuda(inv_freq)
    return part, torch.empty((part.shape[1], 0), dtype=torch.bfloat16, device=part.device)


def _set_rotation(a, part, rotate) -> None:
    if part is None:
        a.qkv_part = None; a.qkv_splits = 0; a.qkv_split_stride = 0; a.qkv_row_stride = 0
        a.inv_freq = None; a.rotary_dim = 0
        return
    inv_freq, rotary_dim = rotate
    a.q = None; a.q_stride = 0
    a.qkv_part = part.data_ptr(); a.qkv_splits = part.shape[0]
    a.qkv_split_stride = part.stride(0); a.qkv_row_stride = part.stride(1)
    a.inv_freq = inv_freq.data_ptr() if inv_freq is not None else None
    a.rotary_dim = rotary_dim if inv_freq is not None else 0


def attn_decode_tma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                    len_after: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                    softcap: float, window: int, ring_rows: int, n_splits: int = 1,
                    variant: str = "mma", rotate=None) -> torch.Tensor:
    """Decode attention with pages staged in shared memory by bulk copies (see attention_decode.cu).
    ``variant``: "mma" (tensor cores, the product path) or "lanes" (scalar, kept for comparison).
    ``rotate`` = (inv_freq or None, rotary_dim), "mma" only: ``q`` is then the float32 partial sums
    [splits, batch, (n_heads + 2 n_kv_heads) * head_dim] of the q/k/v product; the kernel adds them, rotates q and k
    at the new token's position, and writes k and v to the cache itself (no separate rotation kernel)."""
    _cuda(q, k_pool, v_pool, page_table, len_after)
    part = None
    if rotate is not None:
        part, q = _decode_partials(q, n_heads, n_kv_heads, head_dim, variant, rotate)
    _rows_contig(q, "attention: q")
    B = q.shape[0]
    if not attn_decode_takes(q.dtype, n_heads, n_kv_heads, head_dim):
        raise KernelError(f"attn_decode_tma does not take {q.dtype}, {n_heads}/{n_kv_heads} heads, head_dim {head_dim}")
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1 or page_table.shape[0] < B:
        raise KernelError("attention: page_table must be int32 [batch, pages]")
    if len_after.dtype != torch.int32 or len_after.numel() < B:
        raise KernelError("attention: len_after must be int32 [batch]")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE_ROWS, head_dim) or k_pool.shape != v_pool.shape \
            or not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.dtype != q.dtype:
        raise KernelError("attention: pools must be contiguous [pages, n_kv_heads, PAGE_ROWS, head_dim] of q's dtype")
    out = torch.empty((B, n_heads * head_dim), dtype=q.dtype, device=q.device)
    scratch = None
    if n_splits > 1:
        scratch = torch.empty(B * n_heads * n_splits * (head_dim + 2), dtype=torch.float32, device=q.device)
    a = _DecodeArgs()
    a.q = q.data_ptr(); a.q_stride = q.stride(0)
    a.k_pool = k_pool.data_ptr(); a.v_pool = v_pool.data_ptr()
    a.page_table = page_table.data_ptr(); a.pt_stride = page_table.stride(0)
    a.len_after = len_after.data_ptr(); a.out = out.data_ptr()
    a.partial = scratch.data_ptr() if scratch is not None else None
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = head_dim; a.page_rows = PAGE_ROWS
    a.ring_rows = ring_rows; a.window = window or 0; a.n_splits = n_splits
    a.scale = scale; a.cap = softcap or 0.0
    fused_fold = variant == "mma" and head_dim >= 64 and n_splits > 1 and B * n_kv_heads <= _TICKET_SLOTS
    a.tickets = _tickets(q.device).data_ptr() if fused_fold else None
    _set_rotation(a, part, rotate)
    lib = build.load("attention_decode")
    fn = lib.tb_attn_decode if variant == "mma" else lib.tb_attn_decode_lanes
    _check(lib, fn(ctypes.byref(a), c_int(code(q.dtype)), c_int(B), _stream()), "attn_decode",
           2 if (n_splits > 1 and not fused_fold) else 1)
    return out


def attn_decode_stream(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                       len_after: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                       softcap: float, window: int, ring_rows: int, n_ctas: Optional[int] = None,
                       rotate=None) -> torch.Tensor:
    """Decode attention on tensor cores with all pages of the launch dealt out evenly to ``n_ctas`` CTAs
    (default: one per SM), wherever the sequences end: the time of a launch follows the sum of the lengths,
    not the longest one (see attention_decode.cu).  ``rotate``: as in :func:`attn_decode_tma`."""
    _cuda(q, k_pool, v_pool, page_table, len_after)
    part = None
    if rotate is not None:
        part, q = _decode_partials(q, n_heads, n_kv_heads, head_dim, "mma", rotate)
    _rows_contig(q, "attention: q")
    B = q.shape[0]
    if not attn_decode_stream_takes(q.dtype, n_heads, n_kv_heads, head_dim, B):
        raise KernelError(f"attn_decode_stream does not take {q.dtype}, {n_heads}/{n_kv_heads} heads, "
                          f"head_dim {head_dim}, batch {B}")
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.stride(1) != 1 or page_table.shape[0] < B:
        raise KernelError("attention: page_table must be int32 [batch, pages]")
    if len_after.dtype != torch.int32 or len_after.numel() < B:
        raise KernelError("attention: len_after must be int32 [batch]")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE_ROWS, head_dim) or k_pool.shape != v_pool.shape \
            or not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.dtype != q.dtype:
        raise KernelError("attention: pools must be contiguous [pages, n_kv_heads, PAGE_ROWS, head_dim] of q's dtype")
    lib = build.load("attention_decode")
    if n_ctas is None:
        n_ctas = int(lib.tb_attn_decode_stream_ctas(c_int(sm_count(q.device)), c_int(head_dim)))
    lib.tb_attn_decode_stream_scratch_floats.restype = c_longlong
    need = int(lib.tb_attn_decode_stream_scratch_floats(c_int(n_ctas), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim)))
    out = torch.empty((B, n_heads * head_dim), dtype=q.dtype, device=q.device)
    scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    a = _DecodeArgs()
    a.q = q.data_ptr(); a.q_stride = q.stride(0)
    a.k_pool = k_pool.data_ptr(); a.v_pool = v_pool.data_ptr()
    a.page_table = page_table.data_ptr(); a.pt_stride = page_table.stride(0)
    a.len_after = len_after.data_ptr(); a.out = out.data_ptr()
    a.partial = scratch.data_ptr()
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = head_dim; a.page_rows = PAGE_ROWS
    a.ring_rows = ring_rows; a.window = window or 0; a.n_splits = 0
    a.scale = scale; a.cap = softcap or 0.0
    a.tickets = _tickets(q.device).data_ptr()
    _set_rotation(a, part, rotate)
    _check(lib, lib.tb_attn_decode_stream(ctypes.byref(a), c_int(code(q.dtype)), c_int(B), c_int(n_ctas), _stream()),
           "attn_decode_stream")
    return out


def attn_decode_rotates(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether :func:`attn_decode` can take the q/k/v partial sums and rotate by itself (``rotate=``)."""
    return attn_decode_takes(dtype, n_heads, n_kv_heads, head_dim) and head_dim >= 64


def attn_decode_stream_takes(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, batch: int) -> bool:
    return (attn_decode_takes(dtype, n_heads, n_kv_heads, head_dim) and head_dim >= 64
            and batch <= 1024 and batch * n_kv_heads <= _TICKET_SLOTS)


def attn_decode_error() -> int:
    """Reads and clears the decode attention's error word (synchronises): 0, or 1 a bounded wait ran out, 2 the
    shared-memory block began less aligned than budgeted, 3 a CTA of the stream partition had more runs than its
    list holds.  After an error the ticket counters are zeroed again (a launch that gave up may have left them
    half counted)."""
    v = int(build.load("attention_decode").tb_attn_decode_error())
    if v:
        for t in _TICKETS.values():
            t.zero_()
    return v


def choose_decode_splits(batch: int, n_kv_heads: int, pages: int, sms: int) -> int:
    """In how many pieces decode attention cuts a sequence's pages.  A CTA serves one (sequence, kv head,
    piece); all CTAs of a launch are about equally long, so the launch takes ceil(CTAs / SMs) rounds.
    Among the piece counts that keep at least 4 pages per piece, take the one that wastes least of the
    last round (ties: fewer pieces)."""
    items = max(1, batch * n_kv_heads)
    best, best_eff = 1, 0.0
    for s in range(1, max(1, pages // 4) + 1):
        if s > 64:
            break
        ctas = items * s
        eff = ctas / (((ctas + sms - 1) // sms) * sms)
        # a piece pays its start-up and its share of the final fold: about four pages' worth (measured)
        per = (pages + s - 1) // s
        eff *= per / (per + 4.0)
        if eff > best_eff + 1e-9:
            best, best_eff = s, eff
    return best


_DECODE_PARTITION = None          # None: chosen per launch; "split" or "stream": forced (tests, comparisons)


def set_decode_partition(mode: Optional[str]) -> Optional[str]:
    """Forces decode attention's partition ("split", "stream") or gives the choice back (None); returns the
    previous setting.  Set it before an engine captures its decode graphs."""
    global _DECODE_PARTITION
    if mode not in (None, "split", "stream"):
        raise KernelError(f"decode partition {mode!r}: None, 'split' or 'stream'")
    was, _DECODE_PARTITION = _DECODE_PARTITION, mode
    return was


def decode_partition_is_stream(batch: int, n_kv_heads: int, pages: int, splits: int, uneven: int, sms: int) -> bool:
    """Whether decode attention deals its pages out as one stream (else every sequence is cut into ``splits``
    pieces).  A streaming launch costs about ten pages' time more (its CTAs walk several sequences: page prefix,
    a rotation and a fold per run), so it is taken when the pieces of the longest sequence are at least that much
    longer than an even share: ``uneven`` quarters of a piece's pages are saved at least.  And when cutting
    every sequence would take more than two rounds of CTAs: each round pays its start-up again."""
    per = (pages + splits - 1) // splits
    return uneven * per >= 4 * 10 or batch * n_kv_heads * splits > 2 * sms


def attn_decode_plan(batch: int, n_kv_heads: int, len_bucket: int, ring_rows: int, uneven: int, device) -> Tuple[bool, int]:
    """(whether the pages of a decode launch are dealt out as one stream, else in how many pieces every sequence
    is cut), from what a captured step may depend on."""
    rows = min(len_bucket, ring_rows) if ring_rows else len_bucket
    pages = max(1, (rows + PAGE_ROWS - 1) // PAGE_ROWS)
    sms = sm_count(device)
    splits = choose_decode_splits(batch, n_kv_heads, pages, sms)
    stream = decode_partition_is_stream(batch, n_kv_heads, pages, splits, int(uneven), sms)
    if _DECODE_PARTITION is not None:
        stream = _DECODE_PARTITION == "stream"
    return stream, splits


def attn_decode(q, k_pool, v_pool, page_table, len_after, n_heads, n_kv_heads, head_dim, scale, softcap, window,
                ring_rows, len_bucket: int, uneven: int = 0, rotate=None) -> torch.Tensor:
    """Decode attention, kernel and partition chosen here.  ``len_bucket``: an upper bound of the longest
    context of the batch (the engine passes a power of two so that the choice is stable across steps).
    ``uneven``: how much the batch's contexts differ in length (``engine.unevenness``, 0..3); if enough, the pages
    are dealt out to the CTAs as one stream, so that the launch's time follows the sum of the lengths and not
    the longest one."""
    B = q.shape[0] if rotate is None else q.shape[1]
    dt = q.dtype if rotate is None else torch.bfloat16
    stream, splits = attn_decode_plan(B, n_kv_heads, len_bucket, ring_rows, uneven, q.device)
    if stream and attn_decode_stream_takes(dt, n_heads, n_kv_heads, head_dim, B):
        return attn_decode_stream(q, k_pool, v_pool, page_table, len_after, n_heads, n_kv_heads, head_dim, scale,
                                  softcap, window, ring_rows, rotate=rotate)
    if attn_decode_takes(dt, n_heads, n_kv_heads, head_dim):
        variant = "lanes" if head_dim < 64 else "mma"     # a 64-byte row has no swizzled box for the tensor-core kernel
        return attn_decode_tma(q, k_pool, v_pool, page_table, len_after, n_heads, n_kv_heads, head_dim, scale,
                               softcap, window, ring_rows, splits, variant, rotate)
    if rotate is not None:
        raise KernelError("attention: this shape's decode kernel does not rotate by itself")
    return attn_decode_simt(q, k_pool, v_pool, page_table, len_after, n_heads, n_kv_heads, head_dim, scale,
                            softcap, window, ring_rows, splits)
