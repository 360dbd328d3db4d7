"""Python face of the CUDA kernels: argument checks, then a ctypes call on the
current CUDA stream.  Nothing here computes; a tensor on the CPU, of the wrong
type or not contiguous is an error, never a detour through another
implementation.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_TYPE = {torch.float32: F32, torch.bfloat16: BF16}

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


class KernelError(RuntimeError):
    pass


launches = 0  # launcher calls that succeeded since import (each is one or two kernels)


def _check(code: int, what: str) -> None:
    global launches
    if code == 0:
        launches += 1
        return
    if code == -1:
        raise KernelError(f"{what}: bad argument")
    if code == -2:
        raise KernelError(f"{what}: size or option not supported by this kernel")
    if code == -3:
        raise KernelError(f"{what}: CUDA driver call failed")
    if code <= -10:
        raise KernelError(f"{what}: refused with code {code}")
    raise KernelError(f"{what}: CUDA error {code}")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    # the raw handle of the current stream of the current device (torch.cuda.current_stream() builds a
    # Stream object around the same number, several microseconds a call)
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _dev(t: torch.Tensor, name: str, dtype=None, contiguous=True):
    if _pending is not None and t.dtype == torch.float32 and t.data_ptr() == _pending[0].data_ptr():
        resolve_pending()   # an operand whose last matrix product is still in planes: add them first
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def _code(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _TYPE:
        raise KernelError(f"{name}: dtype {t.dtype} is not supported (float32 or bfloat16)")
    return _TYPE[t.dtype]


_sigs_done = set()
_timings = None  # name -> [calls, milliseconds] while kernel timing is on


def enable_timing(on: bool = True) -> None:
    """Per-launcher CUDA-event timers (each call is synchronised: for profiling only)."""
    global _timings
    _timings = {} if on else None


def timing_report() -> dict:
    """{launcher: (calls, total ms)} since enable_timing(True)."""
    return {k: tuple(v) for k, v in (_timings or {}).items()}


_fns = {}   # (library, function, macros) -> the ctypes function with its signature set


def _fn(lib_name: str, fn_name: str, argtypes, macros=None, extra_flags=(), tag=None):
    key = (lib_name, fn_name, tuple(sorted(macros.items())) if macros else None, extra_flags)
    fn = _fns.get(key)
    if fn is None:
        lib = load_library(lib_name, macros, extra_flags)
        fn = getattr(lib, fn_name)
        if (id(lib), fn_name) not in _sigs_done:
            fn.argtypes = argtypes
            fn.restype = c_int
            _sigs_done.add((id(lib), fn_name))
        _fns[key] = fn
    if _timings is None:
        return fn

    def timed(*args):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        rc = fn(*args)
        e.record()
        e.synchronize()
        rec = _timings.setdefault(fn_name if tag is None else f"{fn_name} {tag}", [0, 0.0])
        rec[0] += 1
        rec[1] += s.elapsed_time(e)
        return rc
    return timed


# ------------------------------------------------------------------ elementwise

def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None,
                 scale: float = 1.0) -> torch.Tensor:
    """float32 rows ``table[ids] * scale`` (the start of the residual stream)."""
    _dev(table, "table"); _dev(ids, "ids", torch.int32)
    V, H = table.shape
    T = ids.numel()
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _dev(out, "out", torch.float32)
    fn = _fn("elementwise", "bw_embed_gather",
             [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(table), _code(table, "table"), _ptr(ids), _ptr(out), T, H, V, float(scale), _stream()), "embed_gather")
    return out


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: Optional[float] = None) -> torch.Tensor:
    """In place on float32 ``logits``: times ``scale``, then ``softcap * tanh(x / softcap)`` if a cap is given."""
    _dev(logits, "logits", torch.float32)
    if softcap is not None and not softcap > 0:
        raise KernelError("logit_transform: the soft cap must be positive")
    fn = _fn("elementwise", "bw_logit_transform", [c_void_p, c_ll, c_float, c_float, c_void_p])
    _check(fn(_ptr(logits), logits.numel(), float(scale), float(softcap or 0.0), _stream()), "logit_transform")
    return logits


# ------------------------------------------------------------------ sums left to the reader
#
# For up to DEFER_MAX_TOKENS tokens a product that is ADDED to a float32 tensor (the
# residual stream) can leave its K splits unsummed, as planes in a buffer of this module
# (gemm_tc_deferred): no CTA then waits for another's partial sums.  The planes are added by
# whichever kernel reads the tensor next: rmsnorm adds them while it normalises; every other
# function of this module adds them with a kernel of its own first (through _dev); code that reads
# the tensor by other means calls resolve_pending() before.  At most one sum is outstanding.

DEFER_SUMS = os.environ.get("BW_DEFER_SUMS", "1") != "0"
# Linear.add_to leaves sums open up to this many tokens (measured on a B200: 4 % less step time at 1 to 16
# tokens, 1.5 % at 24 to 64, 0.5 % at 128, nothing at 256)
DEFER_MAX_TOKENS = int(os.environ.get("BW_DEFER_MAX_TOKENS", "128"))
_pending = None          # (target tensor, planes [S, M, N]) or None
_plane_buffers = {}
PLANE_BUFFER_ELEMS = 8 << 20
_plane_generation = 0    # counts the products that left planes: whoever keeps planes for later checks that they are still the last


def _plane_buffer(device: torch.device) -> torch.Tensor:
    buf = _plane_buffers.get(device)
    if buf is None:
        buf = _plane_buffers[device] = torch.empty(PLANE_BUFFER_ELEMS, dtype=torch.float32, device=device)
    return buf


def pending_target() -> Optional[torch.Tensor]:
    """The tensor whose last product is still in planes (None: nothing is outstanding)."""
    return None if _pending is None else _pending[0]


def resolve_pending() -> None:
    """Adds an outstanding sum into its tensor (a no-op when nothing is outstanding)."""
    global _pending
    if _pending is None:
        return
    target, planes = _pending
    _pending = None
    fn = _fn("elementwise", "bw_add_planes", [c_void_p, c_void_p, c_int, c_ll, c_ll, c_void_p])
    _check(fn(_ptr(target), _ptr(planes), planes.shape[0], planes.stride(0), target.numel(), _stream()), "add_planes")


def discard_pending(t: Optional[torch.Tensor] = None) -> None:
    """Forgets an outstanding sum into ``t`` (None: into whatever tensor): it is not read again."""
    global _pending
    if _pending is not None and (t is None or _pending[0].data_ptr() == t.data_ptr()):
        _pending = None


def gemm_tc_planes(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   force_splits: int = 0) -> torch.Tensor:
    """x @ w.T (+ bias) for up to GEMM_PLANES_MAX_TOKENS tokens as float32 planes [S, M, N] that
    add up to it (in plane order; the bias is in plane 0), in this module's plane buffer: valid until
    the next call.  An outstanding sum is resolved first."""
    resolve_pending()
    _dev(x, "x", torch.bfloat16, contiguous=False); _dev(w, "w", torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    if not gemm_tc_supports(x, w) or w.shape[1] != K or M > GEMM_PLANES_MAX_TOKENS:
        raise KernelError("gemm_tc_planes: bfloat16 operands the tensor-core product takes, at most "
                          f"{GEMM_PLANES_MAX_TOKENS} tokens")
    if bias is not None:
        _dev(bias, "bias")
        if bias.numel() != N:
            raise KernelError("gemm: bias must have N entries")
    buf = _plane_buffer(x.device)
    n = c_int(0)
    fn = _fn("gemm_tc", "bw_gemm_tc_planes", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_ll, c_int, c_int, c_int,
                                               c_ll, c_int, ctypes.POINTER(c_int), c_void_p],
             macros=_gemm_macros(), tag=f"planes{M}x{N}x{K}" if _timings is not None else None)
    global _plane_generation
    _plane_generation += 1
    _check(fn(_ptr(x), _ptr(w), _ptr(bias), _code(bias, "bias") if bias is not None else 0, _ptr(buf), buf.numel(),
              M, N, K, x.stride(0), int(force_splits), ctypes.byref(n), _stream()), "gemm_tc_planes")
    return buf[:n.value * M * N].view(n.value, M, N)


def planes_generation() -> int:
    """A number that changes with every product that leaves planes in this module's buffer."""
    return _plane_generation


def gemm_tc_deferred(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out += x @ w.T (+ bias), the sum left to the next reader of ``out`` (float32 [M, N], contiguous)."""
    global _pending
    if out.dtype != torch.float32 or not out.is_contiguous() or out.shape != (x.shape[0], w.shape[0]):
        raise KernelError("gemm_tc_deferred: out must be contiguous float32 [M, N]")
    planes = gemm_tc_planes(x, w, bias)
    _pending = (out, planes)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    global _pending
    mine = None              # an outstanding sum into x: added by the kernel below instead of one of its own
    if _pending is not None and _pending[0].data_ptr() == x.data_ptr() and _pending[0].shape == x.shape:
        mine, _pending = _pending, None
    keep = mine is not None  # the sum stays outstanding unless the kernel below adds it into x
    try:
        out = _rmsnorm(x, w, eps, out_dtype, rows, out, None if mine is None else mine[1])
        keep = keep and rows is not None     # with chosen rows x is left as it is
        return out
    finally:
        if keep:
            _pending = mine


def _rmsnorm(x, w, eps, out_dtype, rows, out, planes):
    _dev(x, "x", torch.float32); _dev(w, "w")
    H = x.shape[-1]
    if w.numel() != H:
        raise KernelError(f"rmsnorm: gain has {w.numel()} elements, rows have {H}")
    n = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _dev(rows, "rows", torch.int32)
    if out is None:
        out = torch.empty((n, H), dtype=out_dtype, device=x.device)
    _dev(out, "out", out_dtype)
    if planes is not None:
        fn = _fn("elementwise", "bw_add_rmsnorm", [c_void_p, c_void_p, c_int, c_ll, c_void_p, c_int, c_void_p, c_void_p,
                                                   c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_ptr(x), _ptr(planes), planes.shape[0], planes.stride(0), _ptr(w), _code(w, "w"), _ptr(rows), _ptr(out),
                  _code(out, "out"), n, H, float(eps), _stream()), "add_rmsnorm")
        return out
    fn = _fn("elementwise", "bw_rmsnorm",
             [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(x), _ptr(w), _code(w, "w"), _ptr(rows), _ptr(out), _code(out, "out"), n, H,
              float(eps), _stream()), "rmsnorm")
    return out


def swiglu(gu: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    _dev(gu, "gate_up")
    T, I2 = gu.shape
    if I2 % 2:
        raise KernelError("swiglu: input width must be even (gate | up)")
    out = torch.empty((T, I2 // 2), dtype=out_dtype or gu.dtype, device=gu.device)
    fn = _fn("elementwise", "bw_swiglu", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(gu), _code(gu, "gate_up"), _ptr(out), _code(out, "out"), T, I2 // 2, _stream()), "swiglu")
    return out


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """cos and sin of ``pos * inv_freq`` per token: float32 [T, rotary_dim] (cos, then sin)."""
    _dev(positions, "positions", torch.int32); _dev(inv_freq, "inv_freq", torch.float32)
    T = positions.numel()
    table = torch.empty((T, rotary_dim), dtype=torch.float32, device=positions.device)
    fn = _fn("elementwise", "bw_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(positions), _ptr(inv_freq), _ptr(table), rotary_dim, T, _stream()), "rope_table")
    return table


def kv_slots(positions: torch.Tensor, req_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int,
             num_pages: int) -> torch.Tensor:
    """int32 [T]: ``page * page_size + slot`` of every token's position in its request's block table
    (-1 where the table names no page): where the token's keys and values go, for every layer of
    the cache group."""
    _dev(positions, "positions", torch.int32); _dev(req_of_token, "req_of_token", torch.int32)
    _dev(block_table, "block_table", torch.int32)
    T = positions.numel()
    out = torch.empty(T, dtype=torch.int32, device=positions.device)
    fn = _fn("elementwise", "bw_kv_slots", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(positions), _ptr(req_of_token), _ptr(block_table), block_table.shape[1], page_size, num_pages,
              _ptr(out), T, _stream()), "kv_slots")
    return out


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, req_of_token: torch.Tensor,
                block_table: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                k_pages: torch.Tensor, v_pages: torch.Tensor, nh: int, nkv: int, hd: int,
                q_out: Optional[torch.Tensor] = None, append: bool = True,
                table: Optional[torch.Tensor] = None, paired: bool = False) -> torch.Tensor:
    """Rotates q and k heads of ``qkv`` [T, (nh+2nkv)*hd], returns q [T, nh*hd] in the
    pages' dtype, and writes rotated k and raw v to pages [num_pages, nkv, page, hd].
    ``table``: the step's cos/sin table from :func:`rope_table` (else computed here).
    ``paired``: the q and k heads of ``qkv`` are in the order of :func:`rotary_row_order`.
    ``qkv`` may be planes [S, T, width] from :func:`gemm_tc_planes`: they are added while they are read."""
    n_planes, plane_stride = 1, 0
    if qkv.dim() == 3:
        n_planes, plane_stride = qkv.shape[0], qkv.stride(0)
        qkv = qkv[0]
    _dev(qkv, "qkv"); _dev(positions, "positions", torch.int32)
    _dev(req_of_token, "req_of_token", torch.int32); _dev(block_table, "block_table", torch.int32)
    _dev(k_pages, "k_pages"); _dev(v_pages, "v_pages", k_pages.dtype)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise KernelError(f"rope_append: qkv width {qkv.shape[1]} != (nh + 2 nkv) * hd = {(nh + 2 * nkv) * hd}")
    num_pages, pk, page_size, phd = k_pages.shape
    if pk != nkv or phd != hd or v_pages.shape != k_pages.shape:
        raise KernelError("rope_append: pages must be [num_pages, nkv, page_size, head_dim]")
    if rotary_dim:
        _dev(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("rope_append: inv_freq must have rotary_dim / 2 entries")
    if q_out is None:
        q_out = torch.empty((T, nh * hd), dtype=k_pages.dtype, device=qkv.device)
    _dev(q_out, "q_out", k_pages.dtype)
    if table is not None:
        _dev(table, "table", torch.float32)
        if tuple(table.shape) != (T, rotary_dim):
            raise KernelError("rope_append: the cos/sin table must be [T, rotary_dim]")
    fn = _fn("elementwise", "bw_rope_append",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_ll, c_void_p])
    _check(fn(_ptr(qkv), _code(qkv, "qkv"), _ptr(positions), _ptr(req_of_token), _ptr(block_table),
              block_table.shape[1], _ptr(inv_freq), _ptr(table), rotary_dim, _ptr(q_out), _ptr(k_pages), _ptr(v_pages),
              _code(k_pages, "pages"), T, nh, nkv, hd, page_size, num_pages if append else 0, int(paired),
              n_planes, plane_stride, _stream()),
           "rope_append")
    return q_out


# ------------------------------------------------------------------ matrix products

def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
              accumulate: bool = False) -> torch.Tensor:
    """out (=|+=) x @ w.T (+ bias) with float32 FMAs on the CUDA cores."""
    _dev(x, "x", contiguous=False); _dev(w, "w")
    if x.dtype != w.dtype:
        raise KernelError(f"gemm: x is {x.dtype} but w is {w.dtype}")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x has {K} columns, w has {K2}")
    if x.stride(1) != 1:
        raise KernelError("gemm: x rows must be contiguous")
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    _dev(out, "out", contiguous=False)
    if out.shape != (M, N) or out.stride(1) != 1:
        raise KernelError("gemm: out must be [M, N] with contiguous rows")
    if bias is not None:
        _dev(bias, "bias")
        if bias.numel() != N:
            raise KernelError("gemm: bias must have N entries")
    fn = _fn("gemm_simt", "bw_gemm_simt",
             [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
              c_int, c_void_p])
    _check(fn(_ptr(x), _ptr(w), _code(x, "x"), _ptr(bias), _code(bias, "bias") if bias is not None else 0,
              _ptr(out), _code(out, "out"), M, N, K, x.stride(0), out.stride(0), int(accumulate), _stream()),
           "gemm_simt")
    return out


# ------------------------------------------------------------------ attention

def attention_simt(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, positions: torch.Tensor,
                   req_of_token: torch.Tensor, block_table: torch.Tensor, nh: int, window: Optional[int],
                   scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _dev(q, "q"); _dev(k_pages, "k_pages", q.dtype); _dev(v_pages, "v_pages", q.dtype)
    _dev(positions, "positions", torch.int32); _dev(req_of_token, "req_of_token", torch.int32)
    _dev(block_table, "block_table", torch.int32)
    num_pages, nkv, page_size, hd = k_pages.shape
    T = q.shape[0]
    if q.shape[1] != nh * hd:
        raise KernelError("attention: q must be [T, nh * head_dim]")
    if out is None:
        out = torch.empty_like(q)
    fn = _fn("attention_simt", "bw_attention_simt",
             [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
              c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pages), _ptr(v_pages), _code(q, "q"), _ptr(positions), _ptr(req_of_token),
              _ptr(block_table), block_table.shape[1], _ptr(out), T, nh, nkv, hd, page_size, num_pages,
              int(window or 0), float(scale), _stream()), "attention_simt")
    return out


# ------------------------------------------------------------------ sampling

def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
           u: Optional[torch.Tensor]) -> torch.Tensor:
    """One token per row of ``logits`` [R, V]; greedy where temperature is None or <= 0."""
    _dev(logits, "logits", torch.float32, contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be [R, V] with contiguous rows")
    R, V = logits.shape
    for name, t in (("temperature", temperature), ("top_p", top_p), ("u", u)):
        if t is not None:
            _dev(t, name, torch.float32)
            if t.numel() != R:
                raise KernelError(f"sample: {name} must have one entry per row")
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    fn = _fn("sampling", "bw_sample",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p])
    _check(fn(_ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(u), _ptr(out), R, V, logits.stride(0),
              _stream()), "sample")
    return out


def repetition_penalty(logits: torch.Tensor, ids: torch.Tensor, begin: torch.Tensor, penalty: torch.Tensor) -> torch.Tensor:
    """In place on ``logits`` [R, V]: each distinct id of row r's history ``ids[begin[r]:begin[r+1]]``
    has its logit divided by ``penalty[r]`` when positive, multiplied when not; penalty <= 1 is off."""
    _dev(logits, "logits", torch.float32, contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("repetition_penalty: logits must be [R, V] with contiguous rows")
    R, V = logits.shape
    _dev(ids, "ids", torch.int32)
    _dev(begin, "begin", torch.int32)
    _dev(penalty, "penalty", torch.float32)
    if begin.numel() != R + 1 or penalty.numel() != R:
        raise KernelError("repetition_penalty: begin needs R + 1 entries and penalty R")
    fn = _fn("sampling", "bw_repetition_penalty",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p])
    _check(fn(_ptr(logits), _ptr(ids), _ptr(begin), _ptr(penalty), R, V, logits.stride(0), _stream()),
           "repetition_penalty")
    return logits


def log_prob(logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """log softmax(logits[r])[target[r]] for each row, float32 [R].  ``target`` int32 in [0, V)
    (checked by the caller on the host)."""
    _dev(logits, "logits", torch.float32, contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("log_prob: logits must be [R, V] with contiguous rows")
    R, V = logits.shape
    _dev(target, "target", torch.int32)
    if target.numel() != R:
        raise KernelError("log_prob: one target per row")
    out = torch.empty((R,), dtype=torch.float32, device=logits.device)
    fn = _fn("sampling", "bw_log_prob", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p])
    _check(fn(_ptr(logits), _ptr(target), _ptr(out), R, V, logits.stride(0), _stream()), "log_prob")
    return out


# ------------------------------------------------------------------ dispatch

_GEMM_TC_ARGS = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_int, c_int,
                 c_void_p, c_ll, c_void_p, c_ll, c_int, c_void_p]
_WORKSPACE_BYTES = 64 << 20
_COUNTERS = 1 << 16
_workspaces = {}
GEMM_FUSED_REDUCE_MAX_TOKENS = 16  # up to here gemm_tc sums its K splits inside the kernel
GEMM_PLANES_MAX_TOKENS = 256       # up to here gemm_tc_planes leaves them as planes
SWIGLU_BLOCK = 16  # gate/up rows of a fused SwiGLU weight alternate in blocks of this many


def _read_gemm_macros():
    v = os.environ.get("BW_GEMM_NARROW")
    if not v:
        return None
    st, ctas = v.split(",")
    return {"GEMM_NARROW_STAGES": int(st), "GEMM_NARROW_CTAS": int(ctas)}


_GEMM_MACROS = _read_gemm_macros()


def _gemm_macros():
    """Build options of the tensor-core product from the environment (read when this module is loaded), for
    measurements: BW_GEMM_NARROW="<stages>,<CTAs per SM>" of the kernel for up to 16 tokens (default: the source's)."""
    return _GEMM_MACROS


def _workspace(device: torch.device):
    """Scratch for split-K, one per device, made at first use: float32 partial sums and
    int32 counters (zero between launches; the kernel returns them to zero)."""
    ws = _workspaces.get(device)
    if ws is None:
        ws = (torch.empty(_WORKSPACE_BYTES // 4, dtype=torch.float32, device=device),
              torch.zeros(_COUNTERS, dtype=torch.int32, device=device))
        _workspaces[device] = ws
    return ws


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up weights -> [2I, K] with 16 gate rows, the 16 up rows of the same
    features, and so on: the layout of gemm_tc's fused SwiGLU epilogue (I % 16 == 0)."""
    I, K = gate.shape
    if I % SWIGLU_BLOCK or up.shape != gate.shape:
        raise KernelError("interleave_gate_up: both [I, K] with I a multiple of 16")
    g = gate.reshape(I // SWIGLU_BLOCK, SWIGLU_BLOCK, K)
    u = up.reshape(I // SWIGLU_BLOCK, SWIGLU_BLOCK, K)
    return torch.stack([g, u], dim=1).reshape(2 * I, K).contiguous()


def gemm_tc_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes this product: bfloat16, inner size and row
    stride multiples of 8 elements, 16-byte aligned (what a TMA descriptor can express)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous():
        return False
    K = x.shape[1]
    return (K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
            accumulate: bool = False, force_splits: int = 0, swiglu: bool = False) -> torch.Tensor:
    """out (=|+=) x @ w.T (+ bias) on the tcgen05 tensor cores (bfloat16 in, float32 sums).
    ``swiglu``: ``w`` is a gate/up weight from :func:`interleave_gate_up`; the result is
    bfloat16 [M, N / 2] = silu(gate) * up, computed in the epilogue."""
    _dev(x, "x", torch.bfloat16, contiguous=False); _dev(w, "w", torch.bfloat16)
    if not gemm_tc_supports(x, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with K and the row stride multiples of 8 "
                          "and 16-byte aligned")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x has {K} columns, w has {K2}")
    n_out = N
    if swiglu:
        if N % (2 * SWIGLU_BLOCK) or bias is not None or accumulate:
            raise KernelError("gemm_tc: the SwiGLU epilogue needs N = 2 I with I a multiple of 16, no bias, no accumulate")
        n_out, out_dtype = N // 2, torch.bfloat16
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, n_out), dtype=out_dtype or x.dtype, device=x.device)
    _dev(out, "out", contiguous=False)
    if out.shape != (M, n_out) or out.stride(1) != 1 or (swiglu and out.dtype != torch.bfloat16):
        raise KernelError("gemm: out must be [M, N] with contiguous rows")
    if bias is not None:
        _dev(bias, "bias")
        if bias.numel() != N:
            raise KernelError("gemm: bias must have N entries")
    ws, counters = _workspace(x.device)
    fn = _fn("gemm_tc", "bw_gemm_tc", _GEMM_TC_ARGS, macros=_gemm_macros(), tag=f"{M}x{N}x{K}" if _timings is not None else None)
    _check(fn(_ptr(x), _ptr(w), _ptr(bias), _code(bias, "bias") if bias is not None else 0, _ptr(out),
              _code(out, "out"), M, N, K, x.stride(0), out.stride(0), int(accumulate), int(swiglu), _ptr(ws),
              ws.numel(), _ptr(counters), counters.numel(), int(force_splits), _stream()), "gemm_tc")
    return out


def rotary_row_order(nh: int, nkv: int, hd: int, rotary_dim: int) -> torch.Tensor:
    """Row order of a fused q/k/v weight for :func:`gemm_tc_rope`: in every q and k head rows 2j
    and 2j + 1 are channels j and j + rotary_dim / 2; the other rows and the v heads stay."""
    half = rotary_dim // 2
    head = torch.arange(hd)
    head[:rotary_dim] = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)
    plain = torch.arange(hd)
    rows = [head + h * hd for h in range(nh + nkv)] + [plain + h * hd for h in range(nh + nkv, nh + 2 * nkv)]
    return torch.cat(rows)


_GEMM_TC_ROPE_ARGS = ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll] + [c_void_p] * 5 + [c_int] * 5
                      + [c_void_p, c_ll, c_void_p, c_ll, c_int, c_void_p])


def gemm_tc_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], table: Optional[torch.Tensor],
                 kv_slot: Optional[torch.Tensor], k_pages: torch.Tensor, v_pages: torch.Tensor, nh: int, nkv: int,
                 hd: int, rotary_dim: int, force_splits: int = 0) -> torch.Tensor:
    """The q/k/v projection, the rotation and the append to the cache in one kernel: ``w`` (and
    ``bias``) in the row order of :func:`rotary_row_order`; ``table`` from :func:`rope_table`;
    ``kv_slot`` from :func:`kv_slots` (None: nothing is appended).  Returns the rotated queries
    [T, nh * hd] (bfloat16); rotated keys and raw values are written to the pages
    [num_pages, nkv, page_size, hd] (bfloat16)."""
    _dev(x, "x", torch.bfloat16, contiguous=False); _dev(w, "w", torch.bfloat16)
    _dev(k_pages, "k_pages", torch.bfloat16); _dev(v_pages, "v_pages", torch.bfloat16)
    if not gemm_tc_supports(x, w):
        raise KernelError("gemm_tc_rope: operands must be bfloat16 with K and the row stride multiples of 8 "
                          "and 16-byte aligned")
    T, K = x.shape
    if w.shape != ((nh + 2 * nkv) * hd, K):
        raise KernelError(f"gemm_tc_rope: w must be [(nh + 2 nkv) * hd, K] = [{(nh + 2 * nkv) * hd}, {K}]")
    num_pages, pk, page_size, phd = k_pages.shape
    if pk != nkv or phd != hd or v_pages.shape != k_pages.shape:
        raise KernelError("gemm_tc_rope: pages must be [num_pages, nkv, page_size, head_dim]")
    if rotary_dim % 2 or not 0 <= rotary_dim <= hd or hd % 16:
        raise KernelError("gemm_tc_rope: rotary_dim must be even and at most head_dim, head_dim a multiple of 16")
    if rotary_dim:
        _dev(table, "table", torch.float32)
        if tuple(table.shape) != (T, rotary_dim):
            raise KernelError("gemm_tc_rope: the cos/sin table must be [T, rotary_dim]")
    if kv_slot is not None:
        _dev(kv_slot, "kv_slot", torch.int32)
        if kv_slot.numel() != T:
            raise KernelError("gemm_tc_rope: kv_slot must have one entry per token")
    if bias is not None:
        _dev(bias, "bias")
        if bias.numel() != w.shape[0]:
            raise KernelError("gemm_tc_rope: bias must have one entry per row of w")
    q_out = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=x.device)
    ws, counters = _workspace(x.device)
    fn = _fn("gemm_tc", "bw_gemm_tc_rope", _GEMM_TC_ROPE_ARGS, macros=_gemm_macros(),
             tag=f"rope{T}x{w.shape[0]}x{K}" if _timings is not None else None)
    _check(fn(_ptr(x), _ptr(w), _ptr(bias), _code(bias, "bias") if bias is not None else 0, T, K, x.stride(0),
              _ptr(table), _ptr(kv_slot), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), nh, nkv, hd, rotary_dim,
              page_size, _ptr(ws), ws.numel(), _ptr(counters), counters.numel(), int(force_splits), _stream()),
           "gemm_tc_rope")
    return q_out


def gemm_pair_mode(mode: int) -> int:
    """When products of more than 256 tokens run on CTA pairs: 0 never, 1 when estimated faster (the
    default), 2 whenever possible.  Returns the mode before (-1: not set yet, i.e. the default)."""
    fn = _fn("gemm_tc", "bw_gemm_tc_pair_mode", [c_int], macros=_gemm_macros())
    return fn(int(mode))


def gemm_tc_status() -> int:
    """0 if no bounded wait in the tensor-core kernels ever gave up (synchronises the device)."""
    lib = load_library("gemm_tc", _gemm_macros())
    lib.bw_gemm_tc_status.restype = c_int
    return int(lib.bw_gemm_tc_status())


MAX_GROUP_BF16 = 16   # query heads per kv head that the bfloat16 attention kernels stack in one tile


def check_attention_supported(dtype: torch.dtype, head_dim: int, group: int = 1) -> None:
    """Raises for a geometry no attention kernel of this dtype takes (known when a model is built)."""
    if head_dim <= 0 or head_dim > 256:
        raise KernelError(f"attention: head_dim {head_dim} is not supported (1..256)")
    if dtype == torch.bfloat16 and head_dim % 16:
        raise KernelError(f"attention: the bfloat16 kernels take head sizes in steps of 16, got {head_dim}")
    if dtype == torch.bfloat16 and group > MAX_GROUP_BF16:
        raise KernelError(f"attention: {group} query heads per kv head exceed the bfloat16 kernels' limit of "
                          f"{MAX_GROUP_BF16}")


class UnrotatedQKV:
    """The q/k/v product of a step in which every request has ONE token, left as float32 planes
    (:func:`gemm_tc_planes`, rows in the order of :func:`rotary_row_order`), with what the rotation needs:
    :func:`paged_attention` rotates the queries, and rotates and appends the keys and values, inside its
    key-slice kernel where that kernel runs; ``materialise()`` does it with :func:`rope_append` elsewhere."""

    def __init__(self, planes: torch.Tensor, table: Optional[torch.Tensor], rotary_dim: int, append: bool, materialise):
        self.planes, self.table, self.rotary_dim, self.append, self.materialise = planes, table, rotary_dim, append, materialise
        self.generation = _plane_generation    # the planes are this module's buffer: good until the next such product


def attention_takes_unrotated(hd: int, page_size: int) -> bool:
    """Whether the decode attention can rotate and append by itself (:class:`UnrotatedQKV`): the TMA
    key-slice kernel's sizes.  BW_ATTN_FUSED_ROPE=0 in the environment says no."""
    return (os.environ.get("BW_ATTN_FUSED_ROPE", "1") != "0" and hd % 64 == 0 and hd <= 256
            and page_size in (8, 16, 32, 64))


def paged_attention(q, k_pages: torch.Tensor, v_pages: torch.Tensor, batch,
                    block_table: torch.Tensor, nh: int, window: Optional[int], scale: float) -> torch.Tensor:
    """Causal attention of the batch's tokens over the paged cache (which already
    holds this step's keys and values, unless ``q`` is an :class:`UnrotatedQKV`).  float32: the
    CUDA-core kernel; bfloat16: the tensor-core kernel built for this head size."""
    if isinstance(q, UnrotatedQKV):
        if batch.T == batch.R and attention_takes_unrotated(k_pages.shape[3], k_pages.shape[2]):
            return attention_mma(q, k_pages, v_pages, batch, block_table, nh, window, scale)
        q = q.materialise()
    if q.dtype == torch.float32:
        return attention_simt(q, k_pages, v_pages, batch.positions, batch.req_of_token, block_table, nh,
                              window, scale)
    return attention_mma(q, k_pages, v_pages, batch, block_table, nh, window, scale)


_ATTN_MMA_ARGS = [c_void_p] * 8 + [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_int, c_float,
                                   c_void_p, c_int, c_ll, c_void_p, c_int, c_int, c_int, c_void_p]


_sm_counts = {}


def num_sms(device=None) -> int:
    """SMs of the device (148, the B200's, where there is no device to ask)."""
    if device is None or not torch.cuda.is_available():
        return 148
    device = torch.device(device)
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def plan_attention_work(q_len, q_start, kv_len, G: int, nkv: int, window: Optional[int], hd: int = 128,
                        rows_tile: int = 64, page_size: int = 16, static_bound: Optional[int] = None,
                        sms: int = 148):
    """The work lists of the tensor-core attention as plain lists (host arithmetic only):
    ``rows`` items (request, first token, 0, 0) for segments of more than 16 stacked rows (tokens x
    heads of a group), cut into tiles of ``rows_tile`` rows and ordered longest first; ``keys`` items
    (request, slice, slices of the request, first slot of its partial results) for the others (decode
    tokens), cut into key slices so that the GPU is filled; ``merge`` items (request, 0, slices, first
    slot) for requests with more than one slice; and the number of partial-result slots."""
    tpt = rows_tile // G   # tokens of one tile of stacked rows
    rows_items, keys_items, merge_items = [], [], []
    n_small = sum(1 for n in q_len if n * G <= 16)
    # CTAs of the key-slice kernel that fit on the GPU at once (shared memory bound)
    if hd % 64 == 0 and page_size in (8, 16, 32, 64):   # the TMA-fed kernel: 2 stages of unpadded tiles
        smem = 2 * 2 * 64 * hd * 2 + 16 * (hd * 2 + 16) + 2048
    else:
        smem = (16 + 4 * 64) * (hd * 2 + 16)
    slots = sms * max(1, min(8, (227 * 1024) // (smem + 1024)))
    heads = max(1, n_small * nkv)
    if heads <= slots:
        want = slots // heads            # one full wave: all slices run side by side, no tail
    else:
        want = -(-4 * slots // heads)    # many short CTAs: at least four waves smooth the tail
    total_slices = 0
    for r, n_q in enumerate(q_len):
        if n_q * G > 16:
            rows_items += [(r, t0, 0, 0) for t0 in range(0, n_q, tpt)]
            continue
        span = static_bound or kv_len[r]
        if window:
            span = min(span, window + n_q)
        tiles = -(-span // 64)
        n = max(1, min(want, tiles // 2, 64))
        keys_items += [(r, s, n, total_slices) for s in range(n)]
        if n > 1:
            merge_items.append((r, 0, n, total_slices))
        total_slices += n
    # the tiles with the most keys to walk (the latest tokens) go first, so the last wave is light
    rows_items.sort(key=lambda it: -(q_start[it[0]] + it[1]))
    return rows_items, keys_items, merge_items, total_slices


def attention_work(batch, G: int, nkv: int, window: Optional[int], hd: int = 128, rows_tile: int = 64,
                   page_size: int = 16):
    """The work lists of :func:`plan_attention_work` for this batch and group size on the device,
    made once per step and shared by all layers.  With ``batch.static_bound`` (graph replay) the
    number of key slices depends on that bound, not on the lengths."""
    key = ("attn_work", G, nkv, window, hd, rows_tile, page_size)
    cached = batch.static_extras.get(key)
    if cached is not None:
        return cached
    R = batch.R
    rows_items, keys_items, merge_items, total_slices = plan_attention_work(
        batch.h_q_len[:R], batch.h_q_start[:R], batch.h_kv_len[:R], G, nkv, window, hd, rows_tile, page_size,
        batch.static_bound, num_sms(batch.token_ids.device))
    dev = batch.token_ids.device

    def up(items):
        if not items:
            return None
        return torch.tensor(items, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)

    work = (up(rows_items), len(rows_items), up(keys_items), len(keys_items), up(merge_items),
            len(merge_items), total_slices if merge_items else 0, max((m[2] for m in merge_items), default=0))
    batch.static_extras[key] = work
    return work


def attention_mma(q, k_pages: torch.Tensor, v_pages: torch.Tensor, batch, block_table: torch.Tensor,
                  nh: int, window: Optional[int], scale: float) -> torch.Tensor:
    _dev(k_pages, "k_pages", torch.bfloat16); _dev(v_pages, "v_pages", torch.bfloat16)
    _dev(block_table, "block_table", torch.int32)
    num_pages, nkv, page_size, hd = k_pages.shape
    raw = q if isinstance(q, UnrotatedQKV) else None
    if raw is not None:
        planes = _dev(raw.planes, "qkv planes", torch.float32)
        if raw.generation != _plane_generation:
            raise KernelError("attention: the unrotated q/k/v planes were overwritten by a later product")
        if batch.T != batch.R:
            raise KernelError("attention: unrotated q/k/v only with one token per request")
        if planes.dim() != 3 or planes.shape[2] != (nh + 2 * nkv) * hd or nh % nkv or planes.shape[1] != batch.R:
            raise KernelError("attention: unrotated q/k/v must be planes [S, requests, (nh + 2 nkv) * head_dim]")
        if raw.rotary_dim:
            _dev(raw.table, "table", torch.float32)
            if tuple(raw.table.shape) != (planes.shape[1], raw.rotary_dim):
                raise KernelError("attention: the cos/sin table must be [T, rotary_dim]")
        q = None
        out = torch.empty((planes.shape[1], nh * hd), dtype=torch.bfloat16, device=planes.device)
    else:
        _dev(q, "q", torch.bfloat16)
        if q.shape[1] != nh * hd or nh % nkv:
            raise KernelError("attention: q must be [T, nh * head_dim] with nh a multiple of the kv heads")
        out = torch.empty_like(q)
    G = nh // nkv
    check_attention_supported(torch.bfloat16, hd, G)
    # prompt portions: the tcgen05 kernel (128-row tiles) where it takes the geometry, else mma.sync (64-row tiles)
    use_tc = attention_tc_supports(hd, G, page_size)
    rows_w, n_rows, keys_w, n_keys, merge_w, n_merge, slices, merge_max = attention_work(
        batch, G, nkv, window, hd, rows_tile=128 if use_tc else 64, page_size=page_size)
    part_o = part_ml = None
    if n_merge:
        part_o = torch.empty((slices * nkv * 16, hd), dtype=torch.float32, device=out.device)
        part_ml = torch.empty((slices * nkv * 16, 2), dtype=torch.float32, device=out.device)
    if raw is not None and n_rows:
        raise KernelError("attention: unrotated q/k/v only with one token per request")
    if use_tc and n_rows:
        tc = _fn("attention_tc", "bw_attention_tc", _ATTN_TC_ARGS, macros=attention_tc_macros(hd))
        _check(tc(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(batch.cu_q), _ptr(batch.q_start),
                  _ptr(batch.kv_len), _ptr(block_table), block_table.shape[1], _ptr(rows_w), n_rows, q.shape[0],
                  nh, nkv, page_size, num_pages, int(window or 0), float(scale), _stream()), "attention_tc")
        n_rows = 0
        if not n_keys:
            return out
    fn = _fn("attention_mma", "bw_attention_mma", _ATTN_MMA_ARGS, macros=attention_mma_macros(hd))
    _check(fn(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(batch.cu_q), _ptr(batch.q_start),
              _ptr(batch.kv_len), _ptr(block_table), block_table.shape[1], _ptr(rows_w), n_rows, _ptr(keys_w),
              n_keys, _ptr(merge_w), n_merge, _ptr(part_o), _ptr(part_ml), nh, nkv, page_size, num_pages,
              int(window or 0), float(scale),
              _ptr(raw.planes if raw is not None else None), raw.planes.shape[0] if raw is not None else 0,
              raw.planes.stride(0) if raw is not None else 0, _ptr(raw.table if raw is not None else None),
              raw.rotary_dim if raw is not None else 0, int(raw.append) if raw is not None else 0, merge_max,
              _stream()), "attention_mma")
    return out


_ATTN_TC_ARGS = [c_void_p] * 8 + [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]


def attention_tc_supports(hd: int, G: int, page_size: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes this geometry (head size a multiple of 64,
    pages of 8, 16, 32 or 64 tokens).  BW_ATTN_TC=0 in the environment keeps the mma.sync kernel."""
    import os
    if os.environ.get("BW_ATTN_TC", "1") == "0":
        return False
    return hd % 64 == 0 and hd <= 256 and G <= 128 and page_size in (8, 16, 32, 64)


def attention_mma_macros(hd: int) -> dict:
    """The build of the mma.sync attention for this head size.  BW_ATTN_MERGE_FEW=n in the environment sets up
    to how many slices the slice merge without barriers takes (for measurements; default: the source's)."""
    macros = _ATTN_MMA_MACROS.get(hd)
    if macros is None:
        macros = {"HEAD_DIM": hd}
        if os.environ.get("BW_ATTN_MERGE_FEW"):
            macros["ATTN_MERGE_FEW"] = int(os.environ["BW_ATTN_MERGE_FEW"])
        _ATTN_MMA_MACROS[hd] = macros
    return macros


_ATTN_MMA_MACROS = {}


def attention_tc_macros(hd: int) -> dict:
    """The build of the tcgen05 prompt attention for this head size.  BW_ATTN_RELAXED_ORDER=1 in the
    environment selects the variant whose MMA warp does not wait for the P V product that reads a
    buffer before it overwrites it (for measuring what the wait costs; never the default)."""
    import os
    macros = {"HEAD_DIM": hd}
    if os.environ.get("BW_ATTN_RELAXED_ORDER", "0") == "1":
        macros["ATTN_STRICT_ORDER"] = 0
    return macros


def attention_tc_status() -> int:
    """0 if no bounded wait in the tcgen05 attention kernels ever gave up (synchronises the device)."""
    total = 0
    for key, lib in list(_loaded_libs().items()):
        if key.startswith("attention_tc"):
            lib.bw_attention_tc_status.restype = c_int
            total |= int(lib.bw_attention_tc_status())
    return total


def _loaded_libs():
    from . import build
    return build._loaded
