"""Python face of the CUDA kernels: argument checks, then a ctypes call on the
current CUDA stream.  Nothing here computes; a tensor on the CPU, of the wrong
type or not contiguous is an error, never a detour through another
implementation.
"""
from __future__ import annotations

import ctypes
import math
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


def embed_positions(table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                    copies: int = 1, scale: float = 1.0) -> torch.Tensor:
    """float32 [T, copies * H]: ``table[ids] * scale`` plus, with ``inv_freq`` (float32 [ceil(H / 2)]), a vector of the
    token's position (entry 2i: sin(pos * inv_freq[i]), entry 2i + 1: the cosine), written ``copies`` times side by
    side: the start of a residual stream that is kept as several copies."""
    _dev(table, "table"); _dev(ids, "ids", torch.int32); _dev(positions, "positions", torch.int32)
    V, H = table.shape
    T = ids.numel()
    if inv_freq is not None:
        _dev(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != (H + 1) // 2:
            raise KernelError("embed_positions: inv_freq must have ceil(H / 2) entries")
    if positions.numel() != T or copies < 1:
        raise KernelError("embed_positions: one position per token, at least one copy")
    out = torch.empty((T, copies * H), dtype=torch.float32, device=table.device)
    fn = _fn("elementwise", "bw_embed_positions",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_ptr(table), _code(table, "table"), _ptr(ids), _ptr(positions), _ptr(inv_freq), _ptr(out), T, H, V, float(scale),
              int(copies), _stream()), "embed_positions")
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
# A product that is WRITTEN to a float32 tensor can be left open the same way (gemm_tc_deferred(...,
# overwrite=True)): the tensor's own values then do not count, the planes are all of it; hc_step takes
# such a sum (and an added one) for its y while it reads it.

DEFER_SUMS = os.environ.get("BW_DEFER_SUMS", "1") != "0"
# Linear.add_to leaves sums open up to this many tokens (measured on a B200: 4 % less step time at 1 to 16
# tokens, 1.5 % at 24 to 64, 0.5 % at 128, nothing at 256)
DEFER_MAX_TOKENS = int(os.environ.get("BW_DEFER_MAX_TOKENS", "128"))
_pending = None          # (target tensor, planes [S, M, N], overwrite) or None
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
    target, planes, overwrite = _pending
    _pending = None
    fn = _fn("elementwise", "bw_sum_planes" if overwrite else "bw_add_planes", [c_void_p, c_void_p, c_int, c_ll, c_ll, c_void_p])
    _check(fn(_ptr(target), _ptr(planes), planes.shape[0], planes.stride(0), target.numel(), _stream()), "add_planes")


def discard_pending(t: Optional[torch.Tensor] = None) -> None:
    """Forgets an outstanding sum into ``t`` (None: into whatever tensor): it is not read again."""
    global _pending
    if _pending is not None and (t is None or _pending[0].data_ptr() == t.data_ptr()):
        _pending = None


def gemm_tc_planes(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   force_splits: int = 0, after: int = 0) -> torch.Tensor:
    """x @ w.T (+ bias) for up to GEMM_PLANES_MAX_TOKENS tokens as float32 planes [S, M, N] that
    add up to it (in plane order; the bias is in plane 0), in this module's plane buffer: valid until
    the next call.  An outstanding sum is resolved first, unless ``after`` > 0: then the planes start that many
    floats into the buffer and what lies before them stays (:func:`gemm_tc_deferred` chains two sums so)."""
    if not after:
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
    buf = _plane_buffer(x.device)[after:]
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


def gemm_tc_deferred(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                     overwrite: bool = False) -> None:
    """out += x @ w.T (+ bias), the sum left to the next reader of ``out`` (float32 [M, N], contiguous);
    ``overwrite``: out = x @ w.T (+ bias) instead (what ``out`` holds does not count)."""
    global _pending
    if out.dtype != torch.float32 or not out.is_contiguous() or out.shape != (x.shape[0], w.shape[0]):
        raise KernelError("gemm_tc_deferred: out must be contiguous float32 [M, N]")
    if (_pending is not None and not overwrite and _pending[0].data_ptr() == out.data_ptr() and _pending[0].shape == out.shape
            and _pending[1].numel() % 64 == 0 and _pending[1].numel() * 4 <= PLANE_BUFFER_ELEMS
            and _pending[1].data_ptr() == _plane_buffer(x.device).data_ptr()):
        # a second sum into the same tensor (a block whose two sublayers both add to the stream): its planes go
        # behind the first's, and the reader adds them all in one pass, in plane order
        target, first, ow = _pending
        more = gemm_tc_planes(x, w, bias, after=first.numel())
        both = _plane_buffer(x.device)[:first.numel() + more.numel()].view(first.shape[0] + more.shape[0], *first.shape[1:])
        _pending = (target, both, ow)
        return
    planes = gemm_tc_planes(x, w, bias)
    _pending = (out, planes, bool(overwrite))


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    global _pending
    mine = None              # an outstanding sum into x: added by the kernel below instead of one of its own
    if (_pending is not None and _pending[0].data_ptr() == x.data_ptr() and _pending[0].shape == x.shape
            and not _pending[2]):
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
    # (x may be a range of columns of a wider tensor when nothing is to be added to it)
    _dev(x, "x", torch.float32, contiguous=planes is not None); _dev(w, "w")
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("rmsnorm: x must be [rows, H] with contiguous rows")
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
    fn = _fn("elementwise", "bw_rmsnorm_ld",
             [c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(x), x.stride(0), _ptr(w), _code(w, "w"), _ptr(rows), _ptr(out), _code(out, "out"), n, H,
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


ACT_SILU, ACT_CLAMPED_SWISH, ACT_RELU2, ACT_GELU_TANH = 0, 1, 2, 3   # the activation codes of csrc/common.cuh
GATED_ACTIVATIONS = {"silu": ACT_SILU, "clamped_swish": ACT_CLAMPED_SWISH, "gelu_tanh": ACT_GELU_TANH}
UNARY_ACTIVATIONS = {"relu2": ACT_RELU2}
GEMM_TC_GATED_ACTIVATIONS = (ACT_SILU, ACT_CLAMPED_SWISH, ACT_GELU_TANH)   # what gemm_tc's fused gate/up epilogue computes
GEMM_TC_GATED_BIAS = True                                   # ... and whether it takes biases on gate and up (interleaved like the rows)


def glu(gu: torch.Tensor, act: int, limit: float = 0.0, alpha: float = 1.0, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """[T, 2I] (gate | up) -> [T, I]: ACT_SILU ``silu(gate) * up``; ACT_CLAMPED_SWISH, with g = min(gate, limit) and
    u = clamp(up, -limit, limit): ``g * sigmoid(alpha * g) * (u + 1)``; ACT_GELU_TANH ``gelu_tanh(gate) * up``.  Float32 arithmetic."""
    _dev(gu, "gate_up")
    T, I2 = gu.shape
    if I2 % 2:
        raise KernelError("glu: input width must be even (gate | up)")
    out = torch.empty((T, I2 // 2), dtype=out_dtype or gu.dtype, device=gu.device)
    fn = _fn("elementwise", "bw_glu", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p])
    _check(fn(_ptr(gu), _code(gu, "gate_up"), _ptr(out), _code(out, "out"), T, I2 // 2, int(act), float(limit), float(alpha),
              _stream()), "glu")
    return out


def unary_act(x: torch.Tensor, act: int, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Element by element: ACT_RELU2 ``max(x, 0) ** 2`` (float32 arithmetic)."""
    _dev(x, "x")
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    fn = _fn("elementwise", "bw_unary_act", [c_void_p, c_int, c_void_p, c_int, c_ll, c_int, c_void_p])
    _check(fn(_ptr(x), _code(x, "x"), _ptr(out), _code(out, "out"), x.numel(), int(act), _stream()), "unary_act")
    return out


def sigmoid_gate(o: torch.Tensor, g: torch.Tensor, nh: int, dv: int) -> torch.Tensor:
    """In place: ``o[t, h, c] *= sigmoid(g[t, h * dv + c])`` for c < dv; o is [T, nh * dpad] with dpad >= dv
    (channels beyond dv become zero); g float32 [T, nh * dv], possibly a column range of a wider tensor."""
    _dev(o, "o"); _dev(g, "g", torch.float32, contiguous=False)
    T = o.shape[0]
    dpad = o.shape[1] // nh
    if o.shape[1] != nh * dpad or dpad < dv or g.shape != (T, nh * dv) or g.stride(1) != 1:
        raise KernelError("sigmoid_gate: o must be [T, nh * dpad], g [T, nh * dv] with contiguous rows")
    fn = _fn("elementwise", "bw_sigmoid_gate", [c_void_p, c_int, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(o), _code(o, "o"), _ptr(g), g.stride(0), T, nh, dv, dpad, _stream()), "sigmoid_gate")
    return o


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, magnitude: float = 1.0) -> torch.Tensor:
    """cos and sin of ``pos * inv_freq`` per token, times ``magnitude``: float32 [T, rotary_dim] (cos, then sin)."""
    _dev(positions, "positions", torch.int32); _dev(inv_freq, "inv_freq", torch.float32)
    T = positions.numel()
    table = torch.empty((T, rotary_dim), dtype=torch.float32, device=positions.device)
    fn = _fn("elementwise", "bw_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(positions), _ptr(inv_freq), _ptr(table), rotary_dim, T, float(magnitude), _stream()), "rope_table")
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
                   scale: float, out: Optional[torch.Tensor] = None, chunk: Optional[int] = None,
                   sink: Optional[torch.Tensor] = None, gate: Optional[tuple] = None,
                   dist: Optional[torch.Tensor] = None, keep_first: int = 0, softcap: Optional[float] = None,
                   rel: Optional[torch.Tensor] = None) -> torch.Tensor:
    _dev(q, "q"); _dev(k_pages, "k_pages", q.dtype); _dev(v_pages, "v_pages", q.dtype)
    _check_sink(sink, nh)
    _check_dist(dist, nh)
    _check_rel(rel, nh, dist)
    g, g_ld, g_dv = _gate_args(gate, q.shape[0], nh, k_pages.shape[3])
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
              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_int,
              c_float, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pages), _ptr(v_pages), _code(q, "q"), _ptr(positions), _ptr(req_of_token),
              _ptr(block_table), block_table.shape[1], _ptr(out), T, nh, nkv, hd, page_size, num_pages,
              int(window or 0), int(chunk or 0), float(scale), _ptr(sink), _ptr(g), g_ld, g_dv, _ptr(dist),
              int(keep_first or 0), float(softcap or 0.0), _ptr(rel), rel.shape[1] if rel is not None else 0,
              _stream()), "attention_simt")
    return out


def _gate_args(gate: Optional[tuple], T: int, nh: int, hd: int):
    """``gate`` = (float32 tensor [T, nh * dv], possibly a column range of a wider one; dv): what the attention
    kernels take as pointer, row stride and value size.  (g [T, nh], dv, "head"): one number per head; the kernels
    get the value size negated for it."""
    if gate is None:
        return None, 0, 0
    g, dv = gate[0], gate[1]
    _dev(g, "gate", torch.float32, contiguous=False)
    if len(gate) > 2 and gate[2] == "head":
        if g.shape != (T, nh) or g.stride(1) != 1 or not 0 < dv <= hd:
            raise KernelError(f"attention: a gate per head must be float32 [T, nh] with contiguous rows and dv <= {hd}")
        return g, g.stride(0), -int(dv)
    if g.shape != (T, nh * dv) or g.stride(1) != 1 or not 0 < dv <= hd:
        raise KernelError(f"attention: the gate must be float32 [T, nh * dv] with contiguous rows and dv <= {hd}")
    return g, g.stride(0), int(dv)


def _check_sink(sink: Optional[torch.Tensor], nh: int) -> None:
    if sink is not None:
        _dev(sink, "sink", torch.float32)
        if sink.numel() != nh:
            raise KernelError(f"attention: the sink must have one float32 entry per query head ({nh})")


def _check_dist(dist: Optional[torch.Tensor], nh: int) -> None:
    if dist is not None:
        _dev(dist, "dist", torch.float32)
        if tuple(dist.shape) != (2, nh):
            raise KernelError(f"attention: the distance bias must be float32 [2, {nh}] (r1 of every head, then r2)")


def _check_rel(rel: Optional[torch.Tensor], nh: int, dist: Optional[torch.Tensor] = None) -> None:
    if rel is not None:
        _dev(rel, "rel", torch.float32)
        if rel.dim() != 2 or rel.shape[0] != nh or rel.shape[1] < 1:
            raise KernelError(f"attention: the table of biases by distance must be float32 [{nh}, distances]")
        if dist is not None:
            raise KernelError("attention: a table of biases by distance does not go with the logarithmic distance bias")


def distance_bucket_table(rows: int, far: float) -> torch.Tensor:
    """int64 [n]: the row of a table of ``rows`` learned biases that stands for the distance d = 0 .. n - 1 between a
    query and a key: distances below rows / 2 have a row each, larger ones share rows on a logarithmic scale that
    reaches the last row at distance ``far``: min(rows - 1, half + floor(ln(d / half) / ln(far / half) * (rows - half))),
    half = rows // 2.  n - 1 is the first distance that takes the last row (every larger one takes it too), so entry
    n - 1 stands for all of them.  Host arithmetic in float64."""
    half = rows // 2
    if rows < 1 or (rows > 1 and half >= 1 and not far > half):
        raise KernelError(f"distance_bucket_table: {rows} rows need a farthest distance above {half}, got {far}")
    out = []
    d = 0
    while True:
        if d < half or half == 0:
            b = min(d, rows - 1)
        else:
            b = min(rows - 1, half + int(math.floor(math.log(d / half) / math.log(far / half) * (rows - half))))
        out.append(b)
        if b >= rows - 1 or d > 1 << 24:
            break
        d += 1
    return torch.tensor(out, dtype=torch.int64)


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
_GEMM_TC_ACT_ARGS = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_int, c_int,
                     c_float, c_float, c_void_p, c_ll, c_void_p, c_ll, c_int, c_void_p]
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
            accumulate: bool = False, force_splits: int = 0, swiglu: bool = False,
            act: Optional[int] = None, limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """out (=|+=) x @ w.T (+ bias) on the tcgen05 tensor cores (bfloat16 in, float32 sums).
    ``swiglu``: ``w`` is a gate/up weight from :func:`interleave_gate_up`; the result is
    bfloat16 [M, N / 2] = silu(gate) * up, computed in the epilogue; ``act`` = ACT_CLAMPED_SWISH (with its
    ``limit`` and ``alpha``) or ACT_GELU_TANH puts that gated activation in its place (:func:`glu`); a ``bias`` (interleaved
    like the rows) is added to gate and up before it.  Without ``swiglu``,
    ``act`` = ACT_RELU2 squares the positive part of every sum of a result that is written (not added)."""
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
        if N % (2 * SWIGLU_BLOCK) or accumulate:
            raise KernelError("gemm_tc: the SwiGLU epilogue needs N = 2 I with I a multiple of 16 and no accumulate")
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
    if act is not None and not (swiglu and act == ACT_SILU):
        if accumulate:
            raise KernelError("gemm_tc: an activation goes with a result that is written, not added")
        fn = _fn("gemm_tc", "bw_gemm_tc_act", _GEMM_TC_ACT_ARGS, macros=_gemm_macros(),
                 tag=f"act{M}x{N}x{K}" if _timings is not None else None)
        _check(fn(_ptr(x), _ptr(w), _ptr(bias), _code(bias, "bias") if bias is not None else 0, _ptr(out),
                  _code(out, "out"), M, N, K, x.stride(0), out.stride(0), int(swiglu), int(act), float(limit), float(alpha),
                  _ptr(ws), ws.numel(), _ptr(counters), counters.numel(), int(force_splits), _stream()), "gemm_tc_act")
        return out
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


ATTENTION_SIMT_MAX_HEAD_DIM = 1024   # the CUDA-core kernel's limit; the tensor-core kernels are built for head sizes up to 256
MAX_GROUP_BF16 = 16   # query heads per kv head that the bfloat16 attention kernels stack in one tile


def check_attention_supported(dtype: torch.dtype, head_dim: int, group: int = 1) -> None:
    """Raises for a geometry no attention kernel of this dtype takes (known when a model is built)."""
    if head_dim <= 0 or head_dim > ATTENTION_SIMT_MAX_HEAD_DIM:
        raise KernelError(f"attention: head_dim {head_dim} is not supported (1..{ATTENTION_SIMT_MAX_HEAD_DIM})")
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
                    block_table: torch.Tensor, nh: int, window: Optional[int], scale: float,
                    chunk: Optional[int] = None, sink: Optional[torch.Tensor] = None,
                    gate: Optional[tuple] = None, dist: Optional[torch.Tensor] = None,
                    keep_first: int = 0, softcap: Optional[float] = None,
                    rel: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of the batch's tokens over the paged cache (which already
    holds this step's keys and values, unless ``q`` is an :class:`UnrotatedQKV`).  float32: the
    CUDA-core kernel; bfloat16: the tensor-core kernel built for this head size.  A query sees the keys
    from ``first_visible(position, window, chunk)`` on: the latest ``window`` keys, and none before the
    start of its own block of ``chunk`` positions (blocks are counted from position 0).  ``sink`` (float32, one
    entry per query head): the softmax of a row has one more term exp(sink) that has no key and no value.
    ``gate`` = (g float32 [T, nh * dv], dv): channel c < dv of every head's output is multiplied by
    sigmoid(g[t, head * dv + c]) as it is written; channels from dv on (padding) become zero; (g [T, nh], dv, "head"):
    one gate number per head.  ``dist`` (float32 [2, nh]: r1 of every head, then r2): r1 ln(1 + r2 (i - j)) is taken off
    the score of query position i and key position j.  ``keep_first``: the first so many keys of a sequence stay
    visible beyond the window.  ``softcap``: the scaled score s becomes softcap * tanh(s / softcap) before any bias.
    ``rel`` (float32 [nh, n]): rel[head, min(i - j, n - 1)] is added to the score (a learned bias per distance, its last
    entry standing for every larger distance; :func:`distance_bucket_table` says which distances share a learned row)."""
    if (softcap or rel is not None) and isinstance(q, UnrotatedQKV):
        q = q.materialise()
    if isinstance(q, UnrotatedQKV):
        if batch.T == batch.R and attention_takes_unrotated(k_pages.shape[3], k_pages.shape[2]):
            return attention_mma(q, k_pages, v_pages, batch, block_table, nh, window, scale, chunk, sink, gate)
        q = q.materialise()
    if q.dtype == torch.float32:
        return attention_simt(q, k_pages, v_pages, batch.positions, batch.req_of_token, block_table, nh,
                              window, scale, chunk=chunk, sink=sink, gate=gate, dist=dist, keep_first=keep_first,
                              softcap=softcap, rel=rel)
    if nh // k_pages.shape[1] > MAX_GROUP_BF16 or k_pages.shape[3] > 256:
        # more query heads per kv head than a tile of the tensor-core kernels stacks, or a head size beyond the ones
        # they are built for (a wide latent row): the CUDA-core kernel in bfloat16
        return attention_simt(q, k_pages, v_pages, batch.positions, batch.req_of_token, block_table, nh,
                              window, scale, chunk=chunk, sink=sink, gate=gate, dist=dist, keep_first=keep_first,
                              softcap=softcap, rel=rel)
    return attention_mma(q, k_pages, v_pages, batch, block_table, nh, window, scale, chunk, sink, gate, dist, keep_first,
                         softcap, rel)


_ATTN_MMA_ARGS = [c_void_p] * 8 + [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                   c_void_p, c_int, c_ll, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_ll, c_int,
                                   c_void_p, c_int, c_float, c_void_p, c_int, c_void_p]


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
                        sms: int = 148, chunk: Optional[int] = None, keep_first: int = 0):
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
        if window:   # (kept first keys lie in tiles of their own before the window's)
            span = min(span, window + n_q + (-(-keep_first // 64) * 64 if keep_first else 0))
        if chunk:   # a query sees no key before the start of its block of positions
            span = min(span, chunk + n_q)
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
                   page_size: int = 16, chunk: Optional[int] = None, keep_first: int = 0):
    """The work lists of :func:`plan_attention_work` for this batch and group size on the device,
    made once per step and shared by all layers.  With ``batch.static_bound`` (graph replay) the
    number of key slices depends on that bound, not on the lengths."""
    key = ("attn_work", G, nkv, window, hd, rows_tile, page_size, chunk, keep_first)
    cached = batch.static_extras.get(key)
    if cached is not None:
        return cached
    R = batch.R
    rows_items, keys_items, merge_items, total_slices = plan_attention_work(
        batch.h_q_len[:R], batch.h_q_start[:R], batch.h_kv_len[:R], G, nkv, window, hd, rows_tile, page_size,
        batch.static_bound, num_sms(batch.token_ids.device), chunk, keep_first)
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
                  nh: int, window: Optional[int], scale: float, chunk: Optional[int] = None,
                  sink: Optional[torch.Tensor] = None, gate: Optional[tuple] = None,
                  dist: Optional[torch.Tensor] = None, keep_first: int = 0, softcap: Optional[float] = None,
                  rel: Optional[torch.Tensor] = None) -> torch.Tensor:
    _dev(k_pages, "k_pages", torch.bfloat16); _dev(v_pages, "v_pages", torch.bfloat16)
    _check_sink(sink, nh)
    _check_dist(dist, nh)
    _check_rel(rel, nh, dist)
    if softcap and dist is not None:
        raise KernelError("attention: a soft cap on the scores does not go with the logarithmic distance bias")
    rel_len = rel.shape[1] if rel is not None else 0
    keep_first = int(keep_first or 0) if window else 0
    g, g_ld, g_dv = _gate_args(gate, batch.T, nh, k_pages.shape[3])
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
    if hd > 256:
        raise KernelError(f"attention: the tensor-core kernels are built for head sizes up to 256, got {hd}")
    # prompt portions: the tcgen05 kernel (128-row tiles) where it takes the geometry, else mma.sync (64-row tiles)
    use_tc = attention_tc_supports(hd, G, page_size)
    rows_w, n_rows, keys_w, n_keys, merge_w, n_merge, slices, merge_max = attention_work(
        batch, G, nkv, window, hd, rows_tile=128 if use_tc else 64, page_size=page_size, chunk=chunk, keep_first=keep_first)
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
                  nh, nkv, page_size, num_pages, int(window or 0), int(chunk or 0), float(scale), _ptr(sink), _ptr(g), g_ld, g_dv,
                  _ptr(dist), keep_first, float(softcap or 0.0), _ptr(rel), rel_len, _stream()), "attention_tc")
        n_rows = 0
        if not n_keys:
            return out
    fn = _fn("attention_mma", "bw_attention_mma", _ATTN_MMA_ARGS, macros=attention_mma_macros(hd))
    _check(fn(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(batch.cu_q), _ptr(batch.q_start),
              _ptr(batch.kv_len), _ptr(block_table), block_table.shape[1], _ptr(rows_w), n_rows, _ptr(keys_w),
              n_keys, _ptr(merge_w), n_merge, _ptr(part_o), _ptr(part_ml), nh, nkv, page_size, num_pages,
              int(window or 0), int(chunk or 0), float(scale),
              _ptr(raw.planes if raw is not None else None), raw.planes.shape[0] if raw is not None else 0,
              raw.planes.stride(0) if raw is not None else 0, _ptr(raw.table if raw is not None else None),
              raw.rotary_dim if raw is not None else 0, int(raw.append) if raw is not None else 0, merge_max,
              _ptr(sink), _ptr(g), g_ld, g_dv, _ptr(dist), keep_first, float(softcap or 0.0), _ptr(rel), rel_len,
              _stream()), "attention_mma")
    return out


_ATTN_TC_ARGS = [c_void_p] * 8 + [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                  c_void_p, c_ll, c_int, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p]


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


# ------------------------------------------------------------------ norm after a sublayer, stream sums

def rmsnorm_add(x: torch.Tensor, w: torch.Tensor, eps: float, stream: torch.Tensor) -> torch.Tensor:
    """``stream += x / rms(x) * w`` row by row (float32 [T, H] both): the norm that follows a sublayer."""
    _dev(x, "x", torch.float32); _dev(w, "w"); _dev(stream, "stream", torch.float32)
    if x.shape != stream.shape or w.numel() != x.shape[-1]:
        raise KernelError("rmsnorm_add: x and stream must be [T, H], the gain [H]")
    fn = _fn("elementwise", "bw_rmsnorm_add", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(x), _ptr(w), _code(w, "w"), _ptr(stream), x.shape[0], x.shape[1], float(eps), _stream()), "rmsnorm_add")
    return stream


def rmsnorm_add_norm(x: torch.Tensor, w: torch.Tensor, eps: float, stream: torch.Tensor, w_next: torch.Tensor,
                     eps_next: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``stream += x / rms(x) * w`` and, in the same kernel, the next norm of the new stream:
    returns ``stream / rms(stream) * w_next`` in ``out_dtype``."""
    _dev(x, "x", torch.float32); _dev(w, "w"); _dev(stream, "stream", torch.float32); _dev(w_next, "w_next", w.dtype)
    if x.shape != stream.shape or w.numel() != x.shape[-1] or w_next.numel() != x.shape[-1]:
        raise KernelError("rmsnorm_add_norm: x and stream must be [T, H], the gains [H]")
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    fn = _fn("elementwise", "bw_rmsnorm_add_norm", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                                    c_float, c_float, c_void_p])
    _check(fn(_ptr(x), _ptr(w), _ptr(stream), _ptr(w_next), _code(w, "w"), _ptr(out), _code(out, "out"), x.shape[0], x.shape[1],
              float(eps), float(eps_next), _stream()), "rmsnorm_add_norm")
    return out


def add_into(target: torch.Tensor, other: torch.Tensor) -> torch.Tensor:
    """``target += other`` (float32, same shape)."""
    _dev(target, "target", torch.float32); _dev(other, "other", torch.float32)
    if target.shape != other.shape:
        raise KernelError("add_into: shapes differ")
    fn = _fn("elementwise", "bw_add_planes", [c_void_p, c_void_p, c_int, c_ll, c_ll, c_void_p])
    _check(fn(_ptr(target), _ptr(other), 1, other.numel(), target.numel(), _stream()), "add_planes")
    return target


def scale_add(stream: torch.Tensor, a: torch.Tensor, ga: torch.Tensor, b: Optional[torch.Tensor] = None,
              gb: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``stream += a * ga (+ b * gb)``: sublayers' outputs (float32 [T, H]) times a gain per channel (float32 [H]) on
    their way into the stream; the two products are added to each other first."""
    _dev(stream, "stream", torch.float32); _dev(a, "a", torch.float32); _dev(ga, "ga", torch.float32)
    T, H = stream.shape
    if a.shape != (T, H) or ga.numel() != H or (b is None) != (gb is None):
        raise KernelError("scale_add: a (and b) must have the stream's shape, the gains its width")
    if b is not None:
        _dev(b, "b", torch.float32); _dev(gb, "gb", torch.float32)
        if b.shape != (T, H) or gb.numel() != H:
            raise KernelError("scale_add: b must have the stream's shape, its gain the width")
    fn = _fn("elementwise", "bw_scale_add", [c_void_p] * 5 + [c_int, c_int, c_void_p])
    _check(fn(_ptr(stream), _ptr(a), _ptr(ga), _ptr(b), _ptr(gb), T, H, _stream()), "scale_add")
    return stream


def scale_add_norm2(stream: torch.Tensor, pending: Optional[tuple], w1: torch.Tensor, eps1: float,
                    w2: Optional[torch.Tensor], eps2: float, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
    """One pass over the stream's rows: with ``pending`` = (a, ga, b, gb) (b and gb may be None) first
    ``stream += a * ga + b * gb`` as :func:`scale_add` makes it, then two RMS norms of the new rows, ``stream / rms *
    w1`` and (``w2`` given) ``stream / rms * w2``, in ``out_dtype``.  Returns (h1, h2 or None).  ``rows`` (int32): only
    these rows are made, and the stream is left as it is (the model's last norm on the rows whose logits are wanted)."""
    _dev(stream, "stream", torch.float32); _dev(w1, "w1")
    T, H = stream.shape
    n = T
    if rows is not None:
        _dev(rows, "rows", torch.int32)
        n = rows.numel()
    a = ga = b = gb = None
    if pending is not None:
        a, ga, b, gb = pending
        _dev(a, "a", torch.float32); _dev(ga, "ga", torch.float32)
        if a.shape != (T, H) or ga.numel() != H or (b is None) != (gb is None):
            raise KernelError("scale_add_norm2: a (and b) must have the stream's shape, the gains its width")
        if b is not None:
            _dev(b, "b", torch.float32); _dev(gb, "gb", torch.float32)
            if b.shape != (T, H) or gb.numel() != H:
                raise KernelError("scale_add_norm2: b must have the stream's shape, its gain the width")
    if w1.numel() != H or (w2 is not None and (w2.numel() != H or w2.dtype != w1.dtype)):
        raise KernelError("scale_add_norm2: the norms' gains must have the stream's width and one type")
    h1 = torch.empty((n, H), dtype=out_dtype, device=stream.device)
    h2 = torch.empty((n, H), dtype=out_dtype, device=stream.device) if w2 is not None else None
    if w2 is not None:
        _dev(w2, "w2")
    fn = _fn("elementwise", "bw_scale_add_norm2", [c_void_p] * 7 + [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                                                  c_float, c_float, c_void_p])
    _check(fn(_ptr(stream), _ptr(a), _ptr(ga), _ptr(b), _ptr(gb), _ptr(w1), _ptr(w2), _code(w1, "w1"), _ptr(h1), _ptr(h2),
              _code(h1, "out"), _ptr(rows), n, H, float(eps1), float(eps2), _stream()), "scale_add_norm2")
    return h1, h2


# ------------------------------------------------------------------ q/k norm + rotation + append

def qk_norm_rope_append(qkv: torch.Tensor, batch, block_table: torch.Tensor, table: Optional[torch.Tensor],
                        rotary_dim: int, interleaved: bool, q_gain: Optional[torch.Tensor],
                        k_gain: Optional[torch.Tensor], eps: float, k_pages: torch.Tensor, v_pages: torch.Tensor,
                        nh: int, nkv: int, dq: int, dv: int, append: bool = True) -> torch.Tensor:
    """``qkv`` float32 [T, nh*dq + nkv*dq + nkv*dv] -> queries [T, nh * dpad] in the pages' dtype, keys and
    values to the pages [num_pages, nkv, page_size, dpad] of the tokens' positions (dpad >= dq, dv; the
    channels beyond a head's own size are written as zeros).  With gains: all query channels of a token
    are divided by their common root mean square and multiplied by ``q_gain`` (the same for the keys)
    before the rotation.  ``table``: :func:`rope_table` of the step; ``interleaved``: channel 2i turns with
    2i + 1, else channel i with i + rotary_dim / 2."""
    _dev(qkv, "qkv", torch.float32); _dev(block_table, "block_table", torch.int32)
    _dev(k_pages, "k_pages"); _dev(v_pages, "v_pages", k_pages.dtype)
    T = qkv.shape[0]
    num_pages, pk, page_size, dpad = k_pages.shape
    if qkv.shape[1] != nh * dq + nkv * dq + nkv * dv or pk != nkv or v_pages.shape != k_pages.shape:
        raise KernelError("qk_norm_rope_append: qkv must be [T, nh*dq + nkv*dq + nkv*dv], pages [num_pages, nkv, page, dpad]")
    for name, g, n in (("q_gain", q_gain, nh * dq), ("k_gain", k_gain, nkv * dq)):
        if g is not None:
            _dev(g, name, torch.float32)
            if g.numel() != n:
                raise KernelError(f"qk_norm_rope_append: {name} must have {n} entries")
    if rotary_dim:
        _dev(table, "table", torch.float32)
        if tuple(table.shape) != (T, rotary_dim):
            raise KernelError("qk_norm_rope_append: the cos/sin table must be [T, rotary_dim]")
    q_out = torch.empty((T, nh * dpad), dtype=k_pages.dtype, device=qkv.device)
    fn = _fn("qk_norm_rope", "bw_qk_norm_rope_append",
             [c_void_p] * 4 + [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p]
             + [c_int] * 9 + [c_void_p])
    _check(fn(_ptr(qkv), _ptr(batch.positions), _ptr(batch.req_of_token), _ptr(block_table), block_table.shape[1],
              _ptr(table), int(rotary_dim), int(interleaved), _ptr(q_gain), _ptr(k_gain), float(eps), _ptr(q_out),
              _ptr(k_pages), _ptr(v_pages), _code(k_pages, "pages"), T, nh, nkv, dq, dv, dpad, page_size,
              num_pages if append else 0, _stream()), "qk_norm_rope_append")
    return q_out


def head_norm_rope_append(qkv: torch.Tensor, batch, block_table: torch.Tensor, table: Optional[torch.Tensor],
                          rotary_dim: int, interleaved: bool, q_gain: Optional[torch.Tensor],
                          k_gain: Optional[torch.Tensor], eps: float, k_pages: torch.Tensor, v_pages: torch.Tensor,
                          nh: int, nkv: int, dq: int, dv: int, has_kv: bool = True, append: bool = True,
                          q_temp: Optional[tuple] = None, v_eps: float = 0.0,
                          v_mix: Optional[tuple] = None) -> torch.Tensor:
    """:func:`qk_norm_rope_append` with the norm taken per head: every query head is divided by its own root mean
    square and multiplied by ``q_gain`` (float32 [dq], shared by the heads; ``k_gain`` for the key heads).
    ``qkv`` float32 [T, >= nh*dq (+ nkv*dq + nkv*dv with ``has_kv``)]: further columns (a gate's projection) are
    left alone.  ``q_temp`` = (coef, every): after norm and rotation the queries of a token at position p are
    multiplied by ``1 + coef * log(1 + n)``, n the whole periods of ``every`` positions in p + 1.  Without ``has_kv`` (a run that reads another
    run's keys and values) nothing is appended.  ``v_eps`` > 0: every value head is divided by
    sqrt(mean(v^2) + v_eps) on its way into the cache.  ``v_mix`` = (v_first float32 [T, nkv * dv], possibly a column
    range of a wider tensor; lam, a float32 number on the device): the values are cached as (1 - lam) v + lam v_first."""
    _dev(qkv, "qkv", torch.float32); _dev(block_table, "block_table", torch.int32)
    vf = lam = None
    if v_mix is not None:
        vf, lam = v_mix
        _dev(vf, "v_first", torch.float32, contiguous=False); _dev(lam, "lam", torch.float32)
        if vf.shape != (qkv.shape[0], nkv * dv) or vf.stride(1) != 1 or lam.numel() != 1 or not has_kv:
            raise KernelError("head_norm_rope_append: v_first must be float32 [T, nkv * dv] with contiguous rows, lam one number")
    _dev(k_pages, "k_pages"); _dev(v_pages, "v_pages", k_pages.dtype)
    T = qkv.shape[0]
    num_pages, pk, page_size, dpad = k_pages.shape
    need = nh * dq + (nkv * (dq + dv) if has_kv else 0)
    if qkv.shape[1] < need or pk != nkv or v_pages.shape != k_pages.shape:
        raise KernelError("head_norm_rope_append: qkv must be [T, >= nh*dq (+ nkv*dq + nkv*dv)], pages [num_pages, nkv, page, dpad]")
    for name, g in (("q_gain", q_gain), ("k_gain", k_gain)):
        if g is not None:
            _dev(g, name, torch.float32)
            if g.numel() != dq:
                raise KernelError(f"head_norm_rope_append: {name} must have {dq} entries")
    if rotary_dim:
        _dev(table, "table", torch.float32)
        if tuple(table.shape) != (T, rotary_dim):
            raise KernelError("head_norm_rope_append: the cos/sin table must be [T, rotary_dim]")
    coef, every = (float(q_temp[0]), float(q_temp[1])) if q_temp is not None else (0.0, 1.0)
    q_out = torch.empty((T, nh * dpad), dtype=k_pages.dtype, device=qkv.device)
    fn = _fn("qk_norm_rope", "bw_head_norm_rope_append",
             [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_float,
              c_float, c_void_p, c_void_p, c_void_p] + [c_int] * 10 + [c_float, c_void_p, c_ll, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.stride(0), _ptr(batch.positions), _ptr(batch.req_of_token), _ptr(block_table),
              block_table.shape[1], _ptr(table), int(rotary_dim), int(interleaved), _ptr(q_gain), _ptr(k_gain), float(eps),
              coef, every, _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _code(k_pages, "pages"), T, nh, nkv, dq, dv, dpad,
              page_size, num_pages if (append and has_kv) else 0, int(has_kv), float(v_eps or 0.0), _ptr(vf),
              vf.stride(0) if vf is not None else 0, _ptr(lam), _stream()),
           "head_norm_rope_append")
    return q_out


# ------------------------------------------------------------------ rows that look at the token before them

def embed_bigram(table: torch.Tensor, second: torch.Tensor, batch, prev_token: torch.Tensor, buckets: int, mul_prev: int,
                 mul_cur: int, scale: float = 1.0) -> torch.Tensor:
    """float32 [T, H]: ``table[id] * scale + second[row]``, row = (previous token * mul_prev + id * mul_cur) mod
    ``buckets``, or row ``buckets`` for a sequence's first token.  The previous token of a portion's first token comes
    from ``prev_token`` (int32 [slots], indexed by the request's slot), which then takes the portion's last token."""
    _dev(table, "table"); _dev(second, "second table", table.dtype); _dev(prev_token, "prev_token", torch.int32)
    V, H = table.shape
    if tuple(second.shape) != (buckets + 1, H) or buckets <= 0:
        raise KernelError(f"embed_bigram: the second table must be [{buckets + 1}, {H}]")
    out = torch.empty((batch.T, H), dtype=torch.float32, device=table.device)
    fn = _fn("rowstate", "bw_embed_bigram", [c_void_p, c_void_p, c_int] + [c_void_p] * 7 + [c_int] * 4 + [c_ll, c_ll, c_float, c_void_p])
    _check(fn(_ptr(table), _ptr(second), _code(table, "table"), _ptr(batch.token_ids), _ptr(batch.positions),
              _ptr(batch.req_of_token), _ptr(batch.cu_q), _ptr(batch.state_slot), _ptr(prev_token), _ptr(out), batch.T, H, V,
              int(buckets), int(mul_prev), int(mul_cur), float(scale), _stream()), "embed_bigram")
    return out


def rmsnorm_shift(x: torch.Tensor, gain: torch.Tensor, shift: torch.Tensor, state: torch.Tensor, batch, eps: float,
                  out_dtype: torch.dtype, want_h: bool = True):
    """(h, hs): ``h = x / rms(x) * gain`` and ``hs_t = h_t + (h_{t-1} - h_t) * shift`` with zeros before a sequence's
    first token.  ``state`` (float32 [slots, H]) holds h of every request's last token so far: a portion's first token
    reads it, and it takes the portion's last h.  ``want_h=False``: only hs is written (h is None)."""
    # an outstanding sum into x: in a step of single tokens (no row reads its neighbour) the kernel adds it while it
    # norms; else a kernel of its own does first (the check of x below would ask for it)
    global _pending
    planes = None
    if (_pending is not None and _pending[0].data_ptr() == x.data_ptr() and _pending[0].shape == x.shape
            and not _pending[2] and batch.T == batch.R and x.dim() == 2 and x.shape[0] == batch.T):
        planes, _pending = _pending[1], None
    else:
        resolve_pending()
    _dev(x, "x", torch.float32); _dev(gain, "gain", torch.float32); _dev(shift, "shift", torch.float32)
    _dev(state, "state", torch.float32)
    T, H = x.shape
    if gain.numel() != H or shift.numel() != H or state.dim() != 2 or state.shape[1] != H or T != batch.T:
        raise KernelError("rmsnorm_shift: gain and shift [H], state [slots, H], one row of x per token of the batch")
    h = torch.empty((T, H), dtype=out_dtype, device=x.device) if want_h else None
    hs = torch.empty((T, H), dtype=out_dtype, device=x.device)
    fn = _fn("rowstate", "bw_rmsnorm_shift", [c_void_p, c_void_p, c_int, c_ll] + [c_void_p] * 9 + [c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(x), _ptr(planes), 0 if planes is None else planes.shape[0], 0 if planes is None else planes.stride(0),
              _ptr(gain), _ptr(shift), _ptr(state), _ptr(batch.positions), _ptr(batch.req_of_token),
              _ptr(batch.cu_q), _ptr(batch.state_slot), _ptr(h), _ptr(hs), _code(hs, "out"), T, H, float(eps), _stream()),
           "rmsnorm_shift")
    return h, hs


def concat2_cast(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """[T, 2H] in ``out_dtype``: the float32 tensors a and b [T, H] side by side."""
    _dev(a, "a", torch.float32); _dev(b, "b", torch.float32)
    if a.shape != b.shape or a.dim() != 2:
        raise KernelError("concat2_cast: two float32 tensors [T, H]")
    T, H = a.shape
    out = torch.empty((T, 2 * H), dtype=out_dtype, device=a.device)
    fn = _fn("rowstate", "bw_concat2_cast", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(a), _ptr(b), _ptr(out), _code(out, "out"), T, H, _stream()), "concat2_cast")
    return out


# ------------------------------------------------------------------ latent attention

def latent_prep(proj: torch.Tensor, q_off: int, kv_off: int, batch, block_table: torch.Tensor, table: torch.Tensor,
                c_gain: torch.Tensor, eps: float, k_pages: torch.Tensor, H: int, d: int, dr: int, rank: int,
                append: bool = True, q_src: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """From the projections of a step (float32 [T, ...]: H query heads of d plain + dr rotated channels at column
    ``q_off``; the latent's rank channels and the shared key part's dr channels at ``kv_off``): appends
    [rms_norm(latent) * c_gain, rotated key part, zeros] to the tokens' cache rows and returns the queries
    [T, H * dpad] with channels [rank, rank + dr) of every head filled (the rotated parts; channels [0, rank) are left
    for :func:`headwise_linear`).  ``q_src``: the float32 tensor that holds the queries at ``q_off`` where that is not
    ``proj`` (queries made by a product of their own).  ``interleaved``: the rotation pairs channel 2j with channel 2j + 1
    instead of channel c with channel c + dr / 2."""
    _dev(proj, "proj", torch.float32); _dev(block_table, "block_table", torch.int32); _dev(table, "table", torch.float32)
    q_src = proj if q_src is None else _dev(q_src, "q_src", torch.float32)
    if q_src.shape[0] != proj.shape[0]:
        raise KernelError("latent_prep: queries and latent must have the same rows")
    _dev(c_gain, "c_gain", torch.float32); _dev(k_pages, "k_pages")
    T = proj.shape[0]
    num_pages, nkv, page_size, dpad = k_pages.shape
    if nkv != 1 or dpad < rank + dr or tuple(table.shape) != (T, dr) or c_gain.numel() != rank:
        raise KernelError("latent_prep: pages [num_pages, 1, page, >= rank + dr], table [T, dr], gain [rank]")
    q = torch.empty((T, H * dpad), dtype=k_pages.dtype, device=proj.device)
    fn = _fn("latent", "bw_latent_prep", [c_void_p, c_ll, c_int, c_void_p, c_ll, c_int, c_int] + [c_void_p] * 3 +
             [c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p] + [c_int] * 9 + [c_void_p])
    _check(fn(_ptr(q_src), q_src.stride(0), int(q_off), _ptr(proj), proj.stride(0), int(kv_off), int(interleaved),
              _ptr(batch.positions), _ptr(batch.req_of_token),
              _ptr(block_table), block_table.shape[1], _ptr(table), _ptr(c_gain), float(eps), _ptr(q), _ptr(k_pages),
              _code(k_pages, "pages"), T, H, d, dr, rank, dpad, page_size, num_pages if append else 0, _stream()), "latent_prep")
    return q


def headwise_linear(x: torch.Tensor, x_off: int, x_hs: int, w: torch.Tensor, y: torch.Tensor, y_off: int, y_hs: int,
                    gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[t, y_off + h * y_hs + o] = sum_i x[t, x_off + h * x_hs + i] * w[h, o, i]`` for every head h: one small
    product per head.  w [H, n_out, n_in]; x float32 or bfloat16, w and y of one type (float32 sums in a fixed order).
    ``gate`` (float32 [T, H * n_out], possibly a range of columns of a wider tensor): the result is multiplied by
    sigmoid(gate[t, h * n_out + o]) before it is rounded and written."""
    _dev(x, "x", contiguous=False); _dev(w, "w"); _dev(y, "y", contiguous=False)
    H, n_out, n_in = w.shape
    T = x.shape[0]
    if gate is not None:
        _dev(gate, "gate", torch.float32, contiguous=False)
        if gate.shape != (T, H * n_out) or gate.stride(1) != 1:
            raise KernelError("headwise_linear: the gate must be float32 [T, H * n_out] with contiguous rows")
    if (x.dim() != 2 or y.dim() != 2 or y.shape[0] != T or x.stride(1) != 1 or y.stride(1) != 1
            or x_off + (H - 1) * x_hs + n_in > x.shape[1] or y_off + (H - 1) * y_hs + n_out > y.shape[1]):
        raise KernelError("headwise_linear: x [T, >= x_off + (H - 1) x_hs + n_in], y [T, >= y_off + (H - 1) y_hs + n_out]")
    fn = _fn("latent", "bw_headwise_linear", [c_void_p, c_int, c_ll, c_int, c_void_p, c_int, c_void_p, c_int, c_ll, c_int,
                                              c_int, c_int, c_int, c_int, c_void_p, c_ll, c_void_p])
    _check(fn(c_void_p(x.data_ptr() + x_off * x.element_size()), _code(x, "x"), x.stride(0), int(x_hs), _ptr(w), _code(w, "w"),
              c_void_p(y.data_ptr() + y_off * y.element_size()), _code(y, "y"), y.stride(0), int(y_hs), T, H, n_in, n_out,
              _ptr(gate), gate.stride(0) if gate is not None else 0, _stream()), "headwise_linear")
    return y


# ------------------------------------------------------------------ several copies of the stream (hyper-connections)

HC_MAX_STREAMS = 8   # the most copies of the stream that hc_step takes (csrc/hyper.cu is built for 1 to 8)


def hc_step(streams: torch.Tensor, S: int, y: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
            out_w: Optional[torch.Tensor] = None, in_w: Optional[torch.Tensor] = None,
            gain: Optional[torch.Tensor] = None, eps: float = 0.0, rows: Optional[torch.Tensor] = None,
            out_dtype: torch.dtype = torch.float32) -> Optional[torch.Tensor]:
    """One step of a stream kept as ``S`` copies (``streams`` float32 [T, S * H], updated in place):

        with ``y`` [T, H]:   x_t <- sum_s mix[s, t] x_s + out_w[t] * y      (all copies at once, from the old ones)
        with ``in_w`` [S]:   returns norm(sum_s in_w[s] x_s) for the next sublayer, the norm being
                             u / sqrt(mean(u^2) + eps) * gain (float32 [H]); without ``gain`` the sum itself, float32.

    ``rows``: only those rows are computed and ``streams`` is left as it is (the last read of a model)."""
    global _pending
    _dev(streams, "streams", torch.float32)
    T = streams.shape[0]
    H = streams.shape[1] // S
    planes, y_valid = None, True
    if (y is not None and _pending is not None and _pending[0].data_ptr() == y.data_ptr() and _pending[0].shape == y.shape):
        # y's last product is still in planes: the kernel adds them while it reads y (or takes them for y)
        (_, planes, overwrite), _pending = _pending, None
        y_valid = not overwrite
    if streams.shape[1] != S * H:
        raise KernelError("hc_step: streams must be [T, S * H]")
    for name, t, n in (("y", y, T * H), ("mix", mix, S * S), ("out_w", out_w, S), ("in_w", in_w, S), ("gain", gain, H)):
        if t is not None:
            _dev(t, name, torch.float32)
            if t.numel() != n:
                raise KernelError(f"hc_step: {name} must have {n} float32 entries")
    if y is not None and (mix is None or out_w is None):
        raise KernelError("hc_step: a write needs mix and out_w")
    n = T
    if rows is not None:
        _dev(rows, "rows", torch.int32)
        n = rows.numel()
    out = None
    if in_w is not None:
        out = torch.empty((n, H), dtype=out_dtype if gain is not None else torch.float32, device=streams.device)
    fn = _fn("hyper", "bw_hc_step", [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_ll, c_int,
                                                      c_void_p])
    _check(fn(_ptr(streams), _ptr(y), _ptr(mix), _ptr(out_w), _ptr(in_w), _ptr(gain), _ptr(rows), _ptr(out),
              _code(out, "out") if out is not None else F32, n, S, H, float(eps), int(rows is None and y is not None),
              _ptr(planes), planes.shape[0] if planes is not None else 0, planes.stride(0) if planes is not None else 0,
              int(y_valid), _stream()), "hc_step")
    return out


# ------------------------------------------------------------------ gated linear attention

GLA_MAX_KEY_DIM = 256


def gla_decay(proj: torch.Tensor, x_off: int, w: torch.Tensor, b: torch.Tensor, tau: float) -> torch.Tensor:
    """``sigmoid(x w.T + b) ** (1 / tau)`` in float32, x being ``rank`` columns of ``proj`` from ``x_off`` on
    (w [C, rank], b [C]): the decay of every key channel of every token, float32 [T, C]."""
    _dev(proj, "proj", torch.float32); _dev(w, "w"); _dev(b, "b", w.dtype)
    T = proj.shape[0]
    C, rank = w.shape
    if x_off + rank > proj.shape[1] or b.numel() != C:
        raise KernelError("gla_decay: the first projection lies outside proj, or the bias has the wrong size")
    a = torch.empty((T, C), dtype=torch.float32, device=proj.device)
    fn = _fn("gla", "bw_gla_decay", [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float,
                                     c_void_p])
    _check(fn(_ptr(proj), proj.stride(0), x_off, _ptr(w), _ptr(b), _code(w, "w"), _ptr(a), T, C, rank, float(tau), _stream()),
           "gla_decay")
    return a


def gla_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: torch.Tensor, batch, state: torch.Tensor,
             heads: int, dk: int, dv: int, q_scale: float, k_scale: Optional[torch.Tensor] = None,
             scalar_decay: bool = False, ones_col: bool = False) -> torch.Tensor:
    """The recurrence ``S <- diag(a) S + k v^T, o = S^T (q_scale q)`` over the step's tokens, request by request
    in order, from and into ``state`` [slots, heads, dk, dv] (float32) at the requests' slots.  ``proj`` float32
    [T, ld] holds q, k, v at the given column offsets (head-major); ``decay`` float32 [T, heads * dk] holds a
    (:func:`gla_decay`).  Returns o float32 [T, heads * dv].  For a memory with one decay per head and a normaliser:
    ``scalar_decay``: ``decay`` is [T, heads]; ``k_scale`` float32 [T, heads]: the keys are multiplied by it as they are
    read; ``ones_col``: ``dv`` counts one more value column than ``proj`` holds, the constant 1, so that the state's
    last column is n <- a n + k and the output's last column n . q.  The state's rows may be longer than ``dv`` (padding that
    stays zero): with a length that is a multiple of 4 the kernel moves a lane's columns of a row in one access."""
    _dev(proj, "proj", torch.float32); _dev(decay, "decay", torch.float32); _dev(state, "state", torch.float32)
    T = proj.shape[0]
    if dk > GLA_MAX_KEY_DIM:
        raise KernelError(f"gla_scan: key size {dk} exceeds {GLA_MAX_KEY_DIM}")
    if (decay.shape != (T, heads if scalar_decay else heads * dk) or state.dim() != 4 or tuple(state.shape[1:3]) != (heads, dk)
            or state.shape[3] < dv):
        raise KernelError("gla_scan: decay must be [T, heads * dk] ([T, heads] with scalar_decay), state [slots, heads, dk, >= dv]")
    if k_scale is not None:
        _dev(k_scale, "k_scale", torch.float32)
        if k_scale.shape != (T, heads):
            raise KernelError("gla_scan: k_scale must be [T, heads]")
    if max(q_off + heads * dk, k_off + heads * dk, v_off + heads * (dv - int(ones_col))) > proj.shape[1]:
        raise KernelError("gla_scan: q, k or v lie outside the projection's columns")
    o = torch.empty((T, heads * dv), dtype=torch.float32, device=proj.device)
    fn = _fn("gla", "bw_gla_scan", [c_void_p, c_ll, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(proj), proj.stride(0), q_off, k_off, v_off, _ptr(decay), _ptr(batch.cu_q), _ptr(batch.state_slot),
              _ptr(state), _ptr(o), batch.R, heads, dk, dv, float(q_scale), _ptr(k_scale), int(scalar_decay),
              int(ones_col), int(state.shape[3]), _stream()), "gla_scan")
    return o


def gla_gate(o: torch.Tensor, proj: torch.Tensor, g_off: int, gain: torch.Tensor, heads: int, dv: int, eps: float,
             out_dtype: torch.dtype) -> torch.Tensor:
    """Per token and head ``o / rms(o) * gain * silu(g)`` with g at column ``g_off`` of ``proj``."""
    _dev(o, "o", torch.float32); _dev(proj, "proj", torch.float32); _dev(gain, "gain", torch.float32)
    T = o.shape[0]
    if o.shape[1] != heads * dv or gain.numel() != dv or g_off + heads * dv > proj.shape[1]:
        raise KernelError("gla_gate: o must be [T, heads * dv], the gain [dv], the gate inside the projection")
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=o.device)
    fn = _fn("gla", "bw_gla_gate", [c_void_p, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_float, c_void_p])
    _check(fn(_ptr(o), _ptr(proj), proj.stride(0), g_off, _ptr(gain), _ptr(out), _code(out, "out"), T, heads, dv,
              float(eps), _stream()), "gla_gate")
    return out


# ------------------------------------------------------------------ matrix memory with exponential gates

def mlstm_gates(proj: torch.Tensor, i_off: int, f_off: int, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float, batch,
                m_state: torch.Tensor, heads: int):
    """The gates of a step's tokens, request by request in order, from and into ``m_state`` [slots, heads] (float32):
    with i = cap tanh((z_i + b_i) / cap), f = log_sigmoid(cap tanh((z_f + b_f) / cap)) (z at columns ``i_off`` /
    ``f_off`` of ``proj``, float32) and m <- max(f + m, i): returns a = exp(f + m_before - m), b = exp(i - m),
    e = exp(-m), each float32 [T, heads]."""
    _dev(proj, "proj", torch.float32); _dev(bias_i, "bias_i", torch.float32); _dev(bias_f, "bias_f", torch.float32)
    _dev(m_state, "m_state", torch.float32)
    T = proj.shape[0]
    if (bias_i.numel() != heads or bias_f.numel() != heads or m_state.dim() != 2 or m_state.shape[1] != heads
            or max(i_off, f_off) + heads > proj.shape[1]):
        raise KernelError("mlstm_gates: biases [heads], m_state [slots, heads], the gates inside the projection")
    a, b, e = (torch.empty((T, heads), dtype=torch.float32, device=proj.device) for _ in range(3))
    fn = _fn("mlstm", "bw_mlstm_gates", [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_float] + [c_void_p] * 6 +
             [c_int, c_int, c_void_p])
    _check(fn(_ptr(proj), proj.stride(0), int(i_off), int(f_off), _ptr(bias_i), _ptr(bias_f), float(cap), _ptr(batch.cu_q),
              _ptr(batch.state_slot), _ptr(m_state), _ptr(a), _ptr(b), _ptr(e), batch.R, heads, _stream()), "mlstm_gates")
    return a, b, e


def mlstm_out(o: torch.Tensor, e: torch.Tensor, proj: torch.Tensor, g_off: int, gain: torch.Tensor, heads: int, dv: int,
              eps: float, out_dtype: torch.dtype, den_eps: float = 1e-6) -> torch.Tensor:
    """Per token and head, from the scan's output ``o`` float32 [T, heads * (dv + 1)] whose last column per head is
    n . q: ``u = o[:dv] / (max(|n . q|, e) + den_eps)``, then ``u / rms(u) * gain * sigmoid(g)`` with the gain per channel
    of all heads (float32 [heads * dv]) and g at column ``g_off`` of ``proj``."""
    _dev(o, "o", torch.float32); _dev(e, "e", torch.float32); _dev(proj, "proj", torch.float32); _dev(gain, "gain", torch.float32)
    T = o.shape[0]
    if o.shape[1] != heads * (dv + 1) or e.shape != (T, heads) or gain.numel() != heads * dv or g_off + heads * dv > proj.shape[1]:
        raise KernelError("mlstm_out: o [T, heads * (dv + 1)], e [T, heads], gain [heads * dv], the gate inside the projection")
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=o.device)
    fn = _fn("mlstm", "bw_mlstm_out", [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                       c_float, c_float, c_void_p])
    _check(fn(_ptr(o), _ptr(e), _ptr(proj), proj.stride(0), int(g_off), _ptr(gain), _ptr(out), _code(out, "out"), T, heads, dv,
              float(eps), float(den_eps), _stream()), "mlstm_out")
    return out


# ------------------------------------------------------------------ routed feed-forward

_moe_tile = None


def moe_tile_rows() -> int:
    """Rows of a tile of regrouped tokens (an expert's stretch of rows is padded to a multiple of it)."""
    global _moe_tile
    if _moe_tile is None:
        _moe_tile = int(_fn("moe", "bw_moe_tile_rows", [])())
    return _moe_tile


def moe_max_tiles(rows: int, experts: int, tile_rows: Optional[int] = None) -> int:
    """Tiles that ``rows`` regrouped rows can take at most, whatever the routing."""
    return -(-rows // (tile_rows or moe_tile_rows())) + experts


_moe_tc_tile = None


def moe_tc_tile_rows() -> int:
    """Rows of a tile of the tcgen05 grouped product."""
    global _moe_tc_tile
    if _moe_tc_tile is None:
        _moe_tc_tile = int(_fn("moe_tc", "bw_moe_tc_tile_rows", [])())
    return _moe_tc_tile


def moe_gemm_tc_supports(H: int, F: int) -> bool:
    """Whether the tcgen05 grouped products take an expert of size F on width H (bfloat16): inner sizes that
    are multiples of 8 (TMA rows), gate/up rows interleaved in blocks of 16.  BW_MOE_TC=0 keeps the CUDA cores."""
    return os.environ.get("BW_MOE_TC", "1") != "0" and H % 8 == 0 and F % 16 == 0


def moe_gemm_tc(a: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, gated: bool = False,
                out_dtype: Optional[torch.dtype] = None, act: int = ACT_SILU, limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """The grouped product on the tensor cores: a bfloat16 [tiles * 128, K], w bfloat16 [E, N, K]; row r gets
    ``a[r] @ w[e].T`` with e the expert of r's tile.  ``gated``: w's rows alternate 16 gate rows / 16 up rows
    (:func:`interleave_gate_up` per expert) and the result is bfloat16 [rows, N / 2] = silu(gate) * up, or the
    gated activation ``act`` with its ``limit`` and ``alpha`` (:func:`glu`)."""
    _dev(a, "a", torch.bfloat16); _dev(w, "w", torch.bfloat16); _dev(tile_expert, "tile_expert", torch.int32)
    rows, K = a.shape
    E, N, K2 = w.shape
    if K != K2 or rows != tile_expert.numel() * moe_tc_tile_rows():
        raise KernelError("moe_gemm_tc: a must be [tiles * 128, K], w [E, N, K]")
    out_dtype = torch.bfloat16 if gated else (out_dtype or torch.bfloat16)
    out = torch.empty((rows, N // 2 if gated else N), dtype=out_dtype, device=a.device)
    fn = _fn("moe_tc", "bw_moe_gemm_tc", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_float, c_float, c_void_p])
    _check(fn(_ptr(a), _ptr(w), int(gated), _ptr(tile_expert), _ptr(out), _code(out, "out"), tile_expert.numel(), E, N, K,
              int(act), float(limit), float(alpha), _stream()), "moe_gemm_tc")
    return out


def moe_tc_status() -> int:
    """0 if no bounded wait of the tcgen05 grouped product ever gave up (synchronises the device)."""
    return int(_fn("moe_tc", "bw_moe_tc_status", [])())


def moe_route(logits: torch.Tensor, top: int, softmax: bool = False, renormalize: bool = False,
              bias: Optional[torch.Tensor] = None, renorm_eps: float = 0.0):
    """float32 router logits [T, E] -> (chosen experts int32 [T, top], their weights float32 [T, top]):
    scores are sigmoid(logit) (or the softmax over the experts), the ``top`` largest are chosen (lowest
    index on ties) in falling order, optionally renormalised to sum 1 (divided by their sum + ``renorm_eps``).
    ``bias`` (float32 [E]): the choice goes by score + bias, the weights stay the scores."""
    _dev(logits, "logits", torch.float32)
    T, E = logits.shape
    _check_route_bias(bias, E)
    sel = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    wt = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    fn = _fn("moe", "bw_moe_route", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), T, E, int(top), int(softmax), int(renormalize), _ptr(bias), float(renorm_eps), _ptr(sel), _ptr(wt),
              _stream()), "moe_route")
    return sel, wt


def _check_route_bias(bias: Optional[torch.Tensor], E: int) -> None:
    if bias is not None:
        _dev(bias, "bias", torch.float32)
        if bias.numel() != E:
            raise KernelError(f"moe_route: the bias must have one float32 entry per router output ({E})")


MOE_FUSED_FRONT_MAX_ROWS = 128   # up to this many (token, choice) rows one block routes, plans and regroups (the kernel takes 1,024)


def moe_route_plan_scatter(logits: torch.Tensor, x: torch.Tensor, top: int, tile_rows: int, softmax: bool = False,
                           renormalize: bool = False, scale_input: bool = False, experts: Optional[int] = None,
                           bias: Optional[torch.Tensor] = None, renorm_eps: float = 0.0):
    """:func:`moe_route`, :func:`moe_plan` and :func:`moe_scatter` as one kernel, for steps of few tokens.
    Returns (weights [T, top], place of every (token, choice), expert of every tile, the regrouped operand).
    ``experts``: how many of the router's outputs are experts with weights (default: all); a choice beyond
    them has no place (-1)."""
    _dev(logits, "logits", torch.float32); _dev(x, "x")
    T, E_total = logits.shape
    E = E_total if experts is None else int(experts)
    _check_route_bias(bias, E_total)
    H = x.shape[1]
    n = T * top
    if n > MOE_FUSED_FRONT_MAX_ROWS or x.shape[0] != T:
        raise KernelError("moe_route_plan_scatter: too many rows for one block, or x and logits disagree")
    max_tiles = moe_max_tiles(n, E, tile_rows)
    dev = logits.device
    sel = torch.empty((T, top), dtype=torch.int32, device=dev)
    wt = torch.empty((T, top), dtype=torch.float32, device=dev)
    pos_of = torch.empty(n, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    xs = torch.empty((max_tiles * tile_rows, H), dtype=x.dtype, device=dev)
    fn = _fn("moe", "bw_moe_route_plan_scatter", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p,
                                                  c_void_p, c_int, c_int,
                                                  c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(logits), T, E, E_total, int(top), int(softmax), int(renormalize), _ptr(bias), float(renorm_eps), _ptr(sel), _ptr(wt),
              int(tile_rows), max_tiles,
              _ptr(pos_of), _ptr(tile_expert), _ptr(x), _code(x, "x"), _ptr(xs), H, int(scale_input), _stream()),
           "moe_route_plan_scatter")
    return wt, pos_of, tile_expert, xs


def moe_plan(sel: torch.Tensor, experts: int, tile_rows: Optional[int] = None):
    """(row of every (token, choice) in the regrouped order int32 [T * top], expert of every tile of
    ``tile_rows`` rows int32 [max_tiles], -1 for idle tiles).  A choice that names no expert below ``experts``
    (an expert without weights) gets no row: -1."""
    _dev(sel, "sel", torch.int32)
    n = sel.numel()
    tile_rows = tile_rows or moe_tile_rows()
    max_tiles = moe_max_tiles(n, experts, tile_rows)
    pos_of = torch.empty(n, dtype=torch.int32, device=sel.device)
    tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=sel.device)
    fn = _fn("moe", "bw_moe_plan", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(sel), n, int(experts), int(tile_rows), max_tiles, _ptr(pos_of), _ptr(tile_expert), _stream()), "moe_plan")
    return pos_of, tile_expert


def moe_scatter(x: torch.Tensor, pos_of: torch.Tensor, wt: torch.Tensor, rows: int, scale_input: bool) -> torch.Tensor:
    """The regrouped operand [rows, H]: row ``pos_of[t * top + k]`` = x[t] (times the choice's weight)."""
    _dev(x, "x"); _dev(pos_of, "pos_of", torch.int32); _dev(wt, "wt", torch.float32)
    T, H = x.shape
    top = pos_of.numel() // max(T, 1)
    xs = torch.empty((rows, H), dtype=x.dtype, device=x.device)
    fn = _fn("moe", "bw_moe_scatter", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), _code(x, "x"), _ptr(pos_of), _ptr(wt), _ptr(xs), pos_of.numel(), H, top, int(scale_input), _stream()),
           "moe_scatter")
    return xs


def moe_gemm(a: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, w2: Optional[torch.Tensor] = None,
             out_dtype: Optional[torch.dtype] = None, act: int = ACT_SILU, limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """Row r of the result is ``a[r] @ w[e].T`` with e the expert of r's tile; with ``w2`` it is
    ``silu(a[r] @ w[e].T) * (a[r] @ w2[e].T)``, or the gated activation ``act`` (:func:`glu`) of the two.
    a [rows, K], w (w2) [E, N, K]."""
    _dev(a, "a"); _dev(w, "w", a.dtype); _dev(tile_expert, "tile_expert", torch.int32)
    if w2 is not None:
        _dev(w2, "w2", a.dtype)
        if w2.shape != w.shape:
            raise KernelError("moe_gemm: both weights must be [E, N, K]")
    rows, K = a.shape
    E, N, K2 = w.shape
    if K != K2 or rows != tile_expert.numel() * moe_tile_rows():
        raise KernelError("moe_gemm: a must be [tiles * tile rows, K], w [E, N, K]")
    out = torch.empty((rows, N), dtype=out_dtype or a.dtype, device=a.device)
    fn = _fn("moe", "bw_moe_gemm", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                    c_float, c_float, c_void_p])
    _check(fn(_ptr(a), _ptr(w), _ptr(w2), _code(a, "a"), _ptr(tile_expert), _ptr(out), _code(out, "out"),
              tile_expert.numel(), N, K, int(act), float(limit), float(alpha), _stream()), "moe_gemm")
    return out


def moe_combine(y: torch.Tensor, pos_of: torch.Tensor, wt: torch.Tensor, out: torch.Tensor, scale_output: bool,
                mode: str = "write", gain: Optional[torch.Tensor] = None, eps: float = 0.0,
                x: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t]`` (= | +=) the sum over t's choices, in order, of (weight *) ``y[pos_of[t * top + k]]``;
    mode "norm_add": the sum is divided by its root mean square, multiplied by ``gain`` and added.
    ``x`` [T, H]: what a choice without a place (``pos_of`` < 0: an expert that returns its input) contributes."""
    _dev(y, "y", torch.float32); _dev(pos_of, "pos_of", torch.int32); _dev(wt, "wt", torch.float32)
    _dev(out, "out", torch.float32)
    T, H = out.shape
    modes = {"write": 0, "add": 1, "norm_add": 2}
    if mode not in modes or y.shape[1] != H or (mode == "norm_add" and gain is None):
        raise KernelError("moe_combine: bad mode or shapes")
    if gain is not None:
        gain = _dev(gain, "gain", torch.float32)
    if x is not None:
        _dev(x, "x")
        if x.shape != (T, H):
            raise KernelError("moe_combine: x must be [T, H]")
    fn = _fn("moe", "bw_moe_combine", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                       c_float, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(y), _ptr(pos_of), _ptr(wt), pos_of.numel() // max(T, 1), int(scale_output), _ptr(out), T, H, modes[mode],
              _ptr(gain), float(eps), _ptr(x), _code(x, "x") if x is not None else F32, _stream()), "moe_combine")
    return out
