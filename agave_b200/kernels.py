"""Python face of the CUDA library: one function per exported kernel launcher.

Each function takes torch CUDA tensors, checks what the C side cannot see
(device, dtype, contiguity), and launches on torch's current stream, so the
calls can be recorded into a CUDA graph.  There is no fallback: without the
compiled library, or on a tensor that is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from . import perf as _perf_mod
from .csrc import build as _build

F32, BF16 = 0, 1
ACT = {"gelu_tanh": 0, "silu": 1, "relu2": 2, "gelu_erf": 3}   # 2, 3: on a plain product only

_lib = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The loaded CUDA library (compiled on first use)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.library_path()
                try:
                    lib = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"the CUDA library {path} could not be loaded: {e}") from None
                lib.agv_last_error.restype = ctypes.c_char_p
                lib.agv_attention_prefill_tc_vt_cols.restype = ctypes.c_longlong
                if os.environ.get("AGAVE_B200_DEPENDENT_LAUNCH", "1") == "0":
                    # kernels then start only after the one before has ended, which
                    # makes per-kernel durations in a profiler additive
                    lib.agv_set_dependent_launch(0)
                _lib = lib
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelError(library().agv_last_error().decode("utf-8", "replace"))


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} has no kernels (float32 and bfloat16 do)")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("a tensor handed to a CUDA kernel is not on a CUDA device")
    return ctypes.c_void_p(t.data_ptr())


NVTX = os.environ.get("AGAVE_B200_NVTX", "0") == "1"     # name every launch for a profiler
_launches = 0
_perf = None          # an active agave_b200.perf.PerfCounters, or None


def _span(op: str, nbytes: int = 0, flops: int = 0):
    """A timing span around one launch while operations are being timed."""
    if _perf is None or torch.cuda.is_current_stream_capturing():
        # (a recording holds no timing events)
        return _perf_mod.NvtxSpan(op) if NVTX else _perf_mod.NULL_SPAN
    return _perf.span(op, nbytes, flops)


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)



_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    # called exactly once per kernel launch: the count is what bench.py reports
    global _launches
    _launches += 1
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))     # the same handle, without the
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)   # Stream object around it


def launch_count() -> int:
    """Kernels of this library launched (or recorded into a graph) so far."""
    return _launches


def _dense(t: torch.Tensor, what: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")


def _f32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{what} must be float32, got {t.dtype}")


def device_arch() -> int:
    rc = library().agv_device_arch()
    if rc < 0:
        _check(rc)
    return rc


# ------------------------------------------------------------------ embedding
def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    """out[t, :] = table[tokens[t], :] * scale, 32-bit."""
    _i32(tokens, "tokens"); _f32(out, "out"); _dense(table, "table"); _dense(out, "out")
    T, (V, H) = tokens.numel(), table.shape
    assert out.shape == (T, H)
    with _span("embed", T * H * table.element_size() + _nbytes(out)):
        _check(library().agv_embed(_ptr(tokens), _ptr(table), dtype_code(table.dtype), _ptr(out),
                                   T, H, V, ctypes.c_float(scale), _stream()))


def add_position_rows(positions: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
                      scale: float = 1.0) -> None:
    """out[t, :] += table[positions[t], :] * scale (out 32-bit): a learned vector per
    position joins the stream."""
    _i32(positions, "positions"); _f32(out, "out"); _dense(table, "table"); _dense(out, "out")
    T, (R, H) = positions.numel(), table.shape
    assert out.shape == (T, H)
    with _span("embed", T * H * table.element_size() + 2 * _nbytes(out)):
        _check(library().agv_add_position_rows(_ptr(positions), _ptr(table),
                                               dtype_code(table.dtype), _ptr(out), T, H, R,
                                               ctypes.c_float(scale), _stream()))


def rope_table(positions: torch.Tensor, rotary_dim: int, theta: float, factor: float,
               cos: torch.Tensor, sin: torch.Tensor) -> None:
    """cos, sin [T, rotary_dim/2] of (p / factor) * theta^(-2i/rotary_dim)."""
    _i32(positions, "positions"); _f32(cos, "cos"); _f32(sin, "sin")
    T = positions.numel()
    assert cos.shape == (T, rotary_dim // 2) and sin.shape == cos.shape
    with _span("rope_table", _nbytes(cos, sin)):
        _check(library().agv_rope_table(_ptr(positions), _ptr(cos), _ptr(sin), T, rotary_dim,
                                        ctypes.c_double(theta), ctypes.c_double(factor), _stream()))


def rope_table_freqs(positions: torch.Tensor, freqs: torch.Tensor, mult: float,
                     cos: torch.Tensor, sin: torch.Tensor) -> None:
    """cos, sin [T, n] = mult * cos / sin(p * freqs[i]); freqs [n] 64-bit on the device."""
    _i32(positions, "positions"); _f32(cos, "cos"); _f32(sin, "sin")
    if freqs.dtype != torch.float64:
        raise KernelError("freqs must be float64")
    T, half = positions.numel(), freqs.numel()
    assert cos.shape == (T, half) and sin.shape == cos.shape
    _dense(cos, "cos"); _dense(sin, "sin"); _dense(freqs, "freqs")
    with _span("rope_table", _nbytes(cos, sin)):
        _check(library().agv_rope_table_freqs(_ptr(positions), _ptr(freqs), _ptr(cos), _ptr(sin),
                                              T, half, ctypes.c_double(mult), _stream()))


# ---------------------------------------------------------------------- norms
def norm_residual(h: Optional[torch.Tensor], y: Optional[torch.Tensor],
                  w_post: Optional[torch.Tensor], w_next: Optional[torch.Tensor],
                  x: Optional[torch.Tensor], eps_post: float = 0.0, eps_next: float = 0.0,
                  rows: Optional[torch.Tensor] = None, add_residual: bool = True) -> None:
    """The norm family in one launch.

    y None:  x = norm(h[rows]; w_next)               (rows optional)
    else:    b = y (summed over a leading split axis if y is 3-D);
             b = norm(b; w_post) if w_post; h += b if add_residual;
             x = norm(h or b; w_next) if w_next, else x = b if x is given.
    h is the 32-bit residual stream [R, H]; w_* are 32-bit and already hold
    1 + w where the norm is zero-centred.
    """
    _f32(h, "h"); _f32(w_post, "w_post"); _f32(w_next, "w_next"); _i32(rows, "rows")
    n_splits, split_stride, y_code = 1, 0, F32
    if y is not None:
        _dense(y, "y")
        y_code = dtype_code(y.dtype)
        if y.dim() == 3:
            n_splits, R, H = y.shape
            split_stride = R * H
        else:
            R, H = y.shape
    else:
        H = h.shape[-1]
        R = rows.numel() if rows is not None else h.shape[0]
    if h is not None:
        _dense(h, "h")
    x_code = F32
    if x is not None:
        _dense(x, "x")
        x_code = dtype_code(x.dtype)
        assert x.shape == (R, H), (x.shape, R, H)
    with _span("norm", _nbytes(y, x) + (R * H * 4 * (2 if y is not None and add_residual else 1)
                                         if h is not None else 0)):
        _check(library().agv_norm_residual(
            _ptr(h), _ptr(y), y_code, n_splits, ctypes.c_longlong(split_stride), _ptr(w_post),
            _ptr(w_next), _ptr(x), x_code, _ptr(rows), R, H, ctypes.c_float(eps_post),
            ctypes.c_float(eps_next), 1 if (add_residual and y is not None) else 0, _stream()))


def layer_norm_join(h: Optional[torch.Tensor], y: Optional[torch.Tensor],
                    w_post: Optional[torch.Tensor], b_post: Optional[torch.Tensor],
                    w_next: Optional[torch.Tensor], b_next: Optional[torch.Tensor],
                    x: Optional[torch.Tensor], eps_post: float = 0.0, eps_next: float = 0.0,
                    mult: float = 1.0, rows: Optional[torch.Tensor] = None,
                    add_residual: bool = True, rms: bool = False) -> None:
    """The layer-norm family in one launch (mean and variance, weight and bias).

    y None:  x = N(h[rows]; w_next, b_next)               (rows optional)
    else:    b = y (summed over a leading split axis if y is 3-D);
             b = N(b; w_post, b_post) if w_post; b *= mult; h += b if add_residual;
             x = N(h or b; w_next, b_next) if w_next, else x = b if x is given.
    h is the 32-bit residual stream [R, H]; weights and biases are 32-bit.  ``rms``: the
    mean is not taken off (an RMS norm with an optional bias and the multiplier)."""
    for t, n in ((h, "h"), (w_post, "w_post"), (b_post, "b_post"), (w_next, "w_next"),
                 (b_next, "b_next")):
        _f32(t, n)
    _i32(rows, "rows")
    n_splits, split_stride, y_code = 1, 0, F32
    if y is not None:
        _dense(y, "y")
        y_code = dtype_code(y.dtype)
        if y.dim() == 3:
            n_splits, R, H = y.shape
            split_stride = R * H
        else:
            R, H = y.shape
    else:
        H = h.shape[-1]
        R = rows.numel() if rows is not None else h.shape[0]
    if h is not None:
        _dense(h, "h")
    x_code = F32
    if x is not None:
        _dense(x, "x")
        x_code = dtype_code(x.dtype)
        assert x.shape == (R, H), (x.shape, R, H)
    with _span("norm", _nbytes(y, x) + (R * H * 4 * (2 if y is not None and add_residual else 1)
                                         if h is not None else 0)):
        _check(library().agv_layer_norm_join(
            _ptr(h), _ptr(y), y_code, n_splits, ctypes.c_longlong(split_stride), _ptr(w_post),
            _ptr(b_post), _ptr(w_next), _ptr(b_next), _ptr(x), x_code, _ptr(rows), R, H,
            ctypes.c_float(eps_post), ctypes.c_float(eps_next), ctypes.c_float(mult),
            1 if (add_residual and y is not None) else 0, 1 if rms else 0, _stream()))


def soft_cap(z: torch.Tensor, cap: float) -> None:
    """z <- cap * tanh(z / cap) in place (32-bit logits)."""
    _f32(z, "z"); _dense(z, "z")
    with _span("soft_cap", 2 * _nbytes(z)):
        _check(library().agv_soft_cap(_ptr(z), ctypes.c_longlong(z.numel()), ctypes.c_float(cap),
                                      _stream()))


# ------------------------------------------------------ routed feed-forward
def moe_route(x: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor],
              n_groups: int, keep: int, top: int, ids: torch.Tensor, wts: torch.Tensor,
              bias: Optional[torch.Tensor] = None, softmax_top: bool = False,
              softmax_all: bool = False, scale: float = 1.0) -> None:
    """ids, wts [T, top]: the experts each token of x [T, H] uses and their weights.
    s = sigmoid(W_r x) in 32-bit; s + correction chooses (only among the experts of the
    ``keep`` groups, of ``n_groups`` equal ones, whose two largest choice scores sum highest),
    s itself weighs.  ``bias`` [E] (32-bit) is added to the logits first; ``softmax_top``: the
    logits themselves choose and the weights are the softmax over the chosen logits;
    ``softmax_all``: s is the softmax over all the logits, s + correction chooses and the chosen
    s, divided by their sum (+ 1e-20) and times ``scale``, weigh."""
    T, H = x.shape
    E = w_router.shape[0]
    assert w_router.shape == (E, H) and x.stride(1) == 1 and x.dtype == w_router.dtype
    _dense(w_router, "w_router"); _f32(correction, "correction"); _i32(ids, "ids"); _f32(wts, "wts")
    _dense(ids, "ids"); _dense(wts, "wts"); _f32(bias, "bias")
    assert ids.shape == (T, top) and wts.shape == (T, top)
    assert bias is None or bias.shape == (E,)
    with _span("router", _nbytes(x, w_router), 2 * T * E * H):
        assert not (softmax_top and softmax_all)
        _check(library().agv_moe_route_mode(
            _ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(w_router), _ptr(correction), _ptr(bias),
            2 if softmax_all else 1 if softmax_top else 0, ctypes.c_float(scale),
            dtype_code(x.dtype), T, H, E, n_groups, keep, top, _ptr(ids), _ptr(wts), _stream()))


def moe_identity(x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, n_experts: int,
                 y: torch.Tensor) -> None:
    """For every (token, choice) pair whose id is at or beyond ``n_experts`` (an identity
    expert): y[choice, token, :] = weight * x[token, :]; y [top, T, H] 32-bit.  The other rows
    are the experts' to write."""
    T, H = x.shape
    top = ids.shape[1]
    _i32(ids, "ids"); _f32(wts, "wts"); _f32(y, "y"); _dense(ids, "ids"); _dense(wts, "wts")
    _dense(y, "y")
    assert x.stride(1) == 1 and ids.shape == wts.shape == (T, top) and y.shape == (top, T, H)
    with _span("experts_identity", _nbytes(x)):
        _check(library().agv_moe_identity(_ptr(x), ctypes.c_longlong(x.stride(0)),
                                          dtype_code(x.dtype), _ptr(ids), _ptr(wts), T, top,
                                          n_experts, H, _ptr(y), _stream()))


def gelu_mul_rows(z: torch.Tensor, e: torch.Tensor, out: torch.Tensor) -> None:
    """out [T, n] = gelu_tanh(z [T, n]) * e [T, n]; e is 32-bit and may be a column slice of a
    wider tensor."""
    T, n = z.shape
    _f32(e, "e"); _dense(z, "z"); _dense(out, "out")
    assert e.shape == (T, n) and e.stride(1) == 1 and out.shape == (T, n)
    with _span("token_side_gate", _nbytes(z, out) + T * n * 4):
        _check(library().agv_gelu_mul_rows(_ptr(z), dtype_code(z.dtype), _ptr(e),
                                           ctypes.c_longlong(e.stride(0)), _ptr(out),
                                           dtype_code(out.dtype), T, n, _stream()))


def row_gate(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y [T, H] (32-bit) *= sigmoid(x[t, :] . w) row by row: one gate value per token."""
    T, K = x.shape
    assert w.numel() == K and w.dtype == x.dtype and x.stride(1) == 1
    _f32(y, "y"); _dense(y, "y"); _dense(w, "w")
    assert y.shape[0] == T and y.dim() == 2
    with _span("gate", 2 * _nbytes(y) + _nbytes(x)):
        _check(library().agv_row_gate(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(w),
                                      dtype_code(x.dtype), _ptr(y), T, K, y.shape[1], _stream()))


class MoePlan:
    """Where the (token, choice) pairs of a step lie once sorted by expert (device arrays;
    see ``csrc/moe.cu``)."""
    __slots__ = ("T", "top", "E", "tile", "rows", "tiles", "tok", "dst", "wpos", "pos_of", "tile_e")


def moe_plan(ids: torch.Tensor, wts: torch.Tensor, n_experts: int, tile: int = 0) -> MoePlan:
    """``tile``: rows per tile, 64 or 128 (0: 128 where an expert gets some hundred rows on
    average, so that padding every expert's run to the tile costs little, else 64)."""
    T, top = ids.shape
    lib = library()
    p = MoePlan()
    p.T, p.top, p.E = T, top, n_experts
    p.tile = tile or (128 if T * top >= 96 * n_experts else 64)
    p.rows = lib.agv_moe_plan_rows(T, top, n_experts, p.tile)
    p.tiles = lib.agv_moe_plan_tiles(T, top, n_experts, p.tile)
    dev = ids.device
    ints = torch.empty(2 * p.rows + T * top + p.tiles, dtype=torch.int32, device=dev)
    p.tok, p.dst = ints[:p.rows], ints[p.rows:2 * p.rows]
    p.pos_of = ints[2 * p.rows:2 * p.rows + T * top]
    p.tile_e = ints[2 * p.rows + T * top:]
    p.wpos = torch.empty(p.rows, dtype=torch.float32, device=dev)
    _check(lib.agv_moe_plan(_ptr(ids), _ptr(wts), T, top, n_experts, p.tile, _ptr(p.tok), _ptr(p.dst),
                            _ptr(p.wpos), _ptr(p.pos_of), _ptr(p.tile_e), _stream()))
    return p


def moe_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan: MoePlan,
                w2: Optional[torch.Tensor] = None, activation: str = "silu",
                gather: bool = False, scatter: bool = False, op: str = "experts") -> None:
    """The experts' product over a plan: out[pos] = a[row(pos)] w[e(pos)]^T, or with w2 the
    gated pair.  w, w2: [E, N, K].  ``gather``: a's rows are tokens (row = the pair's token),
    else sorted positions.  ``scatter``: out is [top * T, N] and a pair's row, times its
    weight, goes to [choice * T + token]; else out's rows are sorted positions."""
    E, N, K = w.shape
    _dense(w, "w")
    assert a.stride(1) == 1 and out.stride(1) == 1 and a.shape[1] == K and out.shape[1] == N
    assert a.dtype == w.dtype
    if w2 is not None:
        _dense(w2, "w2")
        assert w2.shape == w.shape and w2.dtype == w.dtype
    pairs = plan.T * plan.top
    n = 2 if w2 is not None else 1
    with _span(op, n * min(E, pairs) * N * K * w.element_size() + pairs * (K + N) * a.element_size(),
               2 * n * pairs * N * K):
        _check(library().agv_moe_grouped(
            _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(plan.tok) if gather else None,
            _ptr(plan.tok), _ptr(w), _ptr(w2), _ptr(out), ctypes.c_longlong(out.stride(0)),
            _ptr(plan.dst) if scatter else None, _ptr(plan.wpos) if scatter else None,
            _ptr(plan.tile_e), plan.tiles, plan.tile, N, K, dtype_code(a.dtype),
            dtype_code(out.dtype), ACT[activation], _stream()))


def moe_grouped_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``moe_grouped_tc`` takes these operands: bfloat16, K and the row stride
    multiples of 8, 16-byte aligned."""
    return (_MOE_TC and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and
            w.shape[2] % 8 == 0 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and
            w.data_ptr() % 16 == 0)


_MOE_TC = os.environ.get("AGAVE_B200_MOE_TENSOR_CORES", "1") != "0"


def moe_gather_rows(x: torch.Tensor, plan: MoePlan, xs: torch.Tensor) -> None:
    """xs [plan.rows, H] = the rows of x [T, H] in the plan's sorted order (zeros where the
    plan pads), bfloat16."""
    T, H = x.shape
    assert x.dtype == torch.bfloat16 and xs.dtype == torch.bfloat16 and x.stride(1) == 1
    _dense(xs, "xs")
    assert xs.shape == (plan.rows, H)
    with _span("experts_gather", _nbytes(xs) * 2):
        _check(library().agv_moe_gather_rows(_ptr(x), ctypes.c_longlong(x.stride(0)),
                                             _ptr(plan.tok), _ptr(xs), plan.rows, H, _stream()))


def moe_grouped_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan: MoePlan,
                   w2: Optional[torch.Tensor] = None, activation: str = "silu",
                   scatter: bool = False, op: str = "experts") -> None:
    """``moe_grouped`` in bfloat16 on the tensor cores; a's rows are sorted positions
    ([plan.rows, K]).  Gated: out [plan.rows, N] bfloat16.  Plain: out 32-bit, with
    ``scatter`` [top * T, N] rows at [choice * T + token] times the pair's weight."""
    E, N, K = w.shape
    _dense(w, "w")
    assert a.shape == (plan.rows, K) and a.stride(1) == 1 and out.stride(1) == 1
    assert out.shape[1] == N and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if w2 is not None:
        _dense(w2, "w2")
        assert w2.shape == w.shape and w2.dtype == w.dtype and out.dtype == torch.bfloat16
        assert not scatter and out.shape[0] == plan.rows
    else:
        assert out.dtype == torch.float32
    pairs = plan.T * plan.top
    n = 2 if w2 is not None else 1
    with _span(op, n * min(E, pairs) * N * K * 2 + pairs * (K + N) * 2, 2 * n * pairs * N * K):
        _check(library().agv_moe_grouped_tc(
            _ptr(a), ctypes.c_longlong(a.stride(0)), plan.rows, _ptr(plan.tok), _ptr(w), _ptr(w2),
            E, _ptr(out), ctypes.c_longlong(out.stride(0)), _ptr(plan.dst) if scatter else None,
            _ptr(plan.wpos) if scatter else None, _ptr(plan.tile_e), plan.tiles, plan.tile, N, K,
            ACT[activation], _stream()))


def moe_tc_status() -> int:
    """0, or the code of the first bounded wait of the grouped tensor-core kernel that gave
    up since the last call (this call synchronises the device)."""
    torch.cuda.synchronize()
    return library().agv_moe_tc_status()


# ------------------------------------------------------------ matrix products
def _linear_cost(x, w, w2, out):
    """(bytes, flops) of a projection: weights and operands once, 2 T N K flops."""
    T, K = x.shape
    N = w.shape[0]
    n = 2 if w2 is not None else 1
    return (n * N * K * w.element_size() + T * K * x.element_size() + _nbytes(out),
            2 * n * T * N * K)


def linear_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                w2: Optional[torch.Tensor] = None, activation: str = "gelu_tanh",
                op: str = "linear") -> None:
    """out = x w^T, or act(x w^T) * (x w2^T); FFMA kernel (the 32-bit path)."""
    M, K = x.shape
    N = w.shape[0]
    assert w.shape == (N, K) and out.shape == (M, N)
    assert x.stride(1) == 1 and out.stride(1) == 1
    _dense(w, "w")
    if w2 is not None:
        _dense(w2, "w2")
        assert w2.shape == w.shape and w2.dtype == w.dtype
    if x.dtype != w.dtype:
        raise KernelError(f"linear: input {x.dtype} and weight {w.dtype} differ")
    with _span(op, *_linear_cost(x, w, w2, out)):
        _check(library().agv_linear_simt(
            _ptr(x), _ptr(w), _ptr(w2), _ptr(out), M, N, K, ctypes.c_longlong(x.stride(0)),
            ctypes.c_longlong(out.stride(0)), dtype_code(x.dtype), dtype_code(out.dtype),
            ACT[activation], _stream()))


# ------------------------------------------------------------------ attention
def qk_norm_rope_store(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                       wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                       positions: Optional[torch.Tensor],
                       k_pool: Optional[torch.Tensor] = None, v_pool: Optional[torch.Tensor] = None,
                       page_table: Optional[torch.Tensor] = None,
                       slots: Optional[torch.Tensor] = None, lens: Optional[torch.Tensor] = None,
                       seq_index: Optional[torch.Tensor] = None, page: int = 0,
                       cap: int = 0, partial: Optional[torch.Tensor] = None,
                       vt: Optional[torch.Tensor] = None, cu_seqlens: Optional[torch.Tensor] = None,
                       max_len: int = 0, value_dim: int = 0, q_temp=None) -> None:
    """In place on qkv [T, (nh + 2 nkv) * hd]: per-head norm of q and k, rotation,
    and (if pools are given) the store of k and v rows into the paged cache.
    ``partial`` [S, T, (nh + 2 nkv) * hd] (32-bit partial sums of the projection)
    replaces qkv as the input; qkv then only receives the result.  ``vt`` (from
    ``prefill_values_scratch``) also receives the values transposed, for the prompt
    attention; that needs seq_index, positions, cu_seqlens and the greatest length.
    ``value_dim``: the size of a v head where it differs from head_dim (the row is then
    nh * hd + nkv * hd + nkv * value_dim wide); n_kv_heads may be 0 (queries alone).
    ``q_temp`` = (coef, every): every q head is multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1) at position p."""
    T = qkv.shape[0]
    n_splits = 0
    hdv = value_dim or head_dim
    if partial is not None:
        _f32(partial, "partial"); _dense(partial, "partial")
        assert partial.dim() == 3 and partial.shape[1] == T
        assert partial.shape[2] == (n_heads + n_kv_heads) * head_dim + n_kv_heads * hdv
        n_splits = partial.shape[0]
    assert qkv.stride(1) == 1
    _f32(wq, "wq"); _f32(wk, "wk"); _f32(cos, "cos"); _f32(sin, "sin")
    for t, n in ((positions, "positions"), (page_table, "page_table"), (slots, "slots"),
                 (lens, "lens"), (seq_index, "seq_index")):
        _i32(t, n)
    if k_pool is not None:
        _dense(k_pool, "k_pool"); _dense(v_pool, "v_pool")
        assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype
    max_pages = page_table.shape[1] if page_table is not None else 0
    n_seq = 0
    if vt is not None:
        _dense(vt, "vt"); _i32(cu_seqlens, "cu_seqlens")
        assert vt.dtype == torch.bfloat16 and vt.shape[0] == n_kv_heads * head_dim
        n_seq = cu_seqlens.numel() - 1
    with _span("qk_norm_rope", 2 * _nbytes(qkv) + _nbytes(partial, vt)):
        coef, every = q_temp if q_temp is not None else (0.0, 1)
        _check(library().agv_qk_norm_rope_store_ex(
            _ptr(qkv), dtype_code(qkv.dtype), ctypes.c_longlong(qkv.stride(0)), _ptr(partial),
            n_splits, T, n_heads, n_kv_heads, head_dim, _ptr(wq), _ptr(wk), ctypes.c_float(eps),
            _ptr(cos), _ptr(sin), rotary_dim, _ptr(positions), _ptr(k_pool), _ptr(v_pool),
            _ptr(page_table), _ptr(slots), _ptr(lens), _ptr(seq_index), max_pages, page, cap,
            _ptr(vt), ctypes.c_longlong(vt.shape[1] if vt is not None else 0), _ptr(cu_seqlens),
            n_seq, max_len, hdv, ctypes.c_float(coef), int(every), _stream()))


_FUSED_QKV = os.environ.get("AGAVE_B200_FUSED_QKV_PREFILL", "1") != "0"


def qkv_prefill_supported(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int) -> bool:
    """Whether ``qkv_prefill`` takes a prompt step of these sizes: bfloat16 on the tensor
    cores, head sizes 64, 128 or 256 rotated whole or not at all, and enough tiles (128
    tokens x 256 weight rows) that a CTA works on several: the epilogue of one tile then
    runs under the products of the next.  With about one tile per CTA it is exposed, and
    the plain product followed by the norm / rotation / store kernel, whose thousands of
    warps hide their memory trips, is faster (1B sizes, 2,048 tokens: 149 against 156 us a
    layer; 4B: 441 against 433; 27B: 1,624 against 1,612).  ``AGAVE_B200_FUSED_QKV_PREFILL``
    = 0 turns it off, = 2 takes it whenever the sizes allow."""
    if not _FUSED_QKV or x.shape[0] <= 128 or not linear_tc_supported(x, w):
        return False
    tiles = ((w.shape[0] + 255) // 256) * ((x.shape[0] + 127) // 128)
    if tiles * 2 < 3 * n_sms() and os.environ.get("AGAVE_B200_FUSED_QKV_PREFILL") != "2":
        return False
    return (bool(
        library().agv_qkv_prefill_tc_supported(head_dim, rotary_dim, w.shape[1],
                                               ctypes.c_longlong(x.stride(0)),
                                               ctypes.c_longlong(w.shape[0]))))


def qkv_prefill(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, n_heads: int, n_kv_heads: int,
                head_dim: int, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
                cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                positions: torch.Tensor, seq_index: torch.Tensor,
                k_pool: Optional[torch.Tensor] = None, v_pool: Optional[torch.Tensor] = None,
                page_table: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                lens: Optional[torch.Tensor] = None, page: int = 0, cap: int = 0,
                vt: Optional[torch.Tensor] = None, cu_seqlens: Optional[torch.Tensor] = None) -> None:
    """qkv [T, (nh + 2 nkv) * hd] = x w^T with the per-head norm of q and k, the rotation, the
    store of k and v into the paged cache (if pools are given) and the transposed copy of
    the values (if ``vt`` is given) all done in the product's epilogue."""
    T, K = x.shape
    N = (n_heads + 2 * n_kv_heads) * head_dim
    assert w.shape == (N, K) and qkv.shape == (T, N) and qkv.dtype == torch.bfloat16
    assert x.stride(1) == 1 and qkv.stride(1) == 1
    _dense(w, "w")
    _f32(wq, "wq"); _f32(wk, "wk"); _f32(cos, "cos"); _f32(sin, "sin")
    for t, n in ((positions, "positions"), (page_table, "page_table"), (slots, "slots"),
                 (lens, "lens"), (seq_index, "seq_index"), (cu_seqlens, "cu_seqlens")):
        _i32(t, n)
    if cos is not None:
        _dense(cos, "cos"); _dense(sin, "sin")
        assert cos.shape == (T, head_dim // 2)
    if k_pool is not None:
        _dense(k_pool, "k_pool"); _dense(v_pool, "v_pool")
        assert k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16
    if vt is not None:
        _dense(vt, "vt")
        assert vt.dtype == torch.bfloat16 and vt.shape[0] == n_kv_heads * head_dim
    max_pages = page_table.shape[1] if page_table is not None else 0
    with _span("qkv", *_linear_cost(x, w, None, qkv)):
        _check(library().agv_qkv_prefill_tc(
            _ptr(x), _ptr(w), T, K, ctypes.c_longlong(x.stride(0)), _ptr(qkv),
            ctypes.c_longlong(qkv.stride(0)), n_heads, n_kv_heads, head_dim, _ptr(wq), _ptr(wk),
            ctypes.c_float(eps), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(k_pool), _ptr(v_pool),
            _ptr(page_table), _ptr(slots), _ptr(lens), _ptr(seq_index), max_pages, page, cap,
            _ptr(vt), ctypes.c_longlong(vt.shape[1] if vt is not None else 0), _ptr(cu_seqlens),
            _stream()))


def attention_prefill_simt(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                           positions: torch.Tensor, seq_index: torch.Tensor,
                           cu_seqlens: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                           scale: float, window: int, value_dim: int = 0,
                           sinks: Optional[torch.Tensor] = None,
                           dist_bias: Optional[torch.Tensor] = None,
                           keep_first: int = 0) -> None:
    """Prompts that start at 0; q [T, nh*hd], k [T, nkv*hd], v [T, nkv*hdv] row-strided
    views (hdv = value_dim or head_dim), out [T, nh*hdv]; ``sinks`` [nh]: a logit per query
    head that joins its softmax denominator once; ``dist_bias`` [nh, n]: added to the scaled
    score of a key at distance min(t - j, n - 1)."""
    T = q.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
    _dense(out, "out"); _f32(sinks, "sinks"); _f32(dist_bias, "dist_bias")
    if dist_bias is not None:
        _dense(dist_bias, "dist_bias")
        assert dist_bias.dim() == 2 and dist_bias.shape[0] == n_heads
    _i32(positions, "positions"); _i32(seq_index, "seq_index"); _i32(cu_seqlens, "cu_seqlens")
    _check(library().agv_attention_prefill_simt_ex(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(k), _ptr(v),
        ctypes.c_longlong(k.stride(0)), _ptr(out), dtype_code(q.dtype), _ptr(positions),
        _ptr(seq_index), _ptr(cu_seqlens), T, n_heads, n_kv_heads, head_dim,
        ctypes.c_float(scale), window, value_dim or head_dim, ctypes.c_longlong(v.stride(0)),
        _ptr(sinks), _ptr(dist_bias), dist_bias.shape[1] if dist_bias is not None else 0,
        int(keep_first), _stream()))


def attention_paged_simt(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor,
                         v_pool: torch.Tensor, page_table: torch.Tensor, slots: torch.Tensor,
                         positions: torch.Tensor, seq_index: torch.Tensor, page: int, cap: int,
                         n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                         window: int, value_dim: int = 0,
                         sinks: Optional[torch.Tensor] = None,
                         dist_bias: Optional[torch.Tensor] = None, v_row: int = 0,
                         keep_first: int = 0) -> None:
    """Queries against the paged cache; their own keys are already stored.  ``v_row``: the
    elements between two positions' value rows where that is not nkv * hdv (values that are
    the leading part of the key rows: v_pool is then k_pool)."""
    T = q.shape[0]
    assert q.stride(1) == 1
    _f32(sinks, "sinks"); _f32(dist_bias, "dist_bias")
    if dist_bias is not None:
        _dense(dist_bias, "dist_bias")
        assert dist_bias.dim() == 2 and dist_bias.shape[0] == n_heads
    _dense(out, "out"); _dense(k_pool, "k_pool"); _dense(v_pool, "v_pool")
    for t, n in ((positions, "positions"), (page_table, "page_table"), (slots, "slots"),
                 (seq_index, "seq_index")):
        _i32(t, n)
    assert k_pool.dtype == q.dtype
    _check(library().agv_attention_paged_simt_ex(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(out), dtype_code(q.dtype), _ptr(k_pool),
        _ptr(v_pool), _ptr(page_table), _ptr(slots), _ptr(positions), _ptr(seq_index),
        page_table.shape[1], page, cap, T, n_heads, n_kv_heads, head_dim,
        ctypes.c_float(scale), window, value_dim or head_dim, _ptr(sinks), _ptr(dist_bias),
        dist_bias.shape[1] if dist_bias is not None else 0, int(v_row), int(keep_first),
        _stream()))


# ------------------------------------------- rows of stacked projections, latent attention
def _cache_args(view, ctx):
    if view is None:
        return [ctypes.c_void_p(0)] * 6 + [0, 0, 0]
    return [_ptr(view.k_pool), _ptr(view.v_pool), _ptr(view.page_table), _ptr(ctx.slots),
            _ptr(ctx.lens), _ptr(ctx.seq_index), view.page_table.shape[1], view.page, view.cap]


def _row_input(row, partial, T, W):
    """(row pointer, row stride, partial pointer, n_splits) of a stacked projection's output:
    [T, W] in the compute dtype, or [S, T, W] 32-bit partial sums."""
    if partial is not None:
        _f32(partial, "partial"); _dense(partial, "partial")
        assert partial.dim() == 3 and partial.shape[1:] == (T, W)
        return ctypes.c_void_p(0), 0, _ptr(partial), partial.shape[0]
    assert row.shape == (T, W) and row.stride(1) == 1
    return _ptr(row), row.stride(0), ctypes.c_void_p(0), 0


def proj_norm_store(out: torch.Tensor, nq: int, nk: int, nv: int, wq: torch.Tensor,
                    wk: torch.Tensor, eps: float, positions: torch.Tensor, view=None, ctx=None,
                    partial: Optional[torch.Tensor] = None,
                    v_first: Optional[torch.Tensor] = None, v_mix: float = 0.0) -> None:
    """out [T, nq + nk + nv] = q | k | v of a stacked projection with q and k each RMS-normed
    over their whole width (weights wq [nq], wk [nk], 32-bit); the input is ``partial``
    ([S, T, W] 32-bit partial sums) or out itself.  With ``view`` (a cache entry's pools) the
    k and v parts also go to the cache rows of the tokens' positions.  With ``v_first``
    [T, nv] (rows of another tensor) the values become (1 - v_mix) v + v_mix v_first."""
    T, W = out.shape
    assert W == nq + nk + nv and out.stride(1) == 1
    _f32(wq, "wq"); _f32(wk, "wk"); _i32(positions, "positions")
    rp, ld, pp, ns = _row_input(out, partial, T, W)
    cache = _cache_args(view, ctx)
    if view is not None:
        assert view.k_pool.dtype == out.dtype
    if v_first is not None:
        assert v_first.shape == (T, nv) and v_first.stride(1) == 1 and v_first.dtype == out.dtype
    with _span("qk_norm_rope", 2 * _nbytes(out) + _nbytes(partial)):
        _check(library().agv_proj_norm_store(
            rp, ctypes.c_longlong(ld), pp, ns, _ptr(out), ctypes.c_longlong(out.stride(0)),
            dtype_code(out.dtype), T, nq, nk, nv, _ptr(wq), _ptr(wk), ctypes.c_float(eps),
            _ptr(positions), *cache, _ptr(v_first),
            ctypes.c_longlong(v_first.stride(0) if v_first is not None else 0),
            ctypes.c_float(v_mix), _stream()))


def latent_prepare(out: torch.Tensor, q_width: int, q_latent: bool, heads: int, d: int, r: int,
                   R: int, G: int, w_q: Optional[torch.Tensor], w_c: torch.Tensor, eps: float,
                   cos: torch.Tensor, sin: torch.Tensor, interleaved: bool,
                   positions: torch.Tensor, view=None, ctx=None,
                   partial: Optional[torch.Tensor] = None) -> None:
    """out [T, q_width + R + r + G] = Q | c | kr | g of a latent-attention mixer's stacked
    projection: c RMS-normed (w_c [R]), kr rotated by position, c | kr stored as the cache row
    (``view``), g passed through, and Q either normed as a latent (``q_latent``, w_q
    [q_width]) or, as [heads, d + r], with the last r of every head rotated."""
    T, W = out.shape
    assert W == q_width + R + r + G and out.stride(1) == 1
    _f32(w_q, "w_q"); _f32(w_c, "w_c"); _f32(cos, "cos"); _f32(sin, "sin")
    _i32(positions, "positions"); _dense(cos, "cos"); _dense(sin, "sin")
    assert cos.shape == (T, r // 2) and sin.shape == cos.shape
    rp, ld, pp, ns = _row_input(out, partial, T, W)
    cache = _cache_args(view, ctx)
    if view is not None:
        assert view.k_pool.dtype == out.dtype and view.k_pool.shape[-1] * view.k_pool.shape[-2] == R + r
    del cache[1]                                 # one pool: the latent rows
    with _span("qk_norm_rope", 2 * _nbytes(out) + _nbytes(partial)):
        _check(library().agv_latent_prepare(
            rp, ctypes.c_longlong(ld), pp, ns, _ptr(out), ctypes.c_longlong(out.stride(0)),
            dtype_code(out.dtype), T, q_width, 1 if q_latent else 0, heads, d, r, R, G,
            _ptr(w_q), _ptr(w_c), ctypes.c_float(eps), _ptr(cos), _ptr(sin),
            1 if interleaved else 0, _ptr(positions), *cache, _stream()))


def rotate_heads(x: torch.Tensor, heads: int, head_width: int, r: int, cos: torch.Tensor,
                 sin: torch.Tensor, interleaved: bool) -> None:
    """x [T, heads * head_width] in place: the last r of every head rotated by the tables."""
    T = x.shape[0]
    assert x.shape[1] == heads * head_width and x.stride(1) == 1
    _f32(cos, "cos"); _f32(sin, "sin"); _dense(cos, "cos"); _dense(sin, "sin")
    assert cos.shape == (T, r // 2)
    with _span("qk_norm_rope", 2 * T * heads * r * x.element_size()):
        _check(library().agv_rotate_heads(_ptr(x), ctypes.c_longlong(x.stride(0)),
                                          dtype_code(x.dtype), T, heads, head_width, r, _ptr(cos),
                                          _ptr(sin), 1 if interleaved else 0, _stream()))


def assemble_keys(k_plain: torch.Tensor, kr: torch.Tensor, k_out: torch.Tensor, heads: int,
                  d: int, r: int) -> None:
    """k_out [T, heads * (d + r)]: head a is k_plain[t, a * d:(a + 1) * d] followed by kr[t]."""
    T = k_out.shape[0]
    assert k_plain.shape == (T, heads * d) and kr.shape == (T, r) and k_out.shape[1] == heads * (d + r)
    assert k_plain.stride(1) == 1 and kr.stride(1) == 1 and k_plain.dtype == kr.dtype == k_out.dtype
    _dense(k_out, "k_out")
    with _span("qk_norm_rope", 2 * _nbytes(k_out)):
        _check(library().agv_assemble_keys(_ptr(k_plain), ctypes.c_longlong(k_plain.stride(0)),
                                           _ptr(kr), ctypes.c_longlong(kr.stride(0)), _ptr(k_out),
                                           dtype_code(k_out.dtype), T, heads, d, r, _stream()))


def heads_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tail: int = 0,
                 gate: Optional[torch.Tensor] = None, op: str = "heads_linear") -> None:
    """out[t, a, :N] = w[a] x[t, a, :K]: x [T, heads, K + tail] and out [T, heads, N + tail] are
    views with unit innermost stride, w [heads, N, K] dense; out in x's dtype or 32-bit.  The
    ``tail`` values behind a head's inputs are copied behind its outputs.  ``gate`` [T, heads]
    or [T, heads * N]: every output is multiplied by the sigmoid of its (head's) logit."""
    T, A, K = x.shape
    K -= tail
    N = w.shape[1]
    assert w.shape == (A, N, K) and out.shape == (T, A, N + tail) and x.dtype == w.dtype
    assert x.stride(2) == 1 and out.stride(2) == 1
    _dense(w, "w")
    out_f32 = out.dtype == torch.float32 and x.dtype != torch.float32
    assert out_f32 or out.dtype == x.dtype
    per_head = 0
    if gate is not None:
        assert gate.shape in ((T, A), (T, A * N)) and gate.stride(1) == 1 and gate.dtype == x.dtype
        per_head = 1 if gate.shape[1] == A and N != 1 else 0
    with _span(op, _nbytes(w, x, out), 2 * T * A * N * K):
        _check(library().agv_heads_linear(
            _ptr(x), ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(x.stride(1)), _ptr(w),
            _ptr(out), ctypes.c_longlong(out.stride(0)), ctypes.c_longlong(out.stride(1)),
            dtype_code(x.dtype), 1 if out_f32 else 0, T, A, N, K, int(tail), _ptr(gate),
            ctypes.c_longlong(gate.stride(0) if gate is not None else 0), per_head, _stream()))


def gate_sigmoid(out: torch.Tensor, g: torch.Tensor) -> None:
    """out [T, n] *= sigmoid(g [T, m]) in place; each g value covers n / m neighbours."""
    T, n = out.shape
    m = g.shape[1]
    assert g.shape[0] == T and n % m == 0 and out.stride(1) == 1 and g.stride(1) == 1
    assert out.dtype == g.dtype
    with _span("gate", 2 * _nbytes(out) + _nbytes(g)):
        _check(library().agv_gate_sigmoid(_ptr(out), ctypes.c_longlong(out.stride(0)), _ptr(g),
                                          ctypes.c_longlong(g.stride(0)), dtype_code(out.dtype),
                                          T, n, n // m, _stream()))


def relu2(z: torch.Tensor) -> None:
    """z <- max(z, 0)^2 in place."""
    _dense(z, "z")
    with _span("activation", 2 * _nbytes(z)):
        _check(library().agv_relu2(_ptr(z), ctypes.c_longlong(z.numel()), dtype_code(z.dtype),
                                   _stream()))


def linear_activated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, activation: str,
                     op: str = "linear") -> None:
    """out = act(x w^T); "relu2" is the squared relu, "gelu_erf" the erf GELU."""
    if activation not in ("relu2", "gelu_erf"):
        raise KernelError(f"linear_activated: unknown activation {activation!r}")
    # the activation is the product's epilogue, where the sum is finished: one range of K, or
    # (decoding through a layer with few row tiles) the ranges of one cluster
    if linear_tc_supported(x, w) and out.dtype == torch.bfloat16:
        c = 0
        if x.shape[0] <= 16:
            tiles, kb, sms = (w.shape[0] + 127) // 128, (w.shape[1] + 63) // 64, n_sms()
            c = 4 if tiles * 4 <= sms and kb >= 8 else 2 if tiles * 2 <= sms and kb >= 4 else 0
        linear_tc(x, w, out, None, activation, splits=max(c, 1), cluster=c, op=op)
    else:
        linear_simt(x, w, out, None, activation, op=op)


# ------------------------------------------------------- gated delta rule
def _state_args(state: torch.Tensor):
    """(pointer, row stride) of a fixed-size state [n_slots, numel]."""
    _f32(state, "state")
    assert state.dim() == 2 and state.stride(1) == 1
    return _ptr(state), ctypes.c_longlong(state.stride(0))


def delta_prepare(row: Optional[torch.Tensor], partial: Optional[torch.Tensor], T: int, ctx,
                  state: torch.Tensor, conv_off: int, n_qk_heads: int, n_heads: int,
                  head_dim: int, value_dim: int, taps: int, decay_rank: int, gate_rank: int,
                  conv_w: torch.Tensor, unit_eps: float, q_mult: float, qkv: torch.Tensor,
                  beta: torch.Tensor, low_a: torch.Tensor, low_g: torch.Tensor) -> None:
    """From a token's row  q | k | v | b | a1 | g1  of the stacked projection ([T, W] in the
    compute dtype or ``partial`` [S, T, W] 32-bit sums): the causal convolution over ``taps``
    tokens and silu on q, k and v (its earlier inputs come from the step's rows or, before
    the step, from ``state`` at ``conv_off``, which is brought up to date), unit q and k heads
    (q times ``q_mult``), beta = sigmoid(b).  qkv [T, 2 G d + H dv] and beta [T, H] are 32-bit;
    low_a [T, ra] and low_g [T, rg] are the two bottlenecks in the compute dtype."""
    C = 2 * n_qk_heads * head_dim + n_heads * value_dim
    W = C + n_heads + decay_rank + gate_rank
    rp, ld, pp, ns = _row_input(row, partial, T, W)
    _f32(conv_w, "conv_w"); _dense(conv_w, "conv_w"); _f32(qkv, "qkv"); _f32(beta, "beta")
    _dense(qkv, "qkv"); _dense(beta, "beta"); _dense(low_a, "low_a"); _dense(low_g, "low_g")
    assert conv_w.shape == (C, taps) and qkv.shape == (T, C) and beta.shape == (T, n_heads)
    assert low_a.shape == (T, decay_rank) and low_g.shape == (T, gate_rank)
    dt = low_a.dtype
    assert low_g.dtype == dt and (row is None or row.dtype == dt)
    sp, ss = _state_args(state)
    with _span("delta_prepare", _nbytes(row, partial, qkv, beta, low_a, low_g)):
        _check(library().agv_delta_prepare(
            rp, ctypes.c_longlong(ld), pp, ns, dtype_code(dt), T, ctx.batch, n_qk_heads, n_heads,
            head_dim, value_dim, taps, decay_rank, gate_rank, _ptr(conv_w),
            ctypes.c_float(unit_eps), ctypes.c_float(q_mult), sp, ss, ctypes.c_longlong(conv_off),
            _ptr(ctx.slots), _ptr(ctx.cu_seqlens), _ptr(ctx.seq_index), _ptr(ctx.positions),
            0 if ctx.mode == "decode" else 1, _ptr(qkv), _ptr(beta), _ptr(low_a), _ptr(low_g),
            _stream()))


def delta_scan(qkv: torch.Tensor, beta: torch.Tensor, a: torch.Tensor, dt_bias: torch.Tensor,
               neg_a: torch.Tensor, out: torch.Tensor, ctx, state: torch.Tensor,
               n_qk_heads: int, n_heads: int, head_dim: int, value_dim: int) -> None:
    """The recurrence  S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q  over the
    step's tokens, sequence by sequence, with g = exp(neg_a[h] * softplus(a + dt_bias)); S
    [H, dv, d] of each sequence is read from and written to ``state``.  All 32-bit."""
    T = qkv.shape[0]
    for t, n in ((qkv, "qkv"), (beta, "beta"), (a, "a"), (dt_bias, "dt_bias"), (neg_a, "neg_a"),
                 (out, "out")):
        _f32(t, n); _dense(t, n)
    assert a.shape == (T, n_heads * head_dim) and out.shape == (T, n_heads * value_dim)
    assert dt_bias.numel() == n_heads * head_dim and neg_a.numel() == n_heads
    sp, ss = _state_args(state)
    flops = 6 * T * n_heads * head_dim * value_dim
    lib = library()
    lib.agv_delta_scan_work.restype = ctypes.c_longlong
    # scratch for what does not depend on the state (k, the decay, their products), per head
    work = ctx.new(int(lib.agv_delta_scan_work(T, n_heads, head_dim)), dtype=torch.float32)
    with _span("delta_scan", _nbytes(qkv, beta, a, out) + 2 * work.numel() * 4, flops):
        _check(lib.agv_delta_scan(_ptr(qkv), _ptr(beta), _ptr(a), _ptr(dt_bias), _ptr(neg_a),
                                  _ptr(out), T, ctx.batch, n_qk_heads, n_heads, head_dim,
                                  value_dim, sp, ss, _ptr(ctx.slots), _ptr(ctx.cu_seqlens),
                                  _ptr(work), _stream()))


def delta_out(o: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, eps: float, n_heads: int,
              value_dim: int, ctx, y: torch.Tensor) -> None:
    """y[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * sigmoid(gate[t, h, :]); o and gate are
    32-bit [T, H * dv], y is in the compute dtype."""
    T = o.shape[0]
    _f32(o, "o"); _f32(gate, "gate"); _f32(w, "w"); _dense(o, "o"); _dense(gate, "gate")
    _dense(y, "y")
    assert o.shape == gate.shape == y.shape == (T, n_heads * value_dim) and w.numel() == value_dim
    with _span("delta_out", _nbytes(o, gate, y)):
        _check(library().agv_delta_out(_ptr(o), _ptr(gate), _ptr(w), ctypes.c_float(eps), T,
                                       n_heads, value_dim, _ptr(ctx.seq_index), _ptr(ctx.slots),
                                       _ptr(y), dtype_code(y.dtype), _stream()))



# ------------------------------------------------------- matrix memory (mLSTM)
def mlstm_state_numel(n_heads: int, head_dim: int, value_dim: int) -> int:
    """32-bit values a sequence's matrix memory takes: S [H, d, dv], n [H, d] and the running
    maximum m, of which every eight columns of a head keep a copy [H, ceil(dv / 8)] (the CTAs
    of the scan take multiples of eight columns and none reads what another writes)."""
    return (n_heads * head_dim * value_dim + n_heads * head_dim +
            n_heads * ((value_dim + 7) // 8))


def _f32_row_input(row, partial, T, W):
    """(row pointer, stride, partial pointer, n_splits) of a 32-bit stacked projection."""
    if partial is not None:
        _f32(partial, "partial"); _dense(partial, "partial")
        assert partial.dim() == 3 and partial.shape[1:] == (T, W)
        return ctypes.c_void_p(0), ctypes.c_longlong(0), _ptr(partial), partial.shape[0]
    _f32(row, "row")
    assert row.shape == (T, W) and row.stride(1) == 1
    return _ptr(row), ctypes.c_longlong(row.stride(0)), ctypes.c_void_p(0), 0


def mlstm_prepare(row: Optional[torch.Tensor], partial: Optional[torch.Tensor], T: int,
                  n_heads: int, head_dim: int, value_dim: int, bias_i: torch.Tensor,
                  bias_f: torch.Tensor, cap: float, q_mult: float, qkv: torch.Tensor,
                  gates: torch.Tensor) -> None:
    """From a token's row  q | k | v | g | i | f  of the stacked projection (32-bit [T, W] or
    ``partial`` [S, T, W]): qkv [T, 2 H d + H dv] = q * q_mult | k | v and gates [T, 2 H] =
    the log input gates cap * tanh((i + b_i) / cap), then the log forget gates
    logsigmoid(cap * tanh((f + b_f) / cap)); all 32-bit."""
    H, d, dv = n_heads, head_dim, value_dim
    W = 2 * H * d + 2 * H * dv + 2 * H
    rp, ld, pp, ns = _f32_row_input(row, partial, T, W)
    for t, n in ((bias_i, "bias_i"), (bias_f, "bias_f"), (qkv, "qkv"), (gates, "gates")):
        _f32(t, n); _dense(t, n)
    assert qkv.shape == (T, 2 * H * d + H * dv) and gates.shape == (T, 2 * H)
    assert bias_i.numel() == H and bias_f.numel() == H
    with _span("mlstm_prepare", _nbytes(row, partial, qkv, gates)):
        _check(library().agv_mlstm_prepare(rp, ld, pp, ns, T, H, d, dv, _ptr(bias_i),
                                           _ptr(bias_f), ctypes.c_float(cap),
                                           ctypes.c_float(q_mult), _ptr(qkv), _ptr(gates),
                                           _stream()))


def mlstm_scan(qkv: torch.Tensor, gates: torch.Tensor, num: torch.Tensor, den: torch.Tensor, ctx,
               state: torch.Tensor, n_heads: int, head_dim: int, value_dim: int) -> None:
    """The recurrence  m' = max(f + m, i); S <- exp(f + m - m') S + exp(i - m') k v^T; n likewise
    with k  over the step's tokens, sequence by sequence; S, n and m of each sequence are read
    from and written to ``state``.  num [T, H * dv] receives S^T q, den [T, H, 2] receives n . q
    and exp(-m'): the read-out is num / (max(|n . q|, exp(-m')) + eps).  All 32-bit."""
    T = qkv.shape[0]
    H, d, dv = n_heads, head_dim, value_dim
    for t, n in ((qkv, "qkv"), (gates, "gates"), (num, "num"), (den, "den")):
        _f32(t, n); _dense(t, n)
    assert qkv.shape == (T, 2 * H * d + H * dv) and gates.shape == (T, 2 * H)
    assert num.shape == (T, H * dv) and den.shape == (T, H, 2)
    sp, ss = _state_args(state)
    lib = library()
    assert lib.agv_mlstm_state_numel(H, d, dv) == mlstm_state_numel(H, d, dv)
    with _span("mlstm_scan", _nbytes(qkv, gates, num, den), 6 * T * H * d * dv):
        _check(lib.agv_mlstm_scan(_ptr(qkv), _ptr(gates), _ptr(num), _ptr(den), T, ctx.batch, H,
                                  d, dv, sp, ss, _ptr(ctx.slots), _ptr(ctx.cu_seqlens),
                                  _stream()))


def mlstm_out(num: torch.Tensor, den: torch.Tensor, den_eps: float, row: Optional[torch.Tensor],
              partial: Optional[torch.Tensor], weight: torch.Tensor, eps: float, n_heads: int,
              head_dim: int, value_dim: int, y: torch.Tensor) -> None:
    """o = num / (max(|den[..., 0]|, den[..., 1]) + den_eps);  y[t, h, :] = o[t, h, :] /
    rms(o[t, h, :]) * weight[h, :] * sigmoid(g[t, h, :]), g the gate's logits in the stacked
    projection (``row`` / ``partial`` as in ``mlstm_prepare``); num and den 32-bit, y in the
    compute dtype."""
    T = num.shape[0]
    H, d, dv = n_heads, head_dim, value_dim
    rp, ld, pp, ns = _f32_row_input(row, partial, T, 2 * H * d + 2 * H * dv + 2 * H)
    for t, n in ((num, "num"), (den, "den"), (weight, "weight")):
        _f32(t, n); _dense(t, n)
    _dense(y, "y")
    assert num.shape == y.shape == (T, H * dv) and den.shape == (T, H, 2)
    assert weight.numel() == H * dv
    with _span("mlstm_out", _nbytes(num, den, y) + T * H * dv * 4):
        _check(library().agv_mlstm_out(_ptr(num), _ptr(den), ctypes.c_float(den_eps), rp, ld, pp,
                                       ns, _ptr(weight), ctypes.c_float(eps), T, H, d, dv,
                                       _ptr(y), dtype_code(y.dtype), _stream()))


# ------------------------------------------- attention with a short convolution
def conv_rope_store(row: Optional[torch.Tensor], partial: Optional[torch.Tensor],
                    out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                    value_dim: int, taps: int, conv_w: torch.Tensor,
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                    gate: bool, state: Optional[torch.Tensor], state_off: int, ctx,
                    view=None) -> None:
    """From a token's row  q | k | v | g  of the stacked projection (32-bit rows or partial
    sums; k and v absent when ``n_kv_heads`` is 0, g without ``gate``): a causal convolution
    over ``taps`` tokens on every channel of q, k and v (earlier inputs from the step's rows
    or, before the step, from the ring in ``state`` at ``state_off``, which is brought up to
    date), the rotation of the first ``rotary_dim`` dimensions of every q and k head, the store
    of k and v in the cache entry ``view``; out [T, W] receives q | k | v | g in the compute
    dtype."""
    T, W = out.shape
    C = n_heads * head_dim + n_kv_heads * (head_dim + value_dim)
    assert W == C + (n_heads * value_dim if gate else 0) and out.stride(1) == 1
    rp, ld, pp, ns = _f32_row_input(row, partial, T, W)
    _f32(conv_w, "conv_w"); _dense(conv_w, "conv_w"); _f32(cos, "cos"); _f32(sin, "sin")
    assert conv_w.shape == (C, taps)
    if rotary_dim:
        _dense(cos, "cos"); _dense(sin, "sin")
        assert cos.shape == (T, rotary_dim // 2) and sin.shape == cos.shape
    if state is not None:
        sp, ss = _state_args(state)
    else:
        sp, ss = ctypes.c_void_p(0), ctypes.c_longlong(0)
    cache = _cache_args(view, ctx)
    if view is None:
        cache[3:6] = [_ptr(ctx.slots), _ptr(ctx.lens), _ptr(ctx.seq_index)]
    else:
        assert view.k_pool.dtype == out.dtype
    with _span("conv_rope_store", _nbytes(row, partial, out)):
        _check(library().agv_conv_rope_store(
            rp, ld, pp, ns, dtype_code(out.dtype), T, n_heads, n_kv_heads, head_dim, value_dim,
            taps, _ptr(conv_w), _ptr(cos), _ptr(sin), rotary_dim, 1 if gate else 0, sp, ss,
            ctypes.c_longlong(state_off), _ptr(ctx.cu_seqlens), _ptr(ctx.positions), *cache,
            _ptr(out), ctypes.c_longlong(out.stride(0)), _stream()))


# ------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _f32(logits, "logits"); _i32(out, "out")
    B, V = logits.shape
    assert logits.stride(1) == 1
    with _span("argmax", B * V * 4):
        _check(library().agv_argmax(_ptr(logits), ctypes.c_longlong(logits.stride(0)), B, V,
                                    _ptr(out), _stream()))


def history_append(tokens: torch.Tensor, slots: torch.Tensor, hist: torch.Tensor,
                   hist_len: torch.Tensor) -> None:
    """hist[slot, hist_len[slot]++] = token for every entry with a slot."""
    for t, n in ((tokens, "tokens"), (slots, "slots"), (hist, "hist"), (hist_len, "hist_len")):
        _i32(t, n)
    _dense(hist, "hist")
    _check(library().agv_history_append(_ptr(tokens), _ptr(slots), _ptr(hist), _ptr(hist_len),
                                        hist.shape[1], slots.numel(), _stream()))


def take_tokens(tokens: torch.Tensor, prev: torch.Tensor, take: torch.Tensor,
                vocab_size: int) -> None:
    """tokens[b] = prev[b] for every b if take[0] is set (on the device)."""
    for t, n in ((tokens, "tokens"), (prev, "prev"), (take, "take")):
        _i32(t, n)
    assert prev.numel() >= tokens.numel() and take.numel() >= 1
    _check(library().agv_take_tokens(_ptr(tokens), _ptr(prev), _ptr(take), tokens.numel(),
                                     vocab_size, _stream()))


SAMPLING_WORDS = 8


def sampling_words(temperature: float, top_k: int, top_p: float, seed: int,
                   penalty: float):
    """The sampling options as the int32 words the kernels read from the device
    (``dev_params``): [1 / temperature, top_k, top_p, seed low, seed high, penalty]."""
    import numpy as np
    w = np.zeros(SAMPLING_WORDS, dtype=np.int32)
    f = w.view(np.float32)
    f[0] = 1.0 / temperature if temperature > 0 else 1.0
    w[1] = int(top_k)
    f[2] = top_p
    w[3:5] = np.array([seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF], dtype=np.uint32).view(np.int32)
    f[5] = penalty
    return w


def repeat_penalty(logits: torch.Tensor, slots: torch.Tensor, hist: torch.Tensor,
                   hist_len: torch.Tensor, penalty: float,
                   dev_params: Optional[torch.Tensor] = None) -> None:
    """Penalise, in place, every id in each row's slot history, once per occurrence.
    ``dev_params`` (``sampling_words`` on the device) replaces ``penalty`` at run time."""
    _f32(logits, "logits"); _i32(dev_params, "dev_params")
    for t, n in ((slots, "slots"), (hist, "hist"), (hist_len, "hist_len")):
        _i32(t, n)
    B, V = logits.shape
    _dense(hist, "hist")
    _check(library().agv_repeat_penalty(_ptr(logits), ctypes.c_longlong(logits.stride(0)), B, V,
                                        _ptr(slots), _ptr(hist), _ptr(hist_len), hist.shape[1],
                                        ctypes.c_float(penalty), _ptr(dev_params), _stream()))


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float, top_k: int, top_p: float,
           seed: int, seq_ids: torch.Tensor, steps: torch.Tensor,
           dev_params: Optional[torch.Tensor] = None) -> None:
    """out[b] drawn from logits[b]; ``dev_params`` (``sampling_words`` on the device)
    replaces temperature, top_k, top_p and seed at run time."""
    _f32(logits, "logits"); _i32(out, "out"); _i32(steps, "steps"); _i32(dev_params, "dev_params")
    if dev_params is not None:
        assert dev_params.numel() >= SAMPLING_WORDS
    if seq_ids.dtype != torch.int64:
        raise KernelError("seq_ids must be int64")
    B, V = logits.shape
    assert logits.stride(1) == 1
    with _span("sample", B * V * 4):
        _check(library().agv_sample(_ptr(logits), ctypes.c_longlong(logits.stride(0)), B, V,
                                    _ptr(out), ctypes.c_float(temperature), int(top_k),
                                    ctypes.c_float(top_p), ctypes.c_ulonglong(seed & (2**64 - 1)),
                                    _ptr(seq_ids), _ptr(steps), _ptr(dev_params), _stream()))


def linear_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
              w2: Optional[torch.Tensor] = None, activation: str = "gelu_tanh",
              splits: int = 1, token_tile: int = 0, cluster: int = 0,
              op: str = "linear") -> None:
    """bfloat16 product on the tensor cores (tcgen05 + TMA).

    out [T, N] in bfloat16 or 32-bit.  With splits > 1, K is cut into ranges that
    run in CTAs of their own.  ``cluster`` = c (2..8, dividing splits): every c CTAs
    of a tile add their partial sums through distributed shared memory and out is
    [splits / c, T, N] (plain [T, N] when splits == c).  ``cluster`` = 0: out is
    [splits, T, N] 32-bit partial sums (use ``linear_tc_splits`` for the real count).
    """
    T, K = x.shape
    N = w.shape[0]
    assert w.shape == (N, K) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.stride(1) == 1
    _dense(w, "w")
    if w2 is not None:
        _dense(w2, "w2")
        assert w2.shape == w.shape and w2.dtype == w.dtype
    cluster = int(cluster)
    groups = splits // cluster if cluster else splits
    if groups > 1:
        assert out.dim() == 3 and out.shape == (groups, T, N) and out.is_contiguous()
        ldc = N
    else:
        assert out.shape == (T, N) and out.stride(1) == 1
        ldc = out.stride(0)
    with _span(op, *_linear_cost(x, w, w2, out)):
        _check(library().agv_linear_tc(
            _ptr(x), _ptr(w), _ptr(w2), _ptr(out), T, N, K, ctypes.c_longlong(x.stride(0)),
            ctypes.c_longlong(ldc), dtype_code(out.dtype), ACT[activation], splits, cluster,
            token_tile, _stream()))


ARGMAX_MAX_ROWS = 128


def linear_argmax_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``linear_argmax`` takes these operands (else: the product, then ``argmax``)."""
    return linear_tc_supported(x, w) and x.shape[0] <= ARGMAX_MAX_ROWS


def linear_argmax(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = first index of the greatest element of (x w^T)[t, :], bfloat16 on the
    tensor cores; the [T, N] product is never written.  At most 128 rows of x."""
    T, K = x.shape
    N = w.shape[0]
    assert w.shape == (N, K) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.stride(1) == 1 and T <= ARGMAX_MAX_ROWS
    _dense(w, "w"); _i32(out, "out")
    assert out.numel() >= T and out.is_contiguous()
    global _launches
    with _span("lm_head_argmax", N * K * 2 + T * K * 2, 2 * T * N * K):
        _check(library().agv_linear_tc_argmax(_ptr(x), _ptr(w), _ptr(out), T, N, K,
                                              ctypes.c_longlong(x.stride(0)), _stream()))
    _launches += 1            # the product and the kernel that reads its keys out


def linear_tc_splits(K: int, splits: int) -> int:
    return library().agv_linear_tc_splits(K, splits)


def linear_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and
            w.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and
            w.data_ptr() % 16 == 0)


def linear_tc_status() -> int:
    """0, or the code of the first bounded wait of a tensor-core kernel that gave
    up since the last call (this call synchronises the device)."""
    torch.cuda.synchronize()
    return library().agv_linear_tc_status()


def selftest_bounded_wait(limit: int = 2000, ctas: int = 4):
    """Runs the unit kernel whose mbarrier waits all run out after ``limit`` polls;
    returns (status code, clock cycles the first wait took).  The kernel follows the
    tensor-core kernels' give-up protocol: record a code, stop, free tensor memory,
    return."""
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cycles = torch.zeros(1, dtype=torch.int32, device="cuda")
    _check(library().agv_selftest_bounded_wait(ctypes.c_uint(limit), ctas, _ptr(status),
                                               _ptr(cycles), _stream()))
    torch.cuda.synchronize()
    return int(status.item()), int(cycles.item()) & 0xFFFFFFFF


# ------------------------------------------------------------------ dispatch
_n_sms = None


def n_sms() -> int:
    """Streaming multiprocessors of the current device (read once)."""
    global _n_sms
    if _n_sms is None:
        _n_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _n_sms

_PREFILL_TC = os.environ.get("AGAVE_B200_PREFILL_ATTENTION", "tcgen05") != "mma"

def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
           w2: Optional[torch.Tensor] = None, activation: str = "gelu_tanh",
           op: str = "linear") -> None:
    """out = x w^T (or the gated pair).  Which kernel runs follows from the dtype and the
    weight's shape; how K is cut into ranges (and with it the order of the 32-bit sums)
    also follows from the number of rows of x, so a token's result is the same in any
    company up to that summation order."""
    if linear_tc_supported(x, w) and (w2 is None or out.dtype == torch.bfloat16):
        c = 0
        if w2 is not None and x.shape[0] <= 64:
            # decoding through a gated layer with few 64-feature tiles: two or four
            # CTAs per tile, each on a range of K, joined by a cluster
            tiles = (w.shape[0] + 63) // 64
            kb = (w.shape[1] + 63) // 64
            sms = n_sms()
            c = 4 if tiles * 4 <= sms and kb >= 8 else 2 if tiles * 2 <= 2 * sms and kb >= 4 else 0
        linear_tc(x, w, out, w2, activation, splits=max(c, 1), cluster=c, op=op)
    else:
        linear_simt(x, w, out, w2, activation, op=op)


def plan_splits(T: int, N: int, K: int, cheap_sum: bool = False):
    """(groups, cluster size) of the ranges K is cut into so that about one CTA per
    SM is busy when the weight has few row tiles (decoding through narrow
    layers).  The CTAs of a cluster add their sums in the kernel; the groups are
    left to the consumer.  ``cheap_sum``: the consumer adds partial sums in the
    loads it makes anyway (the q/k norm kernel), so up to eight groups are better
    than a cluster, whose exchange costs about 2 us.  Prompts are not cut."""
    if T > 64:
        tile = 128 if T <= 128 else 256
        ctas = ((N + 127) // 128) * ((T + tile - 1) // tile)
        kb = (K + 63) // 64
        if T <= 512:
            # short prompts have one or two token tiles: without a cut a narrow weight
            # would run on a dozen CTAs; the partial sums (fewer, the more tokens there
            # are to write them for) are left to the consumer
            most = 16 if T <= 128 else 8 if T <= 256 else 4
            want = min(kb // 2, n_sms() // ctas, most)
            return (linear_tc_splits(K, want), 0) if want >= 2 else (1, 0)
        # long prompts: only a long K over few tiles is cut, in two, with the partial
        # sums left to the consumer (a cluster's exchange is slow for wide tiles)
        if ctas <= n_sms() // 2 + 6 and kb >= 32:
            return 2, 0
        return 1, 0
    tile = 16 if T <= 16 else 32 if T <= 32 else 64
    ctas = ((N + 127) // 128) * ((T + tile - 1) // tile)
    kb = (K + 63) // 64
    want = min(kb, (n_sms() + ctas - 1) // ctas)
    if ctas >= 100 or want < 2:
        return 1, 0
    if T > 16:
        # tiles of 32 and 64 tokens: a cluster's exchange grows with the tile, the
        # consumer's extra reads do not matter yet
        return linear_tc_splits(K, min(want, 16)), 0
    if cheap_sum:
        return linear_tc_splits(K, min(want, 8)), 0
    if want <= 8 or kb < 64:
        # a single cluster per tile adds its ranges in the kernel
        c = min(want, 8)
        return 1, c
    # a long K: more ranges than a cluster holds; the consumer adds the partial sums
    return linear_tc_splits(K, min(want, 16)), 0


def linear_partial(x: torch.Tensor, w: torch.Tensor, cheap_sum: bool = False,
                   op: str = "linear") -> torch.Tensor:
    """x w^T in 32-bit for a consumer that adds over a leading axis: [G, T, N] on
    the tensor-core path (G >= 1 groups of ranges of K; the ranges of a group
    are added inside the kernel by a cluster), else [T, N] in x's dtype.
    ``cheap_sum``: see ``plan_splits``."""
    T, K = x.shape
    N = w.shape[0]
    if linear_tc_supported(x, w):
        groups, csize = plan_splits(T, N, K, cheap_sum)
        out = torch.empty((groups, T, N), dtype=torch.float32, device=x.device)
        linear_tc(x, w, out if groups > 1 else out[0], splits=groups * max(csize, 1),
                  cluster=csize, op=op)
        return out
    out = torch.empty((T, N), dtype=x.dtype, device=x.device)
    linear_simt(x, w, out, op=op)
    return out


GEMV_FEW_MAX_ROWS = 4
# Decode steps of at most this many tokens run their projections as dot products with the
# joins in their prologues (five kernels a layer instead of seven); measured at the 1B
# sizes: one token gains 18 %, two gain 3 %, four lose 22 %.
FEW_TOKENS = int(os.environ.get("AGAVE_B200_FEW_TOKENS", "2"))


def gemv_few_supported(T: int, N: int, K: int, ldx: int = 8, join: bool = False) -> bool:
    """Whether ``gemv_few`` takes these sizes (one to four rows; see the kernel)."""
    return bool(library().agv_gemv_few_supported(T, N, K, ctypes.c_longlong(ldx), 1 if join else 0))


def gemv_few(w: torch.Tensor, out: torch.Tensor, x: Optional[torch.Tensor] = None,
             w2: Optional[torch.Tensor] = None, activation: str = "gelu_tanh",
             h_in: Optional[torch.Tensor] = None, h_out: Optional[torch.Tensor] = None,
             y: Optional[torch.Tensor] = None, w_post: Optional[torch.Tensor] = None,
             w_next: Optional[torch.Tensor] = None, eps_post: float = 0.0, eps_next: float = 0.0,
             op: str = "linear") -> None:
    """A projection of one to four tokens, one dot product per warp and output row:
    out [T, N] = x w^T in 32-bit, or with w2 the gated pair in bfloat16.  x [T, K]
    bfloat16, or None: then x = bfloat16(norm(h_out; w_next)) with
    h_out = h_in + norm(y; w_post) (or h_in + y, or h_in itself without y) formed in the
    kernel's prologue; h_out (another buffer than h_in) receives the joined stream."""
    N, K = w.shape
    _dense(w, "w")
    assert w.dtype == torch.bfloat16 and out.stride(-1) == 1
    T = out.shape[0]
    if x is not None:
        assert x.shape == (T, K) and x.dtype == torch.bfloat16 and x.stride(1) == 1
    else:
        assert h_in is not None and h_in.shape == (T, K) and w_next is not None
        _f32(h_in, "h_in"); _f32(h_out, "h_out"); _f32(y, "y"); _f32(w_post, "w_post")
        _f32(w_next, "w_next"); _dense(h_in, "h_in")
        for t in (h_out, y):
            if t is not None:
                _dense(t, "join operand")
                assert t.shape == (T, K)
    if w2 is not None:
        _dense(w2, "w2")
        assert w2.shape == w.shape and out.dtype == torch.bfloat16
    else:
        assert out.dtype == torch.float32
    assert out.shape == (T, N)
    nbytes = (2 if w2 is not None else 1) * N * K * 2 + _nbytes(x, h_in, y, out)
    with _span(op, nbytes, 2 * T * N * K * (2 if w2 is not None else 1)):
        _check(library().agv_gemv_few(
            _ptr(w), _ptr(w2), N, K, T, _ptr(x), ctypes.c_longlong(x.stride(0) if x is not None else 0),
            _ptr(h_in), _ptr(h_out), _ptr(y), _ptr(w_post), _ptr(w_next), ctypes.c_float(eps_post),
            ctypes.c_float(eps_next), _ptr(out), ctypes.c_longlong(out.stride(0)), ACT[activation],
            _stream()))


def attention_prefill_mma(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                          cu_seqlens: torch.Tensor, max_len: int, n_heads: int, n_kv_heads: int,
                          head_dim: int, scale: float, window: int,
                          sinks: Optional[torch.Tensor] = None, value_dim: int = 0,
                          dist_bias: Optional[torch.Tensor] = None, keep_first: int = 0) -> None:
    """Prompts that start at 0 on the tensor cores (bfloat16, head sizes in steps
    of 8 up to 256); q, k, v are row-strided views, out is dense.  ``value_dim``: the value
    head size where it differs from the keys'; ``dist_bias`` [nh, n]: see
    ``attention_prefill_simt``."""
    _f32(sinks, "sinks"); _f32(dist_bias, "dist_bias")
    assert q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
    _dense(out, "out"); _i32(cu_seqlens, "cu_seqlens")
    if dist_bias is not None:
        _dense(dist_bias, "dist_bias")
        assert dist_bias.dim() == 2 and dist_bias.shape[0] == n_heads
    _check(library().agv_attention_prefill_mma_ex3(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(k), _ptr(v),
        ctypes.c_longlong(k.stride(0)), _ptr(out), _ptr(cu_seqlens), cu_seqlens.numel() - 1,
        max_len, n_heads, n_kv_heads, head_dim, ctypes.c_float(scale), window, _ptr(sinks),
        value_dim or head_dim, ctypes.c_longlong(v.stride(0)), _ptr(dist_bias),
        dist_bias.shape[1] if dist_bias is not None else 0, int(keep_first), _stream()))


def prefill_values_scratch(T: int, B: int, n_kv_heads: int, head_dim: int,
                           device: torch.device) -> torch.Tensor:
    """The buffer the tcgen05 prompt attention reads the values from, transposed:
    [nkv * hd, columns], every sequence padded to a multiple of 64 columns."""
    cols = library().agv_attention_prefill_tc_vt_cols(T, B)
    return torch.empty((n_kv_heads * head_dim, cols), dtype=torch.bfloat16, device=device)


def transpose_values(v: torch.Tensor, vt: torch.Tensor, cu_seqlens: torch.Tensor, max_len: int,
                     n_kv_heads: int, head_dim: int) -> None:
    """vt (from ``prefill_values_scratch``) = the values v [T, nkv * hd] (row-strided
    view) transposed, every sequence padded with zeros to a multiple of 64 columns."""
    assert v.dtype == torch.bfloat16 and vt.dtype == torch.bfloat16 and v.stride(1) == 1
    _dense(vt, "vt"); _i32(cu_seqlens, "cu_seqlens")
    _check(library().agv_transpose_values(
        _ptr(v), ctypes.c_longlong(v.stride(0)), _ptr(vt), ctypes.c_longlong(vt.shape[1]),
        _ptr(cu_seqlens), cu_seqlens.numel() - 1, max_len, n_kv_heads, head_dim, _stream()))


def attention_prefill_tc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                         cu_seqlens: torch.Tensor, max_len: int, n_heads: int, n_kv_heads: int,
                         head_dim: int, scale: float, window: int,
                         vt: Optional[torch.Tensor] = None,
                         sinks: Optional[torch.Tensor] = None,
                         dist_bias: Optional[torch.Tensor] = None, keep_first: int = 0) -> None:
    """Prompts that start at 0 on the tcgen05 tensor cores (bfloat16, head sizes in
    steps of 16 up to 256); q, k, v are row-strided views, out is dense.  ``vt``:
    the values already transposed (by ``qk_norm_rope_store``); else this call
    transposes them."""
    assert q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
    assert k.stride(0) == v.stride(0)
    _dense(out, "out"); _i32(cu_seqlens, "cu_seqlens")
    T, B = q.shape[0], cu_seqlens.numel() - 1
    ready = vt is not None
    if vt is None:
        vt = prefill_values_scratch(T, B, n_kv_heads, head_dim, q.device)
    _dense(vt, "vt")
    _f32(sinks, "sinks"); _f32(dist_bias, "dist_bias")
    if dist_bias is not None:
        _dense(dist_bias, "dist_bias")
        assert dist_bias.dim() == 2 and dist_bias.shape[0] == n_heads
    _check(library().agv_attention_prefill_tc_ex3(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(k), _ptr(v),
        ctypes.c_longlong(k.stride(0)), _ptr(out), _ptr(vt), ctypes.c_longlong(vt.shape[1]),
        1 if ready else 0, _ptr(cu_seqlens), B, T, max_len, n_heads, n_kv_heads, head_dim,
        ctypes.c_float(scale), window, _ptr(sinks), _ptr(dist_bias),
        dist_bias.shape[1] if dist_bias is not None else 0, int(keep_first), _stream()))


def attention_tc_status() -> int:
    """0, or the code of the first bounded wait of the tcgen05 attention kernel that
    gave up since the last call (this call synchronises the device)."""
    torch.cuda.synchronize()
    return library().agv_attention_tc_status()


# A prompt step of at most this many tokens runs the mma.sync attention: the tcgen05
# kernel's CTAs take 128 query rows each, so a short prompt gives it a handful of CTAs with
# a long set-up each (a 128-token step: 586 against 624 us over six layers; from 256 tokens
# on the tcgen05 kernel is ahead).
PREFILL_TC_MIN_TOKENS = 192


def attention_prefill_wants_transposed_values(qkv: torch.Tensor, head_dim: int,
                                              value_dim: int = 0) -> bool:
    """Whether ``attention_prefill`` on views of this projection output will take the
    tcgen05 kernel, which reads the values transposed."""
    return ((value_dim or head_dim) == head_dim and _PREFILL_TC and qkv.shape[0] > PREFILL_TC_MIN_TOKENS and qkv.dtype == torch.bfloat16 and
            head_dim % 16 == 0 and head_dim <= 256 and qkv.stride(0) % 8 == 0 and
            qkv.data_ptr() % 16 == 0)


def attention_prefill(q, k, v, out, ctx, n_heads, n_kv_heads, head_dim, scale, window,
                      vt=None, value_dim: int = 0, sinks=None, dist_bias=None,
                      op: str = "attention", keep_first: int = 0) -> None:
    """Prompt attention of one layer in bfloat16: the tcgen05 kernel for head sizes
    in steps of 16 up to 256, the mma.sync kernel for the other multiples of 8; else
    (and for value heads of another size than the keys') the one-warp-per-(token, head)
    kernel.  ``sinks`` [nh]: a logit per query head that joins its denominator once."""
    hdv = value_dim or head_dim
    aligned = (q.dtype == torch.bfloat16 and head_dim <= 256 and hdv <= 256 and
               q.stride(0) % 8 == 0 and k.stride(0) % 8 == 0 and v.stride(0) % 8 == 0 and
               q.data_ptr() % 16 == 0 and k.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0)
    # the tcgen05 kernel does not know value heads of their own size
    same = hdv == head_dim and k.stride(0) == v.stride(0)
    if not window:
        keep_first = 0                    # (without a window every key is visible anyway)
    with _span(op, *_attention_cost(ctx, q, k, v, out, n_heads, head_dim, window)):
        if (aligned and same and head_dim % 16 == 0 and _PREFILL_TC and scale > 0 and
                q.shape[0] > PREFILL_TC_MIN_TOKENS):
            attention_prefill_tc(q, k, v, out, ctx.cu_seqlens, ctx.max_new, n_heads, n_kv_heads,
                                 head_dim, scale, window, vt=vt, sinks=sinks, dist_bias=dist_bias,
                                 keep_first=keep_first)
        elif aligned and head_dim % 8 == 0 and hdv % 8 == 0:
            attention_prefill_mma(q, k, v, out, ctx.cu_seqlens, ctx.max_new, n_heads,
                                  n_kv_heads, head_dim, scale, window, sinks=sinks,
                                  value_dim=hdv, dist_bias=dist_bias, keep_first=keep_first)
        else:
            attention_prefill_simt(q, k, v, out, ctx.positions, ctx.seq_index, ctx.cu_seqlens,
                                   n_heads, n_kv_heads, head_dim, scale, window, value_dim=hdv,
                                   sinks=sinks, dist_bias=dist_bias, keep_first=keep_first)


def _attention_cost(ctx, q, k, v, out, n_heads, head_dim, window, n_kv_heads=0):
    """(bytes, flops) of one layer's attention, from the lengths the host knows
    (``ctx.lens_host``; zeros when a step does not carry them)."""
    if _perf is None:
        return 0, 0
    lens = getattr(ctx, "lens_host", None)
    if lens is None:
        return _nbytes(q, k, v, out), 0
    window = abs(window)          # (a mask of blocks is counted as a window of its size)
    seen = 0                      # (query, key) pairs
    kv_rows = 0                   # cache rows a decode step reads
    for n in lens:
        n = int(n)
        if n <= 0:
            continue
        if ctx.mode == "decode":
            vis = min(n, window) if window else n
            seen += vis
            kv_rows += vis
        elif window and n > window:
            seen += window * (window + 1) // 2 + (n - window) * window
        else:
            seen += n * (n + 1) // 2
    esz = out.element_size()
    nbytes = _nbytes(q, k, v, out) + 2 * kv_rows * n_kv_heads * head_dim * esz
    return nbytes, 4 * n_heads * head_dim * seen


def attention_decode_plan(head_dim: int, dtype: torch.dtype, max_keys: int):
    """(chunk length, number of chunks) the split decode attention uses."""
    chunk, n = ctypes.c_int(0), ctypes.c_int(0)
    _check(library().agv_attention_decode_plan(head_dim, dtype_code(dtype), max_keys,
                                               ctypes.byref(chunk), ctypes.byref(n)))
    return chunk.value, n.value


_counters = {}


def _decode_counters(device: torch.device, n: int) -> torch.Tensor:
    """Arrival counters of the split decode attention: zero between launches (the
    kernel resets what it counted), so one buffer per device serves every layer."""
    t = _counters.get(device)
    if t is None or t.numel() < n:
        t = _counters[device] = torch.zeros(max(n, 65536), dtype=torch.int32, device=device)
    return t


def attention_decode_status() -> int:
    """0, or 1 + the tile at which a bounded wait of the decode attention for a tile of keys
    and values gave up first since the last call (this call synchronises the device)."""
    return library().agv_attention_decode_status()


DECODE_TILES = {"auto": 0, "copies": 1, "tma": 2}


def attention_decode_tiles(form: str) -> str:
    """How the tensor-core decode attention brings its key / value tiles: "auto" (from the
    sizes), "copies" (16-byte copies by all threads) or "tma" (the cache's pages as TMA
    boxes, wherever the cache's geometry allows).  Returns the setting before."""
    before = library().agv_attention_decode_set_tiles(DECODE_TILES[form])
    if before < 0:
        raise KernelError("attention_decode_set_tiles failed")
    return {v: k for k, v in DECODE_TILES.items()}[before]


def prepare_device(device: torch.device) -> None:
    """Allocate what the kernels share on a device before any graph is recorded."""
    _decode_counters(device, 65536)


def attention_decode_split(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor,
                           v_pool: torch.Tensor, page_table: torch.Tensor, slots: torch.Tensor,
                           positions: torch.Tensor, page: int, cap: int, n_heads: int,
                           n_kv_heads: int, head_dim: int, scale: float, window: int,
                           max_keys: int, part_acc: Optional[torch.Tensor] = None,
                           part_ml: Optional[torch.Tensor] = None,
                           sinks: Optional[torch.Tensor] = None,
                           dist_bias: Optional[torch.Tensor] = None, keep_first: int = 0) -> None:
    """One query per batch entry against the paged cache, keys split into chunks
    whose partial results go through scratch memory (allocated here if not given)."""
    B = q.shape[0]
    assert q.stride(1) == 1
    _dense(out, "out"); _dense(k_pool, "k_pool"); _dense(v_pool, "v_pool")
    for t, n in ((positions, "positions"), (page_table, "page_table"), (slots, "slots")):
        _i32(t, n)
    assert k_pool.dtype == q.dtype and out.dtype == q.dtype
    _, n_splits = attention_decode_plan(head_dim, q.dtype, max_keys)
    if part_acc is None:
        part_acc = torch.empty((B, n_heads, n_splits, head_dim), dtype=torch.float32,
                               device=q.device)
        part_ml = torch.empty((B, n_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    assert part_acc.numel() >= B * n_heads * n_splits * head_dim
    assert part_ml.numel() >= B * n_heads * n_splits * 2
    _f32(part_acc, "part_acc"); _f32(part_ml, "part_ml")
    counters = _decode_counters(q.device, B * n_heads)
    _f32(sinks, "sinks"); _f32(dist_bias, "dist_bias")
    if dist_bias is not None:
        _dense(dist_bias, "dist_bias")
        assert dist_bias.dim() == 2 and dist_bias.shape[0] == n_heads
    _check(library().agv_attention_decode_ex3(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(out), dtype_code(q.dtype), _ptr(k_pool),
        _ptr(v_pool), _ptr(page_table), _ptr(slots), _ptr(positions), page_table.shape[1], page,
        cap, B, n_heads, n_kv_heads, head_dim, ctypes.c_float(scale), window, max_keys,
        _ptr(part_acc), _ptr(part_ml), _ptr(counters), _ptr(sinks), _ptr(dist_bias),
        dist_bias.shape[1] if dist_bias is not None else 0, int(keep_first), _stream()))


_FUSED_DECODE = os.environ.get("AGAVE_B200_FUSED_DECODE_ATTENTION", "1") != "0"


def attention_decode_fused_supported(dtype: torch.dtype, head_dim: int, rotary_dim: int) -> bool:
    """Whether ``attention_decode_fused`` takes a layer of these sizes."""
    return (_FUSED_DECODE and dtype == torch.bfloat16 and bool(
        library().agv_attention_decode_fused_supported(BF16, head_dim, rotary_dim)))


def attention_decode_fused(partial: torch.Tensor, wq: Optional[torch.Tensor],
                           wk: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                           sin: Optional[torch.Tensor], store_kv: bool, out: torch.Tensor, view,
                           ctx, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                           window: int, sinks: Optional[torch.Tensor] = None, q_temp=None,
                           q_only: bool = False) -> None:
    """Decode attention of one layer with the q/k norm, the rotation and the cache store
    of the new position inside the attention kernel: ``partial`` [G, B, (nh + 2 nkv) *
    hd] are the projection's 32-bit partial sums ([G, B, nh * hd] with ``q_only``: a layer
    that attends to keys and values another layer stored).  ``sinks`` [nh]: a logit per
    query head joining its denominator once; ``q_temp`` = (coef, every): the query
    temperature 1 + coef * ln(floor((p + 1) / every) + 1)."""
    _f32(partial, "partial"); _dense(partial, "partial"); _dense(out, "out")
    _f32(wq, "wq"); _f32(wk, "wk"); _f32(cos, "cos"); _f32(sin, "sin"); _f32(sinks, "sinks")
    G, B, width = partial.shape
    assert width == (n_heads + (0 if q_only else 2 * n_kv_heads)) * head_dim
    assert out.dtype == torch.bfloat16 and not (q_only and store_kv)
    assert view.k_pool.dtype == torch.bfloat16
    if cos is not None:
        _dense(cos, "cos"); _dense(sin, "sin")
        assert cos.shape == (B, head_dim // 2) and sin.shape == cos.shape
    max_keys = max(1, min(abs(window), ctx.max_len) if window else ctx.max_len)
    _, n_splits = attention_decode_plan(head_dim, torch.bfloat16, max_keys)
    # the tensor-core form leaves at most one partial result per cluster, and at most 16
    # clusters share a sequence, however long the context may get
    n_splits = min(n_splits, 16)
    part_acc = torch.empty((B, n_heads, n_splits, head_dim), dtype=torch.float32,
                           device=out.device)
    part_ml = torch.empty((B, n_heads, n_splits, 2), dtype=torch.float32, device=out.device)
    counters = _decode_counters(out.device, B * n_heads)
    with _span("attention", *_attention_cost(ctx, partial, None, None, out, n_heads, head_dim,
                                             window, n_kv_heads)):
        coef, every = q_temp if q_temp is not None else (0.0, 1)
        _check(library().agv_attention_decode_fused_ex(
            _ptr(partial), G, _ptr(wq), _ptr(wk), ctypes.c_float(eps), _ptr(cos), _ptr(sin),
            1 if store_kv else 0, _ptr(out), _ptr(view.k_pool), _ptr(view.v_pool),
            _ptr(view.page_table), _ptr(ctx.slots), _ptr(ctx.positions),
            view.page_table.shape[1], view.page, view.cap, B, n_heads, n_kv_heads, head_dim,
            ctypes.c_float(scale), window, max_keys, _ptr(part_acc), _ptr(part_ml),
            _ptr(counters), _ptr(sinks), ctypes.c_float(coef), int(every), 1 if q_only else 0,
            _stream()))


def attention_decode(q, out, view, ctx, n_heads, n_kv_heads, head_dim, scale, window,
                     value_dim: int = 0, sinks=None, dist_bias=None,
                     values_in_keys: bool = False, op: str = "attention",
                     keep_first: int = 0) -> None:
    """Decode attention of one layer: the split kernel for head sizes in steps of
    16 up to 512, else (and for value heads of another size than the keys') the
    one-warp-per-head kernel."""
    hdv = value_dim or head_dim
    if not window:
        keep_first = 0
    with _span(op, *_attention_cost(ctx, q, None, None, out, n_heads, head_dim, window,
                                    n_kv_heads)):
        if (head_dim % 16 == 0 and head_dim <= 512 and hdv == head_dim and not values_in_keys
                and not (keep_first and dist_bias is not None)):
            # (kept first keys are walked before the window's)
            max_keys = min(abs(window) + keep_first, ctx.max_len) if window else ctx.max_len
            attention_decode_split(q, out, view.k_pool, view.v_pool, view.page_table, ctx.slots,
                                   ctx.positions, view.page, view.cap, n_heads, n_kv_heads,
                                   head_dim, scale, window, max(1, max_keys), sinks=sinks,
                                   dist_bias=dist_bias, keep_first=keep_first)
        else:
            attention_paged_simt(q, out, view.k_pool, view.v_pool, view.page_table, ctx.slots,
                                 ctx.positions, ctx.seq_index, view.page, view.cap, n_heads,
                                 n_kv_heads, head_dim, scale, window, value_dim=hdv, sinks=sinks,
                                 dist_bias=dist_bias,
                                 v_row=n_kv_heads * head_dim if values_in_keys else 0,
                                 keep_first=keep_first)
