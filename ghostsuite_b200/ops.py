"""Kernel entry points on torch CUDA tensors.

Each function validates shapes, hands raw device pointers to ``libghost_b200.so`` on torch's current
stream, and returns torch tensors.  torch is used for memory and stream lookup only; the
arithmetic runs in the library's kernels.  Scratch memory comes from a grow-only arena per
(device, stream), so no allocation happens in steady state and nothing is freed while kernels that
use it may still be queued.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _lib

_BF16 = torch.bfloat16
_F32 = torch.float32

_arenas: Dict[Tuple[int, int], torch.Tensor] = {}


_timing: Optional[list] = None


def start_kernel_timing() -> None:
    """Bracket every library call with CUDA events on the launching stream (opt-in; used by the
    benchmark to attribute device time and algorithmic work to kernel groups)."""
    global _timing
    _timing = []


def stop_kernel_timing() -> dict:
    """Synchronise and return ``{'ops': {name: {calls, ms, flops, bytes, bound}}, 'share': {...}}``."""
    global _timing
    records, _timing = _timing or [], None
    torch.cuda.synchronize()
    out: Dict[str, dict] = {}
    for name, bound, flops, nbytes, e0, e1 in records:
        r = out.setdefault(name, {"calls": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0, "bound": bound})
        r["calls"] += 1
        r["ms"] += e0.elapsed_time(e1)
        r["flops"] += flops
        r["bytes"] += nbytes
    total = sum(r["ms"] for r in out.values()) or 1.0
    return {"ops": out, "share": {k: round(v["ms"] / total, 4) for k, v in out.items()},
            "total_ms": total}


class _Timed:
    """``with _Timed(name, bound, flops, bytes):`` around the library calls of one op."""

    def __init__(self, name: str, bound: str, flops: float, nbytes: float):
        self.rec = (name, bound, float(flops), float(nbytes))

    def __enter__(self):
        if _timing is not None:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if _timing is not None and exc[0] is None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            _timing.append(self.rec + (self.e0, e1))
        return False


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("ghostsuite_b200 kernels need CUDA tensors (no CPU fallback exists)")


class _Arena:
    """Bump allocator over one cached uint8 tensor; reset at the start of every public op."""

    def __init__(self, device: torch.device):
        self.device = device
        self.key = (device.index if device.index is not None else torch.cuda.current_device(),
                    _stream_ptr())
        self.requests = []

    def plan(self, nbytes: int) -> int:
        """Reserve nbytes (256-byte aligned); returns the offset."""
        off = sum(self.requests)
        self.requests.append((int(nbytes) + 255) // 256 * 256)
        return off

    def commit(self) -> int:
        total = sum(self.requests) + 256
        buf = _arenas.get(self.key)
        if buf is None or buf.numel() < total:
            # grow-only; the old buffer stays referenced by torch's caching allocator semantics
            # (stream-ordered reuse), so queued kernels that still read it are safe
            buf = torch.empty(max(total, 1 << 20), dtype=torch.uint8, device=self.device)
            _arenas[self.key] = buf
        base = buf.data_ptr()
        return (base + 255) // 256 * 256


def _dt_flag(t: torch.Tensor) -> int:
    if t.dtype == _F32:
        return 1
    if t.dtype == _BF16:
        return 0
    raise ValueError(f"unsupported dtype {t.dtype}: the kernels take float32 or bfloat16")


def _as3d(x: torch.Tensor) -> torch.Tensor:
    """[N, d] -> [N, 1, d]; [N, ..., d] -> [N, T, d] (contiguous).  float16 / float64 inputs are
    widened / narrowed to float32 first (the kernels take float32 and bfloat16)."""
    if x.dtype in (torch.float16, torch.float64):
        x = x.float()
    if x.dim() <= 2:
        x = x.unsqueeze(1)
    else:
        x = x.reshape(x.shape[0], -1, x.shape[-1])
    return x.contiguous()


def _tma_ready(x: torch.Tensor) -> bool:
    return x.dtype == _BF16 and x.shape[-1] % 8 == 0 and x.data_ptr() % 16 == 0


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def _cast(lib, src: torch.Tensor, samples: int, T: int, dst_ptr: int, ld_dst: int, cpad: int,
          kinds: Tuple[int, ...], row_stack: bool) -> None:
    k = tuple(kinds) + (0,) * (3 - len(kinds))
    _lib.check(lib.ghost_cast_split_bf16(src.data_ptr(), _dt_flag(src), samples, T, src.shape[-1],
                                         src.shape[-1], dst_ptr, ld_dst, cpad, len(kinds),
                                         k[0], k[1], k[2], 1 if row_stack else 0, _stream_ptr()))


# hi/lo layouts of an fp32 operand pair so that  sum_k L[k] R[k] = hi*hi + lo*hi + hi*lo
_SPLIT_LEFT = (0, 1, 0)
_SPLIT_RIGHT = (0, 0, 1)


# --------------------------------------------------------------------------------------------
# Linear / Conv1D weight dot product: Gram path
# --------------------------------------------------------------------------------------------
def gram_dot(A: torch.Tensor, G: torch.Tensor, n_val: int, round_mode: int = 0,
             scale: float = 1.0) -> torch.Tensor:
    """Full ``[n_val, n_train]`` dot-product matrix through the fused Gram kernel.

    bf16 inputs are used as they are (copied only if their feature size is not a multiple of 8);
    fp32 inputs are split into bf16 hi/lo parts so the result keeps fp32-class accuracy.
    """
    lib = _lib.load()
    _require_cuda(A, G)
    A, G = _as3d(A), _as3d(G)
    N, T, d = A.shape
    p = G.shape[-1]
    n_train = N - n_val
    if n_train <= 0:
        raise ValueError("No training samples to compute dot product, check batch sizes.")
    if n_val <= 0:
        raise ValueError("gram_dot needs at least one validation sample")
    if G.shape[0] != N or G.shape[1] != T:
        raise ValueError(f"activation {tuple(A.shape)} and out-grad {tuple(G.shape)} disagree")
    M = torch.empty((n_val, n_train), dtype=_F32, device=A.device)
    arena = _Arena(A.device)
    ops = []
    for x in (A, G):
        f = x.shape[-1]
        if x.dtype == _F32:
            cp = _pad8(f)
            off_t = arena.plan(n_train * T * 3 * cp * 2)
            off_v = arena.plan(n_val * T * 3 * cp * 2)
            ops.append(("split", x, cp, off_t, off_v))
        elif _tma_ready(x):
            ops.append(("asis", x, f, 0, 0))
        else:
            cp = _pad8(f)
            off_t = arena.plan(N * T * cp * 2)
            ops.append(("copy", x, cp, off_t, 0))
    base = arena.commit()
    # algorithmic work (the fp32 hi/lo split executes three times this on the tensor pipe)
    timer = _Timed("ghost_gram_kernel", "tensor", 2.0 * n_train * T * n_val * T * (d + p),
                   float(A.element_size()) * N * T * (d + p))
    timer.__enter__()
    ptrs = []
    for kind, x, cp, off_t, off_v in ops:
        if kind == "asis":
            pt = x.data_ptr()
            pv = pt + n_train * T * x.shape[-1] * 2
            ptrs.append((pt, pv, x.shape[-1], x.shape[-1], x.shape[-1]))
        elif kind == "copy":
            _cast(lib, x, N, T, base + off_t, cp, cp, (0,), False)
            pt = base + off_t
            ptrs.append((pt, pt + n_train * T * cp * 2, cp, cp, cp))
        else:
            _cast(lib, x[:n_train], n_train, T, base + off_t, 3 * cp, cp, _SPLIT_LEFT, False)
            _cast(lib, x[n_train:], n_val, T, base + off_v, 3 * cp, cp, _SPLIT_RIGHT, False)
            ptrs.append((base + off_t, base + off_v, 3 * cp, 3 * cp, 3 * cp))
    (at, av, ka, ld_at, ld_av), (gt, gv, kg, ld_gt, ld_gv) = ptrs
    _lib.check(lib.ghost_gram_dot_bf16(at, av, gt, gv, n_train, n_val, T, ka, kg, ld_at, ld_av,
                                       ld_gt, ld_gv, int(round_mode), float(scale), M.data_ptr(),
                                       _stream_ptr()))
    timer.__exit__(None, None, None)
    return M


# --------------------------------------------------------------------------------------------
# train-gradient recovery and the per-sample-gradient path
# --------------------------------------------------------------------------------------------
def _xty_operands(lib, arena: _Arena, X: torch.Tensor, Y: torch.Tensor, samples: int, T: int):
    """Plan bf16 operands for the token-contracted GEMMs.  Returns a closure that materialises them
    after ``arena.commit()`` and yields (x_ptr, y_ptr, ldx, ldy, T_eff)."""
    split = X.dtype == _F32 or Y.dtype == _F32
    plans = []
    for x, kinds in ((X, _SPLIT_LEFT), (Y, _SPLIT_RIGHT)):
        f = x.shape[-1]
        cp = _pad8(f)
        if split:
            plans.append(("split", x, cp, arena.plan(samples * 3 * T * cp * 2), kinds))
        elif _tma_ready(x):
            plans.append(("asis", x, f, 0, kinds))
        else:
            plans.append(("copy", x, cp, arena.plan(samples * T * cp * 2), kinds))

    def materialise(base: int):
        out = []
        for kind, x, cp, off, kinds in plans:
            if kind == "asis":
                out.append((x.data_ptr(), x.shape[-1]))
            elif kind == "copy":
                _cast(lib, x, samples, T, base + off, cp, cp, (0,), True)
                out.append((base + off, cp))
            else:
                _cast(lib, x, samples, T, base + off, cp, cp, kinds, True)
                out.append((base + off, cp))
        return out[0][0], out[1][0], out[0][1], out[1][1], (3 * T if split else T)

    return materialise, split


def wgrad(X: torch.Tensor, Y: torch.Tensor, scale: float, out_dtype: torch.dtype,
          out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """``scale * sum over all rows of X^T Y`` -> ``[X.shape[-1], Y.shape[-1]]`` in ``out_dtype``.

    ``X``/``Y`` are ``[samples, T, cols]`` (train samples only).
    """
    lib = _lib.load()
    _require_cuda(X, Y)
    X, Y = _as3d(X), _as3d(Y)
    S, T, m = X.shape
    n = Y.shape[-1]
    if Y.shape[0] != S or Y.shape[1] != T:
        raise ValueError("wgrad operands disagree on the token layout")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=X.device)
        accumulate = False
    arena = _Arena(X.device)
    ws_bytes = int(lib.ghost_wgrad_workspace_bytes(m, n))
    off_ws = arena.plan(ws_bytes)
    mat, _ = _xty_operands(lib, arena, X, Y, S, T)
    base = arena.commit()
    with _Timed("xty_gemm_pair_kernel[wgrad]", "tensor", 2.0 * S * T * m * n, 2.0 * S * T * (m + n)):
        xp, yp, ldx, ldy, T_eff = mat(base)
        _lib.check(lib.ghost_wgrad_bf16(xp, yp, S * T_eff, m, n, ldx, ldy, float(scale),
                                        1 if accumulate else 0, out.data_ptr(), _dt_flag(out),
                                        base + off_ws, ws_bytes, _stream_ptr()))
    return out


_PERSAMPLE_NAME = "xty_gemm_pair_kernel+tile_dot_mma_kernel[persample]"


def persample_dot(X: torch.Tensor, Y: torch.Tensor, n_val: int, dot_scale: float = 1.0,
                  want_grad: bool = False, grad_scale: float = 1.0,
                  grad_dtype: Optional[torch.dtype] = None, colsum_of: Optional[str] = None):
    """Dot-product matrix through explicit per-sample weight gradients kept in tensor memory.

    ``X``/``Y``: ``[N, T, cols]``, train first.  Returns ``(M[n_val, n_train], train_grad or None)``
    with ``train_grad = grad_scale * sum_b X_b^T Y_b`` of shape ``[X cols, Y cols]``.  With
    ``colsum_of='X'`` or ``'Y'`` a third value is returned: the per-sample column sums ``[N, cols]``
    (float32) of that operand, taken inside the GEMM pass, or None when the operands are fp32 (their
    bf16 hi/lo split is what the kernel sees).
    """
    lib = _lib.load()
    _require_cuda(X, Y)
    X, Y = _as3d(X), _as3d(Y)
    N, T, m = X.shape
    n = Y.shape[-1]
    n_train = N - n_val
    if n_train <= 0:
        raise ValueError("No training samples to compute dot product, check batch sizes.")
    if n_val <= 0:
        raise ValueError("persample_dot needs at least one validation sample")
    if Y.shape[0] != N or Y.shape[1] != T:
        raise ValueError("persample_dot operands disagree on the token layout")
    M = torch.empty((n_val, n_train), dtype=_F32, device=X.device)
    grad = None
    if want_grad:
        grad = torch.empty((m, n), dtype=grad_dtype or X.dtype, device=X.device)
    arena = _Arena(X.device)
    mat, split = _xty_operands(lib, arena, X, Y, N, T)
    v_f32 = 1 if split else 0
    ws_bytes = int(lib.ghost_persample_workspace_bytes(n_train, n_val, m, n, v_f32))
    off_ws = arena.plan(ws_bytes)
    base = arena.commit()
    if colsum_of not in (None, "X", "Y"):
        raise ValueError("colsum_of must be None, 'X' or 'Y'")
    colsums = None
    cs_flag = 0
    if colsum_of is not None and not split:
        colsums = torch.empty((N, m if colsum_of == "X" else n), dtype=_F32, device=X.device)
        cs_flag = 1 if colsum_of == "X" else 2
    with _Timed(_PERSAMPLE_NAME, "tensor",
                2.0 * N * T * m * n + 2.0 * n_val * n_train * m * n, 2.0 * N * T * (m + n)):
        xp, yp, ldx, ldy, T_eff = mat(base)
        _lib.check(lib.ghost_persample_dot_bf16(
            xp, yp, n_train, n_val, T_eff, m, n, ldx, ldy, float(dot_scale), M.data_ptr(), v_f32,
            grad.data_ptr() if want_grad else None, _dt_flag(grad) if want_grad else 0,
            float(grad_scale), 0, cs_flag, colsums.data_ptr() if colsums is not None else None,
            base + off_ws, ws_bytes, _stream_ptr()))
    if colsum_of is None:
        return M, grad
    return M, grad, colsums


def persample_tiles(X: torch.Tensor, Y: torch.Tensor, sample0: int, samples: int,
                    colsum_of: Optional[str] = None, colsums: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First pass of the per-sample path alone: the bf16 tiles ``X_s^T Y_s`` of samples
    ``[sample0, sample0 + samples)``, laid out ``[tiles, samples, 32768]`` (128 x 256 tiles).  ``X`` /
    ``Y``: contiguous bf16 ``[N, T, cols]`` with column counts that are multiples of 8.  With
    ``colsum_of`` the rows ``sample0 ..`` of ``colsums`` (``[N, cols]`` float32) are filled too."""
    lib = _lib.load()
    N, T, m = X.shape
    n = Y.shape[-1]
    nbytes = int(lib.ghost_persample_tiles_bytes(samples, m, n))
    tiles = torch.empty((nbytes // (samples * 65536), samples, 32768), dtype=_BF16, device=X.device)
    cs_flag = 0 if colsum_of is None else (1 if colsum_of == "X" else 2)
    with _Timed(_PERSAMPLE_NAME, "tensor", 2.0 * samples * T * m * n, 2.0 * samples * T * (m + n)):
        _lib.check(lib.ghost_persample_tiles_bf16(
            X.data_ptr(), Y.data_ptr(), N, T, m, n, m, n, int(sample0), int(samples), cs_flag,
            colsums.data_ptr() if cs_flag else None, tiles.data_ptr(), nbytes, _stream_ptr()))
    return tiles


def tile_dot(V: torch.Tensor, W: torch.Tensor, m: int, n: int, dot_scale: float = 1.0,
             want_grad: bool = False, grad_scale: float = 1.0, grad_dtype: torch.dtype = _BF16,
             M: Optional[torch.Tensor] = None, grad: Optional[torch.Tensor] = None):
    """Second pass alone.  ``W``: train tiles ``[tiles, n_train, 32768]``; ``V``: validation tiles, either
    ``[tiles, n_val, 32768]`` or, as an all-gather over ranks leaves them, ``[ranks, tiles, per_rank,
    32768]`` (validation sample ``r * per_rank + i`` of the result is sample ``i`` of rank ``r``).
    Returns ``(M[n_val, n_train], train_grad[m, n] or None)``, written into ``M`` / ``grad`` when given."""
    lib = _lib.load()
    if V.dim() == 3:
        V = V.unsqueeze(0)
    ranks, tiles, per_rank, _ = V.shape
    n_train = W.shape[1]
    n_val = ranks * per_rank
    if M is None:
        M = torch.empty((n_val, n_train), dtype=_F32, device=W.device)
    if want_grad and grad is None:
        grad = torch.empty((m, n), dtype=grad_dtype, device=W.device)
    with _Timed(_PERSAMPLE_NAME, "tensor", 2.0 * n_val * n_train * m * n, 0.0):
        _lib.check(lib.ghost_tile_dot_bf16(
            V.data_ptr(), ranks, per_rank, W.data_ptr(), n_train, m, n, float(dot_scale), M.data_ptr(),
            grad.data_ptr() if want_grad else None, _dt_flag(grad) if want_grad else 0, float(grad_scale), 0,
            _stream_ptr()))
    return M, (grad if want_grad else None)


# Streaming passes that wait for an all-gather in flight, per (device, stream): the pass of one layer
# is launched when the next layer has launched its own tile passes and all-gather (or by
# ``finish_exchange_jobs``), so the transfer runs under that layer's GEMMs.
_exchange_jobs: Dict[Tuple[int, int], list] = {}

#: how many layers' streaming passes may wait for their all-gather at a time (each holds its tile
#: buffers); a pass is launched when this many later layers have issued theirs
EXCHANGE_DEPTH = 1


def _finish_exchange_job(job: dict) -> None:
    job["work"].wait()               # the current stream waits for the all-gather
    tile_dot(job["V"], job["W"], job["m"], job["n"], job["dot_scale"], job["grad"] is not None,
             job["grad_scale"], _BF16, M=job["M"], grad=job["grad"])
    cb = job["on_ready"]
    job.clear()
    if cb is not None:
        cb()


def finish_exchange_jobs() -> None:
    """Launch the streaming pass of every layer that still waits for its all-gather."""
    for key in list(_exchange_jobs):
        for job in _exchange_jobs.pop(key):
            _finish_exchange_job(job)


def persample_dot_exchanged(X: torch.Tensor, Y: torch.Tensor, n_val_local: int, exchange, dot_scale: float = 1.0,
                            want_grad: bool = False, grad_scale: float = 1.0,
                            grad_dtype: Optional[torch.dtype] = None, colsum_of: Optional[str] = None,
                            on_ready=None):
    """The per-sample path of a rank that holds ``n_val_local`` of the validation samples (the last
    rows of ``X`` / ``Y``): tiles of the local validation samples, an all-gather of them along
    dimension 0 over ``exchange.world`` ranks (``exchange.gather_rows``), tiles of the local train
    samples, then the contraction of ALL validation tiles with the local train tiles.  Returns
    ``(M[world * n_val_local, n_train], train_grad or None, colsums of the LOCAL samples or None)``, or
    None when the shapes are outside what the two-pass entry points take (fp32 operands, a bf16
    train gradient of more than 32 samples, a validation split that does not fit the kernel's row
    blocks).

    With ``on_ready`` and an exchange that has ``gather_rows_async`` the all-gather is not waited
    for: ``M`` and the gradient are filled by a later launch -- when the next call on this stream has
    enqueued its own tile passes, or in :func:`finish_exchange_jobs` -- and ``on_ready()`` is called
    right after that launch has been enqueued."""
    _require_cuda(X, Y)
    if X.dtype != _BF16 or Y.dtype != _BF16:
        return None
    X, Y = _as3d(X), _as3d(Y)
    N, T, m = X.shape
    n = Y.shape[-1]
    n_train = N - n_val_local
    ranks = int(exchange.world)
    if n_train <= 0:
        raise ValueError("No training samples to compute dot product, check batch sizes.")
    if n_val_local <= 0 or Y.shape[0] != N or Y.shape[1] != T or not (_tma_ready(X) and _tma_ready(Y)):
        return None
    gdt = grad_dtype or X.dtype
    if want_grad and gdt != _F32 and n_train > 32:
        return None
    n_val = n_val_local * ranks
    block = 8 if n_val <= 8 else (16 if n_val <= 16 else 32)
    if block % n_val_local != 0 and n_val_local % block != 0:
        return None
    if colsum_of not in (None, "X", "Y"):
        raise ValueError("colsum_of must be None, 'X' or 'Y'")
    colsums = None
    if colsum_of is not None:
        colsums = torch.empty((N, m if colsum_of == "X" else n), dtype=_F32, device=X.device)
    V_loc = persample_tiles(X, Y, n_train, n_val_local, colsum_of, colsums)
    deferred = on_ready is not None and hasattr(exchange, "gather_rows_async")
    if deferred:
        V_all, work = exchange.gather_rows_async(V_loc.unsqueeze(0))
    else:
        V_all = exchange.gather_rows(V_loc.unsqueeze(0))     # [ranks, tiles, n_val_local, 32768]
    W = persample_tiles(X, Y, 0, n_train, colsum_of, colsums)
    if not deferred:
        M, grad = tile_dot(V_all, W, m, n, dot_scale, want_grad, grad_scale, gdt)
        return M, grad, colsums
    M = torch.empty((n_val, n_train), dtype=_F32, device=X.device)
    grad = torch.empty((m, n), dtype=gdt, device=X.device) if want_grad else None
    key = (X.device.index if X.device.index is not None else torch.cuda.current_device(), _stream_ptr())
    queue = _exchange_jobs.setdefault(key, [])
    queue.append({"V": V_all, "W": W, "work": work, "m": m, "n": n, "dot_scale": dot_scale,
                  "grad_scale": grad_scale, "M": M, "grad": grad, "on_ready": on_ready})
    while len(queue) > max(1, int(EXCHANGE_DEPTH)):
        _finish_exchange_job(queue.pop(0))
    return M, grad, colsums


# --------------------------------------------------------------------------------------------
# bias / LayerNorm / small reductions
# --------------------------------------------------------------------------------------------
def colsum(G: torch.Tensor) -> torch.Tensor:
    """Per-sample column sums over tokens: ``[N, T, p] -> [N, p]`` float32."""
    lib = _lib.load()
    _require_cuda(G)
    G = _as3d(G)
    N, T, p = G.shape
    out = torch.empty((N, p), dtype=_F32, device=G.device)
    with _Timed("colsum_kernel", "hbm", 0.0, float(N) * T * p * G.element_size()):
        _lib.check(lib.ghost_colsum(G.data_ptr(), _dt_flag(G), N, T, p, p, out.data_ptr(), _stream_ptr()))
    return out


def small_gram(X: torch.Tensor, n_val: int, scale: float = 1.0) -> torch.Tensor:
    """``M[v, b] = scale * <X[n_train + v], X[b]>`` for per-sample float32 vectors ``X[N, F]``."""
    lib = _lib.load()
    _require_cuda(X)
    if X.dtype != _F32 or X.dim() != 2 or not X.is_contiguous():
        raise ValueError("small_gram takes a contiguous float32 [N, F] tensor")
    n_train = X.shape[0] - n_val
    if n_train <= 0:
        raise ValueError("No training samples to compute dot product, check batch sizes.")
    M = torch.empty((n_val, n_train), dtype=_F32, device=X.device)
    with _Timed("small_gram_kernel", "hbm", 0.0, 4.0 * X.numel()):
        _lib.check(lib.ghost_small_gram_f32(X.data_ptr(), n_train, n_val, X.shape[1], float(scale),
                                            M.data_ptr(), _stream_ptr()))
    return M


def rows_sum(X: torch.Tensor, n_rows: int, scale: float, out_dtype: torch.dtype,
             out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """``scale * X[:n_rows].sum(0)`` cast to ``out_dtype`` (optionally accumulated into ``out``)."""
    lib = _lib.load()
    _require_cuda(X)
    if X.dtype != _F32 or X.dim() != 2 or not X.is_contiguous():
        raise ValueError("rows_sum takes a contiguous float32 [N, F] tensor")
    if out is None:
        out = torch.empty((X.shape[1],), dtype=out_dtype, device=X.device)
        accumulate = False
    with _Timed("rows_sum_kernel", "hbm", 0.0, 4.0 * n_rows * X.shape[1]):
        _lib.check(lib.ghost_rows_sum(X.data_ptr(), int(n_rows), X.shape[1], float(scale), out.data_ptr(),
                                      _dt_flag(out), 1 if accumulate else 0, _stream_ptr()))
    return out


def small_reduce_batch(jobs) -> None:
    """Run many :func:`small_gram` / :func:`rows_sum` reductions in one launch (48 jobs per launch).
    ``jobs``: dicts with ``X`` (contiguous float32 ``[n_train + n_val, F]``), ``n_train``, ``n_val`` and
    optionally ``M`` (float32 ``[n_val, n_train]`` output, with ``dot_scale``) and ``sum_out``
    (float32 / bfloat16 ``[F]`` output, with ``sum_scale``); the outputs are written in place.  A job
    with ``Xv = (gathered, offset, per_rank)`` takes its validation rows from ``gathered[r, offset + i
    * F : ...]`` (row ``r * per_rank + i``; ``gathered`` is a contiguous float32 ``[ranks, pitch]`` tensor, the
    result of one all-gather that carried many jobs' validation rows) and only its train rows from
    ``X``."""
    if not jobs:
        return
    lib = _lib.load()
    arr = (_lib.SmallJob * len(jobs))()
    nbytes = 0.0
    for rec, job in zip(arr, jobs):
        X = job["X"]
        M, out = job.get("M"), job.get("sum_out")
        _require_cuda(X)
        if X.dtype != _F32 or X.dim() != 2 or not X.is_contiguous():
            raise ValueError("small_reduce_batch takes contiguous float32 [N, F] tensors")
        if M is not None and (M.dtype != _F32 or not M.is_contiguous()
                              or M.numel() != job["n_val"] * job["n_train"]):
            raise ValueError("small_reduce_batch: M must be a contiguous float32 [n_val, n_train] tensor")
        if out is not None and (not out.is_contiguous() or out.numel() != X.shape[1]):
            raise ValueError("small_reduce_batch: sum_out must be a contiguous [F] tensor")
        rec.X = X.data_ptr()
        rec.M = M.data_ptr() if M is not None else None
        rec.sum_out = out.data_ptr() if out is not None else None
        rec.n_train, rec.n_val, rec.F = int(job["n_train"]), int(job["n_val"]), int(X.shape[1])
        rec.sum_is_f32 = _dt_flag(out) if out is not None else 1
        rec.dot_scale = float(job.get("dot_scale", 1.0))
        rec.sum_scale = float(job.get("sum_scale", 1.0))
        xv = job.get("Xv")
        if xv is not None:
            gathered, offset, per_rank = xv
            if gathered.dtype != _F32 or gathered.dim() != 2 or not gathered.is_contiguous() \
                    or offset + per_rank * X.shape[1] > gathered.shape[1] \
                    or gathered.shape[0] * per_rank != job["n_val"] or X.shape[0] < job["n_train"]:
                raise ValueError("small_reduce_batch: bad layout of the separate validation rows")
            rec.Xv = gathered.data_ptr() + 4 * int(offset)
            rec.v_rank_pitch = int(gathered.shape[1])
            rec.v_per_rank = int(per_rank)
        else:
            rec.Xv = None
        nbytes += 4.0 * X.numel()
    with _Timed("small_reduce_batch_kernel", "hbm", 0.0, nbytes):
        _lib.check(lib.ghost_small_reduce_batch(arr, len(jobs), _stream_ptr()))


def layernorm_persample(A: torch.Tensor, G: torch.Tensor, eps: float, rms: bool = False
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-sample LayerNorm gamma/beta gradients ``([N, F], [N, F])`` float32 in one pass.  With
    ``rms=True`` the normalisation is RMS norm's (no centring); the second result is then just the
    token sum of the out-grad."""
    lib = _lib.load()
    _require_cuda(A, G)
    if A.dtype != G.dtype:
        common = torch.promote_types(A.dtype, G.dtype)
        A, G = A.to(common), G.to(common)
    A, G = _as3d(A), _as3d(G)
    N, T, F = A.shape
    if G.shape != A.shape:
        raise ValueError("LayerNorm input and out-grad shapes differ")
    gw = torch.empty((N, F), dtype=_F32, device=A.device)
    gb = torch.empty((N, F), dtype=_F32, device=A.device)
    arena = _Arena(A.device)
    ws_bytes = int(lib.ghost_layernorm_workspace_bytes(N, T, F))
    off = arena.plan(ws_bytes)
    base = arena.commit()
    with _Timed("layernorm_persample_kernel", "hbm", 0.0, 2.0 * N * T * F * A.element_size() + 8.0 * N * F):
        fn = lib.ghost_rmsnorm_persample if rms else lib.ghost_layernorm_persample
        _lib.check(fn(A.data_ptr(), G.data_ptr(), _dt_flag(A), N, T, F, float(eps), gw.data_ptr(),
                      gb.data_ptr(), base + off, ws_bytes, _stream_ptr()))
    return gw, gb


# --------------------------------------------------------------------------------------------
# Embedding
# --------------------------------------------------------------------------------------------
def _ids2d(ids: torch.Tensor) -> torch.Tensor:
    ids = ids.reshape(ids.shape[0], -1)
    if ids.dtype != torch.int64:
        ids = ids.long()
    return ids.contiguous()


def embedding_dot(ids: torch.Tensor, G: torch.Tensor, n_val: int, vocab: int,
                  scale: float = 1.0) -> torch.Tensor:
    lib = _lib.load()
    _require_cuda(ids, G)
    ids = _ids2d(ids)
    G = _as3d(G)
    N, T, d = G.shape
    if ids.shape[0] != N or ids.shape[1] != T:
        raise ValueError("embedding ids and out-grad disagree on [batch, tokens]")
    n_train = N - n_val
    if n_train <= 0:
        raise ValueError("No training samples to compute dot product, check batch sizes.")
    M = torch.empty((n_val, n_train), dtype=_F32, device=G.device)
    arena = _Arena(G.device)
    ws_bytes = int(lib.ghost_embedding_dot_workspace_bytes_for(n_val, T, vocab, d))
    off = arena.plan(ws_bytes)
    base = arena.commit()
    with _Timed("emb_dot_kernel", "hbm", 0.0, float(N) * T * d * G.element_size() + 8.0 * N * T):
        _lib.check(lib.ghost_embedding_dot(ids.data_ptr(), G.data_ptr(), _dt_flag(G), n_train, n_val, T,
                                           d, int(vocab), float(scale), M.data_ptr(), base + off,
                                           ws_bytes, _stream_ptr()))
    return M


def embedding_wgrad(ids: torch.Tensor, G: torch.Tensor, n_train: int, vocab: int, pre_scale: float,
                    divisor: float, out: Optional[torch.Tensor] = None,
                    accumulate: bool = False) -> torch.Tensor:
    """Averaged train gradient of an embedding table ``[vocab, d]`` in the dtype of ``G``."""
    lib = _lib.load()
    _require_cuda(ids, G)
    ids = _ids2d(ids)
    G = _as3d(G)
    N, T, d = G.shape
    if out is None:
        out = torch.empty((vocab, d), dtype=G.dtype, device=G.device)
        accumulate = False
    elif out.dtype != G.dtype:
        raise ValueError("embedding_wgrad output must have the dtype of the out-grad")
    arena = _Arena(G.device)
    ws_bytes = int(lib.ghost_embedding_wgrad_workspace_bytes(n_train, T, vocab))
    off = arena.plan(ws_bytes)
    base = arena.commit()
    with _Timed("emb_segsum_kernel", "hbm", 0.0,
                (float(n_train) * T * d + float(vocab) * d) * G.element_size() + 8.0 * n_train * T):
        _lib.check(lib.ghost_embedding_wgrad(ids.data_ptr(), G.data_ptr(), _dt_flag(G), n_train, T, d,
                                             int(vocab), float(pre_scale), float(divisor),
                                             1 if accumulate else 0, out.data_ptr(), base + off,
                                             ws_bytes, _stream_ptr()))
    return out


# --------------------------------------------------------------------------------------------
# GradProj
# --------------------------------------------------------------------------------------------
def prepare_projection(P: torch.Tensor, split: bool) -> torch.Tensor:
    """bf16 copy of a projection matrix ``[k, n]`` laid out for the kernel: columns padded to a
    multiple of 8; for fp32 models the hi/lo split matching ``_SPLIT_RIGHT``."""
    lib = _lib.load()
    _require_cuda(P)
    P = P.contiguous()
    k, n = P.shape
    cp = _pad8(n)
    parts = _SPLIT_RIGHT if split else (0,)
    out = torch.empty((k, len(parts) * cp), dtype=_BF16, device=P.device)
    _cast(lib, P, 1, k, out.data_ptr(), len(parts) * cp, cp, parts, False)
    return out


def gradproj_dense(G: torch.Tensor, A: torch.Tensor, P_r: torch.Tensor, P_c: torch.Tensor,
                   k_r: int, k_c: int, scale: float, out: torch.Tensor) -> torch.Tensor:
    """``out[b] = scale * (G_b P_r^T)^T (A_b P_c^T)`` written into ``out`` (``[B, >= k_r*k_c]`` fp32,
    possibly a column slice of a wider row-major buffer).  ``P_r``/``P_c`` come from
    :func:`prepare_projection` (split layout iff the activations are fp32)."""
    lib = _lib.load()
    _require_cuda(G, A, P_r, P_c, out)
    G, A = _as3d(G), _as3d(A)
    B, T, n_r = G.shape
    n_c = A.shape[-1]
    if A.shape[0] != B or A.shape[1] != T:
        raise RuntimeError("Batch size mismatch between activations and output gradients")
    if out.dtype != _F32 or out.dim() != 2 or out.shape[0] != B or out.stride(1) != 1 \
            or out.shape[1] < k_r * k_c:
        raise ValueError("gradproj output must be a float32 [B, >= k_r*k_c] row-major view")
    split = G.dtype == _F32 or A.dtype == _F32
    arena = _Arena(G.device)
    plans = []
    for x in (G, A):
        cp = _pad8(x.shape[-1])
        if split:
            plans.append(("split", x, cp, arena.plan(B * T * 3 * cp * 2)))
        elif _tma_ready(x):
            plans.append(("asis", x, x.shape[-1], 0))
        else:
            plans.append(("copy", x, cp, arena.plan(B * T * cp * 2)))
    base = arena.commit()
    timer = _Timed("gradproj_kernel", "hbm", 2.0 * B * T * (n_r * k_r + n_c * k_c + k_r * k_c),
                   float(B) * T * (n_r + n_c) * G.element_size() + 2.0 * (k_r * n_r + k_c * n_c)
                   + 4.0 * B * k_r * k_c)
    timer.__enter__()
    ptrs = []
    for kind, x, cp, off in plans:
        if kind == "asis":
            ptrs.append((x.data_ptr(), cp, cp))
        elif kind == "copy":
            _cast(lib, x, B, T, base + off, cp, cp, (0,), False)
            ptrs.append((base + off, cp, cp))
        else:
            _cast(lib, x, B, T, base + off, 3 * cp, cp, _SPLIT_LEFT, False)
            ptrs.append((base + off, 3 * cp, 3 * cp))
    (gp, kr_len, ldg), (ap, kc_len, lda) = ptrs
    if P_r.shape[1] != kr_len or P_c.shape[1] != kc_len:
        raise ValueError("projection matrices were prepared for a different dtype/feature size")
    _lib.check(lib.ghost_gradproj_dense_bf16(gp, ap, B, T, kr_len, kc_len, ldg, lda, P_r.data_ptr(),
                                             P_c.data_ptr(), int(k_r), int(k_c), P_r.shape[1],
                                             P_c.shape[1], float(scale), out.data_ptr(),
                                             out.stride(0), _stream_ptr()))
    timer.__exit__(None, None, None)
    return out


def prepare_embedding_projection(P_i: torch.Tensor) -> torch.Tensor:
    """``P_i [k_i, vocab]`` as the embedding-projection kernel reads it: float32 ``[vocab, k_i]``, so
    that a token id selects one contiguous row (made once per layer)."""
    _require_cuda(P_i)
    return P_i.detach().to(_F32).t().contiguous()


def gradproj_embedding(ids: torch.Tensor, G: torch.Tensor, P_o_prepared: torch.Tensor, P_i_t: torch.Tensor,
                       k_o: int, k_i: int, scale: float = 1.0,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[b] = scale * sum_t (P_o g_bt)(P_i[:, id_bt])^T`` as ``[B, k_o*k_i]`` float32 (written into
    ``out`` when given: a ``[B, >= k_o*k_i]`` row-major view, e.g. a column slice of the engine's
    buffer).  ``P_o_prepared`` comes from :func:`prepare_projection` (split layout iff ``G`` is
    float32), ``P_i_t`` from :func:`prepare_embedding_projection`."""
    lib = _lib.load()
    _require_cuda(ids, G, P_o_prepared, P_i_t)
    ids = _ids2d(ids)
    G = _as3d(G)
    B, T, d = G.shape
    if ids.shape[0] != B or ids.shape[1] != T:
        raise RuntimeError("Batch size mismatch between token ids and output gradients")
    split = G.dtype == _F32
    cp = _pad8(d)
    if P_o_prepared.dtype != _BF16 or P_o_prepared.shape[0] != k_o or P_o_prepared.shape[1] != (3 if split else 1) * cp:
        raise ValueError("P_o was prepared for a different dtype/feature size")
    if P_i_t.dtype != _F32 or P_i_t.dim() != 2 or P_i_t.shape[1] != k_i or not P_i_t.is_contiguous():
        raise ValueError("P_i must be passed as the contiguous float32 [vocab, k_i] transpose")
    if out is None:
        out = torch.empty((B, k_o * k_i), dtype=_F32, device=G.device)
    elif out.dtype != _F32 or out.dim() != 2 or out.shape[0] != B or out.stride(1) != 1 or out.shape[1] < k_o * k_i:
        raise ValueError("embedding projection output must be a float32 [B, >= k_o*k_i] row-major view")
    with _Timed("gradproj_embedding_kernel", "hbm", 2.0 * B * T * (d * k_o + k_o * k_i),
                float(B) * T * (d * G.element_size() + 8 + 4 * k_i) + 4.0 * B * k_o * k_i):
        # _SPLIT_RIGHT lays a float32 matrix out as (hi, hi, lo): the residual part starts at 2 * cp.
        # The kernel covers up to 64 x 64 of a sample's block per launch; larger projections go
        # block by block into the zeroed output.
        chunked = k_o > 64 or k_i > 64
        if chunked:
            out[:, :k_o * k_i].zero_()
        ld_po = P_o_prepared.shape[1]
        for o0 in range(0, k_o, 64):
            for i0 in range(0, k_i, 64):
                _lib.check(lib.ghost_gradproj_embedding(
                    ids.data_ptr(), G.data_ptr(), _dt_flag(G), B, T, d, d,
                    P_o_prepared.data_ptr() + o0 * ld_po * 2, ld_po, cp, 2 * cp if split else 0,
                    P_i_t.data_ptr() + i0 * 4, k_i, P_i_t.shape[0], min(64, k_o - o0), min(64, k_i - i0),
                    float(scale), 1 if chunked else 0, out.data_ptr() + (o0 * k_i + i0) * 4,
                    out.stride(0), k_i, _stream_ptr()))
    return out


#: largest block (rows of either operand) the similarity kernel is used for; beyond it the operands
#: would be re-read once per 16 x 16 output block and a library GEMM is the better tool
SIMILARITY_KERNEL_MAX_ROWS = 128


def projection_similarity(P1: torch.Tensor, P2: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``scale * P1 @ P2.T`` -> ``[n1, n2]`` float32 for two blocks of projection rows (float32 or
    bfloat16, same dtype, unit stride along the projection dimension)."""
    lib = _lib.load()
    _require_cuda(P1, P2)
    if P1.dim() != 2 or P2.dim() != 2 or P1.shape[1] != P2.shape[1]:
        raise ValueError("projection sets have different dimensions")
    if P1.dtype != P2.dtype:
        common = torch.promote_types(P1.dtype, P2.dtype)
        P1, P2 = P1.to(common), P2.to(common)
    if P1.dtype not in (_F32, _BF16):
        P1, P2 = P1.float(), P2.float()
    if P1.stride(1) != 1:
        P1 = P1.contiguous()
    if P2.stride(1) != 1:
        P2 = P2.contiguous()
    n1, D = P1.shape
    n2 = P2.shape[0]
    S = torch.empty((n1, n2), dtype=_F32, device=P1.device)
    with _Timed("proj_similarity_kernel", "hbm", 2.0 * n1 * n2 * D, float(n1 + n2) * D * P1.element_size()):
        _lib.check(lib.ghost_projection_similarity(P1.data_ptr(), P2.data_ptr(), _dt_flag(P1), n1, n2, D,
                                                   P1.stride(0), P2.stride(0), float(scale), S.data_ptr(),
                                                   S.stride(0), _stream_ptr()))
    return S


def launch_count() -> int:
    return _lib.launch_count()


# ------------------------------------------------------------------------------------------------
# benchmark model helper: fused token cross-entropy (not part of the ghost hot path)
# ------------------------------------------------------------------------------------------------
def ce_supported(logits: torch.Tensor) -> bool:
    """True when the fused loss kernels can take this [rows, cols] logit matrix as it is."""
    if not logits.is_cuda or logits.dtype not in (_BF16, _F32) or logits.dim() != 2:
        return False
    vec = 8 if logits.dtype == _BF16 else 4
    return logits.stride(1) == 1 and logits.stride(0) % vec == 0 and logits.data_ptr() % 16 == 0


def ce_forward(logits: torch.Tensor, targets: torch.Tensor, valid_cols: int, ignore_index: int = -100,
               grad_scale: Optional[torch.Tensor] = None):
    """Per-row log-sum-exp over the first ``valid_cols`` columns and per-row loss (0 for ignored
    rows), both float32 ``[rows]``, in one pass over ``logits``.  With ``grad_scale`` (one-element
    float32 device tensor) the kernel also writes ``grad_scale * (softmax - onehot)`` in the logits'
    dtype and returns it as a third value."""
    lib = _lib.load()
    _require_cuda(logits, targets)
    rows, cols = logits.shape
    targets = targets.contiguous()
    lse = torch.empty(rows, dtype=_F32, device=logits.device)
    loss_rows = torch.empty(rows, dtype=_F32, device=logits.device)
    dlogits = torch.empty((rows, cols), dtype=logits.dtype, device=logits.device) if grad_scale is not None else None
    nbytes = float(rows) * valid_cols * logits.element_size() * (1.0 if dlogits is None else 2.0)
    with _Timed("ce_forward_kernel", "hbm", 0.0, nbytes):
        _lib.check(lib.ghost_workload_ce_forward(logits.data_ptr(), _dt_flag(logits), rows, cols, int(valid_cols),
                                                 logits.stride(0), targets.data_ptr(), int(ignore_index),
                                                 lse.data_ptr(), loss_rows.data_ptr(),
                                                 grad_scale.data_ptr() if grad_scale is not None else None,
                                                 dlogits.data_ptr() if dlogits is not None else None,
                                                 _stream_ptr()))
    if grad_scale is None:
        return lse, loss_rows
    return lse, loss_rows, dlogits


def ce_rescale_(dlogits: torch.Tensor, upstream: torch.Tensor) -> torch.Tensor:
    """``dlogits *= upstream[0]`` in place; the kernel returns at once when the factor is exactly 1."""
    lib = _lib.load()
    _require_cuda(dlogits, upstream)
    rows, cols = dlogits.shape
    with _Timed("ce_rescale_kernel", "hbm", 0.0, 0.0):
        _lib.check(lib.ghost_workload_ce_rescale(dlogits.data_ptr(), _dt_flag(dlogits), rows, cols,
                                                 upstream.data_ptr(), _stream_ptr()))
    return dlogits


def ce_backward(logits: torch.Tensor, targets: torch.Tensor, valid_cols: int, lse: torch.Tensor,
                scale: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """``scale * (softmax(logits[:, :valid_cols]) - onehot(targets))`` in the logits' dtype, zero in
    padded columns and ignored rows; ``scale`` is a one-element float32 device tensor."""
    lib = _lib.load()
    _require_cuda(logits, targets, lse, scale)
    rows, cols = logits.shape
    targets = targets.contiguous()
    out = torch.empty((rows, cols), dtype=logits.dtype, device=logits.device)
    with _Timed("ce_backward_kernel", "hbm", 0.0, 2.0 * rows * cols * logits.element_size()):
        _lib.check(lib.ghost_workload_ce_backward(logits.data_ptr(), _dt_flag(logits), rows, cols, int(valid_cols),
                                                  logits.stride(0), targets.data_ptr(), int(ignore_index),
                                                  lse.data_ptr(), scale.data_ptr(), out.data_ptr(), cols,
                                                  _stream_ptr()))
    return out
