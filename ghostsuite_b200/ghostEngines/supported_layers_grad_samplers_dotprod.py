"""Per-layer dot-product and train-gradient functions backed by the sm_100a kernels.

Drop-in for GhostSuite's ``ghostEngines/supported_layers_grad_samplers_dotprod.py``: the registry
``_supported_layers_dotprod`` maps a layer type to ``(dot_fn, train_grad_fn)`` with

    dot_fn(layer, A, B, val_batch_size) -> None      sets  <param>.grad_dot_prod  ([n_train])
    train_grad_fn(layer, A, B_scaled, val_batch_size) -> Tensor | None

exactly as the reference (registry at :596-602 there).  Differences, all additive:

* every parameter also gets ``grad_dot_prod_matrix`` -- the full ``[n_val, n_train]`` float32
  matrix; ``grad_dot_prod`` is its sum over the validation samples, which is the quantity the
  reference defines.  The reference's Conv1D and materialised-Linear branches sum the validation
  batch before the outer product and are therefore only right for one validation sample; here
  every validation sample is treated separately.
* dot products are float32 and computed without the reference's bf16 rounding of intermediates.
* the layer math runs in ``libghost_b200.so``; without a B200 these functions raise.

Two tensor-core paths exist for Linear / Conv1D weights: the Gram ("ghost") kernel and the
per-sample-gradient kernel.  ``layer.use_ghost_computation`` (same attribute as the reference,
computed once and cached; pre-setting it overrides the choice) selects the Gram kernel when True.
"""
from __future__ import annotations

import threading

import torch
import torch.nn.functional as F
from torch import nn

try:  # HF Conv1D is optional at import time; it is a registry key when transformers is present
    from transformers.pytorch_utils import Conv1D as _HFConv1D
except Exception:  # pragma: no cover
    _HFConv1D = None

from .. import ops

#: 'cost'      -- pick the cheaper tensor-core path for the full [n_val, n_train] matrix
#: 'reference' -- GhostSuite's rule, Gram path iff 2*T^2 <= weight.numel()
#: 'gram' / 'persample' -- force one kernel (benchmarks and tests)
PATH_RULE = "cost"

# Measured throughputs behind the 'cost' rule (B200): Gram kernel ~1.2e15 flop/s; per-sample GEMM
# pass ~1.1e15 flop/s plus ~3e12 bytes/s for storing the tiles (the term that matters when a sample
# has few tokens); the streaming kernel reads bf16 tiles at ~4.5e12 bytes/s with its contraction on
# the tensor cores (32 train rows and up to 32 validation rows per
# pass); with fp32 tiles its contraction runs on CUDA cores at ~6e12 (validation x train x
# weight-element) products per second and ~5e12 bytes/s.
_GRAM_FLOPS = 1.2e15
_PERSAMPLE_FLOPS = 1.1e15
_STREAM_BYTES_PER_S = 4.5e12
_TILE_WRITE_BYTES_PER_S = 3.0e12
_DOT_PRODUCTS_PER_S = 6.0e12
_TILE_BYTES_PER_S = 5.0e12


def _token_count(A: torch.Tensor) -> int:
    if A.dim() <= 2:
        return 1
    t = 1
    for s in A.shape[1:-1]:
        t *= int(s)
    return t


def _should_use_ghost_computation(layer: nn.Module, A: torch.Tensor, B: torch.Tensor,
                                  conv: bool = False, val_batch_size: int = None, n_train: int = None):
    """Decide once per layer whether the Gram kernel is used (cached in
    ``layer.use_ghost_computation``, as in the reference at :7-41).

    With ``PATH_RULE == 'reference'`` (or when the batch split is unknown) this is the reference's
    test ``2*T^2 <= weight.numel()``.  With ``'cost'`` the two kernels' tensor work for the full
    matrix is compared: Gram ``2*n_t*n_v*T^2*(d+p)`` flops against the per-sample path's
    ``2*(n_t+n_v)*T*d*p`` flops plus the streaming kernel's passes over the stored tiles.
    """
    if hasattr(layer, "use_ghost_computation"):
        return
    if conv:
        T, d, p = int(A.shape[-1]), int(A.shape[1]), int(B.shape[1])
    else:
        T, d, p = _token_count(A), int(A.shape[-1]), int(B.shape[-1])
    if PATH_RULE in ("gram", "persample"):
        layer.use_ghost_computation = PATH_RULE == "gram"
        return
    if PATH_RULE == "reference" or val_batch_size is None:
        layer.use_ghost_computation = bool(2 * T ** 2 <= layer.weight.numel())
        return
    n_v = int(val_batch_size)
    n_t = int(A.shape[0]) - n_v if n_train is None else int(n_train)
    gram = 2.0 * n_t * n_v * T * T * (d + p) / _GRAM_FLOPS
    if A.dtype == torch.float32:
        gram *= 3.0       # hi/lo split operands: three bf16 products per fp32 product, both paths
        per = (6.0 * (n_t + n_v) * T * d * p / _PERSAMPLE_FLOPS + float(n_v) * n_t * d * p / _DOT_PRODUCTS_PER_S
               + 8.0 * (n_t + n_v) * d * p / _TILE_BYTES_PER_S)
    else:
        vr = 8 if n_v <= 8 else (16 if n_v <= 16 else 32)
        passes = -(-n_v // vr) * -(-n_t // 32)
        per = (2.0 * (n_t + n_v) * T * d * p / _PERSAMPLE_FLOPS
               + 2.0 * d * p * (n_t + n_v) / _TILE_WRITE_BYTES_PER_S
               + 2.0 * d * p * (32 + vr) * passes / _STREAM_BYTES_PER_S)
    layer.use_ghost_computation = bool(gram <= per)


#: optional observer ``fn(param)`` called every time a layer has added its contribution to
#: ``param.train_grad`` (the data-parallel layer uses it to start all-reducing finished gradients
#: while the backward pass is still running)
TRAIN_GRAD_OBSERVER = None


def _create_or_accumulate_train_grad(param: torch.Tensor, grad: torch.Tensor) -> None:
    """``param.train_grad`` is created on first use and added to afterwards (reference :44-69)."""
    assert grad.shape == param.shape, \
        f"Gradient shape ({grad.shape}) does not match parameter shape ({param.shape})"
    grad = grad.detach()
    if hasattr(param, "train_grad"):
        param.train_grad.add_(grad)
    else:
        param.train_grad = grad
    if TRAIN_GRAD_OBSERVER is not None:
        TRAIN_GRAD_OBSERVER(param)


# While a backward pass runs, two kinds of small work are not launched layer by layer but collected
# and run when the pass ends (``finalize_pending_dots``, queued as an autograd callback by the hook
# plumbing): the per-parameter [n_train] vectors (one stacked reduction per matrix shape), and the
# bias / LayerNorm / RMS-norm terms' small reductions -- the [n_val, n_train] Gram of a layer's
# per-sample vectors and the sum of its train rows -- which go out as ONE batched launch instead of
# two launches per parameter.  Their output tensors exist from the moment the hook ran (the
# parameter's ``grad_dot_prod_matrix`` is set at once) and are filled when the pass ends; train
# gradients that come out of the batch are handed to ``_create_or_accumulate_train_grad`` after it.
# Direct callers of the layer functions (no backward pass in flight) get everything at once.
_PENDING_DOTS = None
_PENDING_SMALL = None                 # list of job dicts for ops.small_reduce_batch
_PENDING_LOCK = threading.Lock()      # backward hooks of different devices run on different threads


def begin_deferred_dots() -> bool:
    """Start collecting; returns True when this call opened the lists (its caller must arrange for
    ``finalize_pending_dots`` to run)."""
    global _PENDING_DOTS, _PENDING_SMALL
    with _PENDING_LOCK:
        if _PENDING_DOTS is not None:
            return False
        _PENDING_DOTS = []
        _PENDING_SMALL = []
        return True


def _small_job_for(X: torch.Tensor, n_train: int, n_val: int, want: str):
    """The pending job on ``X`` whose ``want`` output ('M' or 'sum_out') is still free, or a new one
    (the Gram and the row sum of one layer's vectors share a job).  None when nothing is deferred."""
    with _PENDING_LOCK:
        if _PENDING_SMALL is None:
            return None
        for job in reversed(_PENDING_SMALL[-4:]):
            if job["X"] is X and job["n_train"] == n_train and job.get(want) is None:
                return job
        job = {"X": X, "n_train": n_train, "n_val": n_val}
        _PENDING_SMALL.append(job)
        return job


def _gram_of_vectors(X: torch.Tensor, val_batch_size: int) -> torch.Tensor:
    """``[n_val, n_train]`` Gram of per-sample vectors: at once, or as part of the batched launch at
    the end of the backward pass in flight."""
    n_train = X.shape[0] - val_batch_size
    job = _small_job_for(X, n_train, val_batch_size, "M")
    if job is None:
        return ops.small_gram(X, val_batch_size)
    M = torch.empty((val_batch_size, n_train), dtype=torch.float32, device=X.device)
    job["M"], job["n_val"], job["dot_scale"] = M, val_batch_size, 1.0
    return M


def _train_grad_from_vectors(param: torch.Tensor, X: torch.Tensor, n_train: int, scale: float,
                             out_dtype: torch.dtype) -> None:
    """``param.train_grad (+)= scale * X[:n_train].sum(0)``: at once, or from the batched launch."""
    job = _small_job_for(X, n_train, X.shape[0] - n_train, "sum_out")
    if job is None:
        _create_or_accumulate_train_grad(param, ops.rows_sum(X, n_train, scale, out_dtype))
        return
    out = torch.empty((X.shape[1],), dtype=out_dtype, device=X.device)
    job["sum_out"], job["sum_scale"], job["param"] = out, scale, param


def finalize_pending_dots() -> None:
    """Run the collected small reductions in one batched launch, hand their train gradients over,
    then set ``param.grad_dot_prod = param.grad_dot_prod_matrix.sum(0)`` for every collected
    parameter with one stack + one reduction per matrix shape.  A tied parameter keeps its last
    matrix, as it does when every hook overwrites the attribute.  Safe to call when nothing is
    pending."""
    global _PENDING_DOTS, _PENDING_SMALL
    ops.finish_exchange_jobs()       # streaming passes that still wait for their all-gather
    with _PENDING_LOCK:
        pending, _PENDING_DOTS = _PENDING_DOTS, None
        small, _PENDING_SMALL = _PENDING_SMALL, None
    if small:
        _exchange_pending_val_rows(small)        # validation rows of a batch split over ranks
        ops.small_reduce_batch(small)
        for job in small:
            if job.get("param") is not None:
                _create_or_accumulate_train_grad(job["param"], job["sum_out"].view_as(job["param"]))
    if not pending:
        return
    last = {}
    for param, M in pending:
        last[id(param)] = (param, M)
    groups = {}
    for param, M in last.values():
        groups.setdefault((tuple(M.shape), M.dtype, M.device), []).append((param, M))
    for items in groups.values():
        stacked = torch.stack([M for _, M in items])          # [P, n_val, n_train]
        vectors = stacked.sum(dim=1)
        for i, (param, M) in enumerate(items):
            if getattr(param, "grad_dot_prod_matrix", None) is M:
                param.grad_dot_prod = vectors[i]


def _set_dot(param: torch.Tensor, M: torch.Tensor) -> None:
    param.grad_dot_prod_matrix = M
    with _PENDING_LOCK:
        deferred = _PENDING_DOTS is not None
        if deferred:
            _PENDING_DOTS.append((param, M))
    if deferred:
        param.grad_dot_prod = M          # placeholder until the backward pass ends
    else:
        param.grad_dot_prod = M.sum(dim=0)


def _check_batch(A, B, val_batch_size: int) -> int:
    if A is None:
        raise ValueError("Input activations A cannot be None.")
    if B is None:
        raise ValueError("Output gradients B cannot be None.")
    n_train = A.size(0) - val_batch_size
    if n_train <= 0:
        raise ValueError("No training samples to compute dot product, check batch sizes.")
    return n_train


def _grad_dtype(param: torch.Tensor, A: torch.Tensor) -> torch.dtype:
    """Train gradients are produced directly in the parameter's dtype when the kernels can write it
    (float32 / bfloat16), so that ``param.grad = param.train_grad`` also works under autocast, where
    activations are bf16 and parameters fp32 (the reference returns the activation dtype)."""
    if param.dtype in (torch.float32, torch.bfloat16):
        return param.dtype
    return torch.float32 if A.dtype != torch.bfloat16 else torch.bfloat16


def _backprop_scale(layer: nn.Module) -> float:
    """Factor that turns the stored out-grad into the reference's ``B * batch_size``.

    The hook plumbing stores the raw out-grad and records the factor here instead of making a
    scaled copy of the whole tensor; direct callers that pass an already scaled ``B`` leave the
    attribute unset (factor 1).
    """
    return float(getattr(layer, "_ghost_backprop_scale", 1.0))


#: take the bias terms' per-sample column sums of the out-grad inside the per-sample GEMM pass (four
#: extra warps of that kernel read the out-grad rows through L2 while the tensor core works on them)
#: instead of a separate pass over the out-grad from HBM
FUSE_BIAS_COLSUMS = True


def _bias_terms(layer: nn.Module, B: torch.Tensor, val_batch_size: int, colsums=None) -> None:
    """Bias dot products from per-sample column sums of the out-grad (reference :138-146).  The
    per-sample GEMM pass can hand the sums over; otherwise they take one pass over B."""
    if colsums is None:
        colsums = ops.colsum(B)                   # [N, p] float32
    _set_dot(layer.bias, _gram_of_vectors(colsums, val_batch_size))
    layer._ghost_colsums = colsums               # reused by the bias train gradient


# --------------------------------------------------------------------------------------------
# Validation batch split over data-parallel ranks
# --------------------------------------------------------------------------------------------
#: set by ``ghostsuite_b200.dist.exchange_validation``: an object with ``world`` and
#: ``gather_rows(t)`` (all-gather along dimension 0).  Every rank then runs ``1 / world`` of the
#: validation batch through the model and the ranks exchange per-sample GRADIENTS of their validation
#: samples instead of running each other's validation sequences: tiles on the per-sample path of
#: Linear / Conv1D layers, the per-sample vectors of bias and norm layers.  Layers this function does
#: not take (Gram path, embeddings, convolutions, fp32 operands) return False and get the other
#: ranks' validation OPERANDS from the caller.
VALIDATION_EXCHANGE = None

#: let the all-gather of a layer's validation tiles run under the next layer's kernels: the layer's
#: streaming pass, its matrix and its train gradient then come one layer late (the last one when the
#: backward pass ends)
EXCHANGE_OVERLAP = True


#: returned by a train-gradient function whose result is handed to
#: ``_create_or_accumulate_train_grad`` later, by the launch that computes it
DEFERRED = object()


def _with_gathered_val_rows(x: torch.Tensor, n_train: int, ex) -> torch.Tensor:
    """``cat(x[:n_train], all ranks' x[n_train:])`` for per-sample vectors ``x[N_local, F]``."""
    return torch.cat([x[:n_train], ex.gather_rows(x[n_train:].contiguous())], dim=0)


def _gram_of_vectors_exchanged(x: torch.Tensor, n_train: int, n_val: int, ex) -> torch.Tensor:
    """``[n_val, n_train]`` Gram of per-sample vectors whose validation rows are spread over the ranks
    (``x[N_local, F]`` holds this rank's train rows and its own validation rows).  Inside a backward
    pass nothing is sent here: the job joins the batched launch at the end of the pass, and ALL such
    jobs' validation rows cross the ranks in ONE all-gather right before it (a hundred collectives of
    a few kilobytes per step otherwise queue between the layers' tile all-gathers)."""
    with _PENDING_LOCK:
        deferred = _PENDING_SMALL is not None
    if not deferred:
        return _gram_of_vectors(_with_gathered_val_rows(x, n_train, ex), n_val)
    job = _small_job_for(x, n_train, n_val, "M")
    M = torch.empty((n_val, n_train), dtype=torch.float32, device=x.device)
    job["M"], job["n_val"], job["dot_scale"], job["val_exchange"] = M, n_val, 1.0, ex
    return M


def _exchange_pending_val_rows(jobs) -> None:
    """One all-gather for the validation rows of every job that waits for them: each rank sends its
    jobs' rows packed one after the other; job ``j`` then reads row ``r * per_rank + i`` at
    ``gathered[r, offset_j + i * F]`` (``ops.small_reduce_batch``)."""
    waiting = [j for j in jobs if j.get("val_exchange") is not None and j.get("M") is not None]
    if not waiting:
        return
    ex = waiting[0]["val_exchange"]
    parts = [j["X"][j["n_train"]:].reshape(-1) for j in waiting]
    gathered = ex.gather_rows(torch.cat(parts).unsqueeze(0))          # [ranks, floats per rank]
    offset = 0
    for j, part in zip(waiting, parts):
        j["Xv"] = (gathered, offset, j["X"].shape[0] - j["n_train"])
        offset += part.numel()


def dot_product_with_exchange(layer: nn.Module, A: torch.Tensor, B: torch.Tensor, n_val_local: int, ex) -> bool:
    """Dot products of ``layer`` from local operands plus exchanged validation gradients; True when
    the layer was handled (the train-gradient functions then run on the local operands as usual)."""
    world = int(ex.world)
    n_train = A.size(0) - n_val_local
    if world <= 1 or n_train <= 0 or n_val_local <= 0:
        return False
    n_val = n_val_local * world
    if isinstance(layer, nn.LayerNorm):
        gw, gb = _layernorm_vectors(layer, A, B)
        _set_dot(layer.weight, _gram_of_vectors_exchanged(gw, n_train, n_val, ex))
        if layer.bias is not None:
            _set_dot(layer.bias, _gram_of_vectors_exchanged(gb, n_train, n_val, ex))
        return True
    if type(layer) in _SELF_APPLYING and type(layer).__name__.endswith("RMSNorm"):
        gw = _rmsnorm_vectors(layer, A, B)
        _set_dot(layer.weight, _gram_of_vectors_exchanged(gw, n_train, n_val, ex))
        return True
    if _HFConv1D is not None and isinstance(layer, _HFConv1D):
        weight_is_in_by_out = True
    elif isinstance(layer, nn.Linear):
        weight_is_in_by_out = False
    else:
        return False
    A = A.detach()
    B = B.detach()
    _should_use_ghost_computation(layer, A, B, val_batch_size=n_val, n_train=n_train)
    if layer.use_ghost_computation:
        return False
    X, Y = (A, B) if weight_is_in_by_out else (B, A)
    want = bool(getattr(layer.weight, "initially_requires_grad", True))
    has_bias = getattr(layer, "bias", None) is not None
    with _PENDING_LOCK:
        in_backward = _PENDING_DOTS is not None
    holder = {}

    def hand_over(weight=layer.weight):
        if holder.get("grad") is not None:
            _create_or_accumulate_train_grad(weight, holder["grad"])

    res = ops.persample_dot_exchanged(
        X, Y, n_val_local, ex, want_grad=want, grad_scale=_backprop_scale(layer) / n_train,
        grad_dtype=_grad_dtype(layer.weight, A),
        colsum_of=("Y" if weight_is_in_by_out else "X") if (has_bias and FUSE_BIAS_COLSUMS) else None,
        on_ready=hand_over if (in_backward and EXCHANGE_OVERLAP) else None)
    if res is None:
        return False
    M, grad, colsums = res
    if want:
        late = in_backward and EXCHANGE_OVERLAP and hasattr(ex, "gather_rows_async")
        holder["grad"] = grad if late else None
        layer._ghost_cached_train_grad = (A.data_ptr(), B.data_ptr(), A.size(0), DEFERRED if late else grad)
    _set_dot(layer.weight, M)
    if has_bias:
        if colsums is None:
            colsums = ops.colsum(B)
        _set_dot(layer.bias, _gram_of_vectors_exchanged(colsums, n_train, n_val, ex))
        layer._ghost_colsums = colsums               # local rows: reused by the bias train gradient
    return True


# --------------------------------------------------------------------------------------------
# Linear and HF Conv1D
# --------------------------------------------------------------------------------------------
def _dense_dot_product(layer: nn.Module, A: torch.Tensor, B: torch.Tensor, val_batch_size: int,
                       weight_is_in_by_out: bool) -> None:
    n_train = _check_batch(A, B, val_batch_size)
    A = A.detach()
    B = B.detach()
    _should_use_ghost_computation(layer, A, B, val_batch_size=val_batch_size)
    colsums = None
    if val_batch_size > 0:
        if layer.use_ghost_computation:
            M = ops.gram_dot(A, B, val_batch_size)
        else:
            # per-sample path: the train gradient falls out of the same pass
            N = A.size(0)
            X, Y = (A, B) if weight_is_in_by_out else (B, A)
            want = bool(getattr(layer.weight, "initially_requires_grad", True))
            has_bias = FUSE_BIAS_COLSUMS and getattr(layer, "bias", None) is not None
            # the out-grad is Y for [d_in, d_out] weights and X for [d_out, d_in] weights
            res = ops.persample_dot(X, Y, val_batch_size, want_grad=want,
                                    grad_scale=_backprop_scale(layer) / n_train,
                                    grad_dtype=_grad_dtype(layer.weight, A),
                                    colsum_of=("Y" if weight_is_in_by_out else "X") if has_bias else None)
            M, grad = res[0], res[1]
            if has_bias:
                colsums = res[2]
            if want:
                layer._ghost_cached_train_grad = (A.data_ptr(), B.data_ptr(), N, grad)
        _set_dot(layer.weight, M)
    if getattr(layer, "bias", None) is not None and val_batch_size > 0:
        _bias_terms(layer, B, val_batch_size, colsums)


def _dense_train_grad(layer: nn.Module, A: torch.Tensor, B: torch.Tensor, val_batch_size: int,
                      weight_is_in_by_out: bool):
    n_train = A.size(0) - val_batch_size
    if n_train <= 0:
        return None
    cached = layer.__dict__.pop("_ghost_cached_train_grad", None)
    if cached is not None and cached[0] == A.data_ptr() and cached[1] == B.data_ptr() \
            and cached[2] == A.size(0):
        return cached[3]
    scale = _backprop_scale(layer) / n_train
    A_t, B_t = A[:n_train], B[:n_train]
    X, Y = (A_t, B_t) if weight_is_in_by_out else (B_t, A_t)
    return ops.wgrad(X, Y, scale, _grad_dtype(layer.weight, A))


def _compute_linear_dot_product(layer: nn.Linear, A: torch.Tensor, B: torch.Tensor,
                                val_batch_size: int):
    """nn.Linear: weight and bias dot products (reference :75-146)."""
    _dense_dot_product(layer, A, B, val_batch_size, weight_is_in_by_out=False)


def _compute_linear_train_grad(layer: nn.Linear, A: torch.Tensor, B: torch.Tensor,
                               val_batch_size: int):
    """nn.Linear: averaged train gradient ``[d_out, d_in]`` (reference :155-173)."""
    return _dense_train_grad(layer, A, B, val_batch_size, weight_is_in_by_out=False)


def _compute_Conv1D_dot_product(layer: nn.Module, A: torch.Tensor, B: torch.Tensor,
                                val_batch_size: int) -> None:
    """HF Conv1D (weight ``[d_in, d_out]``): dot products (reference :369-471)."""
    if A is not None and A.dim() > 3:
        raise ValueError("Currently we only expect 3D input tensors (batch, seq_len, features). "
                         "Extending this to 4D or higher requires additional handling.")
    _dense_dot_product(layer, A, B, val_batch_size, weight_is_in_by_out=True)


def _compute_Conv1D_train_grad(layer: nn.Module, A: torch.Tensor, B: torch.Tensor,
                               val_batch_size: int):
    """HF Conv1D: averaged train gradient ``[d_in, d_out]`` (reference :474-506)."""
    return _dense_train_grad(layer, A, B, val_batch_size, weight_is_in_by_out=True)


# --------------------------------------------------------------------------------------------
# Embedding
# --------------------------------------------------------------------------------------------
def _compute_embedding_dot_product(layer: nn.Embedding, A: torch.Tensor, B: torch.Tensor,
                                   val_batch_size: int):
    """nn.Embedding: id-equality-masked Gram of the out-grad rows (reference :181-211)."""
    _check_batch(A, B, val_batch_size)
    M = ops.embedding_dot(A.detach(), B.detach(), val_batch_size, layer.weight.shape[0])
    _set_dot(layer.weight, M)


def _compute_embedding_train_grad(layer: nn.Embedding, A: torch.Tensor, B: torch.Tensor,
                                  val_batch_size: int):
    """nn.Embedding: averaged train gradient ``[vocab, d]`` (reference :214-235)."""
    n_train = A.size(0) - val_batch_size
    if n_train <= 0:
        return None
    grad = ops.embedding_wgrad(A, B, n_train, layer.weight.shape[0], _backprop_scale(layer),
                               float(n_train))
    if grad.dtype != layer.weight.dtype:
        grad = grad.to(layer.weight.dtype)
    return grad


# --------------------------------------------------------------------------------------------
# LayerNorm
# --------------------------------------------------------------------------------------------
def _layernorm_vectors(layer: nn.LayerNorm, A: torch.Tensor, B: torch.Tensor):
    if len(layer.normalized_shape) != 1:
        raise ValueError("LayerNorm over more than the last dimension is not supported")
    key = (A.data_ptr(), B.data_ptr(), A.size(0))
    cached = layer.__dict__.get("_ghost_ln_cache")
    if cached is not None and cached[0] == key:
        return cached[1], cached[2]
    gw, gb = ops.layernorm_persample(A.detach(), B.detach(), layer.eps)
    layer._ghost_ln_cache = (key, gw, gb)
    return gw, gb


def _compute_layernorm_dot_product(layer: nn.LayerNorm, A: torch.Tensor, B: torch.Tensor,
                                   val_batch_size: int):
    """nn.LayerNorm: gamma and beta dot products from one pass over A and B (reference :242-300)."""
    if A.size(0) - val_batch_size <= 0:
        return
    gw, gb = _layernorm_vectors(layer, A, B)
    _set_dot(layer.weight, _gram_of_vectors(gw, val_batch_size))
    if layer.bias is not None:
        _set_dot(layer.bias, _gram_of_vectors(gb, val_batch_size))


def _compute_layernorm_train_grad(layer: nn.LayerNorm, A: torch.Tensor, B: torch.Tensor,
                                  val_batch_size: int) -> None:
    """nn.LayerNorm: applies both train gradients itself and returns None (reference :303-366)."""
    n_train = A.size(0) - val_batch_size
    if n_train <= 0:
        raise ValueError("No training samples to compute gradients, check batch sizes.")
    gw, gb = _layernorm_vectors(layer, A, B)
    layer.__dict__.pop("_ghost_ln_cache", None)
    scale = _backprop_scale(layer) / n_train
    _train_grad_from_vectors(layer.weight, gw, n_train, scale, layer.weight.dtype)
    if layer.bias is not None:
        _train_grad_from_vectors(layer.bias, gb, n_train, scale, layer.bias.dtype)
    return None


# --------------------------------------------------------------------------------------------
# RMS norm (nn.RMSNorm, Llama-style *RMSNorm modules).  Not in the reference, whose hook
# registration skips such layers with a warning (autograd_grad_sample_dotprod.py:76-79).
# --------------------------------------------------------------------------------------------
def _rmsnorm_eps(layer: nn.Module, A: torch.Tensor) -> float:
    eps = getattr(layer, "variance_epsilon", None)
    if eps is None:
        eps = getattr(layer, "eps", None)
    if eps is None:
        eps = torch.finfo(A.dtype).eps          # nn.RMSNorm's default
    return float(eps)


def _rmsnorm_vectors(layer: nn.Module, A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    key = (A.data_ptr(), B.data_ptr(), A.size(0))
    cached = layer.__dict__.get("_ghost_ln_cache")
    if cached is not None and cached[0] == key:
        return cached[1]
    gw, _ = ops.layernorm_persample(A.detach(), B.detach(), _rmsnorm_eps(layer, A), rms=True)
    layer._ghost_ln_cache = (key, gw)
    return gw


def _compute_rmsnorm_dot_product(layer: nn.Module, A: torch.Tensor, B: torch.Tensor,
                                 val_batch_size: int):
    """RMS norm: weight dot products from one pass over A and B."""
    if A.size(0) - val_batch_size <= 0:
        return
    _set_dot(layer.weight, _gram_of_vectors(_rmsnorm_vectors(layer, A, B), val_batch_size))


def _compute_rmsnorm_train_grad(layer: nn.Module, A: torch.Tensor, B: torch.Tensor,
                                val_batch_size: int) -> None:
    """RMS norm: applies the averaged train gradient of the weight itself and returns None."""
    n_train = A.size(0) - val_batch_size
    if n_train <= 0:
        raise ValueError("No training samples to compute gradients, check batch sizes.")
    gw = _rmsnorm_vectors(layer, A, B)
    layer.__dict__.pop("_ghost_ln_cache", None)
    scale = _backprop_scale(layer) / n_train
    _train_grad_from_vectors(layer.weight, gw, n_train, scale, layer.weight.dtype)
    return None


def maybe_register_rmsnorm(cls) -> bool:
    """Register a module class as an RMS norm when it looks like one: the name ends in 'RMSNorm'
    and instances carry a 1-D ``weight`` (nn.RMSNorm, transformers' LlamaRMSNorm and its copies)."""
    if cls in _supported_layers_dotprod:
        return cls in _SELF_APPLYING and cls is not nn.LayerNorm
    if not cls.__name__.endswith("RMSNorm"):
        return False
    _supported_layers_dotprod[cls] = (_compute_rmsnorm_dot_product, _compute_rmsnorm_train_grad)
    _SELF_APPLYING.add(cls)
    return True


# --------------------------------------------------------------------------------------------
# Conv2d: every output position is a token of the unfolded (im2col) input
# --------------------------------------------------------------------------------------------
def _conv2d_tokens(layer: nn.Conv2d, A: torch.Tensor, B: torch.Tensor):
    """``(A_tok [N, L, C*kh*kw], B_tok [N, L, out_channels])`` for a Conv2d with groups == 1.  The
    unfold is PyTorch's; the contractions over tokens run in the same kernels as nn.Linear."""
    if layer.groups != 1:
        raise ValueError("Conv2d with groups != 1 is not supported")
    key = (A.data_ptr(), B.data_ptr(), A.size(0))
    cached = layer.__dict__.get("_ghost_conv_tokens")
    if cached is not None and cached[0] == key:
        return cached[1], cached[2]
    A_u = F.unfold(A.detach(), kernel_size=layer.kernel_size, dilation=layer.dilation,
                   padding=layer.padding, stride=layer.stride)               # [N, D, L]
    B_r = B.detach().reshape(B.size(0), B.size(1), -1)                        # [N, p, L]
    A_tok = A_u.transpose(1, 2).contiguous()
    B_tok = B_r.transpose(1, 2).contiguous()
    layer._ghost_conv_tokens = (key, A_tok, B_tok)
    return A_tok, B_tok


def _compute_conv2d_dot_product(layer: nn.Conv2d, A: torch.Tensor, B: torch.Tensor,
                                val_batch_size: int) -> None:
    """nn.Conv2d weight and bias dot products (reference :513-563).  The reference's ghost branch
    for this layer type contracts over output positions instead of features and fails unless
    C*kh*kw == out_channels; both kernels here compute the per-sample-gradient products."""
    if A.size(0) - val_batch_size <= 0:
        raise ValueError("No training samples to compute dot product")
    A_tok, B_tok = _conv2d_tokens(layer, A, B)
    if not hasattr(layer, "use_ghost_computation"):
        _should_use_ghost_computation(layer, A_tok.transpose(1, 2), B_tok.transpose(1, 2), conv=True,
                                      val_batch_size=val_batch_size)
    _dense_dot_product(layer, A_tok, B_tok, val_batch_size, weight_is_in_by_out=False)
    cached = layer.__dict__.get("_ghost_cached_train_grad")
    if cached is not None:       # re-key the cached train gradient to the tensors the hook passes
        layer._ghost_cached_train_grad = (A.data_ptr(), B.data_ptr(), A.size(0), cached[3])


def _compute_conv2d_train_grad(layer: nn.Conv2d, A: torch.Tensor, B: torch.Tensor, val_batch_size: int):
    """nn.Conv2d averaged train gradient in the weight's shape (reference :566-592)."""
    n_train = A.size(0) - val_batch_size
    if n_train <= 0:
        return None
    cached = layer.__dict__.pop("_ghost_cached_train_grad", None)
    if cached is not None and cached[0] == A.data_ptr() and cached[1] == B.data_ptr() and cached[2] == A.size(0):
        grad = cached[3]
    else:
        A_tok, B_tok = _conv2d_tokens(layer, A, B)
        grad = ops.wgrad(B_tok[:n_train], A_tok[:n_train], _backprop_scale(layer) / n_train,
                         _grad_dtype(layer.weight, A))
    layer.__dict__.pop("_ghost_conv_tokens", None)
    return grad.view_as(layer.weight)


_supported_layers_dotprod = {
    nn.Linear: (_compute_linear_dot_product, _compute_linear_train_grad),
    nn.Embedding: (_compute_embedding_dot_product, _compute_embedding_train_grad),
    nn.LayerNorm: (_compute_layernorm_dot_product, _compute_layernorm_train_grad),
    nn.Conv2d: (_compute_conv2d_dot_product, _compute_conv2d_train_grad),
}
if _HFConv1D is not None:
    _supported_layers_dotprod[_HFConv1D] = (_compute_Conv1D_dot_product, _compute_Conv1D_train_grad)
# layer types whose train-gradient function writes ``param.train_grad`` itself and returns None
_SELF_APPLYING = {nn.LayerNorm}
if hasattr(nn, "RMSNorm"):
    maybe_register_rmsnorm(nn.RMSNorm)
