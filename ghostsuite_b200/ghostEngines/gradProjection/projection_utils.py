"""Projection-rank selection and projection-matrix initialisers for GradProj.

Drop-in for GhostSuite's ``ghostEngines/gradProjection/projection_utils.py``: ``choose_ki_ko``
(:12-66), the Gaussian / Rademacher / row-orthonormal initialisers (:69-174) and
``compute_projection_metadata`` (:202-238) return the same values for the same arguments, so that a
projection matrix built here equals the one the reference builds from the same seed on the same
device type.  This is one-time setup and stays in PyTorch.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from ... import ops


def choose_ki_ko(n_i: int, n_o: int, k_total: int, k_min: int = 1) -> Tuple[int, int]:
    """Pick ``(k_i, k_o)`` with ``k_i * k_o ~ k_total``, ``k_i / k_o ~ sqrt(n_o / n_i)`` and both at
    least ``k_min`` (and at most the layer dimension), then search the +-2 neighbourhood for the
    product closest to ``k_total``; the first best candidate in row-major (di, dj) order wins."""
    if min(n_i, n_o) <= 0 or k_total <= 0:
        raise ValueError(f"Invalid dimensions for projection: n_i={n_i}, n_o={n_o}, k_total={k_total}")
    if k_min > min(n_i, n_o):
        raise ValueError(f"k_min={k_min} exceeds layer dimensions (n_i={n_i}, n_o={n_o})")
    ratio = math.sqrt(n_o / max(1, n_i))
    k_i = max(k_min, min(n_i, max(1, int(round(math.sqrt(k_total) * ratio)))))
    k_o = max(k_min, min(n_o, max(1, k_total // k_i)))
    best, best_err = (k_i, k_o), abs(k_i * k_o - k_total)
    for di in range(-2, 3):
        for dj in range(-2, 3):
            ci, co = k_i + di, k_o + dj
            if k_min <= ci <= n_i and k_min <= co <= n_o:
                err = abs(ci * co - k_total)
                if err < best_err:
                    best, best_err = (ci, co), err
    if best[0] < k_min or best[1] < k_min:
        raise ValueError(f"Cannot satisfy k_min={k_min} constraints with k_total={k_total}")
    return best


def _generator(device, seed: Optional[int]):
    if seed is None:
        return None
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def init_projection_matrix_gaussian(rows: int, cols: int, dtype: torch.dtype = torch.float32,
                                    device: torch.device = torch.device("cpu"),
                                    seed: Optional[int] = None) -> torch.Tensor:
    """Gaussian JL matrix ``[rows, cols]`` with entries N(0, 1/rows)."""
    P = torch.randn(rows, cols, dtype=dtype, device=device, generator=_generator(device, seed))
    P = P * (1.0 / math.sqrt(rows))
    P.requires_grad_(False)
    return P


def init_projection_matrix_rademacher(rows: int, cols: int, dtype: torch.dtype = torch.float32,
                                      device: torch.device = torch.device("cpu"),
                                      seed: Optional[int] = None) -> torch.Tensor:
    """Entries +-1/sqrt(rows) with equal probability."""
    bits = torch.randint(0, 2, (rows, cols), dtype=torch.int8, device=device,
                         generator=_generator(device, seed))
    P = (bits * 2 - 1).to(dtype) * (1.0 / math.sqrt(rows))
    P.requires_grad_(False)
    return P


def init_projection_matrix_orthonormal(rows: int, cols: int, dtype: torch.dtype = torch.float32,
                                       device: torch.device = torch.device("cpu"),
                                       seed: Optional[int] = None) -> torch.Tensor:
    """Row-orthonormal ``[rows, cols]`` matrix: reduced QR of a float64 Gaussian ``[cols, rows]``."""
    if rows > cols:
        raise ValueError(f"Cannot create {rows} orthonormal rows in {cols} dimensions")
    M = torch.randn(cols, rows, dtype=torch.float64, device=device, generator=_generator(device, seed))
    Q, _ = torch.linalg.qr(M, mode="reduced")
    P = Q.t().to(dtype)
    P.requires_grad_(False)
    return P


def get_projection_initializer(method: str = "gaussian"):
    table = {
        "gaussian": init_projection_matrix_gaussian,
        "rademacher": init_projection_matrix_rademacher,
        "orthonormal": init_projection_matrix_orthonormal,
    }
    if method not in table:
        raise ValueError(f"Unknown projection method: {method}. Choose from {list(table.keys())}")
    return table[method]


def compute_projection_metadata(layer_name: str, layer: nn.Module, k_i: int, k_o: int) -> dict:
    """Per-layer entry of ``metadata.json``."""
    meta = {"name": layer_name, "type": layer.__class__.__name__, "k_i": k_i, "k_o": k_o,
            "k_total": k_i * k_o}
    if hasattr(layer, "weight"):
        shape = layer.weight.shape
        if isinstance(layer, nn.Linear):
            meta["n_o"], meta["n_i"] = shape
        elif isinstance(layer, nn.Conv1d):
            meta["n_o"] = shape[0]
            meta["n_i"] = shape[1] * shape[2]
        elif layer.__class__.__name__ == "Conv1D":
            meta["n_o"], meta["n_i"] = shape
    elif isinstance(layer, nn.Embedding):
        meta["vocab_size"] = layer.num_embeddings
        meta["n_i"] = layer.num_embeddings
        meta["n_o"] = layer.embedding_dim
    return meta


def projection_similarity(proj_a: torch.Tensor, proj_b: torch.Tensor) -> torch.Tensor:
    """Gradient-similarity scores ``proj_a @ proj_b.T`` between two sets of projected per-sample
    gradients (``[Na, D]``, ``[Nb, D]`` -> ``[Na, Nb]`` float32): the downstream step of the
    reference's examples (Examples/ghost_gradproj_lm.py:190-196;
    Examples/GradProj_LM/plot_error_with_dim.py:69-86), done while the projections are still on the
    device.  Batch-sized blocks (up to ``ops.SIMILARITY_KERNEL_MAX_ROWS`` rows each: the
    ``[B, total_proj_dim]`` buffers ``collect_batch`` returns) go through the library's streaming
    kernel, which reads both operands once; larger sets are a plain dense GEMM and use cuBLAS
    through torch, in full fp32 so that scores do not depend on the TF32 setting.  Host tensors
    are multiplied on the host."""
    if proj_a.shape[-1] != proj_b.shape[-1]:
        raise ValueError("projection sets have different dimensions")
    if proj_a.is_cuda and proj_b.is_cuda and proj_a.dim() == 2 and proj_b.dim() == 2 and \
            max(proj_a.shape[0], proj_b.shape[0]) <= ops.SIMILARITY_KERNEL_MAX_ROWS:
        return ops.projection_similarity(proj_a, proj_b)
    a, b = proj_a.float(), proj_b.float()
    if a.is_cuda:
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            return a @ b.t()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
    return a @ b.t()
