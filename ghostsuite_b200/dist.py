"""Data-parallel use of the ghost engines inside one multi-GPU node.

GradDotProd: the train batch is sharded over ranks, the validation batch is replicated.  Each rank
runs forward/backward on ``cat(train_shard, val)``; afterwards

* the per-parameter dot-product blocks ``[n_val, n_train_local]`` are packed into one buffer and
  all-gathered (a few hundred KB), giving every rank the ``[n_val, n_train_global]`` matrices;
* the recovered train gradients (each the mean over the rank's own shard) are all-reduced in
  flat buckets and averaged.

With a ``mean`` loss every rank divides by its local batch size, so a local out-grad is
``N_global / N_local`` times what a single process over the global batch would see; dot products
are bilinear in the two gradients, hence the optional rescale by ``(N_local / N_global) ** 2``
(``single_process_equivalent=True``).  The averaged train gradient needs no rescale for equal
shards.

GradProj shards the corpus (:func:`shard_indices`) and needs no communication at all.

Only ``torch.distributed`` collectives on local buffers are used (NCCL on GPUs, gloo in the CPU
tests); no kernel reads another GPU's memory.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_items: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, near-equal split of ``range(n_items)``: ``[lo, hi)`` for ``rank``."""
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_indices(n_items: int, rank: int, world: int) -> range:
    """Corpus shard of a GradProj run (contiguous block; no communication needed afterwards)."""
    lo, hi = shard_bounds(n_items, rank, world)
    return range(lo, hi)


def shard_train_batch(x_train: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_bounds(x_train.shape[0], rank, world)
    return x_train[lo:hi]


def _dot_params(module: torch.nn.Module) -> List[Tuple[str, torch.Tensor]]:
    return [(n, p) for n, p in module.named_parameters()
            if hasattr(p, "grad_dot_prod_matrix") and getattr(p, "initially_requires_grad", True)]


def gather_dot_products(module: torch.nn.Module, group=None,
                        single_process_equivalent: bool = True) -> Dict[str, torch.Tensor]:
    """All-gather every parameter's ``[n_val, n_train_local]`` block along the train dimension
    (equal shard sizes) and store the global ``[n_val, n_train_global]`` matrix (and its column sums)
    back on the parameter.  One collective for all parameters."""
    world = dist.get_world_size(group)
    named = _dot_params(module)
    if not named:
        return {}
    packed = torch.stack([p.grad_dot_prod_matrix for _, p in named])       # [P, n_val, n_loc]
    P, n_val, n_loc = packed.shape
    gathered = torch.empty((world * P, n_val, n_loc), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(gathered, packed.contiguous(), group=group)
    full = gathered.view(world, P, n_val, n_loc).permute(1, 2, 0, 3).reshape(P, n_val, world * n_loc)
    if single_process_equivalent:
        n_local = n_val + n_loc
        n_global = n_val + world * n_loc
        full = full * (float(n_local) / float(n_global)) ** 2
    out = {}
    for i, (name, p) in enumerate(named):
        p.grad_dot_prod_matrix = full[i]
        p.grad_dot_prod = full[i].sum(dim=0)
        out[name] = full[i]
    return out


def allreduce_train_grads(module: torch.nn.Module, group=None, bucket_bytes: int = 256 << 20) -> int:
    """Average ``param.train_grad`` over ranks in flat buckets.  Returns the number of collectives."""
    world = dist.get_world_size(group)
    by_dtype: Dict[torch.dtype, List[torch.Tensor]] = {}
    for _, p in module.named_parameters():
        g = getattr(p, "train_grad", None)
        if g is not None:
            by_dtype.setdefault(g.dtype, []).append(g)
    calls = 0
    for dtype, grads in by_dtype.items():
        bucket: List[torch.Tensor] = []
        size = 0

        def flush():
            nonlocal bucket, size, calls
            if not bucket:
                return
            flat = torch.cat([g.reshape(-1) for g in bucket])
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
            flat.mul_(1.0 / world)
            off = 0
            for g in bucket:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g))
                off += n
            calls += 1
            bucket, size = [], 0

        for g in grads:
            bucket.append(g)
            size += g.numel() * g.element_size()
            if size >= bucket_bytes:
                flush()
        flush()
    return calls


def sync_engine(engine, group=None, single_process_equivalent: bool = True) -> None:
    """Call between ``loss.backward()`` and ``engine.prepare_gradients()`` on every rank."""
    gather_dot_products(engine.module, group, single_process_equivalent)
    allreduce_train_grads(engine.module, group)
