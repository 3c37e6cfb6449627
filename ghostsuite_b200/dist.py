"""Data-parallel use of the ghost engines inside one multi-GPU node.

GradDotProd: the train batch is sharded over ranks, the validation batch is replicated.  Each rank
runs forward/backward on ``cat(train_shard, val)``; afterwards

* the per-parameter dot-product blocks ``[n_val, n_train_local]`` are packed into one buffer and
  all-gathered (a few hundred KB), giving every rank the ``[n_val, n_train_global]`` matrices;
* the recovered train gradients (each the mean over the rank's own shard) are all-reduced in
  flat buckets and averaged -- after the backward pass (:func:`allreduce_train_grads`) or, with
  :func:`overlap_train_grad_sync`, bucket by bucket while the backward pass is still running.

With a ``mean`` loss every rank divides by its local batch size, so a local out-grad is
``N_global / N_local`` times what a single process over the global batch would see; dot products
are bilinear in the two gradients, hence the optional rescale by ``(N_local / N_global) ** 2``
(``single_process_equivalent=True``).  The averaged train gradient needs no rescale for equal
shards.

GradProj shards the corpus (:func:`shard_indices`) and needs no communication at all.

With :func:`shard_validation` the validation batch is split over the ranks as well: every rank runs
``cat(train_shard, val_shard)`` through the model, and in each hooked layer the other ranks'
validation rows of the two operands are all-gathered into local buffers before the kernels run.

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
    """Rank ``rank``'s block of the train batch.  The batch must divide by ``world``: the all-gather of
    the dot-product blocks, the ``(N_local / N_global) ** 2`` rescale and the plain average of the
    train gradients all rely on equal shards."""
    n = int(x_train.shape[0])
    if n % world != 0:
        raise ValueError(f"train batch of {n} samples does not divide over {world} ranks; the "
                         "data-parallel GradDotProd path needs equal shards")
    lo, hi = shard_bounds(n, rank, world)
    return x_train[lo:hi]


def _dot_params(module: torch.nn.Module) -> List[Tuple[str, torch.Tensor]]:
    return [(n, p) for n, p in module.named_parameters()
            if hasattr(p, "grad_dot_prod_matrix") and getattr(p, "initially_requires_grad", True)]


def gather_dot_products(module: torch.nn.Module, group=None,
                        single_process_equivalent: bool = True,
                        check_equal_shards: bool = True,
                        n_val_local: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """All-gather every parameter's ``[n_val, n_train_local]`` block along the train dimension
    (equal shard sizes) and store the global ``[n_val, n_train_global]`` matrix (and its column sums)
    back on the parameter.  One collective for all parameters, preceded by a four-integer MIN
    all-reduce that makes unequal shards raise ``ValueError`` on every rank instead of reaching the
    all-gather (``check_equal_shards=False`` skips it when the caller has sharded with
    :func:`shard_train_batch`, which enforces equal shards itself)."""
    world = dist.get_world_size(group)
    named = _dot_params(module)
    if not named:
        return {}
    packed = torch.stack([p.grad_dot_prod_matrix for _, p in named])       # [P, n_val, n_loc]
    P, n_val, n_loc = packed.shape
    if check_equal_shards:
        # a rank with a different shard size would hand the all-gather a buffer of another size
        # (undefined under NCCL): compare sizes first, one tiny collective
        probe = torch.tensor([n_loc, -n_loc, P, -P], dtype=torch.int64, device=packed.device)
        dist.all_reduce(probe, op=dist.ReduceOp.MIN, group=group)
        lo_n, hi_n, lo_p, hi_p = int(probe[0]), -int(probe[1]), int(probe[2]), -int(probe[3])
        if lo_n != hi_n or lo_p != hi_p:
            raise ValueError(f"ranks disagree on the dot-product blocks (train samples per rank {lo_n}..{hi_n}, "
                             f"parameters {lo_p}..{hi_p}); the data-parallel path needs equal shards")
    gathered = torch.empty((world * P, n_val, n_loc), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(gathered, packed.contiguous(), group=group)
    full = gathered.view(world, P, n_val, n_loc).permute(1, 2, 0, 3).reshape(P, n_val, world * n_loc)
    if single_process_equivalent:
        # samples in this rank's loss mean against samples in the single-process loss mean
        n_local = (n_val if n_val_local is None else int(n_val_local)) + n_loc
        n_global = n_val + world * n_loc
        full = full * (float(n_local) / float(n_global)) ** 2
    vectors = full.sum(dim=1)                      # one reduction for all parameters
    out = {}
    for i, (name, p) in enumerate(named):
        p.grad_dot_prod_matrix = full[i]
        p.grad_dot_prod = vectors[i]
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


class OverlappedGradSync:
    """All-reduce of the train gradients started bucket by bucket while the backward pass is still
    running.

    The hooks report every contribution to ``param.train_grad``; a parameter is final once all the
    hooked layers that own it have reported (a tied table gets two contributions).  Final gradients
    are collected into a bucket; a full bucket is flattened and all-reduced asynchronously (NCCL on
    its own stream), and :meth:`finish` flushes the rest, waits and copies the averages back.  The
    order in which parameters become final is the backward order, identical on every rank.
    """

    def __init__(self, module: torch.nn.Module, group=None, bucket_bytes: int = 32 << 20):
        from .ghostEngines import supported_layers_grad_samplers_dotprod as layers
        self._layers = layers
        self.module = module
        self.group = group
        self.bucket_bytes = int(bucket_bytes)
        self.world = dist.get_world_size(group)
        self.avg_op = dist.ReduceOp.AVG if dist.get_backend(group) == "nccl" else dist.ReduceOp.SUM
        # number of hooked layers contributing to each parameter
        self.expected: Dict[int, int] = {}
        for layer in module.modules():
            if type(layer) in layers._supported_layers_dotprod:
                for prm in layer.parameters(recurse=False):
                    if getattr(prm, "initially_requires_grad", prm.requires_grad):
                        self.expected[id(prm)] = self.expected.get(id(prm), 0) + 1
        self._seen: Dict[int, int] = {}
        self._bucket: List[Tuple[int, torch.Tensor]] = []
        self._bucket_size = 0
        self._bucket_dtype = None
        self._inflight: List[Tuple[object, torch.Tensor, List[Tuple[int, torch.Tensor]]]] = []
        self._reduced: set = set()
        self._dirty: set = set()
        layers.TRAIN_GRAD_OBSERVER = self._on_train_grad

    def close(self) -> None:
        if self._layers.TRAIN_GRAD_OBSERVER == self._on_train_grad:
            self._layers.TRAIN_GRAD_OBSERVER = None

    # ------------------------------------------------------------------ during backward
    def _on_train_grad(self, param: torch.Tensor) -> None:
        key = id(param)
        if key not in self.expected:
            return
        seen = self._seen.get(key, 0) + 1
        self._seen[key] = seen
        if seen < self.expected[key]:
            return                                   # another layer still adds to this gradient
        if seen > self.expected[key]:
            # More contributions than hooked layers: a second backward pass before finish() (gradient
            # accumulation) or a module called twice in one forward.  The gradient was queued after
            # its first complete set of contributions and has been added to since, so whatever was
            # (or will be) reduced for it is stale: finish() drops that and reduces the final tensor.
            self._dirty.add(key)
            return
        self._enqueue(key, param.train_grad)

    def _enqueue(self, key: int, g: torch.Tensor) -> None:
        if self._bucket and g.dtype != self._bucket_dtype:
            self._flush()
        self._bucket.append((key, g))
        self._bucket_dtype = g.dtype
        self._bucket_size += g.numel() * g.element_size()
        self._reduced.add(key)
        if self._bucket_size >= self.bucket_bytes:
            self._flush()

    def _flush(self) -> None:
        if not self._bucket:
            return
        entries = self._bucket
        flat = torch.cat([g.reshape(-1) for _, g in entries])
        work = dist.all_reduce(flat, op=self.avg_op, group=self.group, async_op=True)
        self._inflight.append((work, flat, entries))
        self._bucket, self._bucket_size, self._bucket_dtype = [], 0, None

    # ------------------------------------------------------------------ after backward
    def finish(self) -> int:
        """Flush, wait for every bucket, write the averages back.  Gradients that never reported
        (parameters of layers without hooks) and gradients that were added to after they had been
        queued are averaged here in one more bucket.  Returns the number of collectives of this
        pass."""
        dirty = self._dirty
        if dirty:
            kept = [(k, g) for k, g in self._bucket if k not in dirty]
            self._bucket = kept
            self._bucket_size = sum(g.numel() * g.element_size() for _, g in kept)
            self._reduced -= dirty
        n_early = len(self._inflight)          # buckets that went out during the backward pass
        for _, prm in self.module.named_parameters():
            g = getattr(prm, "train_grad", None)
            if g is not None and id(prm) not in self._reduced:
                self._enqueue(id(prm), g)
        self._flush()
        calls = len(self._inflight)
        for i, (work, flat, entries) in enumerate(self._inflight):
            work.wait()
            if self.avg_op == dist.ReduceOp.SUM:
                flat.mul_(1.0 / self.world)
            pieces = flat.split([g.numel() for _, g in entries])
            dst, src = [], []
            for (k, g), pc in zip(entries, pieces):
                # an early bucket's snapshot of a gradient that was added to afterwards is stale: it
                # is not copied back; the same gradient sits, complete, in one of the last buckets
                if i >= n_early or k not in dirty:
                    dst.append(g)
                    src.append(pc.view_as(g))
            if dst:
                torch._foreach_copy_(dst, src)
        self._inflight.clear()
        self._seen.clear()
        self._reduced.clear()
        self._dirty.clear()
        return calls


class ShardedValidation:
    """Splits the validation batch over the ranks.

    Rank ``r`` runs ``cat(train_shard_r, val[r * v : (r + 1) * v])`` (``v = n_val / world``) through the
    model, with the engine built for ``val_batch_size = v``.  In every hooked layer's backward hook this
    object replaces the layer's operands ``A`` and ``B`` (``[n_train_local + v, ...]``) by
    ``cat(train rows, all ranks' validation rows)`` -- one ``all_gather_into_tensor`` per operand
    straight into the tail of a new local buffer -- and reports ``n_val`` validation samples, so the
    layer functions and kernels work exactly as with a replicated validation batch while the model's
    forward and backward pass cover ``1 / world`` of it.  Every rank's loss is a mean over the same
    number of samples, so all gathered out-grads carry the same factor.
    """

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.calls = 0
        self.bytes = 0

    def __call__(self, layer, A: torch.Tensor, B: torch.Tensor, n_val_local: int):
        if self.world == 1:
            return A, B, n_val_local
        n_train = A.shape[0] - n_val_local
        if n_train <= 0 or n_val_local <= 0 or B.shape[0] != A.shape[0]:
            raise ValueError("sharded validation needs train and validation rows in every rank's batch")
        out = []
        for x in (A, B):
            x = x.contiguous()
            full = x.new_empty((n_train + n_val_local * self.world,) + tuple(x.shape[1:]))
            full[:n_train].copy_(x[:n_train])
            dist.all_gather_into_tensor(full[n_train:], x[n_train:], group=self.group)
            self.calls += 1
            self.bytes += full[n_train:].numel() * full.element_size()
            out.append(full)
        return out[0], out[1], n_val_local * self.world


def _require_equal_validation_shards(engine, group=None) -> None:
    """Every all-gather of validation rows hands NCCL one buffer per rank of the same size: ranks that
    hold different numbers of validation samples would stall it.  One two-integer collective when
    the split is installed makes that a ``ValueError`` on every rank instead."""
    n = int(engine.val_batch_size)
    params = [p for p in engine.module.parameters()]
    device = params[0].device if params else torch.device("cpu")
    probe = torch.tensor([n, -n], dtype=torch.int64, device=device)
    dist.all_reduce(probe, op=dist.ReduceOp.MIN, group=group)
    lo, hi = int(probe[0]), -int(probe[1])
    if lo != hi or n <= 0:
        raise ValueError(f"ranks hold {lo}..{hi} validation samples; a split validation batch needs the same "
                         "positive number on every rank")


class ValidationExchange:
    """What the layer functions need to exchange validation gradients (``gather_rows``): an
    all-gather along dimension 0 into a new local tensor, rank-major."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.calls = 0
        self.bytes = 0

    def gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous()
        out = x.new_empty((x.shape[0] * self.world,) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x, group=self.group)
        self.calls += 1
        self.bytes += out.numel() * out.element_size()
        return out

    def gather_rows_async(self, x: torch.Tensor, out: Optional[torch.Tensor] = None):
        """``(out, work)``: the all-gather is enqueued behind what the current stream holds so far and
        nothing waits for it until ``work.wait()``.  ``out`` may be the contiguous tail of a larger
        tensor."""
        x = x.contiguous()
        if out is None:
            out = x.new_empty((x.shape[0] * self.world,) + tuple(x.shape[1:]))
        work = dist.all_gather_into_tensor(out, x, group=self.group, async_op=True)
        self.calls += 1
        self.bytes += out.numel() * out.element_size()
        return out, work


def exchange_validation(engine, group=None, exchange_group=None) -> ValidationExchange:
    """:func:`shard_validation` with the cheaper exchange where a layer allows it: on the per-sample
    path of Linear / Conv1D layers every rank computes the gradient tiles of its own validation
    samples and the ranks all-gather those (``2 * n_val * d * p`` bytes per layer) instead of the
    validation rows of both operands, and no rank repeats another rank's validation GEMMs; bias and
    norm layers exchange their per-sample vectors.  Other layers (Gram path, embeddings) gather
    operands as :class:`ShardedValidation` does.  ``exchange_group`` (same ranks as ``group``) gives the
    tile and vector all-gathers a communicator of their own, so that they do not queue behind the
    gradient all-reduces of :func:`overlap_train_grad_sync`.  Undo with :func:`unshard_validation`."""
    from .ghostEngines import supported_layers_grad_samplers_dotprod as layers
    shard_validation(engine, group)
    ex = ValidationExchange(exchange_group if exchange_group is not None else group)
    layers.VALIDATION_EXCHANGE = ex
    engine._ghost_val_exchange = ex
    return ex


def shard_validation(engine, group=None) -> ShardedValidation:
    """Install :class:`ShardedValidation` for the hooks of ``engine`` (built with the per-rank
    validation count).  Pass ``n_val_local`` to :func:`sync_engine` afterwards; undo with
    :func:`unshard_validation`."""
    from .ghostEngines import autograd_grad_sample_dotprod as plumbing
    _require_equal_validation_shards(engine, group)
    sv = ShardedValidation(group)
    plumbing.VALIDATION_GATHER = sv
    engine._ghost_val_shard = sv
    return sv


def unshard_validation(engine=None) -> None:
    from .ghostEngines import autograd_grad_sample_dotprod as plumbing
    from .ghostEngines import supported_layers_grad_samplers_dotprod as layers
    plumbing.VALIDATION_GATHER = None
    layers.VALIDATION_EXCHANGE = None
    if engine is not None:
        for attr in ("_ghost_val_shard", "_ghost_val_exchange"):
            if hasattr(engine, attr):
                delattr(engine, attr)


def overlap_train_grad_sync(engine, group=None, bucket_bytes: int = 32 << 20) -> OverlappedGradSync:
    """Start all-reducing finished train gradients during the backward pass; :func:`sync_engine`
    then only has to wait for them.  Call once after ``engine.attach``."""
    sync = OverlappedGradSync(engine.module, group, bucket_bytes)
    engine._ghost_grad_sync = sync
    return sync


def sync_engine(engine, group=None, single_process_equivalent: bool = True,
                check_equal_shards: bool = True) -> None:
    """Call between ``loss.backward()`` and ``engine.prepare_gradients()`` on every rank."""
    n_val_local = engine.val_batch_size if getattr(engine, "_ghost_val_shard", None) is not None else None
    gather_dot_products(engine.module, group, single_process_equivalent, check_equal_shards, n_val_local)
    overlapped = getattr(engine, "_ghost_grad_sync", None)
    if overlapped is not None:
        overlapped.finish()
    else:
        allreduce_train_grads(engine.module, group)
