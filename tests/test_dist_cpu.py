"""Multi-rank logic of the data-parallel path on CPU ranks (gloo, world_size 2)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from ghostsuite_b200 import dist as gdist
from oracle.ghost_engine_cpu import OracleDotProdEngine


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q, overlap=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        n_t_global, n_v, d = 8, 3, 12
        model = nn.Sequential(nn.Linear(d, 16), nn.ReLU(), nn.Linear(16, 5))
        X_train = torch.randn(n_t_global, d)
        Y_train = torch.randint(0, 5, (n_t_global,))
        X_val = torch.randn(n_v, d)
        Y_val = torch.randint(0, 5, (n_v,))

        # single-process result over the global batch
        ref = nn.Sequential(nn.Linear(d, 16), nn.ReLU(), nn.Linear(16, 5))
        ref.load_state_dict(model.state_dict())
        e_ref = OracleDotProdEngine(ref, n_v, exact=True)
        e_ref.attach()
        nn.functional.cross_entropy(ref(torch.cat((X_train, X_val))), torch.cat((Y_train, Y_val))).backward()

        # sharded run
        eng = OracleDotProdEngine(model, n_v, exact=True)
        eng.attach()
        xs = gdist.shard_train_batch(X_train, rank, world)
        ys = gdist.shard_train_batch(Y_train, rank, world)
        nn.functional.cross_entropy(model(torch.cat((xs, X_val))), torch.cat((ys, Y_val))).backward()
        for p in model.parameters():     # the CUDA engine produces float32 matrices
            p.grad_dot_prod_matrix = p.grad_dot_prod_matrix.float()
            p.train_grad = p.train_grad.float()

        class E:
            module = model
        if overlap:
            # the hooks of the CUDA engine report every finished train gradient in backward order;
            # tiny buckets force several collectives
            sync = gdist.overlap_train_grad_sync(E, None, bucket_bytes=256)
            for p in reversed(list(model.parameters())):
                sync._on_train_grad(p)
            assert len(sync._inflight) >= 1              # something went out before finish()
        gdist.sync_engine(E, None)
        if overlap:
            sync.close()
        ok = True
        for (name, p), (_, r) in zip(model.named_parameters(), ref.named_parameters()):
            m_err = (p.grad_dot_prod_matrix.double() - r.grad_dot_prod_matrix).norm() / r.grad_dot_prod_matrix.norm()
            g_err = (p.train_grad.double() - r.train_grad.double()).norm() / r.train_grad.double().norm()
            v_err = (p.grad_dot_prod.double() - r.grad_dot_prod_matrix.sum(0)).norm() / r.grad_dot_prod_matrix.sum(0).norm()
            ok = ok and p.grad_dot_prod_matrix.shape == (n_v, n_t_global)
            ok = ok and m_err < 1e-5 and g_err < 1e-5 and v_err < 1e-5
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("overlap", [False, True])
def test_sharded_run_reproduces_single_process_numbers(overlap):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, overlap)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def _run_ranks(target, world=2, args=()):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q) + tuple(args)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(results)


def _worker_unequal(rank, world, port, q):
    """Ranks that hold different numbers of train samples: the gather must raise on every rank
    instead of calling the all-gather with mismatched buffers."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = nn.Linear(4, 3)
        n_loc = 3 + rank                                  # 3 on rank 0, 4 on rank 1
        for p in model.parameters():
            p.initially_requires_grad = True
            p.grad_dot_prod_matrix = torch.ones(2, n_loc)
        try:
            gdist.gather_dot_products(model, None)
            raised = False
        except ValueError as exc:
            raised = "equal shards" in str(exc)
        q.put((rank, raised))
    finally:
        dist.destroy_process_group()


def test_unequal_shards_raise():
    with pytest.raises(ValueError, match="does not divide"):
        gdist.shard_train_batch(torch.zeros(7, 3), 0, 2)
    assert gdist.shard_train_batch(torch.zeros(8, 3), 1, 2).shape[0] == 4
    assert _run_ranks(_worker_unequal) == [(0, True), (1, True)]


def _worker_two_backwards(rank, world, port, q):
    """Gradient accumulation: two backward passes report every parameter twice before the sync.  The
    overlapped path must average the final sums, exactly like the plain bucketed all-reduce."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        n_v, d = 2, 6
        model = nn.Sequential(nn.Linear(d, 8), nn.ReLU(), nn.Linear(8, 3))
        twin = nn.Sequential(nn.Linear(d, 8), nn.ReLU(), nn.Linear(8, 3))
        twin.load_state_dict(model.state_dict())
        g = torch.Generator().manual_seed(10 + rank)      # every rank has its own micro-batches
        micro = [(torch.randn(4 + n_v, d, generator=g), torch.randint(0, 3, (4 + n_v,), generator=g))
                 for _ in range(2)]

        class E:
            module = model

        class T:
            module = twin
        eng = OracleDotProdEngine(model, n_v, exact=True)
        eng.attach()
        ref = OracleDotProdEngine(twin, n_v, exact=True)
        ref.attach()
        sync = gdist.overlap_train_grad_sync(E, None, bucket_bytes=64)     # tiny buckets: sent at once
        for x, y in micro:
            nn.functional.cross_entropy(model(x), y).backward()
            nn.functional.cross_entropy(twin(x), y).backward()
            for p in reversed(list(model.parameters())):                   # what the CUDA hooks report
                sync._on_train_grad(p)
        for m in (model, twin):
            for p in m.parameters():
                p.grad_dot_prod_matrix = p.grad_dot_prod_matrix.float()
                p.train_grad = p.train_grad.float() if p.train_grad.dtype != torch.float32 else p.train_grad
        early = len(sync._inflight)
        gdist.sync_engine(E, None)
        sync.close()
        gdist.gather_dot_products(twin, None)
        gdist.allreduce_train_grads(twin, None)
        ok = early >= 1 and len(sync._dirty) == 0
        for p, r in zip(model.parameters(), twin.parameters()):
            ok = ok and bool(torch.allclose(p.train_grad, r.train_grad, rtol=1e-6, atol=1e-7))
        # and the averages really are cross-rank means: all ranks now hold the same tensors
        flat = torch.cat([p.train_grad.reshape(-1) for p in model.parameters()])
        both = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(both, flat)
        ok = ok and bool(torch.equal(both[0], both[1]))
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_overlapped_sync_with_two_backward_passes():
    assert _run_ranks(_worker_two_backwards) == [(0, True), (1, True)]


def _worker_val_shard(rank, world, port, q):
    """Validation batch split over ranks: after the per-layer gather every rank holds
    cat(own train rows, all validation rows), and the blocks it computes, gathered and rescaled,
    reproduce the single-process matrix over the global batch."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import ghost_oracle as O
        g = torch.Generator().manual_seed(3)
        n_t, n_v, T, d, p = 4, 2, 5, 6, 7
        A = torch.randn(n_t + n_v, T, d, generator=g)            # the global batch, train first
        G = torch.randn(n_t + n_v, T, p, generator=g)
        ids = torch.randint(0, 50, (n_t + n_v, T), generator=g)
        t_lo, t_hi = gdist.shard_bounds(n_t, rank, world)
        v_lo, v_hi = gdist.shard_bounds(n_v, rank, world)
        rows = list(range(t_lo, t_hi)) + list(range(n_t + v_lo, n_t + v_hi))
        n_global, n_local = n_t + n_v, len(rows)
        # a mean loss over the local batch makes every local out-grad n_global / n_local times larger
        G_loc = G[rows] * (n_global / n_local)
        sv = gdist.ShardedValidation(None)
        A_full, G_full, nv = sv(None, A[rows], G_loc, v_hi - v_lo)
        ok = nv == n_v and A_full.shape[0] == (t_hi - t_lo) + n_v
        ok = ok and torch.equal(A_full, torch.cat((A[t_lo:t_hi], A[n_t:])))
        ok = ok and torch.allclose(G_full, torch.cat((G[t_lo:t_hi], G[n_t:])) * (n_global / n_local))
        ids_full, _, _ = sv(None, ids[rows], G_loc, v_hi - v_lo)
        ok = ok and ids_full.dtype == torch.int64 and torch.equal(ids_full, torch.cat((ids[t_lo:t_hi], ids[n_t:])))
        # the local block -> gathered, rescaled -> the global matrix
        lin = nn.Linear(d, p, bias=False)
        lin.weight.initially_requires_grad = True
        lin.weight.grad_dot_prod_matrix = O.linear_dot_exact(A_full, G_full, n_v).float()
        full = gdist.gather_dot_products(lin, None, n_val_local=v_hi - v_lo)["weight"]
        want = O.linear_dot_exact(A, G, n_v)
        ok = ok and full.shape == (n_v, n_t) and float((full.double() - want).norm() / want.norm()) < 1e-5
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_sharded_validation_gather():
    assert _run_ranks(_worker_val_shard) == [(0, True), (1, True)]


def _worker_val_exchange(rank, world, port, q):
    """Validation batch split over ranks with per-sample GRADIENTS exchanged: the all-gather of the
    validation rows of per-sample vectors, blocking and non-blocking (into the tail of a larger
    tensor, waited for when the backward pass ends), gives cat(own train rows, all validation rows)
    in rank order."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ghostsuite_b200.ghostEngines import supported_layers_grad_samplers_dotprod as L
        g = torch.Generator().manual_seed(5)
        n_t, n_v, F = 4, 4, 6
        X = torch.randn(n_t + n_v, F, generator=g)               # per-sample vectors of the global batch
        t_lo, t_hi = gdist.shard_bounds(n_t, rank, world)
        v_lo, v_hi = gdist.shard_bounds(n_v, rank, world)
        x_loc = torch.cat((X[t_lo:t_hi], X[n_t + v_lo:n_t + v_hi]))
        want = torch.cat((X[t_lo:t_hi], X[n_t:]))
        ex = gdist.ValidationExchange(None)
        ok = ex.world == world
        ok = ok and torch.equal(L._with_gathered_val_rows(x_loc, t_hi - t_lo, ex), want)      # nothing deferred
        tiles = torch.arange(2 * 3 * (v_hi - v_lo) * 4, dtype=torch.float32).reshape(1, 2 * 3, v_hi - v_lo, 4) + 1000 * rank
        both = ex.gather_rows(tiles)                              # [ranks, tiles, per rank, elems], rank-major
        ok = ok and both.shape[0] == world and torch.equal(both[rank], tiles[0]) and float(both[1 - rank][0, 0, 0]) == 1000.0 * (1 - rank)
        # inside a backward pass the vectors of all layers cross the ranks in one packed all-gather
        Y = torch.randn(n_t + n_v, 10, generator=g)
        y_loc = torch.cat((Y[t_lo:t_hi], Y[n_t + v_lo:n_t + v_hi]))
        jobs = []
        for vec in (x_loc, y_loc):
            jobs.append({"X": vec, "n_train": t_hi - t_lo, "n_val": n_v, "M": torch.empty(n_v, t_hi - t_lo),
                         "val_exchange": ex})
        jobs.append({"X": x_loc, "n_train": t_hi - t_lo, "n_val": n_v, "sum_out": torch.empty(F)})   # no exchange
        L._exchange_pending_val_rows(jobs)
        ok = ok and "Xv" not in jobs[2] and ex.calls == 3
        for job, full in zip(jobs[:2], (X, Y)):
            gathered, off, per = job["Xv"]
            width = job["X"].shape[1]
            ok = ok and gathered.shape == (world, per * (F + 10)) and per == v_hi - v_lo
            for v in range(n_v):
                row = gathered[v // per, off + (v % per) * width: off + (v % per + 1) * width]
                ok = ok and torch.equal(row, full[n_t + v])
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def _worker_val_unequal(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        class Eng:
            module = nn.Linear(3, 2)
            val_batch_size = 2 + rank
        raised = 0
        for install in (gdist.shard_validation, gdist.exchange_validation):
            try:
                install(Eng(), None)
            except ValueError:
                raised += 1
            finally:
                gdist.unshard_validation()
        Eng.val_batch_size = 2
        ok = raised == 2 and isinstance(gdist.exchange_validation(Eng(), None), gdist.ValidationExchange)
        gdist.unshard_validation()
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_unequal_validation_shards_raise():
    assert _run_ranks(_worker_val_unequal) == [(0, True), (1, True)]


def test_validation_gradient_exchange_of_vectors():
    assert _run_ranks(_worker_val_exchange) == [(0, True), (1, True)]


def test_shard_bounds_cover_everything():
    for n in (1, 7, 8, 65536):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = gdist.shard_bounds(n, r, world)
                seen.extend(range(lo, hi))
            assert seen == list(range(n))
    assert list(gdist.shard_indices(10, 1, 4)) == [3, 4, 5]
