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


def test_shard_bounds_cover_everything():
    for n in (1, 7, 8, 65536):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = gdist.shard_bounds(n, r, world)
                seen.extend(range(lo, hi))
            assert seen == list(range(n))
    assert list(gdist.shard_indices(10, 1, 4)) == [3, 4, 5]
