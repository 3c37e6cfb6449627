"""Pins the CPU oracle against outputs of the reference's own functions (tests/golden)."""
import numpy as np
import pytest
import torch

from conftest import as_dtype
from oracle import ghost_oracle as O

N_T, N_V = 5, 3
N = N_T + N_V


def close(x, ref, rtol, atol=0.0):
    x = torch.as_tensor(np.asarray(x)).double()
    ref = torch.as_tensor(np.asarray(ref)).double()
    assert x.shape == ref.shape
    assert torch.allclose(x, ref, rtol=rtol, atol=atol), (x, ref)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
@pytest.mark.parametrize("nv", [1, N_V])
@pytest.mark.parametrize("ghost", [True, False])
def test_linear_and_conv1d_reference_restatement(golden, tag, nv, ghost):
    A = as_dtype(golden[f"lin_{tag}_A"], tag)
    G = as_dtype(golden[f"lin_{tag}_G"], tag)
    got = O.linear_dot_reference(A, G, nv, ghost).float()
    close(got, golden[f"lin_{tag}_nv{nv}_ghost{int(ghost)}_w"], rtol=2e-2 if tag == "bf16" or ghost else 1e-5,
          atol=1e-2 if tag == "bf16" or ghost else 1e-6)
    got = O.conv1d_dot_reference(A, G, nv, ghost).float()
    close(got, golden[f"c1d_{tag}_nv{nv}_ghost{int(ghost)}_w"], rtol=2e-2, atol=1e-2)
    close(O.bias_dot_reference(G, nv).float(), golden[f"lin_{tag}_nv{nv}_ghost{int(ghost)}_b"],
          rtol=2e-2 if tag == "bf16" else 1e-5, atol=1e-2 if tag == "bf16" else 1e-6)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_exact_matrix_matches_reference_rows(golden, tag):
    """The float64 matrix equals the reference's materialised branch called per validation row."""
    A = as_dtype(golden[f"lin_{tag}_A"], tag)
    G = as_dtype(golden[f"lin_{tag}_G"], tag)
    M = O.linear_dot_exact(A, G, N_V)
    M2 = O.linear_dot_persample_exact(A, G, N_V)
    assert O.rel_fro(M, M2) < 1e-12
    rows = torch.from_numpy(golden[f"lin_{tag}_rows_materialised"])
    assert O.rel_fro(rows, M) < (1e-5 if tag == "f32" else 2e-2)
    # reference at n_val = 1: every branch is algebraically right
    for ghost in (True, False):
        ref1 = torch.from_numpy(golden[f"lin_{tag}_nv1_ghost{int(ghost)}_w"])
        M1 = O.linear_dot_exact(A, G, 1)[0]
        assert O.rel_fro(ref1, M1) < (1e-5 if (tag == "f32" and not ghost) else 2e-2)
        c1 = torch.from_numpy(golden[f"c1d_{tag}_nv1_ghost{int(ghost)}_w"])
        assert O.rel_fro(c1, M1) < 2e-2
    # ghost branch with several validation samples: the vector is the column sum of M
    refv = torch.from_numpy(golden[f"lin_{tag}_nv{N_V}_ghost1_w"])
    assert O.rel_fro(refv, M.sum(0)) < 2e-2
    # bias
    Mb = O.bias_dot_exact(G, N_V)
    refb = torch.from_numpy(golden[f"lin_{tag}_nv{N_V}_ghost1_b"])
    assert O.rel_fro(refb, Mb.sum(0)) < (1e-5 if tag == "f32" else 2e-2)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_train_grads(golden, tag):
    A = as_dtype(golden[f"lin_{tag}_A"], tag)
    G = as_dtype(golden[f"lin_{tag}_G"], tag)
    Gs = G * N
    tol = dict(rtol=1e-5, atol=1e-6) if tag == "f32" else dict(rtol=2e-2, atol=1e-2)
    close(O.linear_train_grad(A, Gs, N_V).float(), golden[f"lin_{tag}_train_grad"], **tol)
    close(O.conv1d_train_grad(A, Gs, N_V).float(), golden[f"c1d_{tag}_train_grad"], **tol)
    close(O.bias_train_grad(Gs.clone(), N_V).float(), golden[f"bias_{tag}_train_grad"], **tol)


def test_linear_2d(golden):
    A = torch.from_numpy(golden["lin2d_A"])
    G = torch.from_numpy(golden["lin2d_G"])
    M = O.linear_dot_exact(A, G, 4)
    assert O.rel_fro(torch.from_numpy(golden["lin2d_nv4_w"]), M.sum(0)) < 2e-2
    close(O.linear_dot_reference(A, G, 4, True), golden["lin2d_nv4_w"], rtol=1e-2, atol=1e-2)
    close(O.bias_dot_exact(G, 4).sum(0), golden["lin2d_nv4_b"], rtol=1e-5, atol=1e-5)
    close(O.linear_train_grad(A, G * 12, 4), golden["lin2d_train_grad"], rtol=1e-5, atol=1e-6)


def test_heuristic(golden):
    for T, d, p, flag in golden["heuristic_table"]:
        assert O.use_gram_rule(int(T), int(d) * int(p)) == bool(flag)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_embedding(golden, tag):
    ids = torch.from_numpy(golden["emb_ids"])
    G = as_dtype(golden[f"emb_{tag}_G"], tag)
    vocab = 11
    for nv in (1, N_V):
        ref = torch.from_numpy(golden[f"emb_{tag}_nv{nv}_w"])
        got = O.embedding_dot_reference(ids, G, nv, vocab)
        close(got, ref, rtol=1e-2, atol=1e-2)
        M = O.embedding_dot_exact(ids, G, nv)
        assert O.rel_fro(ref, M.sum(0)) < 2e-2
    Gs = G * N
    ref = golden[f"emb_{tag}_train_grad"]
    seq = O.embedding_train_grad(ids, Gs, N_V, vocab, sequential=True)
    # the CPU index_add_ is a sequential loop: the explicit loop is bit-identical to it
    assert np.array_equal(seq.float().numpy(), ref)
    fast = O.embedding_train_grad(ids, Gs, N_V, vocab, sequential=False)
    assert np.array_equal(fast.float().numpy(), ref)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_layernorm(golden, tag):
    A = as_dtype(golden[f"ln_{tag}_A"], tag)
    G = as_dtype(golden[f"ln_{tag}_G"], tag)
    eps = float(golden["ln_eps"][0])
    for nv in (1, N_V):
        w, b = O.layernorm_dot_reference(A, G, nv, eps)
        close(w, golden[f"ln_{tag}_nv{nv}_w"], rtol=1e-3, atol=1e-3)
        close(b, golden[f"ln_{tag}_nv{nv}_b"], rtol=1e-3, atol=1e-3)
        Mw, Mb = O.layernorm_dot_exact(A, G, nv, eps)
        assert O.rel_fro(torch.from_numpy(golden[f"ln_{tag}_nv{nv}_w"]), Mw.sum(0)) < 2e-2
        assert O.rel_fro(torch.from_numpy(golden[f"ln_{tag}_nv{nv}_b"]), Mb.sum(0)) < 2e-2
    gw, gb = O.layernorm_train_grad(A, G * N, N_V, eps)
    tol = dict(rtol=1e-5, atol=1e-5) if tag == "f32" else dict(rtol=2e-2, atol=2e-2)
    close(gw.float(), golden[f"ln_{tag}_train_grad_w"], **tol)
    close(gb.float(), golden[f"ln_{tag}_train_grad_b"], **tol)
    # exact per-sample vectors reproduce the train gradients: mean over train of N * gw
    pw, pb = O.layernorm_persample_exact(A, G, eps)
    assert O.rel_fro(torch.from_numpy(golden[f"ln_{tag}_train_grad_w"]),
                     pw[:N_T].sum(0) * N / N_T) < (1e-5 if tag == "f32" else 2e-2)


def test_gradproj_dense(golden):
    A = torch.from_numpy(golden["lin_f32_A"])
    G = torch.from_numpy(golden["lin_f32_G"])
    got = O.gradproj_dense(A, G, torch.from_numpy(golden["gp_P_i"]), torch.from_numpy(golden["gp_P_o"]))
    close(got, golden["gp_linear"], rtol=1e-5, atol=1e-6)
    got = O.gradproj_dense(A, G, torch.from_numpy(golden["gp_c1d_P_i"]),
                           torch.from_numpy(golden["gp_c1d_P_o"]), conv1d=True)
    close(got, golden["gp_c1d"], rtol=1e-5, atol=1e-6)
    # naive: materialise each sample's weight gradient, then project (Examples/ghost_gradproj_mlp.py:52-82)
    grads = torch.einsum("btp,btd->bpd", G.double(), A.double()) * A.shape[0]
    naive = torch.from_numpy(golden["gp_P_o"]).double() @ grads @ torch.from_numpy(golden["gp_P_i"]).double().t()
    close(torch.from_numpy(golden["gp_linear"]), naive, rtol=1e-4, atol=1e-5)


def test_gradproj_embedding(golden):
    """The vectorised restatement against the reference's per-token Python loop."""
    ids = torch.from_numpy(golden["gp_emb_ids"])
    G = torch.from_numpy(golden["gp_emb_G"])
    P_i = torch.from_numpy(golden["gp_emb_P_i"])
    P_o = torch.from_numpy(golden["gp_emb_P_o"])
    got = O.gradproj_embedding(ids, G, P_i, P_o)
    ref = torch.from_numpy(golden["gp_emb"])
    assert got.shape == ref.shape == (3, 4, 5)
    close(got, ref, 1e-5, 1e-6)
    # the definition, token by token
    b, t = 1, 2
    one = torch.outer(P_o @ G[b, t], P_i[:, ids[b, t]])
    full = sum(torch.outer(P_o @ G[b, tt], P_i[:, ids[b, tt]]) for tt in range(G.shape[1]))
    assert one.shape == (4, 5)
    close(got[b], full, 1e-5, 1e-6)


def test_conv2d(golden):
    """Materialised branch of the reference (its ghost branch for Conv2d raises on shape grounds)."""
    assert int(golden["conv_ghost_branch_runs"][0]) == 0
    A = torch.from_numpy(golden["conv_A"])
    G = torch.from_numpy(golden["conv_G"])
    kw = dict(kernel_size=(3, 2), dilation=(1, 2), padding=(1, 0), stride=(2, 1))
    for nv in (1, N_V):
        w, b = O.conv2d_dot_reference(A, G, nv, use_ghost=False, **kw)
        close(w.float(), golden[f"conv_nv{nv}_ghost0_w"], rtol=1e-3, atol=1e-3)
        close(b.float(), golden[f"conv_nv{nv}_ghost0_b"], rtol=1e-3, atol=1e-3)
    Mw, Mb = O.conv2d_dot_exact(A, G, 1, **kw)
    assert O.rel_fro(torch.from_numpy(golden["conv_nv1_ghost0_w"]), Mw[0]) < 2e-2
    assert O.rel_fro(torch.from_numpy(golden["conv_nv1_ghost0_b"]), Mb[0]) < 2e-2
    tg = O.conv2d_train_grad(A, G * N, N_V, (5, 3, 3, 2), **kw)
    close(tg, golden["conv_train_grad"], rtol=1e-5, atol=1e-6)


def test_rmsnorm_oracle_matches_autograd():
    """RMS norm has no reference counterpart: the float64 restatement is pinned against per-sample
    autograd gradients of torch's own nn.RMSNorm."""
    import torch
    from oracle import ghost_oracle as O
    torch.manual_seed(3)
    N, T, F, eps = 4, 6, 10, 1e-5
    norm = torch.nn.RMSNorm(F, eps=eps).double()
    with torch.no_grad():
        norm.weight.uniform_(0.5, 1.5)
    A = torch.randn(N, T, F, dtype=torch.float64)
    G = torch.randn(N, T, F, dtype=torch.float64)
    per = []
    for n in range(N):
        norm.zero_grad()
        (norm(A[n:n + 1]) * G[n:n + 1]).sum().backward()
        per.append(norm.weight.grad.clone())
    per = torch.stack(per)
    got = O.rmsnorm_persample_exact(A, G, eps)
    assert torch.allclose(got, per, rtol=1e-10, atol=1e-12)
    M = O.rmsnorm_dot_exact(A, G, 1, eps)
    assert torch.allclose(M, per[3:] @ per[:3].t(), rtol=1e-10, atol=1e-12)
