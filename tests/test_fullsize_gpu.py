"""Checks at the full sizes of the benchmark configurations, where the CPU oracle would take hours.

They rest on properties that do not depend on the size: two independent kernels must agree (Gram
kernel against per-sample path), a checksum of checksums (the sum over validation samples of a
column of M equals one inner product with the summed validation gradient, which a different
kernel produces), exact float64 values for a seeded subset of (validation, train) pairs, scaling
laws, and bit-exact index work against the CPU's own index_add_.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def ops():
    from ghostsuite_b200 import ops as _ops
    return _ops


def after():
    from ghostsuite_b200 import _lib
    torch.cuda.synchronize()
    _lib.poll_kernel_error()


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def make_gpu(N, T, d, p, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = (torch.randn(N, T, d, generator=g, device="cuda") / d ** 0.5).bfloat16()
    G = (torch.randn(N, T, p, generator=g, device="cuda") / p ** 0.5).bfloat16()
    return A, G


def exact_pairs(A, G, n_t, pairs):
    """float64 <grad_v, grad_b> for a few (v, b) pairs; grad_s = G_s^T A_s."""
    cache = {}

    def grad(s):
        if s not in cache:
            cache[s] = G[s].double().t() @ A[s].double()
        return cache[s]

    return torch.stack([(grad(n_t + v) * grad(b)).sum() for v, b in pairs])


def test_gpt2_cfc_shape_full_size():
    """GPT-2 mlp.c_fc at the benchmark's sizes: 32 train + 8 validation sequences of 1024 tokens,
    768 -> 3072, bf16."""
    n_t, n_v, T, d, p = 32, 8, 1024, 768, 3072
    A, G = make_gpu(n_t + n_v, T, d, p, seed=3)
    M_gram = ops().gram_dot(A, G, n_v)
    M_per, grad = ops().persample_dot(A, G, n_v, want_grad=True, grad_scale=1.0, grad_dtype=torch.float32)
    after()
    assert M_gram.shape == (n_v, n_t) and torch.isfinite(M_gram).all()
    assert rel(M_per, M_gram) < 5e-3                      # independent kernels, both fp32-accumulating
    pairs = [(0, 0), (7, 31), (3, 17), (5, 2)]
    want = exact_pairs(A, G, n_t, pairs)
    got_g = torch.stack([M_gram[v, b] for v, b in pairs])
    got_p = torch.stack([M_per[v, b] for v, b in pairs])
    assert rel(got_g, want) < 2e-2 and rel(got_p, want) < 2e-2
    # train gradient [d, p] (Conv1D orientation: X = A, Y = G) against a float32 GEMM; it is the sum
    # of the per-sample tiles, which are stored in bf16 (one rounding per sample and element)
    ref = torch.einsum("btd,btp->dp", A[:n_t].float(), G[:n_t].float())
    assert rel(grad, ref) < 5e-3
    # checksum of checksums: sum_v M[v, b] = <sum_v grad_v, grad_b>, the summed validation gradient
    # coming from the train-gradient-recovery kernel
    W_val = ops().wgrad(A[n_t:], G[n_t:], 1.0, torch.float32)          # [d, p]
    after()
    check = torch.stack([((A[b].float() @ W_val) * G[b].float()).sum() for b in range(n_t)])
    assert rel(M_per.sum(0), check) < 2e-2
    assert rel(M_gram.sum(0), check) < 2e-2
    # scaling law: doubling the out-grads quadruples every dot product
    M2 = ops().gram_dot(A, (G.float() * 2).bfloat16(), n_v)
    after()
    assert rel(M2, 4 * M_gram) < 1e-5


def test_ghost_linear_microbenchmark_shape_full_size():
    """Single layer 4096 -> 11008 with 256 train and 32 validation samples at T = 128, bf16."""
    n_t, n_v, T, d, p = 256, 32, 128, 4096, 11008
    A, G = make_gpu(n_t + n_v, T, d, p, seed=4)
    M = ops().gram_dot(A, G, n_v)
    after()
    assert torch.isfinite(M).all()
    pairs = [(0, 0), (31, 255), (7, 100), (16, 3), (2, 77), (29, 200)]
    want = exact_pairs(A, G, n_t, pairs)
    got = torch.stack([M[v, b] for v, b in pairs])
    assert rel(got, want) < 2e-2
    W_val = ops().wgrad(G[n_t:], A[n_t:], 1.0, torch.float32)          # Linear orientation: [p, d]
    after()
    check = torch.stack([((G[b].float() @ W_val) * A[b].float()).sum() for b in range(0, n_t, 16)])
    assert rel(M.sum(0)[::16], check) < 2e-2
    # the per-sample path on a slice of the batch must agree with the Gram kernel
    sel = torch.cat((torch.arange(0, 24), torch.arange(n_t, n_t + 8))).cuda()
    M_per, _ = ops().persample_dot(G[sel].contiguous(), A[sel].contiguous(), 8, want_grad=False,
                                   grad_scale=1.0, grad_dtype=torch.float32)
    after()
    assert rel(M_per, M[:8, :24]) < 5e-3


def test_gradproj_llama_q_proj_shape_full_size():
    """Llama-3-8B q_proj: 8 sequences of 4096 tokens, 4096 -> 4096, k_i = k_o = 64, bf16."""
    B, T, n, k = 8, 4096, 4096, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    A = (torch.randn(B, T, n, generator=g, device="cuda") / n ** 0.5).bfloat16()
    G = (torch.randn(B, T, n, generator=g, device="cuda") / n ** 0.5).bfloat16()
    P_i = torch.randn(k, n, generator=g, device="cuda") / k ** 0.5
    P_o = torch.randn(k, n, generator=g, device="cuda") / k ** 0.5
    Pi, Po = ops().prepare_projection(P_i, False), ops().prepare_projection(P_o, False)
    out = torch.empty(B, k * k, device="cuda")
    ops().gradproj_dense(G, A, Po, Pi, k, k, float(B), out)
    after()
    ref = torch.stack([(G[b].float() @ Po.float().t()).t() @ (A[b].float() @ Pi.float().t()) for b in range(B)])
    assert rel(out.view(B, k, k), ref * B) < 1e-3
    out2 = torch.empty(B, k * k, device="cuda")
    ops().gradproj_dense((G.float() * 0.5).bfloat16(), A, Po, Pi, k, k, float(B), out2)
    after()
    assert rel(out2, 0.5 * out) < 1e-5                    # linear in the out-grad (exact power of two)


def test_layernorm_and_bias_gpt2_shape_full_size():
    N, T, F, n_v = 40, 1024, 768, 8
    g = torch.Generator(device="cuda").manual_seed(6)
    A = torch.randn(N, T, F, generator=g, device="cuda").bfloat16()
    G = (torch.randn(N, T, F, generator=g, device="cuda") / 30).bfloat16()
    gw, gb = ops().layernorm_persample(A, G, 1e-5)
    cs = ops().colsum(G)
    after()
    xhat = torch.nn.functional.layer_norm(A.float(), (F,), eps=1e-5)
    assert rel(gw, (G.float() * xhat).sum(1)) < 1e-4
    assert rel(gb, G.float().sum(1)) < 1e-4
    assert rel(cs, G.float().sum(1)) < 1e-4
    M = ops().small_gram(gw, n_v)
    after()
    assert rel(M, gw[N - n_v:].double() @ gw[:N - n_v].double().t()) < 1e-5


def test_embedding_gpt2_vocab_full_size():
    """Token embedding of the benchmark model: 50304-row table, 32 + 8 sequences of 1024 ids."""
    n_t, n_v, T, d, V = 32, 8, 1024, 768, 50304
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 50257, (n_t + n_v, T), generator=g)
    G = (torch.randn(n_t + n_v, T, d, generator=g) / 50).bfloat16()
    M = ops().embedding_dot(ids.cuda(), G.cuda(), n_v, V)
    grad = ops().embedding_wgrad(ids.cuda(), G.cuda(), n_t, V, float(n_t + n_v), float(n_t))
    after()
    # dot products: per validation sample scatter its rows into a [V, d] table, gather at the train ids
    Gd = G.cuda().double()
    idc = ids.cuda()
    want = torch.empty(n_v, n_t, dtype=torch.float64, device="cuda")
    for v in range(n_v):
        table = torch.zeros(V, d, dtype=torch.float64, device="cuda").index_add_(0, idc[n_t + v], Gd[n_t + v])
        want[v] = (table[idc[:n_t]] * Gd[:n_t]).sum(dim=(1, 2))
    assert rel(M, want) < 1e-4
    # train gradient: bit-identical to the CPU's sequential index_add_ (fp32 accumulate, one rounding)
    table = torch.zeros(V, d, dtype=torch.bfloat16)
    table.index_add_(0, ids[:n_t].reshape(-1), (G[:n_t] * float(n_t + n_v)).reshape(-1, d))
    ref = table / float(n_t)
    assert torch.equal(grad.cpu().view(torch.int16), ref.view(torch.int16))
