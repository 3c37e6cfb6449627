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


def _gradproj_case(B, T, n_i, n_o, k, seed, conv1d=False):
    """One GradProj call at a configuration's full size against the float64 oracle evaluated with the
    float32 projection matrices (the kernel's one-time bf16 rounding of P is inside the check)."""
    from oracle import ghost_oracle as O
    torch.cuda.empty_cache()
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = (torch.randn(B, T, n_i, generator=g, device="cuda") / n_i ** 0.5).bfloat16()
    G = (torch.randn(B, T, n_o, generator=g, device="cuda") / n_o ** 0.5).bfloat16()
    P_i = torch.randn(k, n_i, generator=g, device="cuda") / k ** 0.5          # float32, N(0, 1/k)
    P_o = torch.randn(k, n_o, generator=g, device="cuda") / k ** 0.5
    Pi, Po = ops().prepare_projection(P_i, False), ops().prepare_projection(P_o, False)
    out = torch.empty(B, k * k, device="cuda")
    ops().gradproj_dense(G, A, Po, Pi, k, k, float(B), out)
    after()
    # one sample at a time keeps the float64 copies of the operands small
    ref = torch.cat([O.gradproj_dense(A[b:b + 1], G[b:b + 1], P_i, P_o, compute_dtype=torch.float64)
                     for b in range(B)]).double() * B
    err = rel(out.view(B, k, k), ref)
    assert err < 2e-2, err
    out2 = torch.empty(B, k * k, device="cuda")
    ops().gradproj_dense((G.float() * 0.5).bfloat16(), A, Po, Pi, k, k, float(B), out2)
    after()
    assert rel(out2, 0.5 * out) < 1e-5                    # linear in the out-grad (exact power of two)
    return err


def test_gradproj_llama_q_proj_shape_full_size():
    """Llama-3-8B q_proj: 8 sequences of 4096 tokens, 4096 -> 4096, k_i = k_o = 64, bf16."""
    _gradproj_case(8, 4096, 4096, 4096, 64, seed=5)


@pytest.mark.parametrize("n_i,n_o", [(4096, 14336), (14336, 4096), (4096, 1024)],
                         ids=["gate_up_proj", "down_proj", "kv_proj"])
def test_gradproj_llama_other_shapes_full_size(n_i, n_o):
    """The other Linear shapes of a Llama-3-8B block (SwiGLU 14336, 8 KV heads) at 8 x 4096 tokens, k = 64."""
    _gradproj_case(8, 4096, n_i, n_o, 64, seed=8)


@pytest.mark.parametrize("n_i,n_o", [(1024, 4096), (4096, 1024), (1024, 3072), (1024, 1024)],
                         ids=["dense_h_to_4h", "dense_4h_to_h", "query_key_value", "attention_dense"])
def test_gradproj_pythia_shapes_full_size(n_i, n_o):
    """Pythia-410M-shaped Linears at the configuration's 16 x 2048 tokens, k_i = k_o = 32."""
    _gradproj_case(16, 2048, n_i, n_o, 32, seed=9)


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


def make_gpu_chunked(N, T, d, p, seed):
    """Like make_gpu, drawn one sample at a time so that no float32 copy of a whole operand exists
    (the 4096 -> 11008 layer at 288 x 8192 tokens holds 71 GB of bf16 operands)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    A = torch.empty(N, T, d, dtype=torch.bfloat16, device="cuda")
    G = torch.empty(N, T, p, dtype=torch.bfloat16, device="cuda")
    for s in range(N):
        A[s] = torch.randn(T, d, generator=g, device="cuda") / d ** 0.5
        G[s] = torch.randn(T, p, generator=g, device="cuda") / p ** 0.5
    return A, G


def seeded_pairs(n_v, n_t, vals, trains, seed):
    """vals x trains (validation, train) index pairs from a seeded draw without replacement."""
    g = torch.Generator().manual_seed(seed)
    vs = torch.randperm(n_v, generator=g)[:vals].tolist()
    bs = torch.randperm(n_t, generator=g)[:trains].tolist()
    return [(v, b) for v in vs for b in bs]


@pytest.mark.parametrize("name,d,p,linear", [
    ("attn.c_attn", 768, 2304, False), ("attn.c_proj", 768, 768, False),
    ("mlp.c_proj", 3072, 768, False), ("lm_head", 768, 50304, True)])
def test_gpt2_other_layer_shapes_full_size(name, d, p, linear):
    """The remaining dense layers of the GPT-2-small step at 32 train + 8 validation sequences of 1024
    tokens: both dot-product paths against float64 values of 16 seeded pairs, and the train gradient
    of the per-sample pass against a float32 GEMM.  Conv1D layers store [d_in, d_out] (X = A), the
    head is an nn.Linear with [d_out, d_in] (X = out-grad), as the engine calls them."""
    n_t, n_v, T = 32, 8, 1024
    torch.cuda.empty_cache()
    A, G = make_gpu_chunked(n_t + n_v, T, d, p, seed=11)
    X, Y = (G, A) if linear else (A, G)
    M_per, grad = ops().persample_dot(X, Y, n_v, want_grad=True, grad_scale=1.0, grad_dtype=torch.float32)
    M_gram = ops().gram_dot(A, G, n_v)
    after()
    assert torch.isfinite(M_per).all() and torch.isfinite(M_gram).all()
    assert rel(M_per, M_gram) < 5e-3
    pairs = seeded_pairs(n_v, n_t, 4, 4, seed=12)
    want = exact_pairs(A, G, n_t, pairs)
    assert rel(torch.stack([M_per[v, b] for v, b in pairs]), want) < 2e-2
    assert rel(torch.stack([M_gram[v, b] for v, b in pairs]), want) < 2e-2
    Xt, Yt = X[:n_t].reshape(-1, X.shape[-1]), Y[:n_t].reshape(-1, Y.shape[-1])
    ref = Xt.float().t() @ Yt.float()
    assert rel(grad, ref) < 5e-3
    # the split-K train-gradient kernel on the same operands (fp32 accumulation throughout)
    W = ops().wgrad(X[:n_t], Y[:n_t], 1.0, torch.float32)
    after()
    assert rel(W, ref) < 1e-3


@pytest.mark.parametrize("T,gram", [(512, True), (2048, False), (8192, False)])
def test_ghost_linear_microbenchmark_long_sequences_full_size(T, gram):
    """Single layer 4096 -> 11008 with 256 train and 32 validation samples (bf16) at T = 512, 2048 and
    8192: the per-sample path (the product path at these lengths) against float64 values of 64 seeded
    (validation, train) pairs; at T = 512 the Gram kernel as well.  At T = 8192 the operands hold
    71 GB and every sample's token block starts beyond 2^31 elements for most samples, which is what
    this case is for."""
    n_t, n_v, d, p = 256, 32, 4096, 11008
    torch.cuda.empty_cache()
    A, G = make_gpu_chunked(n_t + n_v, T, d, p, seed=13)
    M_per, grad = ops().persample_dot(G, A, n_v, want_grad=True, grad_scale=1.0, grad_dtype=torch.float32)
    after()
    assert M_per.shape == (n_v, n_t) and torch.isfinite(M_per).all()
    pairs = seeded_pairs(n_v, n_t, 8, 8, seed=14)          # 64 pairs, 16 float64 per-sample gradients
    want = exact_pairs(A, G, n_t, pairs)
    got = torch.stack([M_per[v, b] for v, b in pairs])
    assert rel(got, want) < 2e-2
    # the last train and the last validation sample sit at the far end of the buffers
    far = exact_pairs(A, G, n_t, [(n_v - 1, n_t - 1)])
    assert rel(M_per[n_v - 1, n_t - 1].reshape(1), far) < 2e-2
    # train gradient: the per-sample pass sums bf16 tiles; check it on a seeded set of output rows
    # against float64 (a full float32 GEMM reference would need a 105 GB float32 copy at T = 8192)
    rows = torch.randperm(p, generator=torch.Generator().manual_seed(15))[:64].cuda()
    ref = torch.zeros(64, d, dtype=torch.float64, device="cuda")
    for s in range(n_t):
        ref += G[s][:, rows].double().t() @ A[s].double()
    assert rel(grad[rows], ref) < 1e-2
    if gram:
        M_gram = ops().gram_dot(A, G, n_v)
        after()
        assert rel(M_gram, M_per) < 5e-3
        assert rel(torch.stack([M_gram[v, b] for v, b in pairs]), want) < 2e-2
    del A, G
    torch.cuda.empty_cache()
