"""Parity of every CUDA kernel (called through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import as_dtype
from oracle import ghost_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}   # relative Frobenius, per the north star


def ops():
    from ghostsuite_b200 import ops as _ops
    return _ops


def make(N, T, d, p, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    A = (torch.randn(N, T, d, generator=g) / d ** 0.5).to(dtype)
    G = (torch.randn(N, T, p, generator=g) / p ** 0.5).to(dtype)
    return A, G


def after():
    from ghostsuite_b200 import _lib
    torch.cuda.synchronize()
    _lib.poll_kernel_error()


LIN_CASES = [
    # n_train, n_val, T, d, p
    (5, 3, 6, 16, 24),        # several samples per tile, ragged everything
    (64, 16, 1, 512, 1024),   # MLP config: T = 1
    (3, 1, 130, 72, 40),      # T just above one tile, single validation sample
    (2, 2, 300, 200, 136),    # validation rows straddle the 256-wide tile
    (4, 2, 128, 64, 64),      # exactly tile-aligned
    (2, 3, 37, 10, 50),       # feature sizes that are not multiples of 8
    (33, 20, 9, 64, 264),     # 17..32 validation samples share one streaming pass; two train blocks
    (40, 35, 20, 72, 136),    # more than 32 validation samples: two passes over the train tiles
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", LIN_CASES)
def test_gram_dot(case, dtype):
    n_t, n_v, T, d, p = case
    A, G = make(n_t + n_v, T, d, p, dtype)
    M = ops().gram_dot(A.cuda(), G.cuda(), n_v)
    after()
    ref = O.linear_dot_exact(A, G, n_v)
    assert M.shape == (n_v, n_t)
    assert O.rel_fro(M, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", [(5, 3, 130, 72, 40), (4, 2, 256, 128, 64), (9, 2, 300, 200, 136),
                                  (700, 300, 1, 64, 48), (3, 5, 513, 96, 256)])
def test_gram_dot_cta_pair_kernel(case, dtype):
    """The cta_group::2 variant (256 x 256 tile per CTA pair) against the oracle and the
    single-CTA kernel, including ragged tiles and an odd number of tiles."""
    from ghostsuite_b200 import _lib
    lib = _lib.load()
    n_t, n_v, T, d, p = case
    A, G = make(n_t + n_v, T, d, p, dtype, seed=21)
    ref = O.linear_dot_exact(A, G, n_v) if n_t * n_v < 5000 else None
    try:
        _lib.check(lib.ghost_set_gram_pair_mode(2))
        M2 = ops().gram_dot(A.cuda(), G.cuda(), n_v)
        after()
        _lib.check(lib.ghost_set_gram_pair_mode(0))
        M1 = ops().gram_dot(A.cuda(), G.cuda(), n_v)
        after()
    finally:
        _lib.check(lib.ghost_set_gram_pair_mode(1))
    assert O.rel_fro(M2, M1.cpu()) < 1e-5
    if ref is not None:
        assert O.rel_fro(M2, ref) < TOL[dtype]


def test_gram_dot_reference_rounding_mode():
    """round_mode=1 reproduces the reference's bf16-rounded Grams (vector = column sums)."""
    n_t, n_v, T, d, p = 5, 3, 6, 16, 24
    A, G = make(n_t + n_v, T, d, p, torch.bfloat16, seed=3)
    M = ops().gram_dot(A.cuda(), G.cuda(), n_v, round_mode=1)
    after()
    ref = O.linear_dot_reference(A, G, n_v, use_ghost=True)
    assert O.rel_fro(M.sum(0), ref) < 2e-3


def test_gram_dot_golden(golden):
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        A = as_dtype(golden[f"lin_{tag}_A"], tag)
        G = as_dtype(golden[f"lin_{tag}_G"], tag)
        M = ops().gram_dot(A.cuda(), G.cuda(), 3)
        after()
        rows = torch.from_numpy(golden[f"lin_{tag}_rows_materialised"])
        assert O.rel_fro(M, rows) < TOL[dt]
        assert O.rel_fro(M.sum(0), torch.from_numpy(golden[f"lin_{tag}_nv3_ghost1_w"])) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", LIN_CASES)
def test_wgrad(case, dtype):
    n_t, n_v, T, d, p = case
    A, G = make(n_t + n_v, T, d, p, dtype, seed=1)
    N = n_t + n_v
    scale = N / n_t
    out = ops().wgrad(G[:n_t].cuda(), A[:n_t].cuda(), scale, dtype)        # Linear layout [p, d]
    outc = ops().wgrad(A[:n_t].cuda(), G[:n_t].cuda(), scale, dtype)       # Conv1D layout [d, p]
    after()
    ref = torch.einsum("btp,btd->pd", G[:n_t].double(), A[:n_t].double()) * scale
    assert out.shape == (p, d) and out.dtype == dtype
    tol = 1e-4 if dtype == torch.float32 else 1e-2
    assert O.rel_fro(out, ref) < tol
    assert O.rel_fro(outc, ref.t()) < tol
    # against the reference formula in its own dtype
    ref2 = O.linear_train_grad(A, G * N, n_v)
    assert O.rel_fro(out, ref2) < (1e-4 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("case", [(70, 64, 128), (130 * 3, 192, 320), (2700, 448, 64), (5000, 768, 1024),
                                  (64 * 300, 128, 384), (9, 64, 64)])
def test_wgrad_cta_pair_kernel(case):
    """The CTA-pair split-K pass (mode 2: wherever the column counts are multiples of 64, odd tile
    counts included) against the single-CTA pass and the fp64 contraction."""
    from ghostsuite_b200 import _lib
    lib = _lib.load()
    rows, d, p = case
    A, G = make(1, rows, d, p, torch.bfloat16, seed=23)
    ref = torch.einsum("btp,btd->pd", G.double(), A.double())
    res = {}
    try:
        for mode in (0, 2):
            _lib.check(lib.ghost_set_wgrad_pair_mode(mode))
            res[mode] = ops().wgrad(G.cuda(), A.cuda(), 1.0, torch.float32)
            after()
    finally:
        _lib.check(lib.ghost_set_wgrad_pair_mode(1))
    assert O.rel_fro(res[2], ref) < 1e-2
    assert O.rel_fro(res[2], res[0].cpu()) < 1e-5      # same products, another order of fp32 additions


def test_wgrad_accumulate():
    A, G = make(6, 40, 64, 48, torch.bfloat16, seed=5)
    o = ops()
    base = torch.randn(48, 64).to(torch.float32).cuda()
    out = base.clone()
    o.wgrad(G.cuda(), A.cuda(), 0.5, torch.float32, out=out, accumulate=True)
    after()
    ref = base.cpu().double() + 0.5 * torch.einsum("btp,btd->pd", G.double(), A.double())
    assert O.rel_fro(out, ref) < 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", LIN_CASES)
def test_persample_dot(case, dtype):
    n_t, n_v, T, d, p = case
    A, G = make(n_t + n_v, T, d, p, dtype, seed=2)
    N = n_t + n_v
    M, grad = ops().persample_dot(G.cuda(), A.cuda(), n_v, want_grad=True, grad_scale=N / n_t,
                                  grad_dtype=dtype)
    after()
    ref = O.linear_dot_exact(A, G, n_v)
    assert O.rel_fro(M, ref) < TOL[dtype]
    gref = torch.einsum("btp,btd->pd", G[:n_t].double(), A[:n_t].double()) * (N / n_t)
    assert O.rel_fro(grad, gref) < (1e-4 if dtype == torch.float32 else 1e-2)
    # both paths agree with each other far inside the tolerance
    M2 = ops().gram_dot(A.cuda(), G.cuda(), n_v)
    after()
    assert O.rel_fro(M, M2.cpu()) < TOL[dtype]


@pytest.mark.parametrize("case", [(5, 3, 6, 16, 24), (3, 1, 130, 72, 40), (2, 2, 300, 200, 136), (9, 4, 70, 264, 520),
                                  # column counts that take the CTA-pair kernel (multiples of 64, an even
                                  # number of 128-row tiles), T not a multiple of 32
                                  (5, 3, 130, 256, 512), (3, 2, 77, 768, 256), (4, 2, 1024, 512, 1024)])
@pytest.mark.parametrize("which", ["X", "Y"])
def test_persample_dot_column_sums(case, which):
    """Per-sample column sums of one operand taken inside the GEMM pass (the bias terms)."""
    n_t, n_v, T, d, p = case
    A, G = make(n_t + n_v, T, d, p, torch.bfloat16, seed=13)
    M, grad, cs = ops().persample_dot(G.cuda(), A.cuda(), n_v, want_grad=True, grad_scale=1.0,
                                      grad_dtype=torch.float32, colsum_of=which)
    after()
    src = G if which == "X" else A
    assert cs.shape == (n_t + n_v, src.shape[-1])
    assert O.rel_fro(cs, src.double().sum(1)) < 1e-5
    assert O.rel_fro(M, O.linear_dot_exact(A, G, n_v)) < 2e-2
    # fp32 operands reach the kernel as a bf16 hi/lo split: no fused sums
    res = ops().persample_dot(G.float().cuda(), A.float().cuda(), n_v, colsum_of=which)
    assert res[2] is None


@pytest.mark.parametrize("sizes", [(37, 11, 70, 136, 264), (70, 35, 12, 72, 264)])
def test_persample_dot_in_groups(sizes):
    """A small workspace budget forces the train samples through in several groups (and several
    validation / train blocks of the streaming kernel): same numbers as the single-pass run."""
    from ghostsuite_b200 import _lib
    lib = _lib.load()
    n_t, n_v, T, d, p = sizes
    A, G = make(n_t + n_v, T, d, p, torch.bfloat16, seed=11)
    ref = O.linear_dot_exact(A, G, n_v)
    gref = torch.einsum("btp,btd->pd", G[:n_t].double(), A[:n_t].double())
    try:
        for budget in (12 << 30, 2 << 20):
            _lib.check(lib.ghost_set_persample_budget_bytes(budget))
            M, grad, cs = ops().persample_dot(G.cuda(), A.cuda(), n_v, want_grad=True, grad_scale=1.0,
                                              grad_dtype=torch.float32, colsum_of="X")
            after()
            assert O.rel_fro(M, ref) < 2e-2
            assert O.rel_fro(grad, gref) < 1e-2
            assert O.rel_fro(cs, G.double().sum(1)) < 1e-5
    finally:
        _lib.check(lib.ghost_set_persample_budget_bytes(12 << 30))


@pytest.mark.parametrize("case", [(5, 3, 70, 64, 128), (3, 1, 130, 192, 320), (9, 4, 300, 448, 64),
                                  (4, 2, 64, 768, 1024), (33, 20, 9, 64, 256), (37, 11, 70, 128, 384)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_persample_dot_cta_pair_kernel(case, dtype):
    """The CTA-pair tile pass (mode 2: wherever the column counts allow it, odd tile counts and
    several train groups included) stores the same tiles as the single-CTA pass: identical train
    gradient, and dot products equal up to the order of the fp32 additions."""
    from ghostsuite_b200 import _lib
    lib = _lib.load()
    n_t, n_v, T, d, p = case
    A, G = make(n_t + n_v, T, d, p, dtype, seed=17)
    res = {}
    try:
        _lib.check(lib.ghost_set_persample_budget_bytes(8 << 20))
        for mode in (0, 2):
            _lib.check(lib.ghost_set_persample_pair_mode(mode))
            res[mode] = ops().persample_dot(G.cuda(), A.cuda(), n_v, want_grad=True, grad_scale=1.0,
                                            grad_dtype=torch.float32)[:2]
            after()
    finally:
        _lib.check(lib.ghost_set_persample_pair_mode(1))
        _lib.check(lib.ghost_set_persample_budget_bytes(12 << 30))
    assert torch.equal(res[0][1], res[2][1])
    assert O.rel_fro(res[2][0], res[0][0].cpu()) < 1e-5
    assert O.rel_fro(res[2][0], O.linear_dot_exact(A, G, n_v)) < TOL[dtype]
    assert lib.ghost_set_persample_pair_mode(3) < 0


@pytest.mark.parametrize("case", [(5, 8, 70, 64, 128), (12, 8, 64, 256, 512), (7, 16, 33, 192, 320),
                                  (33, 4, 40, 72, 264), (3, 32, 20, 128, 256)])
def test_tile_pass_and_gathered_tile_dot(case):
    """The per-sample path as two calls with the validation tiles laid out as an all-gather over
    ranks leaves them ([ranks][tiles][per rank][128 x 256]): every split of the validation batch
    gives the matrix and the train gradient of the one-call path (same tiles, same kernel)."""
    n_t, n_v, T, d, p = case
    A, G = make(n_t + n_v, T, d, p, torch.bfloat16, seed=50 + n_v)
    Ac, Gc = A.cuda(), G.cuda()
    o = ops()
    gdt = torch.float32 if n_t > 32 else torch.bfloat16
    M_ref, grad_ref, cs_ref = o.persample_dot(Gc, Ac, n_v, dot_scale=1.5, want_grad=True, grad_scale=0.25,
                                              grad_dtype=gdt, colsum_of="X")
    after()
    block = 8 if n_v <= 8 else (16 if n_v <= 16 else 32)
    for ranks in (1, 2, 4, 8):
        per = n_v // ranks
        if per * ranks != n_v or per == 0:
            continue
        assert block % per == 0 or per % block == 0
        cs = torch.full((n_t + n_v, p), float("nan"), device="cuda")
        V = torch.stack([o.persample_tiles(Gc, Ac, n_t + r * per, per, "X", cs) for r in range(ranks)])
        W = o.persample_tiles(Gc, Ac, 0, n_t, "X", cs)
        M, grad = o.tile_dot(V, W, p, d, dot_scale=1.5, want_grad=True, grad_scale=0.25, grad_dtype=gdt)
        after()
        assert O.rel_fro(M, M_ref.cpu()) < 1e-5, ranks
        assert torch.equal(grad, grad_ref), ranks
        assert O.rel_fro(cs, cs_ref.double().cpu()) < 1e-6, ranks
    # a split that does not fit the kernel's blocks of validation rows is refused, not mangled
    if n_v == 16:
        V = torch.zeros(4, W.shape[0], 3, 32768, dtype=torch.bfloat16, device="cuda")      # 12 = 4 x 3
        with pytest.raises(ValueError):
            o.tile_dot(V, W, p, d)
        class FourRanks:
            world = 4

            @staticmethod
            def gather_rows(t):
                return t.repeat(4, 1, 1, 1)

        assert o.persample_dot_exchanged(Gc[:n_t + 3], Ac[:n_t + 3], 3, FourRanks) is None
        res = o.persample_dot_exchanged(Gc[:n_t + 4], Ac[:n_t + 4], 4, FourRanks, want_grad=True,
                                        grad_dtype=torch.float32, colsum_of="X")
        after()
        one = o.persample_dot(Gc[:n_t + 4], Ac[:n_t + 4], 4, want_grad=True, grad_dtype=torch.float32, colsum_of="X")
        # four "ranks" that all hold the same four validation samples: the local block four times
        assert res[0].shape == (16, n_t) and O.rel_fro(res[0], one[0].repeat(4, 1).cpu()) < 1e-5
        assert torch.equal(res[1], one[1]) and O.rel_fro(res[2], one[2].double().cpu()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(8, 6, 24), (12, 1, 10), (5, 300, 520), (3, 1024, 768)])
def test_colsum_and_bias(shape, dtype):
    N, T, p = shape
    g = torch.Generator().manual_seed(4)
    G = torch.randn(N, T, p, generator=g).to(dtype)
    o = ops()
    cs = o.colsum(G.cuda())
    n_v = 2
    M = o.small_gram(cs, n_v)
    bgrad = o.rows_sum(cs, N - n_v, N / (N - n_v), dtype)
    after()
    ref = G.double().sum(1)
    assert O.rel_fro(cs, ref) < 1e-5
    assert O.rel_fro(M, O.bias_dot_exact(G, n_v)) < 1e-4
    assert O.rel_fro(bgrad, O.bias_train_grad((G * N).clone(), n_v)) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(8, 6, 16), (5, 70, 768), (4, 33, 1024), (3, 9, 20), (2, 5, 1536)])
def test_layernorm(shape, dtype):
    N, T, F = shape
    g = torch.Generator().manual_seed(6)
    A = (torch.randn(N, T, F, generator=g) * 1.5 + 0.3).to(dtype)
    G = (torch.randn(N, T, F, generator=g) / F ** 0.5).to(dtype)
    gw, gb = ops().layernorm_persample(A.cuda(), G.cuda(), 1e-5)
    after()
    rw, rb = O.layernorm_persample_exact(A, G, 1e-5)
    assert O.rel_fro(gw, rw) < 1e-4
    assert O.rel_fro(gb, rb) < 1e-4


def test_layernorm_golden(golden):
    eps = float(golden["ln_eps"][0])
    for tag in ("f32", "bf16"):
        A = as_dtype(golden[f"ln_{tag}_A"], tag)
        G = as_dtype(golden[f"ln_{tag}_G"], tag)
        o = ops()
        gw, gb = o.layernorm_persample(A.cuda(), G.cuda(), eps)
        Mw, Mb = o.small_gram(gw, 3), o.small_gram(gb, 3)
        after()
        assert O.rel_fro(Mw.sum(0), torch.from_numpy(golden[f"ln_{tag}_nv3_w"])) < 2e-2
        assert O.rel_fro(Mb.sum(0), torch.from_numpy(golden[f"ln_{tag}_nv3_b"])) < 2e-2
        tw = o.rows_sum(gw, 5, 8 / 5, torch.float32)
        after()
        assert O.rel_fro(tw, torch.from_numpy(golden[f"ln_{tag}_train_grad_w"])) < (1e-5 if tag == "f32" else 2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", [(5, 3, 6, 8, 11), (4, 2, 64, 40, 50), (3, 2, 100, 768, 7), (6, 1, 33, 16, 1000),
                                  # tables that span several 4096-id tiles of the bucket scan, feature counts
                                  # off the 16-byte path, a crowded row in the last, partial tile
                                  (6, 2, 700, 20, 9001), (40, 2, 64, 72, 4099), (12, 3, 50, 264, 12289)])
def test_embedding(case, dtype):
    n_t, n_v, T, d, vocab = case
    N = n_t + n_v
    g = torch.Generator().manual_seed(8)
    ids = torch.randint(0, vocab, (N, T), generator=g)
    if vocab > 4096:
        ids[:, :3] = vocab - 1
        ids[:, 3] = 4095
        ids[:, 4] = 4096
    G = (torch.randn(N, T, d, generator=g) / d ** 0.5).to(dtype)
    o = ops()
    M = o.embedding_dot(ids.cuda(), G.cuda(), n_v, vocab)
    grad = o.embedding_wgrad(ids.cuda(), G.cuda(), n_t, vocab, float(N), float(n_t))
    after()
    assert O.rel_fro(M, O.embedding_dot_exact(ids, G, n_v)) < (1e-5 if dtype == torch.float32 else 1e-4)
    ref = O.embedding_train_grad(ids, G * N, n_v, vocab, sequential=True)
    # index / gather work: bit-exact against the CPU sequential order
    assert torch.equal(grad.cpu().float(), ref.float())


def test_embedding_position_ids_and_golden(golden):
    # position-embedding pattern: every sample has ids 0..T-1 (all buckets hold n_train tokens)
    n_t, n_v, T, d = 40, 2, 16, 24
    ids = torch.arange(T).repeat(n_t + n_v, 1)
    G = torch.randn(n_t + n_v, T, d, generator=torch.Generator().manual_seed(1))
    o = ops()
    M = o.embedding_dot(ids.cuda(), G.cuda(), n_v, T)
    grad = o.embedding_wgrad(ids.cuda(), G.cuda(), n_t, T, float(n_t + n_v), float(n_t))
    after()
    assert O.rel_fro(M, O.embedding_dot_exact(ids, G, n_v)) < 1e-5
    assert torch.equal(grad.cpu(), O.embedding_train_grad(ids, G * (n_t + n_v), n_v, T))
    ids = torch.from_numpy(golden["emb_ids"])
    for tag in ("f32", "bf16"):
        G = as_dtype(golden[f"emb_{tag}_G"], tag)
        M = o.embedding_dot(ids.cuda(), G.cuda(), 3, 11)
        grad = o.embedding_wgrad(ids.cuda(), G.cuda(), 5, 11, 8.0, 5.0)
        after()
        assert O.rel_fro(M.sum(0), torch.from_numpy(golden[f"emb_{tag}_nv3_w"])) < 2e-2
        assert np.array_equal(grad.cpu().float().numpy(), golden[f"emb_{tag}_train_grad"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", [
    # n_t, n_v, T, d, vocab, share of tokens that carry one and the same id
    (6, 3, 200, 64, 50, 0.6),        # validation chain of ~360 tokens, train bucket of ~720
    (64, 2, 48, 24, 48, None),       # position ids: every id 64 times in the train rows (> 32), twice in val
    (40, 2, 1024, 16, 1000, 0.9),    # a train bucket above 32768 tokens: sorted in place in global memory
    (5, 40, 64, 40, 30, 0.5)])       # many validation samples, feature size not a multiple of 16
def test_embedding_with_heavily_repeated_ids(case, dtype):
    """Padding-like batches: one id carried by most tokens.  The dot products go through the
    per-(id, validation sample) pre-summed rows, the train gradient through the big-bucket kernel,
    and the train gradient stays bit-identical to the CPU's sequential index_add_."""
    n_t, n_v, T, d, vocab, share = case
    N = n_t + n_v
    g = torch.Generator().manual_seed(31)
    if share is None:
        ids = torch.arange(T).repeat(N, 1)
    else:
        ids = torch.randint(0, vocab, (N, T), generator=g)
        ids[torch.rand(N, T, generator=g) < share] = 7
    G = (torch.randn(N, T, d, generator=g) / d ** 0.5).to(dtype)
    o = ops()
    M = o.embedding_dot(ids.cuda(), G.cuda(), n_v, vocab)
    grad = o.embedding_wgrad(ids.cuda(), G.cuda(), n_t, vocab, float(N), float(n_t))
    after()
    assert O.rel_fro(M, O.embedding_dot_exact(ids, G, n_v)) < (1e-5 if dtype == torch.float32 else 1e-4)
    ref = O.embedding_train_grad(ids, G * N, n_v, vocab, sequential=True)
    assert torch.equal(grad.cpu().float(), ref.float())


def test_embedding_out_of_range_ids_are_reported():
    """An id outside the table makes the reference's index_add_ raise.  The kernels skip such a token
    and record it; the next poll of the error word raises IndexError."""
    from ghostsuite_b200 import _lib
    n_t, n_v, T, d, vocab = 4, 2, 9, 16, 30
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, vocab, (n_t + n_v, T), generator=g)
    G = torch.randn(n_t + n_v, T, d, generator=g)
    good_M = ops().embedding_dot(ids.cuda(), G.cuda(), n_v, vocab)
    after()                                                   # nothing recorded for valid ids
    for row, col in ((1, 3), (n_t, 4)):                       # a train token, then a validation token
        bad = ids.clone()
        bad[row, col] = vocab
        M = ops().embedding_dot(bad.cuda(), G.cuda(), n_v, vocab)
        torch.cuda.synchronize()
        with pytest.raises(IndexError):
            _lib.poll_kernel_error()
        keep = torch.ones(n_t + n_v, T, 1)
        keep[row, col] = 0
        assert O.rel_fro(M, O.embedding_dot_exact(ids, G * keep, n_v)) < 1e-5
    bad = ids.clone()
    bad[0, 0] = -1
    ops().embedding_wgrad(bad.cuda(), G.cuda(), n_t, vocab, 1.0, float(n_t))
    torch.cuda.synchronize()
    with pytest.raises(IndexError):
        _lib.poll_kernel_error()
    _lib.poll_kernel_error()
    assert torch.isfinite(good_M).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", [(8, 6, 16, 24, 4, 6), (4, 130, 72, 200, 32, 32), (2, 300, 512, 136, 64, 64),
                                  (3, 1, 10, 20, 5, 3), (2, 257, 128, 256, 120, 34)])
def test_gradproj_dense(case, dtype):
    B, T, n_i, n_o, k_i, k_o = case
    A, G = make(B, T, n_i, n_o, dtype, seed=9)
    g = torch.Generator().manual_seed(10)
    P_i = torch.randn(k_i, n_i, generator=g) / k_i ** 0.5
    P_o = torch.randn(k_o, n_o, generator=g) / k_o ** 0.5
    o = ops()
    split = dtype == torch.float32
    Pr = o.prepare_projection(P_o.cuda(), split)
    Pc = o.prepare_projection(P_i.cuda(), split)
    total = k_o * k_i + 7
    buf = torch.full((B, total), 123.0, device="cuda")
    o.gradproj_dense(G.cuda(), A.cuda(), Pr, Pc, k_o, k_i, float(B), buf[:, 3:3 + k_o * k_i])
    after()
    ref = O.gradproj_dense(A, G, P_i, P_o, compute_dtype=torch.float64)
    got = buf[:, 3:3 + k_o * k_i].reshape(B, k_o, k_i)
    assert O.rel_fro(got, ref) < (1e-4 if split else 2e-2)
    # neighbours of the slice are untouched
    assert torch.all(buf[:, :3] == 123.0) and torch.all(buf[:, 3 + k_o * k_i:] == 123.0)


def test_gradproj_golden(golden):
    A = torch.from_numpy(golden["lin_f32_A"])
    G = torch.from_numpy(golden["lin_f32_G"])
    o = ops()
    P_i, P_o = torch.from_numpy(golden["gp_P_i"]), torch.from_numpy(golden["gp_P_o"])
    out = torch.empty(8, 24, device="cuda")
    o.gradproj_dense(G.cuda(), A.cuda(), o.prepare_projection(P_o.cuda(), True),
                     o.prepare_projection(P_i.cuda(), True), 6, 4, 8.0, out)
    after()
    assert O.rel_fro(out.reshape(8, 6, 4), torch.from_numpy(golden["gp_linear"])) < 1e-4
    assert torch.allclose(out.cpu().reshape(8, 6, 4), torch.from_numpy(golden["gp_linear"]), rtol=1e-3, atol=1e-4)
    # Conv1D: the out-grad is projected with P_i, the activations with P_o -> [k_i, k_o]
    P_i, P_o = torch.from_numpy(golden["gp_c1d_P_i"]), torch.from_numpy(golden["gp_c1d_P_o"])
    o.gradproj_dense(G.cuda(), A.cuda(), o.prepare_projection(P_i.cuda(), True),
                     o.prepare_projection(P_o.cuda(), True), 4, 6, 8.0, out)
    after()
    assert O.rel_fro(out.reshape(8, 4, 6), torch.from_numpy(golden["gp_c1d"])) < 1e-4
    assert torch.allclose(out.cpu().reshape(8, 4, 6), torch.from_numpy(golden["gp_c1d"]), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", [
    # B, T, d, vocab, k_i, k_o
    (3, 7, 12, 19, 5, 4),          # the golden case's sizes: everything smaller than one tile
    (4, 130, 72, 300, 32, 32),     # T straddles the 64-token blocks, d not a multiple of 16
    (2, 300, 512, 50, 64, 64),     # heavy id repetition, the largest single-launch block
    (3, 1, 10, 20, 3, 5),          # one token per sample, d with a 2-element tail
    (2, 65, 11, 40, 7, 9),         # odd feature size: the element-wise load path
    (2, 257, 128, 1000, 12, 85),   # k_o > 64: covered block by block
    (2, 33, 64, 64, 70, 66)])      # both larger than 64
def test_gradproj_embedding(case, dtype):
    B, T, d, vocab, k_i, k_o = case
    g = torch.Generator().manual_seed(21)
    ids = torch.randint(0, vocab, (B, T), generator=g)
    G = (torch.randn(B, T, d, generator=g) / d ** 0.5).to(dtype)
    P_i = torch.randn(k_i, vocab, generator=g) / k_i ** 0.5
    P_o = torch.randn(k_o, d, generator=g) / k_o ** 0.5
    o = ops()
    split = dtype == torch.float32
    Po = o.prepare_projection(P_o.cuda(), split)
    PiT = o.prepare_embedding_projection(P_i.cuda())
    total = k_o * k_i + 9
    buf = torch.full((B, total), 55.0, device="cuda")
    o.gradproj_embedding(ids.cuda(), G.cuda(), Po, PiT, k_o, k_i, 1.0, buf[:, 4:4 + k_o * k_i])
    after()
    ref = O.gradproj_embedding(ids, G, P_i, P_o, compute_dtype=torch.float64)
    got = buf[:, 4:4 + k_o * k_i].reshape(B, k_o, k_i)
    assert O.rel_fro(got, ref) < (1e-4 if split else 2e-2)
    assert torch.all(buf[:, :4] == 55.0) and torch.all(buf[:, 4 + k_o * k_i:] == 55.0)
    # a second call into the same buffer overwrites (the kernel adds into a block it zeroed itself)
    o.gradproj_embedding(ids.cuda(), G.cuda(), Po, PiT, k_o, k_i, 2.0, buf[:, 4:4 + k_o * k_i])
    after()
    assert O.rel_fro(buf[:, 4:4 + k_o * k_i].reshape(B, k_o, k_i), 2 * ref) < (1e-4 if split else 2e-2)


def test_gradproj_embedding_golden_and_bad_ids(golden):
    """The reference's per-token loop (golden output), then an id outside the table: the kernel skips
    it and the next poll raises IndexError, as indexing P_i[:, id] does in the reference."""
    ids = torch.from_numpy(golden["gp_emb_ids"])
    G = torch.from_numpy(golden["gp_emb_G"])
    P_i, P_o = torch.from_numpy(golden["gp_emb_P_i"]), torch.from_numpy(golden["gp_emb_P_o"])
    o = ops()
    Po = o.prepare_projection(P_o.cuda(), True)
    PiT = o.prepare_embedding_projection(P_i.cuda())
    out = o.gradproj_embedding(ids.cuda(), G.cuda(), Po, PiT, 4, 5)
    after()
    want = torch.from_numpy(golden["gp_emb"])
    assert O.rel_fro(out.reshape(3, 4, 5), want) < 1e-4
    assert torch.allclose(out.cpu().reshape(3, 4, 5), want, rtol=1e-3, atol=1e-4)
    bad = ids.clone()
    bad[1, 2] = 19                                        # vocab is 19
    out2 = o.gradproj_embedding(bad.cuda(), G.cuda(), Po, PiT, 4, 5)
    torch.cuda.synchronize()
    from ghostsuite_b200 import _lib
    with pytest.raises(IndexError):
        _lib.poll_kernel_error()
    _lib.poll_kernel_error()                              # the word was cleared
    keep = torch.ones(3, 7, dtype=torch.bool)
    keep[1, 2] = False
    ref = O.gradproj_embedding(ids, G * keep.unsqueeze(-1), P_i, P_o, compute_dtype=torch.float64)
    assert O.rel_fro(out2.reshape(3, 4, 5), ref) < 1e-4     # the bad token contributed nothing


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", [(3, 5, 64), (16, 16, 98304), (8, 40, 1000), (33, 17, 4096),
                                  (5, 3, 12345), (1, 1, 7), (16, 8, 917504)])
def test_projection_similarity(case, dtype):
    n1, n2, D = case
    g = torch.Generator().manual_seed(22)
    P1 = torch.randn(n1, D, generator=g).to(dtype)
    P2 = (torch.randn(n2, D, generator=g) + 0.05 * torch.randn(1, D, generator=g)).to(dtype)
    S = ops().projection_similarity(P1.cuda(), P2.cuda(), 0.5)
    after()
    ref = 0.5 * O.projection_similarity(P1, P2)
    assert S.shape == (n1, n2) and S.dtype == torch.float32
    assert O.rel_fro(S, ref) < 1e-4
    # rows of a wider buffer (the engine's [B, total_proj_dim] buffer, a column range of it)
    if D >= 64:
        wide = torch.zeros(n1, D + 24, dtype=dtype, device="cuda")
        wide[:, 8:8 + D] = P1.cuda()
        S2 = ops().projection_similarity(wide[:, 8:8 + D], P2.cuda(), 0.5)
        after()
        assert O.rel_fro(S2, ref) < 1e-4


def test_small_reduce_batch_matches_single_launches():
    """One batched launch for many layers' small reductions against the per-layer kernels: more jobs
    than fit one launch, mixed sizes, Gram only / sum only / both, bf16 and fp32 sums."""
    o = ops()
    g = torch.Generator().manual_seed(23)
    jobs, want = [], []
    for i in range(110):
        n_t, n_v = (5, 3) if i % 3 else (32, 8)
        F = (768, 10, 3072, 37, 1)[i % 5]
        X = torch.randn(n_t + n_v, F, generator=g).cuda()
        job = {"X": X, "n_train": n_t, "n_val": n_v}
        rec = {}
        if i % 4 != 1:
            job["M"] = torch.full((n_v, n_t), 7.0, device="cuda")
            job["dot_scale"] = 0.5
            rec["M"] = o.small_gram(X, n_v, 0.5)
        if i % 4 != 2:
            dt = torch.bfloat16 if i % 2 else torch.float32
            job["sum_out"] = torch.full((F,), 7.0, dtype=dt, device="cuda")
            job["sum_scale"] = 0.25
            rec["sum"] = o.rows_sum(X, n_t, 0.25, dt)
        jobs.append(job)
        want.append(rec)
    from ghostsuite_b200 import _lib
    l0 = _lib.launch_count()
    o.small_reduce_batch(jobs)
    assert _lib.launch_count() - l0 == 3                      # 48 jobs per launch
    after()
    for job, rec in zip(jobs, want):
        if "M" in rec:
            assert torch.equal(job["M"], rec["M"])
        if "sum" in rec:
            assert torch.equal(job["sum_out"], rec["sum"])


def test_error_codes_are_python_exceptions():
    o = ops()
    A = torch.randn(4, 3, 8, device="cuda")
    with pytest.raises(ValueError):
        o.gram_dot(A, A, 4)            # no training samples
    with pytest.raises(ValueError):
        o.small_gram(A.reshape(4, 24), 4)
    with pytest.raises(RuntimeError):
        o.colsum(A.cpu())
    # the two-pass entry points through the raw C ABI: every refusal is GHOST_ERR_INVALID with a message
    from ghostsuite_b200 import _lib
    lib = _lib.load()
    X = torch.zeros(6, 16, 64, dtype=torch.bfloat16, device="cuda")
    tiles = torch.zeros(6 * 32768, dtype=torch.bfloat16, device="cuda")
    M = torch.zeros(64, device="cuda")
    nbytes = lib.ghost_persample_tiles_bytes(6, 64, 64)
    assert nbytes == 6 * 65536 and lib.ghost_persample_tiles_bytes(0, 64, 64) == 0
    args = lambda s0, ns, nb: (X.data_ptr(), X.data_ptr(), 6, 16, 64, 64, 64, 64, s0, ns, 0, None, tiles.data_ptr(), nb, None)
    assert lib.ghost_persample_tiles_bf16(*args(0, 6, nbytes)) == 0
    assert lib.ghost_persample_tiles_bf16(*args(4, 3, nbytes)) == -1 and b"sample range" in lib.ghost_last_error()
    assert lib.ghost_persample_tiles_bf16(*args(0, 6, nbytes - 1)) == -1 and b"too small" in lib.ghost_last_error()
    dot = lambda ranks, per, n_t, grad: lib.ghost_tile_dot_bf16(tiles.data_ptr(), ranks, per, tiles.data_ptr(), n_t, 64, 64, 1.0,
                                                                M.data_ptr(), grad, 0, 1.0, 0, None)
    assert dot(1, 2, 4, None) == 0
    assert dot(4, 3, 4, None) == -1 and b"per rank" in lib.ghost_last_error()
    assert dot(1, 2, 33, tiles.data_ptr()) == -1 and b"32 train samples" in lib.ghost_last_error()
    assert dot(1, 2, 0, None) == -1
    after()


# ------------------------------------------------------------------------------------------------
# benchmark model helper: fused token cross-entropy against torch's own
# ------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(37, 1000, 1000), (64, 50304, 50257), (5, 72, 61)])
def test_fused_token_loss_matches_torch(shape, dtype):
    from ghostsuite_b200.workloads import _FusedTokenLoss
    rows, cols, valid = shape
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(rows, cols, generator=g) * 3).to(dtype).cuda().requires_grad_(True)
    target = torch.randint(0, valid, (rows,), generator=g)
    target[::7] = -100
    target = target.cuda()
    loss = _FusedTokenLoss.apply(logits, target, valid)
    (loss * 1.7).backward()
    ref_logits = logits.detach().float().clone().requires_grad_(True)
    masked = ref_logits[:, :valid]
    ref = torch.nn.functional.cross_entropy(masked, target, ignore_index=-100)
    (ref * 1.7).backward()
    assert abs(loss.item() - ref.item()) <= 2e-5 * max(1.0, abs(ref.item()))
    got = logits.grad.float()
    want = ref_logits.grad
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5       # relative Frobenius; bf16 = one rounding of the result
    assert (got - want).norm() <= tol * want.norm()
    assert torch.count_nonzero(got[:, valid:]) == 0
    assert torch.count_nonzero(got[::7]) == 0
    # a retained graph backpropagated twice with different upstream gradients
    x2 = logits.detach().clone().requires_grad_(True)
    loss2 = _FusedTokenLoss.apply(x2, target, valid)
    loss2.backward(retain_graph=True)
    g1 = x2.grad.float().clone()
    x2.grad = None
    (loss2 * 0.25).backward()
    assert (g1 * 1.7 - want).norm() <= tol * want.norm()
    assert (x2.grad.float() * 4 * 1.7 - want).norm() <= tol * want.norm()
    # logits that need no gradient take the forward-only kernel
    assert abs(_FusedTokenLoss.apply(logits.detach(), target, valid).item() - ref.item()) <= 2e-5 * max(1.0, abs(ref.item()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(6, 5, 64), (9, 33, 768), (3, 17, 4096), (4, 7, 30)])
def test_rmsnorm_persample(shape, dtype):
    N, T, F = shape
    g = torch.Generator().manual_seed(21)
    A = (torch.randn(N, T, F, generator=g) * 2 + 0.3).to(dtype)
    G = torch.randn(N, T, F, generator=g).to(dtype)
    gw, gsum = ops().layernorm_persample(A.cuda(), G.cuda(), 1e-6, rms=True)
    want = O.rmsnorm_persample_exact(A, G, 1e-6)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert O.rel_fro(gw, want) < tol
    assert O.rel_fro(gsum, G.double().sum(1)) < tol
