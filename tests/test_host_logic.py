"""Host-side logic that needs no GPU: deferred reduction of the dot-product vectors, the path rule's
cost model, the flat projection file format."""
import contextlib
import io

import numpy as np
import torch
from torch import nn

from ghostsuite_b200.ghostEngines import supported_layers_grad_samplers_dotprod as L


def test_deferred_dot_vectors_are_reduced_in_one_batch():
    params = [nn.Parameter(torch.zeros(3)) for _ in range(3)]
    mats = [torch.randn(4, 6) for _ in range(4)]
    assert L.begin_deferred_dots() is True
    assert L.begin_deferred_dots() is False              # already collecting
    L._set_dot(params[0], mats[0])
    L._set_dot(params[1], mats[1])
    L._set_dot(params[2], mats[2])
    L._set_dot(params[0], mats[3])                        # a tied parameter: the last hook wins
    assert params[1].grad_dot_prod_matrix is mats[1]
    L.finalize_pending_dots()
    for p, m in zip(params, (mats[3], mats[1], mats[2])):
        assert p.grad_dot_prod_matrix is m
        assert p.grad_dot_prod.shape == (6,)
        assert torch.allclose(p.grad_dot_prod, m.sum(0))
    L.finalize_pending_dots()                             # nothing pending: a no-op
    q = nn.Parameter(torch.zeros(1))
    L._set_dot(q, mats[0])                                # outside a backward pass: reduced at once
    assert torch.allclose(q.grad_dot_prod, mats[0].sum(0))


def _decide(n_t, n_v, T, d, p, rule="cost", dtype=torch.bfloat16):
    layer = nn.Linear(d, p, bias=False, device="meta")
    A = torch.empty(n_t + n_v, T, d, dtype=dtype, device="meta")
    B = torch.empty(n_t + n_v, T, p, dtype=dtype, device="meta")
    old = L.PATH_RULE
    L.PATH_RULE = rule
    try:
        L._should_use_ghost_computation(layer, A, B, val_batch_size=n_v)
    finally:
        L.PATH_RULE = old
    return layer.use_ghost_computation


def test_path_rule_follows_the_measured_crossover():
    # single layer 4096 -> 11008: the Gram kernel wins at T = 128, the per-sample path from T = 512 on
    assert _decide(256, 32, 128, 4096, 11008) is True
    assert _decide(256, 32, 512, 4096, 11008) is False
    assert _decide(64, 8, 2048, 4096, 11008) is False
    assert _decide(16, 2, 8192, 4096, 11008) is False
    # GPT-2 layers at T = 1024 take the per-sample path, the T = 1 MLP the Gram kernel
    for d, p in ((768, 2304), (768, 768), (768, 3072), (3072, 768), (768, 50304)):
        assert _decide(32, 8, 1024, d, p) is False
    assert _decide(64, 16, 1, 512, 1024, dtype=torch.float32) is True
    # the reference's rule 2 T^2 <= numel and the forced rules
    assert _decide(32, 8, 1024, 768, 2304, rule="reference") is False        # 2 * 1024^2 > 1.77 M
    assert _decide(32, 8, 1024, 768, 3072, rule="reference") is True         # 2 * 1024^2 <= 2.36 M
    assert _decide(32, 8, 1024, 768, 50304, rule="reference") is True
    assert _decide(32, 8, 1024, 768, 768, rule="gram") is True
    assert _decide(256, 32, 128, 4096, 11008, rule="persample") is False


def test_flat_projection_file_round_trip(tmp_path):
    from ghostsuite_b200.ghostEngines.gradProjection.gradproj_engine import GradProjLoraEngine, load_projection_bin
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(10, 24), nn.ReLU(), nn.Linear(24, 5))
    with contextlib.redirect_stdout(io.StringIO()):
        eng = GradProjLoraEngine(model, "0,2", 16, 2, 42, "float32", str(tmp_path / "p"), proj_format="bin")
    rows = [torch.randn(n, eng.total_proj_dim) for n in (4, 3, 5)]
    for it, r in enumerate(rows):
        eng.iteration = it
        with contextlib.redirect_stdout(io.StringIO()):
            eng._save_projection(r, batch_indices=list(range(100 * it, 100 * it + r.shape[0])))
    eng.flush()
    data, index = load_projection_bin(str(tmp_path / "p"))
    assert data.shape == (12, eng.total_proj_dim) and index["dtype"] == "float32"
    assert [b["row0"] for b in index["batches"]] == [0, 4, 7]
    assert index["batches"][2]["batch_idx"] == [200, 201, 202, 203, 204]
    assert np.array_equal(np.asarray(data), torch.cat(rows).numpy())
    eng.cleanup()


def test_choose_ki_ko_reproduces_the_reference_table(golden):
    """``choose_ki_ko`` against the (n_i, n_o, k_total, k_min) -> (k_i, k_o) rows that the golden
    script recorded from the reference's projection_utils.choose_ki_ko (:12-66 there)."""
    from ghostsuite_b200.ghostEngines.gradProjection.projection_utils import choose_ki_ko
    table = golden["choose_ki_ko_table"]
    assert table.shape[0] >= 7
    for n_i, n_o, k_total, k_min, k_i, k_o in table.tolist():
        assert choose_ki_ko(n_i, n_o, k_total, k_min) == (k_i, k_o), (n_i, n_o, k_total, k_min)
