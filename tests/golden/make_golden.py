"""Generate the golden fixtures in this directory by running the reference's own code.

Run once in a container that has the reference checkout (it cannot travel to the GPU machine):

    python tests/golden/make_golden.py --reference /path/to/GhostSuite

Every fixture stores the seeded *inputs* next to the reference's *outputs*, so the tests never
depend on RNG streams matching across torch versions.  bf16 tensors are stored as float32 (exact).

The reference functions exercised (paths inside the reference project):
  ghostEngines/supported_layers_grad_samplers_dotprod.py  -- every (dot_fn, train_grad_fn) pair
  ghostEngines/autograd_grad_sample_dotprod.py            -- _compute_train_grad_bias, add_hooks
  ghostEngines/graddotprod_engine.py                      -- 3-step MLP run (engine level)
  ghostEngines/gradProjection/autograd_gradproj.py        -- _compute_dense_proj, _compute_embedding_proj
  ghostEngines/gradProjection/projection_utils.py         -- choose_ki_ko, gaussian initialiser
  ghostEngines/gradProjection/gradproj_engine.py          -- engine-level MLP projection
"""

import argparse
import contextlib
import io
import os
import sys

import numpy as np
import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))


def f32(x):
    return x.detach().to(torch.float32).cpu().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the GhostSuite reference to import from")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import transformers.pytorch_utils as tpu
    from ghostEngines import supported_layers_grad_samplers_dotprod as ref
    from ghostEngines import autograd_grad_sample_dotprod as refhooks
    from ghostEngines import GradDotProdEngine
    from ghostEngines.gradProjection.autograd_gradproj import GradProjHooks
    from ghostEngines.gradProjection import projection_utils as pu
    from ghostEngines.gradProjection.gradproj_engine import GradProjLoraEngine

    torch.manual_seed(20240611)
    out = {}

    n_t, n_v, T, d, p = 5, 3, 6, 16, 24
    N = n_t + n_v

    # ---------------- Linear / Conv1D ----------------
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        A = (torch.randn(N, T, d) / math_sqrt(d)).to(dtype)
        G = (torch.randn(N, T, p) / math_sqrt(p)).to(dtype)
        out[f"lin_{tag}_A"] = f32(A)
        out[f"lin_{tag}_G"] = f32(G)
        for nv in (1, n_v):
            for ghost in (True, False):
                lin = nn.Linear(d, p).to(dtype)
                lin.use_ghost_computation = ghost
                ref._compute_linear_dot_product(lin, A, G, nv)
                out[f"lin_{tag}_nv{nv}_ghost{int(ghost)}_w"] = f32(lin.weight.grad_dot_prod)
                out[f"lin_{tag}_nv{nv}_ghost{int(ghost)}_b"] = f32(lin.bias.grad_dot_prod)
                c1d = tpu.Conv1D(p, d).to(dtype)
                c1d.use_ghost_computation = ghost
                ref._compute_Conv1D_dot_product(c1d, A, G, nv)
                out[f"c1d_{tag}_nv{nv}_ghost{int(ghost)}_w"] = f32(c1d.weight.grad_dot_prod)
                out[f"c1d_{tag}_nv{nv}_ghost{int(ghost)}_b"] = f32(c1d.bias.grad_dot_prod)
        # rows of the full matrix through n_val = 1 calls (exact algebra in the reference)
        rows_w = []
        for v in range(n_v):
            lin = nn.Linear(d, p).to(dtype)
            lin.use_ghost_computation = False
            Av = torch.cat([A[:n_t], A[n_t + v:n_t + v + 1]])
            Gv = torch.cat([G[:n_t], G[n_t + v:n_t + v + 1]])
            ref._compute_linear_dot_product(lin, Av, Gv, 1)
            rows_w.append(f32(lin.weight.grad_dot_prod))
        out[f"lin_{tag}_rows_materialised"] = np.stack(rows_w)
        Gs = G * N
        lin = nn.Linear(d, p).to(dtype)
        out[f"lin_{tag}_train_grad"] = f32(ref._compute_linear_train_grad(lin, A, Gs, n_v))
        c1d = tpu.Conv1D(p, d).to(dtype)
        out[f"c1d_{tag}_train_grad"] = f32(ref._compute_Conv1D_train_grad(c1d, A, Gs, n_v))
        out[f"bias_{tag}_train_grad"] = f32(refhooks._compute_train_grad_bias(Gs.clone(), n_v))

    # 2-D (T = 1) linear, the MLP case
    A2 = torch.randn(12, 16)
    G2 = torch.randn(12, 10)
    out["lin2d_A"] = f32(A2)
    out["lin2d_G"] = f32(G2)
    lin = nn.Linear(16, 10)
    ref._compute_linear_dot_product(lin, A2, G2, 4)
    assert lin.use_ghost_computation is True
    out["lin2d_nv4_w"] = f32(lin.weight.grad_dot_prod)
    out["lin2d_nv4_b"] = f32(lin.bias.grad_dot_prod)
    out["lin2d_train_grad"] = f32(ref._compute_linear_train_grad(lin, A2, G2 * 12, 4))

    # heuristic table
    heur = []
    for (T_, d_, p_) in ((1, 16, 10), (6, 16, 24), (20, 16, 24), (1024, 768, 2304),
                         (1024, 768, 3072), (1024, 768, 768), (1024, 768, 50257)):
        l = nn.Linear(d_, p_, device="meta")
        a = torch.empty(2, T_, d_, device="meta") if T_ > 1 else torch.empty(2, d_, device="meta")
        b = torch.empty(2, T_, p_, device="meta") if T_ > 1 else torch.empty(2, p_, device="meta")
        ref._should_use_ghost_computation(l, a, b)
        heur.append((T_, d_, p_, int(l.use_ghost_computation)))
    out["heuristic_table"] = np.array(heur, dtype=np.int64)

    # ---------------- Embedding ----------------
    vocab, de = 11, 8
    ids = torch.randint(0, vocab, (N, T))
    out["emb_ids"] = ids.numpy()
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        Ge = (torch.randn(N, T, de) / math_sqrt(de)).to(dtype)
        out[f"emb_{tag}_G"] = f32(Ge)
        emb = nn.Embedding(vocab, de).to(dtype)
        for nv in (1, n_v):
            ref._compute_embedding_dot_product(emb, ids, Ge, nv)
            out[f"emb_{tag}_nv{nv}_w"] = f32(emb.weight.grad_dot_prod)
        out[f"emb_{tag}_train_grad"] = f32(ref._compute_embedding_train_grad(emb, ids, Ge * N, n_v))

    # ---------------- LayerNorm ----------------
    Fdim = 16
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        Al = (torch.randn(N, T, Fdim) * 1.5 + 0.3).to(dtype)
        Gl = (torch.randn(N, T, Fdim) / math_sqrt(Fdim)).to(dtype)
        out[f"ln_{tag}_A"] = f32(Al)
        out[f"ln_{tag}_G"] = f32(Gl)
        for nv in (1, n_v):
            ln = nn.LayerNorm(Fdim).to(dtype)
            ref._compute_layernorm_dot_product(ln, Al, Gl, nv)
            out[f"ln_{tag}_nv{nv}_w"] = f32(ln.weight.grad_dot_prod)
            out[f"ln_{tag}_nv{nv}_b"] = f32(ln.bias.grad_dot_prod)
        ln = nn.LayerNorm(Fdim).to(dtype)
        ref._compute_layernorm_train_grad(ln, Al, Gl * N, n_v)
        out[f"ln_{tag}_train_grad_w"] = f32(ln.weight.train_grad)
        out[f"ln_{tag}_train_grad_b"] = f32(ln.bias.train_grad)
    out["ln_eps"] = np.array([nn.LayerNorm(Fdim).eps])

    # ---------------- Conv2d ----------------
    Ac = torch.randn(N, 3, 7, 6)
    conv = nn.Conv2d(3, 5, kernel_size=(3, 2), stride=(2, 1), padding=(1, 0), dilation=(1, 2))
    out[f"conv_A"] = f32(Ac)
    Gc = torch.randn_like(conv(Ac)) / 5.0
    out["conv_G"] = f32(Gc)
    # The reference's ghost branch for Conv2d multiplies a [b, D, D] by a [b, p, p] tensor (it
    # contracts over the output positions instead of the features, :550-554) and raises unless
    # C*kh*kw == out_channels, so only the materialised branch can be recorded.
    try:
        c = nn.Conv2d(3, 5, kernel_size=(3, 2), stride=(2, 1), padding=(1, 0), dilation=(1, 2))
        c.use_ghost_computation = True
        ref._compute_conv2d_dot_product(c, Ac, Gc, 1)
        out["conv_ghost_branch_runs"] = np.array([1])
    except RuntimeError:
        out["conv_ghost_branch_runs"] = np.array([0])
    for nv in (1, n_v):
        c = nn.Conv2d(3, 5, kernel_size=(3, 2), stride=(2, 1), padding=(1, 0), dilation=(1, 2))
        c.use_ghost_computation = False
        ref._compute_conv2d_dot_product(c, Ac, Gc, nv)
        out[f"conv_nv{nv}_ghost0_w"] = f32(c.weight.grad_dot_prod)
        out[f"conv_nv{nv}_ghost0_b"] = f32(c.bias.grad_dot_prod)
    out["conv_train_grad"] = f32(ref._compute_conv2d_train_grad(conv, Ac, Gc * N, n_v))

    # ---------------- GradProj dense ----------------
    k_i, k_o = 4, 6
    P_i = pu.init_projection_matrix_gaussian(k_i, d, seed=42)
    P_o = pu.init_projection_matrix_gaussian(k_o, p, seed=1042)
    out["gp_P_i"] = f32(P_i)
    out["gp_P_o"] = f32(P_o)
    Ag = out["lin_f32_A"]
    Gg = out["lin_f32_G"]
    hooks = GradProjHooks(P_i, P_o, "lin", "Linear")
    lin = nn.Linear(d, p)
    hooks._compute_dense_proj(lin, torch.from_numpy(Ag), torch.from_numpy(Gg))
    out["gp_linear"] = f32(lin._ghost_grad_proj)
    # Conv1D(nf=p, nx=d): weight [d, p]; the reference sizes P_i by weight.shape[1] (= p) and
    # P_o by weight.shape[0] (= d)
    c1d = tpu.Conv1D(p, d)
    P_i_c = pu.init_projection_matrix_gaussian(k_i, p, seed=43)
    P_o_c = pu.init_projection_matrix_gaussian(k_o, d, seed=1043)
    out["gp_c1d_P_i"] = f32(P_i_c)
    out["gp_c1d_P_o"] = f32(P_o_c)
    hooks = GradProjHooks(P_i_c, P_o_c, "c1d", "Linear")
    hooks._compute_dense_proj(c1d, torch.from_numpy(Ag), torch.from_numpy(Gg))
    out["gp_c1d"] = f32(c1d._ghost_grad_proj)

    kk = []
    for (ni, no, kt, km) in ((1024, 4096, 1024, 4), (4096, 14336, 4096, 4), (768, 768, 256, 4),
                             (768, 2304, 256, 8), (10, 20, 16, 2), (4096, 1024, 4096, 4),
                             (16, 24, 24, 1)):
        kk.append((ni, no, kt, km) + tuple(pu.choose_ki_ko(ni, no, kt, km)))
    out["choose_ki_ko_table"] = np.array(kk, dtype=np.int64)

    # ---------------- engine level: GradDotProd on a small MLP, 3 SGD steps ----------------
    torch.manual_seed(7)
    model = nn.Sequential(nn.Linear(10, 8), nn.ReLU(), nn.Linear(8, 4))
    out["mlp_init"] = np.concatenate([f32(q).ravel() for q in model.parameters()])
    Xm = torch.randn(12, 10)
    Ym = torch.randint(0, 4, (12,))
    out["mlp_X"] = f32(Xm)
    out["mlp_Y"] = Ym.numpy()
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    eng = GradDotProdEngine(module=model, val_batch_size=4, loss_reduction="mean",
                            use_dummy_bias=False)
    eng.attach(opt)
    for step in range(3):
        eng.attach_train_batch(Xm[:8], Ym[:8], step, 0)
        loss = nn.functional.cross_entropy(model(Xm), Ym)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        for name, q in model.named_parameters():
            out[f"mlp_step{step}_{name}_dot"] = f32(q.grad_dot_prod)
            out[f"mlp_step{step}_{name}_train_grad"] = f32(q.train_grad)
        eng.aggregate_and_log()
        out[f"mlp_step{step}_agg"] = f32(eng.dot_product_log[-1]["dot_product"])
        eng.prepare_gradients()
        opt.step()
        eng.clear_gradients()
    out["mlp_final"] = np.concatenate([f32(q).ravel() for q in model.parameters()])
    eng.detach()

    # ---------------- engine level: GradProj on a small MLP ----------------
    torch.manual_seed(11)
    gmodel = nn.Sequential()
    gmodel.add_module("fc1", nn.Linear(10, 20))
    gmodel.add_module("relu", nn.ReLU())
    gmodel.add_module("fc2", nn.Linear(20, 5))
    out["gpmlp_init"] = np.concatenate([f32(q).ravel() for q in gmodel.parameters()])
    Xg = torch.randn(4, 10)
    Yg = torch.randint(0, 5, (4,))
    out["gpmlp_X"] = f32(Xg)
    out["gpmlp_Y"] = Yg.numpy()
    with contextlib.redirect_stdout(io.StringIO()):
        geng = GradProjLoraEngine(gmodel, proj_layers="fc", proj_rank_total=16, proj_rank_min=2,
                                  proj_seed=42, proj_dtype="float32", proj_dir="/tmp/_gp_golden",
                                  proj_save_interval=10 ** 9)
        geng.attach()
    out["gpmlp_dims"] = np.array([geng.projection_dims[k] for k in sorted(geng.matched_layers)],
                                 dtype=np.int64)
    for k in sorted(geng.matched_layers):
        out[f"gpmlp_P_i_{k}"] = f32(geng.projection_matrices[k][0])
        out[f"gpmlp_P_o_{k}"] = f32(geng.projection_matrices[k][1])
    gmodel.zero_grad()
    nn.functional.cross_entropy(gmodel(Xg), Yg).backward()
    geng.iteration = 1   # skip the disk write (interval is huge)
    out["gpmlp_proj"] = f32(geng.collect_batch())
    geng.detach()

    # ---------------- GradProj embedding projection (own generator: earlier draws stay as they are) ----
    ge = torch.Generator().manual_seed(31)
    V_e, d_e, T_e, B_e, ki_e, ko_e = 19, 12, 7, 3, 5, 4
    ids_e = torch.randint(0, V_e, (B_e, T_e), generator=ge)
    G_e = torch.randn(B_e, T_e, d_e, generator=ge)
    P_i_e = pu.init_projection_matrix_gaussian(ki_e, V_e, seed=44)
    P_o_e = pu.init_projection_matrix_gaussian(ko_e, d_e, seed=1044)
    emb = nn.Embedding(V_e, d_e)
    GradProjHooks(P_i_e, P_o_e, "emb", "Embedding")._compute_embedding_proj(emb, ids_e, G_e)
    out["gp_emb_ids"] = ids_e.numpy()
    out["gp_emb_G"] = f32(G_e)
    out["gp_emb_P_i"] = f32(P_i_e)
    out["gp_emb_P_o"] = f32(P_o_e)
    out["gp_emb"] = f32(emb._ghost_grad_proj)

    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


def math_sqrt(x):
    return float(x) ** 0.5


if __name__ == "__main__":
    main()
