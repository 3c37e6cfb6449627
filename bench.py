#!/usr/bin/env python
"""Benchmark of the ghost hot path on the GPT-2-small GradDotProd configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the hot path over one synthetic batch: forward and backward of a GPT-2-small
architecture (12 layers, d=768, 12 heads, vocab 50257, random init, bf16) on cat(train, val)
sequences of 1024 uniform-random token ids, with every hooked layer's dot-product matrix [8 x 32]
and train gradient produced by the CUDA kernels inside the backward hooks, then
prepare_gradients, the optimizer step, and aggregate_and_log.  Metric: train tokens per second
(train tokens of the global batch / step time), the definition used for the CPU baseline as well.

The batch is the configuration's: 32 train + 8 validation sequences in total (strong scaling).  With
N > 1 (launched by torch.distributed.run, one rank per GPU) every rank takes 32 / N train sequences
and either the whole validation batch (`val_replicated`) or 8 / N of it, with a per-layer all-gather
of the validation operands (`val_sharded`) or of the validation samples' per-sample gradients
(`val_exchanged`: tiles on the per-sample path, vectors of bias and norm layers); all variants are
timed and the fastest one is the line's `value`.  After backward the per-parameter dot-product blocks are all-gathered and the train
gradients all-reduced over NCCL.  `weak_scaling` is the same step with 32 train sequences on every
GPU.  On the first, untimed step of each variant the gathered results are checked (`dist_check`).

After the timed region the line gains `gradproj` (the GradProj kernel on the Llama-3-8B Linear
shapes and a Pythia-410M-shaped GradProj step, corpus-sharded over the ranks), `reference_gpu` (the
reference's own PyTorch layer functions on the same GPU beside the kernels that replace them) and,
at N = 1, `cpu_baseline`.

`--impl reference` times the reference's own engine on the host cores (the unmodified package from
baseline/_ref when `__graft_entry__.build()` has staged it, else the oracle's restatement of it), on
a bounded sample.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_TRAIN, N_VAL, SEQ = 32, 8, 1024
WORKLOAD = "GradDotProd, GPT-2-small architecture (12L, d768, 12H, vocab 50257, tied head), bf16, " \
           "T=1024, global batch of 32 train + 8 val sequences, full 8x32 dot-product matrix per parameter"
METRIC = "train tokens/sec (ghost dot-prod + train grad, GPT-2 124M)"


# ------------------------------------------------------------------------------------------------
_SAVED_STDOUT = None


def guard_stdout():
    """Point file descriptor 1 at stderr so that library banners and engine log lines do not mix with
    the JSON result; emit() restores it."""
    global _SAVED_STDOUT
    if _SAVED_STDOUT is None:
        sys.stdout.flush()
        _SAVED_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(obj):
    global _SAVED_STDOUT
    sys.stdout.flush()
    if _SAVED_STDOUT is not None:
        os.dup2(_SAVED_STDOUT, 1)
        os.close(_SAVED_STDOUT)
        _SAVED_STDOUT = None
    print(json.dumps(obj), flush=True)


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"tensor": float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 1400.0))),
                "hbm": float(d.get("hbm_gbs", 6650.0)), "source": "measured (sustained bf16 GEMM / copy)"}
    return {"tensor": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons = [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    out["sm_max_mhz"] = float(f[2])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            # under load = samples in the upper half of what was seen
            busy = [x for x in sm if x >= 0.5 * max(sm)]
            out["sm_mhz"] = statistics.median(busy)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ------------------------------------------------------------------------------------------------
# CPU legs: the reference's own engine when it has been staged (baseline/_ref), else the oracle port
# ------------------------------------------------------------------------------------------------
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _reference_package():
    """The reference's unmodified ``ghostEngines`` package from baseline/_ref (staged by
    ``__graft_entry__.build()`` wherever the reference tree is present), or None."""
    if not os.path.isdir(os.path.join(REF_DIR, "ghostEngines")):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        import ghostEngines as ref_pkg                      # noqa: F401  (the reference's top-level name)
        return ref_pkg
    except Exception as exc:                                # e.g. a transformers release it cannot import under
        sys.stderr.write(f"reference package not importable: {exc}\n")
        return None


def cpu_step_factory(n_train: int, n_val: int, seed: int = 0):
    """One GradDotProd step of the full 12-layer model on the host cores.  Returns (step, kind, note).

    kind 'reference': the reference's GradDotProdEngine, hooks and layer functions, unmodified, through
    its public API, on float32 weights -- with bf16 weights its hook plumbing promotes the int64 token
    ids to bf16 (autograd_grad_sample_dotprod.py:116-123 there), position 1023 becomes 1024 and the
    embedding's index_add_ raises; its dot-product functions cast activations and out-grads to bf16
    themselves either way.  kind 'port': the oracle restatement of that path with bf16 weights."""
    from ghostsuite_b200.workloads import GPT2Like, GPT2Config
    torch.manual_seed(seed)
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(seed + 1)
    ids = torch.randint(0, 50257, (n_train + n_val, SEQ), generator=g)
    ref_pkg = _reference_package()
    if ref_pkg is not None:
        model = GPT2Like(GPT2Config(fused_loss=False))
        engine = ref_pkg.GradDotProdEngine(module=model, val_batch_size=n_val, loss_reduction="mean",
                                           use_dummy_bias=True)
        model.ghost_prepare()         # dummy bias on wte / wpe: what the reference's forward swap does for HF GPT-2
        opt = torch.optim.AdamW([p for n, p in model.named_parameters() if "dummy_bias" not in n], lr=1e-4)
        engine.attach(opt)

        def step():
            engine.attach_train_batch(ids[:n_train], ids[:n_train], 0, 0)
            loss, _ = model(ids, labels=ids)
            loss.backward()
            engine.prepare_gradients()
            opt.step()
            engine.aggregate_and_log()
            total = engine.dot_product_log[-1]["dot_product"]
            engine.dot_product_log.clear()
            engine.clear_gradients()
            opt.zero_grad(set_to_none=True)
            return float(total.sum())

        return step, "reference", ("reference's own GradDotProdEngine, float32 weights (it raises on bf16 weights: "
                                   "token ids promoted to bf16), bf16 dot products as the reference casts them")
    from oracle.ghost_engine_cpu import OracleDotProdEngine
    model = GPT2Like(GPT2Config()).to(torch.bfloat16)
    engine = OracleDotProdEngine(model, n_val, use_dummy_bias=True)
    engine.attach()
    opt = torch.optim.AdamW([p for n, p in model.named_parameters() if "dummy_bias" not in n], lr=1e-4)

    def step():
        loss, _ = model(ids, labels=ids)
        loss.backward()
        engine.prepare_gradients()
        opt.step()
        total = engine.aggregate()
        engine.clear_gradients()
        opt.zero_grad(set_to_none=True)
        return float(total.sum())

    return step, "port", "oracle restatement of the reference's path (no staged reference package), bf16 weights"


def run_reference_arm(args, rank: int):
    """The reference's CPU path on the host cores; rank 0 only."""
    if rank != 0:
        return None
    n_train, n_val = 1, 1
    step, kind, note = cpu_step_factory(n_train, n_val)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    val = n_train * SEQ / dt
    sample = (f"{n_train} train + {n_val} val sequences x {SEQ} tokens per step (full 12-layer model, the reference's "
              f"path rule, AdamW step included); {note}")
    cores = torch.get_num_threads()
    return {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "cpu_sample": sample},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def cpu_baseline_leg():
    n_train, n_val = 1, 1
    step, kind, note = cpu_step_factory(n_train, n_val)
    step()
    t0 = time.perf_counter()
    reps = 2
    for _ in range(reps):
        step()
    dt = (time.perf_counter() - t0) / reps
    return {"value": n_train * SEQ / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{n_train} train + {n_val} val sequences x {SEQ} tokens, full 12-layer model, "
                      f"{reps} timed steps after 1 warm-up ({dt:.1f} s/step); {note}"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def _rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch.distributed as dist
    from ghostsuite_b200 import ops, _lib, dist as gdist
    from ghostsuite_b200.ghostEngines import GradDotProdEngine
    from ghostsuite_b200.ghostEngines import supported_layers_grad_samplers_dotprod as L
    from ghostsuite_b200.workloads import GPT2Like, GPT2Config

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a B200: the kernels have no CPU fallback")
    if N_TRAIN % world or N_VAL % world:
        raise ValueError(f"--gpus {world}: the fixed batch of {N_TRAIN} train + {N_VAL} validation sequences "
                         "must divide over the ranks")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _lib.check(_lib.load().ghost_device_check())

    torch.manual_seed(0)
    model = GPT2Like(GPT2Config()).to(torch.bfloat16).to(dev)
    opt = torch.optim.AdamW([p for p in model.parameters()], lr=1e-4, fused=True)
    group = dist.group.WORLD if world > 1 else None
    n_batches = 4

    g = torch.Generator().manual_seed(1)
    val_ids = torch.randint(0, 50257, (N_VAL, SEQ), generator=g)              # the same on every rank
    dev_val = val_ids.to(dev)

    def draw(seed):
        gg = torch.Generator().manual_seed(seed)
        return [torch.randint(0, 50257, (N_TRAIN, SEQ), generator=gg).pin_memory() for _ in range(n_batches)]

    global_train = draw(100)            # strong scaling: one global batch per step, the same on every rank
    weak_train = draw(100 + rank)       # weak scaling: every rank has its own 32 sequences

    # ---------------------------------------------------------------- engine per variant
    state = {"engine": None, "sync": None, "deterministic": False}
    graph_checks = {}

    def attention_backend():
        """The fused attention kernels of PyTorch sum their backward with atomics, so two runs of the
        same batch differ in the last bf16 bits; the result check runs the model with the plain
        matmul-softmax attention, which is deterministic, so that 1e-5 means something."""
        import contextlib
        if not state["deterministic"]:
            return contextlib.nullcontext()
        from torch.nn.attention import sdpa_kernel, SDPBackend
        return sdpa_kernel(SDPBackend.MATH)

    def attach(n_val_engine: int, shard_val: bool):
        if state["engine"] is not None:
            if state["sync"] is not None:
                state["sync"].close()
            gdist.unshard_validation(state["engine"])
            state["engine"].detach()
        for _, prm in model.named_parameters():
            prm.requires_grad = True
        for m in model.modules():                      # the path choice depends on the batch split
            m.__dict__.pop("use_ghost_computation", None)
        eng = GradDotProdEngine(module=model, val_batch_size=n_val_engine, loss_reduction="mean",
                                use_dummy_bias=True)
        eng.attach(opt)
        state["engine"] = eng
        state["sync"] = gdist.overlap_train_grad_sync(eng, group) if world > 1 else None
        if shard_val and world > 1:
            if shard_val == "gradients":
                if args.exchange_own_group and "xgroup" not in state:
                    state["xgroup"] = dist.new_group(ranks=list(range(world)))
                gdist.exchange_validation(eng, group, state.get("xgroup"))
            else:
                gdist.shard_validation(eng, group)
        return eng

    def variant(name):
        """(train rows of this rank, validation rows of this rank, engine's validation count, shard_val)"""
        if name == "weak":
            return None, dev_val, N_VAL, False
        lo, hi = gdist.shard_bounds(N_TRAIN, rank, world)
        if name in ("val_sharded", "val_exchanged"):
            vlo, vhi = gdist.shard_bounds(N_VAL, rank, world)
            return (lo, hi), dev_val[vlo:vhi], vhi - vlo, ("gradients" if name == "val_exchanged" else "operands")
        return (lo, hi), dev_val, N_VAL, False

    def make_step(name, optimise=True):
        rows, x_val, n_val_engine, shard_val = variant(name)
        engine = attach(n_val_engine, shard_val)
        host = weak_train if rows is None else [t[rows[0]:rows[1]] for t in global_train]
        devb = [t.to(dev) for t in host]

        def step(i: int, from_host: bool):
            x_train = host[i % n_batches].to(dev, non_blocking=True) if from_host else devb[i % n_batches]
            engine.attach_train_batch(x_train, x_train, i, i)
            x = torch.cat((x_train, x_val), dim=0)
            with attention_backend():
                loss, _ = model(x, labels=x)
                loss.backward()
            if world > 1:
                gdist.sync_engine(engine, group, check_equal_shards=False)   # shards are equal by construction
            if not optimise:
                return
            engine.prepare_gradients()
            opt.step()
            engine.clear_gradients()            # host-side bookkeeping first, while the GPU is still busy
            opt.zero_grad(set_to_none=True)
            engine.aggregate_and_log()          # device -> host read of the step's result (the step's sync)
            engine.dot_product_log.clear()

        return step, engine, host[0].numel() * 8

    def make_graph_step(name):
        """The variant's step with forward, backward (hooks and their kernels), the collectives of
        `sync_engine`, `prepare_gradients` and the optimizer step captured once in a CUDA graph and
        replayed: at 12 sequences per GPU the eager step is bound by the host (about 21 ms to issue
        its ~1700 launches), not by the GPU.  The library only enqueues kernels and memsets on the
        stream it is given and NCCL collectives can be captured, so a replay refreshes every
        parameter's result matrix and `.grad` in place; the ids are copied into the graph's static
        input before each replay and the aggregated result is read back after it (the step's sync).
        Returns (step, launches per replay) or raises if the capture fails on any rank."""
        rows, x_val, n_val_engine, shard_val = variant(name)
        engine = attach(n_val_engine, shard_val)
        gopt = torch.optim.AdamW([p for p in model.parameters()], lr=1e-4, fused=True, capturable=True)
        host = weak_train if rows is None else [t[rows[0]:rows[1]] for t in global_train]
        devb = [t.to(dev) for t in host]
        n_loc = host[0].shape[0]
        x_static = torch.cat((devb[0], x_val), dim=0).clone()

        def drop_results():
            for prm in model.parameters():
                for attr in ("grad_dot_prod", "grad_dot_prod_matrix"):
                    if hasattr(prm, attr):
                        delattr(prm, attr)

        def body():
            loss, _ = model(x_static, labels=x_static)
            loss.backward()
            if world > 1:
                gdist.sync_engine(engine, group, check_equal_shards=False)
            engine.prepare_gradients()
            gopt.step()

        ok = torch.ones(1, device=dev)
        graph = None
        err = ""
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):             # warm-up on the capture stream (lazy initialisations)
                for _ in range(2):
                    body()
                    engine.clear_gradients()
                    gopt.zero_grad(set_to_none=True)
                    drop_results()
                # the eager result on these parameters and this batch, for the check of the first replay
                loss, _ = model(x_static, labels=x_static)
                loss.backward()
                if world > 1:
                    gdist.sync_engine(engine, group, check_equal_shards=False)
                named = [p for p in model.parameters() if hasattr(p, "grad_dot_prod_matrix")]
                eager_mats = torch.stack([p.grad_dot_prod_matrix for p in named]).clone()
                engine.clear_gradients()
                gopt.zero_grad(set_to_none=True)
                drop_results()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            l0 = _lib.launch_count()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                body()
            launches = _lib.launch_count() - l0
        except Exception as exc:                      # every rank must learn of it before anyone replays
            err = f"{type(exc).__name__}: {exc}"
            ok.zero_()
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            raise RuntimeError("CUDA-graph capture failed" + (f" here: {err}" if err else " on another rank"))
        mats = [prm.grad_dot_prod_matrix for prm in model.parameters() if hasattr(prm, "grad_dot_prod_matrix")]
        # first replay: same parameters, same batch as the eager step above (the fused attention
        # backward is not bit-reproducible, hence a bf16-sized tolerance)
        graph.replay()
        torch.cuda.synchronize()
        graph_checks[name + "_cuda_graph"] = {
            "matrices_rel_err": _rel(torch.stack(mats), eager_mats), "against": "the eager step on the same parameters and batch"}
        graph_checks[name + "_cuda_graph"]["ok"] = graph_checks[name + "_cuda_graph"]["matrices_rel_err"] < 2e-2
        del eager_mats

        def step(i: int, from_host: bool):
            src = host[i % n_batches] if from_host else devb[i % n_batches]
            x_static[:n_loc].copy_(src, non_blocking=True)
            graph.replay()
            total = torch.stack(mats).sum(dim=0)
            return total.sum(dim=0).cpu(), total.cpu()        # the step's device -> host read (and sync)

        return step, launches, host[0].numel() * 8

    def timed(step, from_host: bool, profile: bool):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        l0 = _lib.launch_count()
        if profile:
            ops.start_kernel_timing()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            step(i, from_host)
        e1.record()
        torch.cuda.synchronize()
        prof = ops.stop_kernel_timing() if profile else None
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            dist.barrier()
        return ms, _lib.launch_count() - l0, prof

    # ---------------------------------------------------------------- multi-GPU result check
    def snapshot(engine):
        named = [(n, p) for n, p in model.named_parameters() if hasattr(p, "grad_dot_prod_matrix")]
        mats = torch.stack([p.grad_dot_prod_matrix for _, p in named]).clone()
        grads = {n: p.train_grad.float().clone() for n, p in model.named_parameters() if hasattr(p, "train_grad")}
        engine.clear_gradients()
        for _, p in model.named_parameters():
            for attr in ("grad_dot_prod", "grad_dot_prod_matrix"):
                if hasattr(p, attr):
                    delattr(p, attr)
        return mats, grads

    def local_rerun(name, engine):
        """Rank 0 alone runs every rank's batch of the check step and assembles what the collectives
        should have produced: the blocks side by side (with the loss-normalisation rescale) and the
        mean of the shard gradients."""
        saved = L.TRAIN_GRAD_OBSERVER
        L.TRAIN_GRAD_OBSERVER = None
        try:
            blocks, grad_sum = [], None
            for r in range(world):
                if name == "weak":
                    gg = torch.Generator().manual_seed(100 + r)
                    x_train = torch.randint(0, 50257, (N_TRAIN, SEQ), generator=gg).to(dev)
                else:
                    lo, hi = gdist.shard_bounds(N_TRAIN, r, world)
                    x_train = global_train[0][lo:hi].to(dev)
                x = torch.cat((x_train, dev_val), dim=0)
                with attention_backend():
                    loss, _ = model(x, labels=x)
                    loss.backward()
                m, gr = snapshot(engine)
                blocks.append(m)
                grad_sum = gr if grad_sum is None else {n: grad_sum[n] + gr[n] for n in gr}
            n_loc = blocks[0].shape[-1]
            factor = (float(N_VAL + n_loc) / float(N_VAL + world * n_loc)) ** 2
            return torch.cat(blocks, dim=-1) * factor, {n: v / world for n, v in grad_sum.items()}
        finally:
            L.TRAIN_GRAD_OBSERVER = saved

    def check_variant(name, reference=None):
        """One untimed step of the variant without the optimizer; its gathered matrices and averaged
        train gradients against rank 0's local re-run of all shards (same shapes, same kernels,
        deterministic attention: 1e-5 on the float32 matrices, 1e-2 on the train gradients, which NCCL
        sums in bf16 rank by rank where the re-run averages in float32 -- 2e-3 at two ranks, 3e-3 at four), or
        against another variant's result (`reference`: different batch composition per rank, so the
        model's own bf16 GEMMs differ in the last bits -- the 2e-2 of bf16 parity)."""
        step, engine, _ = make_step(name, optimise=False)
        step(0, False)
        torch.cuda.synchronize()
        mats, grads = snapshot(engine)
        rec = {}
        if reference is None:
            if rank == 0:
                want_m, want_g = local_rerun(name, engine)
                rec["matrices_rel_err"] = _rel(mats, want_m)
                rec["train_grad_rel_err"] = max(_rel(grads[n], want_g[n]) for n in want_g)
                rec["ok"] = rec["matrices_rel_err"] < 1e-5 and rec["train_grad_rel_err"] < 1e-2
                rec["against"] = "rank 0's local re-run of every rank's shard"
            dist.barrier()
        else:
            rec["matrices_rel_err"] = _rel(mats, reference[0])
            rec["train_grad_rel_err"] = max(_rel(grads[n], reference[1][n]) for n in grads)
            rec["ok"] = rec["matrices_rel_err"] < 2e-2 and rec["train_grad_rel_err"] < 2e-2
            rec["against"] = "the val_replicated variant's gathered result"
        return rec, (mats, grads)

    dist_check = None
    if world > 1:
        dist_check = {}
        state["deterministic"] = True
        dist_check["val_replicated"], ref_res = check_variant("val_replicated")
        dist_check["val_sharded"], _ = check_variant("val_sharded", reference=ref_res)
        dist_check["val_exchanged"], _ = check_variant("val_exchanged", reference=ref_res)
        dist_check["weak"], _ = check_variant("weak")
        del ref_res
        state["deterministic"] = False

    # ---------------------------------------------------------------- timed runs
    sampler = ClockSampler(local_rank)
    results = {}
    prof = None
    names = ["val_replicated"] if world == 1 else ["val_replicated", "val_sharded", "val_exchanged", "weak"]
    keep = [v for v in args.only_variants.split(",") if v]
    if keep:
        names = [n for n in names if n == "val_replicated" or n == "weak" or n in keep]
    for name in names:
        step, engine, h2d = make_step(name)
        for i in range(args.warmup):
            step(i, False)
        torch.cuda.synchronize()
        if rank == 0 and name == "val_replicated":
            sampler.start()
        ms_dev, launches, _ = timed(step, False, False)
        rec = {"ms_dev": ms_dev, "launches": launches, "h2d": h2d}
        if name == "val_replicated":
            # the same K steps once more with a CUDA event pair around every library call (the
            # roofline's kernel durations); kept out of `value`: the event records cost ~2 % of the step
            _, _, prof = timed(step, False, True)
        rec["ms_e2e"], _, _ = timed(step, True, False)
        if rank == 0 and name == "val_replicated":
            rec["clocks"] = sampler.stop()
        n_steps_run = max(1, (args.warmup + 2 * args.steps))
        sv = getattr(engine, "_ghost_val_shard", None)
        ex = getattr(engine, "_ghost_val_exchange", None)
        if sv is not None:
            rec["val_gather_calls_per_step"] = (sv.calls + (ex.calls if ex else 0)) / n_steps_run
            rec["val_gather_bytes_per_step"] = (sv.bytes + (ex.bytes if ex else 0)) / n_steps_run
        results[name] = rec
    _lib.poll_kernel_error()

    # the same step with the model's loss through PyTorch ops instead of the library's fused loss kernels
    step, engine, _ = make_step("val_replicated")
    model.cfg.fused_loss = False
    for i in range(max(2, args.warmup // 2)):
        step(i, False)
    ms_torch_loss, _, _ = timed(step, False, False)
    model.cfg.fused_loss = True

    # the fixed-batch step replayed from a CUDA graph (validation replicated; with more than one GPU
    # also with the validation batch sharded)
    graph_note = None
    for base in (["val_replicated"] if world == 1 else
                 [n for n in ("val_replicated", "val_sharded", "val_exchanged") if n in names]):
        try:
            step, graph_launches, h2d = make_graph_step(base)
            for i in range(args.warmup):
                step(i, False)
            torch.cuda.synchronize()
            ms_dev, _, _ = timed(step, False, False)
            ms_e2e, _, _ = timed(step, True, False)
            rec = {"ms_dev": ms_dev, "ms_e2e": ms_e2e, "launches": graph_launches * args.steps, "h2d": h2d}
            sv = getattr(state["engine"], "_ghost_val_shard", None)
            ex = getattr(state["engine"], "_ghost_val_exchange", None)
            if sv is not None:              # counted at capture, in the two warm-up steps and in the eager check step
                rec["val_gather_calls_per_step"] = (sv.calls + (ex.calls if ex else 0)) / 4
                rec["val_gather_bytes_per_step"] = (sv.bytes + (ex.bytes if ex else 0)) / 4
            results[base + "_cuda_graph"] = rec
            names.insert(1, base + "_cuda_graph")
            _lib.poll_kernel_error()
        except Exception as exc:
            graph_note = f"{base}: not measured: {exc}"
            break

    if rank != 0:
        state["engine"].detach()
        return None
    peaks = _peaks()

    def line(name, tokens_per_step):
        r = results[name]
        return {"value": tokens_per_step * args.steps / (r["ms_dev"] * 1e-3), "ms_per_step": r["ms_dev"] / args.steps,
                "e2e": tokens_per_step * args.steps / (r["ms_e2e"] * 1e-3),
                **{k: v for k, v in r.items() if k.startswith("val_gather")}}

    tok_strong = N_TRAIN * SEQ                       # the fixed global batch
    variants = {n: line(n, tok_strong) for n in names if n != "weak"}
    best = max(variants, key=lambda n: variants[n]["value"])
    weak = line("weak", N_TRAIN * SEQ * world) if world > 1 else dict(variants["val_replicated"])
    weak["per_gpu_batch"] = f"{N_TRAIN} train + {N_VAL} val sequences on every GPU"
    h2d_total = results[best]["h2d"] * world
    d2h_bytes = (N_TRAIN * 4 + N_VAL * N_TRAIN * 4) * world
    roof = dominant_kernel_roofline(prof, peaks)
    how = {"val_replicated": "validation batch replicated, eager launches",
           "val_replicated_cuda_graph": "validation batch replicated, step replayed from a CUDA graph",
           "val_sharded": "validation batch sharded, per-layer all-gather of its operands",
           "val_sharded_cuda_graph": "validation batch sharded (per-layer all-gather of its operands), step replayed "
                                     "from a CUDA graph",
           "val_exchanged": "validation batch sharded, per-layer all-gather of its per-sample gradients (tiles / "
                            "vectors; operands for the embeddings)",
           "val_exchanged_cuda_graph": "validation batch sharded (per-layer all-gather of its per-sample gradients), "
                                       "step replayed from a CUDA graph"}[best]
    if world == 1:
        parallelism = f"1 GPU; {how} (the fastest of the variants measured in this run)"
    else:
        parallelism = (f"train batch sharded {N_TRAIN // world} per GPU over {world} GPUs; {how} "
                       "(the fastest of the variants measured in this run)")
    out = {
        "metric": METRIC, "value": variants[best]["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": variants[best]["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": parallelism,
                   "l2": "working set per step (activations + out-grads, > 1 GB per GPU) exceeds the 126 MB L2",
                   "optimizer": "AdamW (fused)", "path_rule": "cost",
                   "vocab_table_rows": "50257 ids; embedding / LM-head table padded to 50304 rows (padded logits masked out of the loss)"},
        "e2e": {"value": variants[best]["e2e"], "unit": "tokens/s", "h2d_bytes_per_step": h2d_total,
                "d2h_bytes_per_step": d2h_bytes},
        "gpu_launches": int(results[best]["launches"]),
        "clocks": results["val_replicated"].get("clocks"),
        "roofline": roof,
        "roofline_pass": "kernel durations from a second pass over the same steps (validation replicated) with CUDA "
                         "events around every library call; `value` is the pass without them",
        "kernel_time_share": prof["share"] if prof else None,
        "library_ms_per_step": (prof["total_ms"] / args.steps) if prof else None,
        "variants": variants,
        "cuda_graph_note": graph_note or "*_cuda_graph: the same step captured once (forward, backward with the hooks, "
                           "collectives, optimizer) and replayed; ids copied in before, result read back after",
        "weak_scaling": weak,
        "ms_per_step_torch_loss": ms_torch_loss / args.steps,
    }
    out["cuda_graph_check"] = graph_checks
    if dist_check is not None:
        dist_check.update(graph_checks)
        out["dist_check"] = "ok" if all(v.get("ok", True) for v in dist_check.values()) else "FAILED"
        out["dist_check_detail"] = dist_check
    state["engine"].detach()
    return out


def hf_gpt2_leg(dev, steps: int = 3):
    """The same GradDotProd step on `transformers.GPT2LMHeadModel` (GPT-2-small configuration, vocabulary
    50257 unpadded, the model's own loss) instead of this package's GPT2Like workload: what a user who
    brings the Hugging Face model gets from the hooks alone.  One GPU, a few steps, CUDA events."""
    from transformers import GPT2Config as HFConfig, GPT2LMHeadModel
    from ghostsuite_b200.ghostEngines import GradDotProdEngine
    torch.manual_seed(0)
    cfg = HFConfig(vocab_size=50257, n_positions=SEQ, n_embd=768, n_layer=12, n_head=12, resid_pdrop=0.0,
                   embd_pdrop=0.0, attn_pdrop=0.0, use_cache=False)
    model = GPT2LMHeadModel(cfg).to(torch.bfloat16).to(dev)
    opt = torch.optim.AdamW(list(model.parameters()), lr=1e-4, fused=True)
    engine = GradDotProdEngine(module=model, val_batch_size=N_VAL, loss_reduction="mean", use_dummy_bias=True)
    engine.attach(opt)
    g = torch.Generator().manual_seed(1)
    x = torch.randint(0, 50257, (N_TRAIN + N_VAL, SEQ), generator=g).to(dev)

    def step(i):
        engine.attach_train_batch(x[:N_TRAIN], x[:N_TRAIN], i, i)
        model(input_ids=x, labels=x).loss.backward()
        engine.prepare_gradients()
        opt.step()
        engine.clear_gradients()
        opt.zero_grad(set_to_none=True)
        engine.aggregate_and_log()
        engine.dot_product_log.clear()

    for i in range(2):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    hooked = len(model.autograd_grad_sample_hooks) // 2
    engine.detach()
    del model, opt, engine
    torch.cuda.empty_cache()
    return {"ms_per_step": ms, "tokens_per_s": N_TRAIN * SEQ / (ms * 1e-3), "hooked_modules": hooked, "steps": steps,
            "note": "transformers.GPT2LMHeadModel, vocabulary 50257 unpadded (its logit GEMMs run on cuBLAS's "
                    "unaligned kernels), loss through the model's own float32 log-softmax"}


def dominant_kernel_roofline(prof, peaks):
    """Roofline of the kernel group with the largest share of library time in the timed region."""
    if not prof or not prof["ops"]:
        return None
    name, rec = max(prof["ops"].items(), key=lambda kv: kv[1]["ms"])
    calls = max(1, rec["calls"])
    avg_s = rec["ms"] * 1e-3 / calls
    if rec["flops"] > 0 and rec["bound"] == "tensor":
        achieved = rec["flops"] / calls / avg_s / 1e12
        traffic = None
        if "persample" in name:
            # ncu capture of the mlp.c_fc shape with the bias column sums inside the GEMM kernel and the
            # tiles stored by the copy engine: 669.7 MB of DRAM traffic per call -- GEMM pass 315.3 MB
            # read (the inputs, once) and 160.1 MB of tile write-back, streaming pass 188.8 MB of tiles
            # read once and 5.6 MB of results -- for 315 MB of input bytes; scaled by input bytes
            traffic = rec["bytes"] / calls * (669.7 / 315.0)
        return {"kernel": name, "bound": "tensor", "achieved": achieved, "peak": peaks["tensor"],
                "unit": "TFLOP/s", "frac": achieved / peaks["tensor"], "traffic": traffic,
                "launches": calls, "avg_ms": avg_s * 1e3, "peak_source": peaks["source"]}
    achieved = rec["bytes"] / calls / avg_s / 1e9
    return {"kernel": name, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
            "frac": achieved / peaks["hbm"], "traffic": None, "launches": calls, "avg_ms": avg_s * 1e3,
            "peak_source": peaks["source"]}


# ------------------------------------------------------------------------------------------------
# the reference's own PyTorch arithmetic on the same GPU, beside the kernels that replace it
# ------------------------------------------------------------------------------------------------
def reference_gpu_leg(dev, reps: int = 5):
    """Per layer: this library's call against the reference's layer functions run on CUDA tensors of
    the same shapes (cuBLAS GEMMs + ATen element-wise kernels of the torch build on this machine).

    `torch_as_is_ms` is one call of the reference function with the whole validation batch: it
    returns the [n_train] vector (and, for Conv1D / the materialised branch, the wrong one for more
    than one validation sample).  `torch_full_matrix_ms` is what producing this library's output
    costs with the reference's functions: one call per validation sample with
    cat(train, that sample) (inputs concatenated outside the timed region), each row correct.  Both
    include the reference's train-gradient function, as `ours_ms` includes the train gradient.
    The reference's functions come from the staged reference package when it is there, else from
    the oracle's restatement of the same torch expressions (`impl` says which)."""
    from ghostsuite_b200 import ops, _lib
    from ghostsuite_b200.ghostEngines import supported_layers_grad_samplers_dotprod as ours
    from transformers.pytorch_utils import Conv1D
    ref_pkg = _reference_package()
    if ref_pkg is not None:
        import importlib
        ref = importlib.import_module("ghostEngines.supported_layers_grad_samplers_dotprod")
        ref_gp = importlib.import_module("ghostEngines.gradProjection.autograd_gradproj")
        impl = "reference package (unmodified layer functions on CUDA tensors)"
    else:
        ref = ref_gp = None
        impl = "oracle restatement of the reference's torch expressions on CUDA tensors"
    from oracle import ghost_oracle as O
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)

    def time_ms(fn, n=reps):
        fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(n):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / n

    def fresh(layer):
        for attr in ("use_ghost_computation", "activations", "backprops"):
            layer.__dict__.pop(attr, None)
        for prm in layer.parameters():
            for attr in ("grad_dot_prod", "grad_dot_prod_matrix", "train_grad"):
                if hasattr(prm, attr):
                    delattr(prm, attr)

    def dense_case(name, kind, n_t, n_v, T, d, p):
        N = n_t + n_v
        A = (torch.randn(N, T, d, generator=g, device=dev) * d ** -0.5).bfloat16()
        G = torch.empty(N, T, p, dtype=torch.bfloat16, device=dev)
        for b in range(N):
            G[b] = torch.randn(T, p, generator=g, device=dev) * p ** -0.5
        if kind == "conv1d":
            layer = Conv1D(p, d).to(dev).bfloat16()
            o_dot, o_grad = ours._compute_Conv1D_dot_product, ours._compute_Conv1D_train_grad
            r_dot = ref._compute_Conv1D_dot_product if ref else None
            r_grad = ref._compute_Conv1D_train_grad if ref else None
        else:
            layer = torch.nn.Linear(d, p, bias=False).to(dev).bfloat16()
            o_dot, o_grad = ours._compute_linear_dot_product, ours._compute_linear_train_grad
            r_dot = ref._compute_linear_dot_product if ref else None
            r_grad = ref._compute_linear_train_grad if ref else None
        for prm in layer.parameters():
            prm.initially_requires_grad = True

        def run_ours_fn():
            fresh(layer)
            layer._ghost_backprop_scale = float(N)
            o_dot(layer, A, G, n_v)
            o_grad(layer, A, G, n_v)

        def run_ref(a, b, nv):
            fresh(layer)
            if ref is not None:
                r_dot(layer, a, b, nv)
                r_grad(layer, a, b, nv)           # the reference passes B * N here; the product is not timed
            elif kind == "conv1d":
                O.conv1d_dot_reference(a, b, nv)
                O.conv1d_train_grad(a, b, nv)
            else:
                O.linear_dot_reference(a, b, nv)
                O.linear_train_grad(a, b, nv)

        rec = {"layer": name, "n_train": n_t, "n_val": n_v, "T": T, "d_in": d, "d_out": p}
        rec["ours_ms"] = time_ms(run_ours_fn)
        rec["ours_path"] = "gram" if layer.use_ghost_computation else "persample"
        rec["torch_as_is_ms"] = time_ms(lambda: run_ref(A, G, n_v))
        rec["torch_path"] = "ghost" if getattr(layer, "use_ghost_computation", 2 * T * T <= d * p) else "materialised"
        rows_ms = 0.0
        n_rows = min(n_v, 4)                      # every row costs the same: time a few, scale to n_val
        for v in range(n_rows):
            a = torch.cat((A[:n_t], A[n_t + v:n_t + v + 1]))
            b = torch.cat((G[:n_t], G[n_t + v:n_t + v + 1]))
            rows_ms += time_ms(lambda: run_ref(a, b, 1), n=2)
            del a, b
        rec["torch_full_matrix_ms"] = rows_ms / n_rows * n_v
        rec["torch_full_matrix_note"] = f"{n_rows} of {n_v} validation rows timed, scaled"
        rec["speedup_vs_torch_as_is"] = rec["torch_as_is_ms"] / rec["ours_ms"]
        rec["speedup_vs_torch_full_matrix"] = rec["torch_full_matrix_ms"] / rec["ours_ms"]
        fresh(layer)
        del A, G, layer
        torch.cuda.empty_cache()
        return rec

    def gradproj_case(name, B, T, n_i, n_o, k):
        A = (torch.randn(B, T, n_i, generator=g, device=dev) * n_i ** -0.5).bfloat16()
        G = (torch.randn(B, T, n_o, generator=g, device=dev) * n_o ** -0.5).bfloat16()
        P_i = torch.randn(k, n_i, generator=g, device=dev) / k ** 0.5
        P_o = torch.randn(k, n_o, generator=g, device=dev) / k ** 0.5
        Pi, Po = ops.prepare_projection(P_i, False), ops.prepare_projection(P_o, False)
        out = torch.empty(B, k * k, device=dev)
        rec = {"layer": name, "batch": B, "T": T, "n_i": n_i, "n_o": n_o, "k": k}
        rec["ours_ms"] = time_ms(lambda: ops.gradproj_dense(G, A, Po, Pi, k, k, float(B), out))
        # the reference multiplies float32 P with the activations and raises on bf16 ones: its input
        # is the float32 copy (made outside the timed region)
        A32, G32 = A.float(), G.float()
        lin = torch.nn.Linear(n_i, n_o, bias=False, device="meta")
        if ref_gp is not None:
            hooks = ref_gp.GradProjHooks(P_i, P_o, name, "Linear")
            fn = lambda: hooks._compute_dense_proj(lin, A32, G32)
        else:
            fn = lambda: O.gradproj_dense(A32, G32, P_i, P_o)
        rec["torch_ms"] = time_ms(fn)
        rec["torch_note"] = "float32 upcast of the bf16 operands (untimed); the reference raises on bf16 operands"
        rec["speedup_vs_torch"] = rec["torch_ms"] / rec["ours_ms"]
        del A, G, A32, G32
        torch.cuda.empty_cache()
        return rec

    cases = [
        dense_case("GPT-2 mlp.c_fc (Conv1D)", "conv1d", N_TRAIN, N_VAL, SEQ, 768, 3072),
        dense_case("GPT-2 lm_head (Linear)", "linear", N_TRAIN, N_VAL, SEQ, 768, 50304),
        dense_case("single layer 4096 -> 11008, T = 128", "linear", 256, 32, 128, 4096, 11008),
        gradproj_case("Llama-3-8B q_proj, GradProj k = 64", 8, 4096, 4096, 4096, 64),
    ]
    _lib.poll_kernel_error()
    return {"impl": impl, "timing": f"CUDA events, {reps} calls each, L2 flushed between calls", "cases": cases}


# ------------------------------------------------------------------------------------------------
# GradProj inside the driver's line: kernel sweep on the Llama-3-8B Linear shapes + a Pythia-410M-shaped step
# ------------------------------------------------------------------------------------------------
LLAMA_LINEARS = (("q_proj", 4096, 4096), ("k_proj", 4096, 1024), ("v_proj", 4096, 1024), ("o_proj", 4096, 4096),
                 ("gate_proj", 4096, 14336), ("up_proj", 4096, 14336), ("down_proj", 14336, 4096))


def gradproj_kernel_sweep(dev, reps: int = 5):
    """gradproj_kernel on the seven Linear shapes of a Llama-3-8B block at 8 x 4096 tokens, k_i = k_o = 64:
    algorithmic bytes (operands once, P, output), CUDA-event time, GB/s against the measured copy
    bandwidth, and the tensor-pipe fraction its 2*B*T*(n_i*k + n_o*k + k*k) flops amount to (the
    kernel's intensity is about k flop/byte, far below the ridge, so HBM is the bound)."""
    from ghostsuite_b200 import ops, _lib
    peaks = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)
    B, T, k = 8, 4096, 64
    rows = []
    for name, n_i, n_o in LLAMA_LINEARS:
        A = (torch.randn(B, T, n_i, generator=g, device=dev) * n_i ** -0.5).bfloat16()
        G = (torch.randn(B, T, n_o, generator=g, device=dev) * n_o ** -0.5).bfloat16()
        Pi = ops.prepare_projection(torch.randn(k, n_i, generator=g, device=dev) / k ** 0.5, False)
        Po = ops.prepare_projection(torch.randn(k, n_o, generator=g, device=dev) / k ** 0.5, False)
        out = torch.empty(B, k * k, device=dev)
        ops.gradproj_dense(G, A, Po, Pi, k, k, float(B), out)
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.gradproj_dense(G, A, Po, Pi, k, k, float(B), out)
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        us = total / reps * 1e3
        nbytes = 2.0 * B * T * (n_i + n_o) + 2.0 * k * (n_i + n_o) + 4.0 * B * k * k
        flops = 2.0 * B * T * (n_i * k + n_o * k + k * k)
        gbs = nbytes / (us * 1e-6) / 1e9
        rows.append({"layer": name, "n_i": n_i, "n_o": n_o, "bytes": nbytes, "us": us, "gbs": gbs,
                     "frac_of_measured_hbm": gbs / peaks["hbm"],
                     "tensor_tflops": flops / (us * 1e-6) / 1e12,
                     "frac_of_measured_tensor": flops / (us * 1e-6) / 1e12 / peaks["tensor"]})
        del A, G
        torch.cuda.empty_cache()
    _lib.poll_kernel_error()
    tot_b = sum(r["bytes"] for r in rows)
    tot_us = sum(r["us"] for r in rows)
    return {"batch": B, "T": T, "k": k, "rows": rows, "block_gbs": tot_b / (tot_us * 1e-6) / 1e9,
            "block_frac_of_measured_hbm": tot_b / (tot_us * 1e-6) / 1e9 / peaks["hbm"],
            "hbm_peak_gbs": peaks["hbm"], "peak_source": peaks["source"]}


# ------------------------------------------------------------------------------------------------
# kernel-level microbenchmarks (used for the ncu captures and the per-kernel roofline table)
# ------------------------------------------------------------------------------------------------
KERNEL_CASES = {
    # name: (kind, dict of sizes)
    "gram_T128": ("gram", dict(n_t=256, n_v=32, T=128, d=4096, p=11008)),       # single-layer config, T = 128
    "gram_T512": ("gram", dict(n_t=256, n_v=32, T=512, d=4096, p=11008)),
    "gram_small": ("gram", dict(n_t=64, n_v=8, T=256, d=2048, p=4096)),          # sized for an ncu capture
    "gram_pair_T128": ("gram_pair", dict(n_t=256, n_v=32, T=128, d=4096, p=11008)),   # cta_group::2 variant
    "gram_pair_T512": ("gram_pair", dict(n_t=256, n_v=32, T=512, d=4096, p=11008)),
    "gram_pair_small": ("gram_pair", dict(n_t=64, n_v=8, T=256, d=2048, p=4096)),
    "persample_cfc": ("persample", dict(n_t=32, n_v=8, T=1024, d=768, p=3072)),  # GPT-2 mlp.c_fc
    "persample_cfc_colsum": ("persample", dict(n_t=32, n_v=8, T=1024, d=768, p=3072, colsum="Y")),
    "persample_cproj_colsum": ("persample", dict(n_t=32, n_v=8, T=1024, d=3072, p=768, colsum="Y")),
    "persample_T512": ("persample", dict(n_t=256, n_v=32, T=512, d=4096, p=11008)),
    "persample_T2048": ("persample", dict(n_t=64, n_v=32, T=2048, d=4096, p=11008)),
    "wgrad_cfc": ("wgrad", dict(n_t=32, n_v=8, T=1024, d=768, p=3072)),
    "wgrad_big": ("wgrad", dict(n_t=64, n_v=0, T=1024, d=4096, p=11008)),
    "layernorm_768": ("layernorm", dict(N=40, T=1024, F=768)),
    "colsum_3072": ("colsum", dict(N=40, T=1024, p=3072)),
    "embedding_wte": ("embedding", dict(n_t=32, n_v=8, T=1024, d=768, vocab=50257)),
    # half of all tokens share one id (padding-like): every such train token walks a chain of ~4096 validation tokens
    "embedding_wpe": ("embedding", dict(n_t=32, n_v=8, T=1024, d=768, vocab=1024, positions=True)),   # GPT-2 position table
    "embedding_repeated_ids": ("embedding", dict(n_t=32, n_v=8, T=1024, d=768, vocab=50257, repeat_frac=0.5)),
    "gradproj_llama_q": ("gradproj", dict(B=8, T=4096, n_i=4096, n_o=4096, k=64)),
    "gradproj_llama_gate": ("gradproj", dict(B=8, T=4096, n_i=4096, n_o=14336, k=64)),
    "gradproj_pythia_fc": ("gradproj", dict(B=16, T=2048, n_i=1024, n_o=4096, k=32)),
    "gradproj_small": ("gradproj", dict(B=8, T=4096, n_i=1024, n_o=2048, k=64)),   # sized for an ncu capture
    # embedding projection of a Pythia-410M-shaped token embedding at the configuration's 16 x 2048 tokens
    "gradproj_embedding_pythia": ("gradproj_embedding", dict(B=16, T=2048, d=1024, vocab=50304, k_i=32, k_o=32)),
    # similarity of one Llama-3-8B-shaped batch of projections ([8, 917504] fp32) against another
    "similarity_llama_batch": ("similarity", dict(n1=8, n2=8, D=917504)),
    "similarity_pythia_batch": ("similarity", dict(n1=16, n2=16, D=98304)),
    "similarity_64_rows": ("similarity", dict(n1=64, n2=64, D=917504)),
}


def run_kernels(args):
    """Times single kernels on seeded N(0,1)/sqrt(d) inputs that exceed the L2 (or with an L2 flush
    between iterations), CUDA events on the launching stream.  Prints one JSON object."""
    from ghostsuite_b200 import ops, _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = _peaks()
    burst = peaks["tensor"]
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        burst = float(json.load(open(path)).get("bf16_tflops", burst))
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    names = args.only.split(",") if args.only else list(KERNEL_CASES)
    g = torch.Generator(device=dev).manual_seed(0)
    results = {}
    for name in names:
        kind, c = KERNEL_CASES[name]

        def rnd(*shape, scale=1.0, dtype=torch.bfloat16):
            return (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)

        _lib.check(_lib.load().ghost_set_gram_pair_mode(2 if kind == "gram_pair" else 0))
        if kind == "gram_pair":
            kind = "gram"
        if kind in ("gram", "persample", "wgrad"):
            N = c["n_t"] + c["n_v"]
            A = rnd(N, c["T"], c["d"], scale=c["d"] ** -0.5)
            G = rnd(N, c["T"], c["p"], scale=c["p"] ** -0.5)
            if kind == "gram":
                fn = lambda: ops.gram_dot(A, G, c["n_v"])
            elif kind == "persample":
                if c.get("colsum"):      # Conv1D orientation: X = activations, Y = out-grad, its column sums fused
                    fn = lambda: ops.persample_dot(A, G, c["n_v"], want_grad=True, grad_scale=1.0,
                                                   grad_dtype=torch.bfloat16, colsum_of=c["colsum"])
                else:
                    fn = lambda: ops.persample_dot(G, A, c["n_v"], want_grad=True, grad_scale=1.0, grad_dtype=torch.bfloat16)
            else:
                fn = lambda: ops.wgrad(G[:c["n_t"]], A[:c["n_t"]], 1.0, torch.bfloat16)
        elif kind == "layernorm":
            A = rnd(c["N"], c["T"], c["F"]); G = rnd(c["N"], c["T"], c["F"])
            fn = lambda: ops.layernorm_persample(A, G, 1e-5)
        elif kind == "colsum":
            G = rnd(c["N"], c["T"], c["p"])
            fn = lambda: ops.colsum(G)
        elif kind == "embedding":
            N = c["n_t"] + c["n_v"]
            ids = torch.randint(0, c["vocab"], (N, c["T"]), generator=g, device=dev)
            if c.get("positions"):       # every sample holds the ids 0 .. T - 1 in order
                ids = torch.arange(c["T"], device=dev).repeat(N, 1)
            if c.get("repeat_frac"):
                hot = torch.rand(N, c["T"], generator=g, device=dev) < c["repeat_frac"]
                ids = torch.where(hot, torch.zeros_like(ids), ids)
            G = rnd(N, c["T"], c["d"])
            fn = lambda: (ops.embedding_dot(ids, G, c["n_v"], c["vocab"]),
                          ops.embedding_wgrad(ids, G, c["n_t"], c["vocab"], float(N), float(c["n_t"])))
        elif kind == "gradproj":
            A = rnd(c["B"], c["T"], c["n_i"], scale=c["n_i"] ** -0.5)
            G = rnd(c["B"], c["T"], c["n_o"], scale=c["n_o"] ** -0.5)
            P_i = ops.prepare_projection(torch.randn(c["k"], c["n_i"], generator=g, device=dev) / c["k"] ** 0.5, False)
            P_o = ops.prepare_projection(torch.randn(c["k"], c["n_o"], generator=g, device=dev) / c["k"] ** 0.5, False)
            out = torch.empty(c["B"], c["k"] * c["k"], device=dev)
            fn = lambda: ops.gradproj_dense(G, A, P_o, P_i, c["k"], c["k"], float(c["B"]), out)
        elif kind == "gradproj_embedding":
            ids = torch.randint(0, c["vocab"], (c["B"], c["T"]), generator=g, device=dev)
            G = rnd(c["B"], c["T"], c["d"], scale=c["d"] ** -0.5)
            P_o = ops.prepare_projection(torch.randn(c["k_o"], c["d"], generator=g, device=dev) / c["k_o"] ** 0.5, False)
            P_i_t = ops.prepare_embedding_projection(torch.randn(c["k_i"], c["vocab"], generator=g, device=dev) / c["k_i"] ** 0.5)
            out = torch.empty(c["B"], c["k_o"] * c["k_i"], device=dev)
            fn = lambda: ops.gradproj_embedding(ids, G, P_o, P_i_t, c["k_o"], c["k_i"], 1.0, out)
        elif kind == "similarity":
            P1 = torch.randn(c["n1"], c["D"], generator=g, device=dev)
            P2 = torch.randn(c["n2"], c["D"], generator=g, device=dev)
            fn = lambda: ops.projection_similarity(P1, P2)
        for _ in range(max(1, args.warmup)):
            fn()
        torch.cuda.synchronize()
        ops.start_kernel_timing()
        for _ in range(args.steps):
            flush_buf.zero_()            # evict the L2 between timed iterations
            fn()
        prof = ops.stop_kernel_timing()
        _lib.poll_kernel_error()
        entry = {"sizes": c, "ops": {}}
        for op_name, rec in prof["ops"].items():
            ms = rec["ms"] / rec["calls"]
            e = {"avg_ms": ms, "calls": rec["calls"]}
            if rec["bound"] == "tensor":
                tf = rec["flops"] / rec["calls"] / (ms * 1e-3) / 1e12
                e.update(bound="tensor", achieved_tflops=tf, frac_of_measured_burst=tf / burst)
            else:
                gb = rec["bytes"] / rec["calls"] / (ms * 1e-3) / 1e9
                e.update(bound="hbm", achieved_gbs=gb, frac_of_measured=gb / peaks["hbm"])
            entry["ops"][op_name] = e
        results[name] = entry
        del fn
        torch.cuda.empty_cache()
    _lib.check(_lib.load().ghost_set_gram_pair_mode(1))
    emit({"mode": "kernels", "peaks": {"tensor_burst_tflops": burst, "hbm_gbs": peaks["hbm"],
                                                    "source": peaks["source"]}, "results": results})


def run_crossover(args):
    """Single Linear layer d_in=4096, d_out=11008 (bf16, N(0,1)/sqrt(d) inputs), n_train=256, n_val=32,
    T swept over 128, 512, 2048, 8192: the Gram kernel against the per-sample-gradient path (which
    also yields the train gradient), CUDA events, operands far larger than the L2.  At T = 8192 the
    operands hold 71 GB; the Gram kernel's 1.66e16 flops take seconds there, so long Gram calls are
    timed once, everything else `--steps` times after one warm-up call."""
    from ghostsuite_b200 import ops, _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    d, p, n_t, n_v = 4096, 11008, 256, 32
    N = n_t + n_v
    peaks = _peaks()
    sampler = ClockSampler(0)
    sampler.start()
    rows = []
    for T in (128, 512, 2048, 8192):
        A = torch.empty(N, T, d, dtype=torch.bfloat16, device=dev)
        G = torch.empty(N, T, p, dtype=torch.bfloat16, device=dev)
        for b in range(N):                     # one sample at a time: no float32 copy of a whole operand
            A[b] = torch.randn(T, d, generator=g, device=dev) * d ** -0.5
            G[b] = torch.randn(T, p, generator=g, device=dev) * p ** -0.5
        rec = {"T": T, "n_train": n_t, "n_val": n_v,
               "gram_flops": 2.0 * n_t * T * n_v * T * (d + p),
               "persample_flops": 2.0 * N * T * d * p + 2.0 * n_v * n_t * d * p}
        results = {}
        for name, fn, flops in (("persample", lambda: ops.persample_dot(G, A, n_v, want_grad=True, grad_scale=1.0,
                                                                        grad_dtype=torch.bfloat16), rec["persample_flops"]),
                                ("gram", lambda: ops.gram_dot(A, G, n_v), rec["gram_flops"])):
            long_call = flops / 1.0e15 > 0.5           # estimated seconds at 1 PFLOP/s
            if not long_call:
                results[name] = fn()
                torch.cuda.synchronize()
            reps = 1 if long_call else max(1, args.steps)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                results[name] = fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            rec[name + "_ms"] = ms
            rec[name + "_calls_timed"] = reps
            rec[name + "_tflops"] = flops / (ms * 1e-3) / 1e12
            rec[name + "_train_tokens_per_s"] = n_t * T / (ms * 1e-3)
        M_per, M_gram = results["persample"][0], results["gram"]
        rec["paths_agree_rel_fro"] = float((M_per.double() - M_gram.double()).norm() / M_gram.double().norm())
        rec["faster"] = "gram" if rec["gram_ms"] < rec["persample_ms"] else "persample"
        rec["reference_rule_picks"] = "gram" if 2 * T * T <= d * p else "persample"
        rec["persample_includes_train_gradient"] = True
        rows.append(rec)
        del A, G, results, M_per, M_gram
        torch.cuda.empty_cache()
    clocks = sampler.stop()
    _lib.poll_kernel_error()
    emit({"mode": "crossover", "layer": {"d_in": d, "d_out": p, "dtype": "bf16"}, "rows": rows, "clocks": clocks,
          "tensor_peak_tflops": peaks["tensor"], "peak_source": peaks["source"]})


def run_mlp(args):
    """GradDotProd on the fp32 MLP 512 -> 1024 -> 1024 -> 10 (Linear + ReLU, cross-entropy), 64 train +
    16 validation samples, SGD: the launch-latency-bound configuration.  Reports microseconds per step
    (forward, backward with hooks, prepare_gradients, optimizer step, aggregate with its device-to-host
    read) for the CUDA engine and for the CPU restatement of the reference's path."""
    from ghostsuite_b200 import _lib
    from ghostsuite_b200.ghostEngines import GradDotProdEngine
    from ghostsuite_b200.workloads import make_mlp
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n_t, n_v = 64, 16

    def run(device, steps, warmup):
        torch.manual_seed(0)
        model = make_mlp().to(device)
        opt = torch.optim.SGD(model.parameters(), lr=0.1)
        on_gpu = device.type == "cuda"
        if on_gpu:
            eng = GradDotProdEngine(module=model, val_batch_size=n_v, loss_reduction="mean")
            eng.attach(opt)
        else:
            from oracle.ghost_engine_cpu import OracleDotProdEngine
            eng = OracleDotProdEngine(model, n_v)
            eng.attach()
        g = torch.Generator().manual_seed(0)
        X = torch.randn(n_t + n_v, 512, generator=g).to(device)
        Y = torch.randint(0, 10, (n_t + n_v,), generator=g).to(device)

        def step(i):
            if on_gpu:
                eng.attach_train_batch(X[:n_t], Y[:n_t], i, i)
            torch.nn.functional.cross_entropy(model(X), Y).backward()
            eng.prepare_gradients()
            opt.step()
            if on_gpu:
                eng.aggregate_and_log()
                eng.dot_product_log.clear()
            else:
                eng.aggregate()
            eng.clear_gradients()
            opt.zero_grad(set_to_none=True)

        for i in range(warmup):
            step(i)
        if on_gpu:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(steps):
            step(i)
        if on_gpu:
            torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / steps
        eng.detach()
        return dt * 1e6

    def run_graph(steps, warmup):
        """The same step with forward, backward (hooks included), prepare_gradients and the optimizer
        step captured once in a CUDA graph and replayed: the hooks' kernels, workspaces and result
        tensors keep their addresses, so each replay refreshes ``param.grad_dot_prod_matrix`` in place
        and only the aggregation (one stacked sum and the device-to-host read) runs eagerly."""
        torch.manual_seed(0)
        model = make_mlp().to(dev)
        opt = torch.optim.SGD(model.parameters(), lr=0.1)
        eng = GradDotProdEngine(module=model, val_batch_size=n_v, loss_reduction="mean")
        eng.attach(opt)
        g = torch.Generator().manual_seed(0)
        X = torch.randn(n_t + n_v, 512, generator=g).to(dev)
        Y = torch.randint(0, 10, (n_t + n_v,), generator=g).to(dev)

        def body():
            torch.nn.functional.cross_entropy(model(X), Y).backward()
            eng.prepare_gradients()
            opt.step()

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                 # warm-up on the capture stream (lazy initialisations)
            for _ in range(3):
                body()
                eng.clear_gradients()
                opt.zero_grad(set_to_none=True)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            body()
        mats = [p_.grad_dot_prod_matrix for p_ in model.parameters() if hasattr(p_, "grad_dot_prod_matrix")]

        def step():
            graph.replay()
            total = torch.stack(mats).sum(dim=0)
            return total.sum(dim=0).cpu()             # the step's device-to-host read (and sync)

        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            out = step()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / steps
        assert out.shape == (n_t,) and bool(torch.isfinite(out).all())
        _lib.poll_kernel_error()
        return dt * 1e6

    l0 = _lib.launch_count()
    gpu_us = run(dev, max(args.steps, 50), max(args.warmup, 5))
    launches = (_lib.launch_count() - l0) / (max(args.steps, 50) + max(args.warmup, 5))
    _lib.poll_kernel_error()
    cpu_us = run(torch.device("cpu"), 20, 3)
    graph_us = run_graph(max(args.steps, 50), max(args.warmup, 5))
    emit({"mode": "mlp", "workload": " ".join(run_mlp.__doc__.split()), "us_per_step": gpu_us,
          "us_per_step_cuda_graph": graph_us, "library_launches_per_step": launches,
          "cpu_baseline": {"us_per_step": cpu_us, "cores": torch.get_num_threads(), "kind": "port"}})


def _next_token_loss(logits, ids):
    """Mean next-token cross-entropy from the library's fused loss kernels (targets shifted, last
    position of every sequence ignored) instead of the model's own fp32 log-softmax."""
    from ghostsuite_b200.workloads import _FusedTokenLoss
    B, T, V = logits.shape
    target = torch.cat((ids[:, 1:], ids.new_full((B, 1), -100)), dim=1).reshape(-1)
    return _FusedTokenLoss.apply(logits.reshape(-1, V), target, V)


def _gradproj_world(local_rank: int, world: int):
    """GradProj shards the corpus with no data-path communication; the process group only serves the
    barrier around the timed region and the max-over-ranks of the step time."""
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return torch.device("cuda", local_rank)


def _gradproj_sync_ms(ms: float, world: int, dev) -> float:
    if world <= 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _gradproj_barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def _gradproj_done(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def gradproj_model_core(steps: int, warmup: int, rank: int, world: int, dev):
    """GradProjLoRA on a Pythia-410M-shaped decoder (24 layers, d=1024, 16 heads, MLP 4096, vocab 50304,
    random init, bf16), sequence 2048, batch 16 per GPU, k_i = k_o = 32 on every attention / MLP Linear,
    projections streamed to pinned host memory and written to disk by the engine's writer thread.
    The engine runs with freeze_weights=True (autograd computes activation gradients only); the loss
    comes from the library's fused cross-entropy kernels.  With world > 1 every rank works on its own
    shard of the corpus (no data-path communication).  Returns the record on rank 0."""
    import contextlib
    import io
    import shutil
    from transformers import GPTNeoXConfig, GPTNeoXForCausalLM
    from ghostsuite_b200 import _lib, ops
    from ghostsuite_b200.ghostEngines.gradProjection.gradproj_engine import GradProjLoraEngine
    torch.manual_seed(0)
    cfg = GPTNeoXConfig(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096,
                        vocab_size=50304, max_position_embeddings=2048, use_cache=False)
    model = GPTNeoXForCausalLM(cfg).to(torch.bfloat16).to(dev)
    out_dir = tempfile.mkdtemp(prefix="gradproj_bench_")
    with contextlib.redirect_stdout(io.StringIO()):
        eng = GradProjLoraEngine(model, proj_layers="attention,mlp", proj_rank_total=1024, proj_rank_min=4,
                                 proj_seed=42, proj_dtype="float32", proj_dir=out_dir, proj_save_interval=1,
                                 proj_dims_override=(32, 32), freeze_weights=True)
        eng.attach()
    B, T = 16, 2048
    g = torch.Generator().manual_seed(1 + rank)          # every rank draws its own shard of the corpus
    batches = [torch.randint(0, 50304, (B, T), generator=g).pin_memory() for _ in range(4)]

    def step(i):
        x = batches[i % 4].to(dev, non_blocking=True)
        _next_token_loss(model(input_ids=x).logits, x).backward()
        first = (i * world + rank) * B                   # corpus rows of this rank's i-th batch
        eng.collect_batch(batch_indices=list(range(first, first + B)))
        eng.clear_gradients()

    for i in range(warmup):
        step(i)
    eng.flush()
    _gradproj_barrier(world)
    l0 = _lib.launch_count()
    t0 = time.perf_counter()
    ops.start_kernel_timing()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    prof = ops.stop_kernel_timing()
    eng.flush()
    wall = time.perf_counter() - t0
    ms = _gradproj_sync_ms(e0.elapsed_time(e1) / steps, world, dev)
    _lib.poll_kernel_error()
    n_files = len([f for f in os.listdir(out_dir) if f.startswith("proj_iter_")])
    total_proj_dim, n_layers = eng.total_proj_dim, len(eng.matched_layers)
    launches = int(_lib.launch_count() - l0)
    eng.cleanup()
    shutil.rmtree(out_dir, ignore_errors=True)
    del model, eng
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    rec = prof["ops"].get("gradproj_kernel", {"ms": 0.0, "calls": 1, "bytes": 0.0})
    peaks = _peaks()
    gbs = rec["bytes"] / (rec["ms"] * 1e-3) / 1e9 if rec["ms"] > 0 else 0.0
    return {"workload": " ".join(gradproj_model_core.__doc__.split()),
            "layers": n_layers, "total_proj_dim": total_proj_dim, "n_gpus": world,
            "scaling": "weak (corpus sharded, no communication)",
            "tokens_per_s": world * B * T / (ms * 1e-3), "tokens_per_s_per_gpu": B * T / (ms * 1e-3),
            "ms_per_step": ms, "steps": steps, "warmup": warmup,
            "wall_ms_per_step_including_disk_flush": wall * 1e3 / steps,
            "gradproj_kernel_ms_per_step": rec["ms"] / steps, "gradproj_kernel_gbs": gbs,
            "gradproj_kernel_frac_of_measured_hbm": gbs / peaks["hbm"],
            "d2h_bytes_per_step": B * total_proj_dim * 4, "files_written": n_files,
            "gpu_launches": launches}


def run_gradproj_model(args, rank: int = 0, world: int = 1, local_rank: int = 0):
    dev = _gradproj_world(local_rank, world)
    rec = gradproj_model_core(args.steps, args.warmup, rank, world, dev)
    _gradproj_done(world)
    if rec is not None:
        emit({"mode": "gradproj_model", **rec})


def run_gradproj_llama(args, rank: int = 0, world: int = 1, local_rank: int = 0):
    """GradProjLoRA on a Llama-3-8B-shaped decoder (32 layers, d=4096, 32 heads / 8 KV heads, SwiGLU 14336,
    vocab 128256, random init, bf16), sequence 4096, k_i = k_o = 64 on all 224 attention / MLP Linears.
    Without recomputation the saved activations of the 32-layer model are about 7.8 MB per token, so
    the configuration's batch of 8 x 4096 tokens would need ~250 GB: run it with --checkpoint --batch 8
    (decoder layers recomputed in the backward pass), or at --batch 2 without.  Weights have
    requires_grad=False (only a one-element dummy bias on the embedding keeps the graph alive), so
    autograd computes activation gradients only."""
    import contextlib
    import io
    import shutil
    from transformers import LlamaConfig, LlamaForCausalLM
    from ghostsuite_b200 import _lib
    from ghostsuite_b200.ghostEngines.gradProjection.gradproj_engine import GradProjLoraEngine
    dev = _gradproj_world(local_rank, world)
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=4096, num_hidden_layers=args.layers, num_attention_heads=32,
                      num_key_value_heads=8, intermediate_size=14336, vocab_size=128256,
                      max_position_embeddings=4096, use_cache=False, attn_implementation="sdpa")
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    if args.checkpoint:
        # recompute each decoder layer in the backward pass: only the layer-boundary activations stay
        # resident, which is what lets the configuration's batch of 8 x 4096 tokens fit
        model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": True})
    out_dir = tempfile.mkdtemp(prefix="gradproj_llama_")
    with contextlib.redirect_stdout(io.StringIO()):
        eng = GradProjLoraEngine(model, proj_layers="self_attn,mlp", proj_rank_total=4096, proj_rank_min=4,
                                 proj_seed=42, proj_dtype="float32", proj_dir=out_dir, proj_save_interval=1,
                                 proj_dims_override=(64, 64), freeze_weights=True)
        eng.attach()
    B, T = args.batch, 4096
    g = torch.Generator().manual_seed(1 + rank)          # every rank draws its own shard of the corpus
    batches = [torch.randint(0, 128256, (B, T), generator=g).pin_memory() for _ in range(2)]

    def step(i):
        x = batches[i % 2].to(dev, non_blocking=True)
        _next_token_loss(model(input_ids=x).logits, x).backward()
        first = (i * world + rank) * B
        eng.collect_batch(batch_indices=list(range(first, first + B)))
        eng.clear_gradients()

    for i in range(args.warmup):
        step(i)
    eng.flush()
    _gradproj_barrier(world)
    from ghostsuite_b200 import ops
    l0 = _lib.launch_count()
    ops.start_kernel_timing()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    prof = ops.stop_kernel_timing()
    eng.flush()
    ms = _gradproj_sync_ms(e0.elapsed_time(e1) / args.steps, world, dev)
    _lib.poll_kernel_error()
    rec = prof["ops"].get("gradproj_kernel", {"ms": 0.0, "calls": 1, "bytes": 0.0})
    peaks = _peaks()
    gbs = rec["bytes"] / (rec["ms"] * 1e-3) / 1e9 if rec["ms"] > 0 else 0.0
    total_proj_dim, n_layers = eng.total_proj_dim, len(eng.matched_layers)
    eng.cleanup()
    shutil.rmtree(out_dir, ignore_errors=True)
    _gradproj_done(world)
    if rank != 0:
        return
    emit({"mode": "gradproj_llama", "workload": " ".join(run_gradproj_llama.__doc__.split()),
                      "layers_projected": n_layers, "total_proj_dim": total_proj_dim, "n_gpus": world,
                      "scaling": "weak (corpus sharded, no communication)",
                      "batch": B, "seq_len": T, "activation_checkpointing": bool(args.checkpoint),
                      "tokens_per_s": world * B * T / (ms * 1e-3), "ms_per_step": ms,
                      "gradproj_kernel_ms_per_step": rec["ms"] / args.steps,
                      "gradproj_kernel_gbs": gbs, "gradproj_kernel_frac_of_measured_hbm": gbs / peaks["hbm"],
                      "d2h_bytes_per_step": B * total_proj_dim * 4,
                      "max_memory_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
                      "gpu_launches": int(_lib.launch_count() - l0)})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="step mode: skip the GradProj and reference-on-GPU legs that follow the timed region")
    ap.add_argument("--batch", type=int, default=2, help="gradproj_llama mode: sequences per step")
    ap.add_argument("--layers", type=int, default=32, help="gradproj_llama mode: decoder layers")
    ap.add_argument("--checkpoint", action="store_true",
                    help="gradproj_llama mode: recompute decoder layers in the backward pass (needed for --batch 8)")
    ap.add_argument("--mode", default="step",
                    choices=["step", "kernels", "crossover", "gradproj_model", "gradproj_llama", "mlp"],
                    help="step: the driver's benchmark line; kernels: per-kernel microbenchmarks; crossover: "
                         "Gram vs per-sample path over T on one Linear layer; gradproj_model: GradProj on a "
                         "Pythia-410M-shaped model")
    ap.add_argument("--only", default="", help="kernels mode: comma-separated case names")
    ap.add_argument("--only-variants", default="",
                    help="multi-GPU step: comma-separated variants to time (val_replicated is always timed)")
    ap.add_argument("--exchange-overlap", type=int, default=-1,
                    help="override the engines' EXCHANGE_OVERLAP switch (0 / 1) for an A/B run")
    ap.add_argument("--exchange-own-group", type=int, default=1,
                    help="1 (default): the validation-gradient exchange uses an NCCL communicator of its own, so "
                         "that its all-gathers do not queue behind the gradient all-reduces; 0: one communicator")
    ap.add_argument("--exchange-depth", type=int, default=-1,
                    help="override ops.EXCHANGE_DEPTH (layers whose streaming pass may wait for its all-gather)")
    ap.add_argument("--fuse-bias-colsums", type=int, default=-1,
                    help="override the engines' FUSE_BIAS_COLSUMS switch (0 / 1) for an A/B run")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    guard_stdout()
    if args.exchange_depth >= 0:
        from ghostsuite_b200 import ops as _ops
        _ops.EXCHANGE_DEPTH = args.exchange_depth
    if args.exchange_overlap >= 0:
        from ghostsuite_b200.ghostEngines import supported_layers_grad_samplers_dotprod as _L3
        _L3.EXCHANGE_OVERLAP = bool(args.exchange_overlap)
    if args.fuse_bias_colsums >= 0:
        from ghostsuite_b200.ghostEngines import supported_layers_grad_samplers_dotprod as _L
        _L.FUSE_BIAS_COLSUMS = bool(args.fuse_bias_colsums)
    if args.mode == "kernels":
        run_kernels(args)
        return
    if args.mode == "crossover":
        run_crossover(args)
        return
    if args.mode == "mlp":
        run_mlp(args)
        return
    if args.mode == "gradproj_model":
        run_gradproj_model(args, rank, world, local_rank)
        return
    if args.mode == "gradproj_llama":
        run_gradproj_llama(args, rank, world, local_rank)
        return
    if args.impl == "reference":
        line = run_reference_arm(args, rank)
        if line is not None:
            emit(line)
        return

    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        line = run_ours(args, rank, world, local_rank)
        dev = torch.device("cuda", local_rank)
        from ghostsuite_b200 import ops as _ops
        _ops._arenas.clear()
        torch.cuda.empty_cache()
        if not args.no_extras:
            # GradProj beside the GradDotProd line: the kernel sweep on rank 0, the model step on every
            # rank (corpus sharded)
            gp_step = gradproj_model_core(max(3, args.steps // 4), 2, rank, world, dev)
            if line is not None:
                line["gradproj"] = {"llama3_8b_linear_shapes": gradproj_kernel_sweep(dev),
                                    "pythia_410m_shaped_step": gp_step}
                line["reference_gpu"] = reference_gpu_leg(dev)
                if world == 1:
                    line["hf_gpt2_lm_head_model"] = hf_gpt2_leg(dev)
        if line is not None and world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()                       # rank 0's extra legs end before any rank tears down
        if line is not None:
            emit(line)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
