#!/usr/bin/env python
"""Benchmark of the ghost hot path on the GPT-2-small GradDotProd configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the hot path over one synthetic batch: forward and backward of a GPT-2-small
architecture (12 layers, d=768, 12 heads, vocab 50257, random init, bf16) on cat(32 train, 8 val)
sequences of 1024 uniform-random token ids, with every hooked layer's dot-product matrix [8 x 32]
and train gradient produced by the CUDA kernels inside the backward hooks, then
prepare_gradients, the optimizer step, and aggregate_and_log.  Metric: train tokens per second
(n_train * T * n_gpus / step time), the definition used for the CPU baseline as well.

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank works on its own 32
train sequences plus the replicated validation batch (weak scaling); after backward the
per-parameter dot-product blocks are all-gathered and the train gradients all-reduced over NCCL.

`--impl reference` times the CPU restatement of the reference's own PyTorch path (the reference is
pure Python and cannot be shipped to the GPU machine) on the host cores, on a bounded sample.
Prints ONE JSON line on rank 0.
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
           "T=1024, 32 train + 8 val sequences per GPU, full 8x32 dot-product matrix per parameter"
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
# CPU legs (oracle port of the reference's PyTorch path)
# ------------------------------------------------------------------------------------------------
def cpu_step_factory(n_train: int, n_val: int, seed: int = 0):
    from ghostsuite_b200.workloads import GPT2Like, GPT2Config
    from oracle.ghost_engine_cpu import OracleDotProdEngine
    torch.manual_seed(seed)
    torch.set_num_threads(os.cpu_count() or 1)
    model = GPT2Like(GPT2Config()).to(torch.bfloat16)
    engine = OracleDotProdEngine(model, n_val, use_dummy_bias=True)
    engine.attach()
    opt = torch.optim.AdamW([p for n, p in model.named_parameters() if "dummy_bias" not in n], lr=1e-4)
    g = torch.Generator().manual_seed(seed + 1)
    ids = torch.randint(0, 50257, (n_train + n_val, SEQ), generator=g)

    def step():
        loss, _ = model(ids, labels=ids)
        loss.backward()
        engine.prepare_gradients()
        opt.step()
        total = engine.aggregate()
        engine.clear_gradients()
        opt.zero_grad(set_to_none=True)
        return float(total.sum())

    return step


def run_reference_arm(args, rank: int):
    """The reference's own CPU path, restated (oracle/), on the host cores; rank 0 only."""
    if rank != 0:
        return None
    n_train, n_val = 1, 1
    step = cpu_step_factory(n_train, n_val)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    val = n_train * SEQ / dt
    sample = (f"{n_train} train + {n_val} val sequences x {SEQ} tokens per step (full 12-layer model, "
              "reference's bf16 arithmetic and path rule, AdamW step included)")
    cores = torch.get_num_threads()
    return {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "cpu_sample": sample},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def cpu_baseline_leg():
    n_train, n_val = 2, 1
    step = cpu_step_factory(n_train, n_val)
    step()
    t0 = time.perf_counter()
    reps = 2
    for _ in range(reps):
        step()
    dt = (time.perf_counter() - t0) / reps
    return {"value": n_train * SEQ / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_train} train + {n_val} val sequences x {SEQ} tokens, full 12-layer model, "
                      f"{reps} timed steps after 1 warm-up ({dt:.1f} s/step)"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def run_ours(args, rank: int, world: int, local_rank: int):
    import torch.distributed as dist
    from ghostsuite_b200 import ops, _lib, dist as gdist
    from ghostsuite_b200.ghostEngines import GradDotProdEngine
    from ghostsuite_b200.workloads import GPT2Like, GPT2Config

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a B200: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _lib.check(_lib.load().ghost_device_check())

    torch.manual_seed(0)
    model = GPT2Like(GPT2Config()).to(torch.bfloat16).to(dev)
    params = [p for p in model.parameters()]
    opt = torch.optim.AdamW(params, lr=1e-4, fused=True)
    engine = GradDotProdEngine(module=model, val_batch_size=N_VAL, loss_reduction="mean", use_dummy_bias=True)
    engine.attach(opt)
    group = dist.group.WORLD if world > 1 else None
    if world > 1:
        gdist.overlap_train_grad_sync(engine, group)      # buckets of finished gradients go out during backward

    g = torch.Generator().manual_seed(1)
    val_ids = torch.randint(0, 50257, (N_VAL, SEQ), generator=g)              # replicated
    g.manual_seed(100 + rank)
    n_batches = 4
    host_train = [torch.randint(0, 50257, (N_TRAIN, SEQ), generator=g).pin_memory() for _ in range(n_batches)]
    host_val = val_ids.pin_memory()
    dev_val = val_ids.to(dev)
    dev_train = [t.to(dev) for t in host_train]
    h2d_bytes = host_train[0].numel() * 8
    d2h_bytes = N_TRAIN * 4 + N_VAL * N_TRAIN * 4

    def step(i: int, from_host: bool):
        if from_host:
            x_train = host_train[i % n_batches].to(dev, non_blocking=True)
        else:
            x_train = dev_train[i % n_batches]
        engine.attach_train_batch(x_train, x_train, i, i)
        x = torch.cat((x_train, dev_val), dim=0)
        loss, _ = model(x, labels=x)
        loss.backward()
        if world > 1:
            gdist.sync_engine(engine, group)
        engine.prepare_gradients()
        opt.step()
        engine.clear_gradients()            # host-side bookkeeping first, while the GPU is still busy
        opt.zero_grad(set_to_none=True)
        engine.aggregate_and_log()          # device -> host read of the step's result (the step's sync)
        engine.dot_product_log.clear()

    def timed(from_host: bool, profile: bool):
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

    for i in range(args.warmup):
        step(i, False)
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_dev, launches, _ = timed(False, False)
    # the same K steps once more with a CUDA event pair around every library call (the roofline's
    # kernel durations); kept out of `value` because the event records cost about 2 % of the step
    _, _, prof = timed(False, True)
    ms_e2e, _, _ = timed(True, False)
    clocks = sampler.stop() if rank == 0 else None
    _lib.poll_kernel_error()

    if rank != 0:
        return None
    tok = N_TRAIN * SEQ * world
    value = tok * args.steps / (ms_dev * 1e-3)
    e2e = tok * args.steps / (ms_e2e * 1e-3)
    peaks = _peaks()
    roof = dominant_kernel_roofline(prof, peaks)
    out = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": f"train batch sharded over {world} GPU(s), val replicated",
                   "l2": "working set per step (activations + out-grads, > 10 GB) exceeds the 126 MB L2",
                   "optimizer": "AdamW (fused)", "path_rule": "cost",
                   "vocab_table_rows": "50257 ids; embedding / LM-head table padded to 50304 rows (padded logits masked out of the loss)"},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roof,
        "roofline_pass": "kernel durations from a second pass over the same steps with CUDA events around every "
                         "library call; `value` is the pass without them",
        "kernel_time_share": prof["share"] if prof else None,
    }
    if world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline_leg()
    return out


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
            # ncu capture of the mlp.c_fc shape: 669 MB of DRAM traffic per call (315 MB inputs read
            # once, 159 MB of tile write-back, 189 MB of tiles read once, 6 MB of results) for
            # 315 MB of input bytes; scaled by input bytes
            traffic = rec["bytes"] / calls * (669.0 / 315.0)
        return {"kernel": name, "bound": "tensor", "achieved": achieved, "peak": peaks["tensor"],
                "unit": "TFLOP/s", "frac": achieved / peaks["tensor"], "traffic": traffic,
                "launches": calls, "avg_ms": avg_s * 1e3, "peak_source": peaks["source"]}
    achieved = rec["bytes"] / calls / avg_s / 1e9
    return {"kernel": name, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
            "frac": achieved / peaks["hbm"], "traffic": None, "launches": calls, "avg_ms": avg_s * 1e3,
            "peak_source": peaks["source"]}


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
    "persample_T512": ("persample", dict(n_t=256, n_v=32, T=512, d=4096, p=11008)),
    "persample_T2048": ("persample", dict(n_t=64, n_v=32, T=2048, d=4096, p=11008)),
    "wgrad_cfc": ("wgrad", dict(n_t=32, n_v=8, T=1024, d=768, p=3072)),
    "wgrad_big": ("wgrad", dict(n_t=64, n_v=0, T=1024, d=4096, p=11008)),
    "layernorm_768": ("layernorm", dict(N=40, T=1024, F=768)),
    "colsum_3072": ("colsum", dict(N=40, T=1024, p=3072)),
    "embedding_wte": ("embedding", dict(n_t=32, n_v=8, T=1024, d=768, vocab=50257)),
    "gradproj_llama_q": ("gradproj", dict(B=8, T=4096, n_i=4096, n_o=4096, k=64)),
    "gradproj_llama_gate": ("gradproj", dict(B=8, T=4096, n_i=4096, n_o=14336, k=64)),
    "gradproj_pythia_fc": ("gradproj", dict(B=16, T=2048, n_i=1024, n_o=4096, k=32)),
    "gradproj_small": ("gradproj", dict(B=8, T=4096, n_i=1024, n_o=2048, k=64)),   # sized for an ncu capture
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
    """Single Linear layer d_in=4096, d_out=11008 (bf16, N(0,1)/sqrt(d) inputs): Gram path against
    per-sample-gradient path over T.  Batch sizes shrink with T so that the Gram path stays within
    seconds; times are reported per (train sample x validation sample) pair and per train token."""
    from ghostsuite_b200 import ops, _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    d, p = 4096, 11008
    rows = []
    for T, n_t, n_v in ((128, 256, 32), (512, 256, 32), (2048, 64, 8), (8192, 16, 2)):
        N = n_t + n_v
        A = (torch.randn(N, T, d, generator=g, device=dev) * d ** -0.5).bfloat16()
        G = (torch.randn(N, T, p, generator=g, device=dev) * p ** -0.5).bfloat16()
        rec = {"T": T, "n_train": n_t, "n_val": n_v}
        for name, fn in (("gram", lambda: ops.gram_dot(A, G, n_v)),
                         ("persample", lambda: ops.persample_dot(G, A, n_v, want_grad=True, grad_scale=1.0,
                                                                 grad_dtype=torch.bfloat16))):
            fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            rec[name + "_ms"] = ms
            rec[name + "_train_tokens_per_s"] = n_t * T / (ms * 1e-3)
        rec["gram_flops"] = 2.0 * n_t * T * n_v * T * (d + p)
        rec["persample_flops"] = 2.0 * N * T * d * p + 2.0 * n_v * n_t * d * p
        rec["faster"] = "gram" if rec["gram_ms"] < rec["persample_ms"] else "persample"
        rec["persample_includes_train_gradient"] = True
        rows.append(rec)
        del A, G
        torch.cuda.empty_cache()
    _lib.poll_kernel_error()
    emit({"mode": "crossover", "layer": {"d_in": d, "d_out": p, "dtype": "bf16"}, "rows": rows})


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


def run_gradproj_model(args, rank: int = 0, world: int = 1, local_rank: int = 0):
    """GradProjLoRA on a Pythia-410M-shaped decoder (24 layers, d=1024, 16 heads, MLP 4096, vocab 50304,
    random init, bf16), sequence 2048, batch 16, k_i = k_o = 32 on every attention / MLP Linear,
    projections streamed to pinned host memory and written to disk by the engine's writer thread.
    Weights have requires_grad=False (autograd computes activation gradients only); the loss comes
    from the library's fused cross-entropy kernels."""
    import contextlib
    import io
    import shutil
    from transformers import GPTNeoXConfig, GPTNeoXForCausalLM
    from ghostsuite_b200 import _lib
    from ghostsuite_b200.ghostEngines.gradProjection.gradproj_engine import GradProjLoraEngine
    dev = _gradproj_world(local_rank, world)
    torch.manual_seed(0)
    cfg = GPTNeoXConfig(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096,
                        vocab_size=50304, max_position_embeddings=2048, use_cache=False)
    model = GPTNeoXForCausalLM(cfg).to(torch.bfloat16).to(dev)
    # projections need activation gradients only: no weight requires grad, a one-element dummy bias on
    # the embedding keeps the graph alive (the reference's loop computes and discards the weight gradients)
    from ghostsuite_b200.ghostEngines.transformers_support import _add_dummy_bias
    for prm in model.parameters():
        prm.requires_grad = False
    _add_dummy_bias(model.get_input_embeddings())
    out_dir = tempfile.mkdtemp(prefix="gradproj_bench_")
    with contextlib.redirect_stdout(io.StringIO()):
        eng = GradProjLoraEngine(model, proj_layers="attention,mlp", proj_rank_total=1024, proj_rank_min=4,
                                 proj_seed=42, proj_dtype="float32", proj_dir=out_dir, proj_save_interval=1,
                                 proj_dims_override=(32, 32))
        eng.attach()
    B, T = 16, 2048
    g = torch.Generator().manual_seed(1 + rank)          # every rank draws its own shard of the corpus
    batches = [torch.randint(0, 50304, (B, T), generator=g).pin_memory() for _ in range(4)]

    def step(i):
        x = batches[i % 4].to(dev, non_blocking=True)
        model.zero_grad(set_to_none=True)
        _next_token_loss(model(input_ids=x).logits, x).backward()
        first = (i * world + rank) * B                   # corpus rows of this rank's i-th batch
        eng.collect_batch(batch_indices=list(range(first, first + B)))
        eng.clear_gradients()

    for i in range(args.warmup):
        step(i)
    eng.flush()
    _gradproj_barrier(world)
    l0 = _lib.launch_count()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    eng.flush()
    wall = time.perf_counter() - t0
    ms = _gradproj_sync_ms(e0.elapsed_time(e1) / args.steps, world, dev)
    _lib.poll_kernel_error()
    n_files = len([f for f in os.listdir(out_dir) if f.startswith("proj_iter_")])
    total_proj_dim, n_layers = eng.total_proj_dim, len(eng.matched_layers)
    eng.cleanup()
    shutil.rmtree(out_dir, ignore_errors=True)
    _gradproj_done(world)
    if rank != 0:
        return
    emit({"mode": "gradproj_model", "workload": " ".join(run_gradproj_model.__doc__.split()),
                      "layers": n_layers, "total_proj_dim": total_proj_dim, "n_gpus": world,
                      "scaling": "weak (corpus sharded, no communication)",
                      "tokens_per_s": world * B * T / (ms * 1e-3), "ms_per_step": ms,
                      "wall_ms_per_step_including_disk_flush": wall * 1e3 / args.steps,
                      "d2h_bytes_per_step": B * total_proj_dim * 4, "files_written": n_files,
                      "gpu_launches": int(_lib.launch_count() - l0)})


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
    from ghostsuite_b200.ghostEngines.transformers_support import _add_dummy_bias
    dev = _gradproj_world(local_rank, world)
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=4096, num_hidden_layers=args.layers, num_attention_heads=32,
                      num_key_value_heads=8, intermediate_size=14336, vocab_size=128256,
                      max_position_embeddings=4096, use_cache=False, attn_implementation="sdpa")
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    for prm in model.parameters():
        prm.requires_grad = False
    _add_dummy_bias(model.get_input_embeddings())
    if args.checkpoint:
        # recompute each decoder layer in the backward pass: only the layer-boundary activations stay
        # resident, which is what lets the configuration's batch of 8 x 4096 tokens fit
        model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": True})
    out_dir = tempfile.mkdtemp(prefix="gradproj_llama_")
    with contextlib.redirect_stdout(io.StringIO()):
        eng = GradProjLoraEngine(model, proj_layers="self_attn,mlp", proj_rank_total=4096, proj_rank_min=4,
                                 proj_seed=42, proj_dtype="float32", proj_dir=out_dir, proj_save_interval=1,
                                 proj_dims_override=(64, 64))
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
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    guard_stdout()
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
        if line is not None:
            emit(line)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
