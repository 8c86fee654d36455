#!/usr/bin/env python
"""Benchmark of the proving hot path on B200: sparse x dense product sumcheck over BN254 Fr.

Workload (one "step" = one whole prove, transcript included): num_var = 26, dense table of 2^26
uniform Fr elements, sparse table of 2^20 int8 values at distinct uniform indices, seed 1.
Metric: Fr-evals/s = (2^26 + 2^20) / seconds per prove.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints one JSON line.  `value` is measured with the inputs resident in HBM; `e2e` goes through
the C ABI with pinned host buffers (host->device copies inside the timed region).  The
reference arm times the CPU restatement of the reference's prover (oracle/) on the host cores,
because the reference is a Rust crate and no Rust toolchain exists on the box.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NUM_VAR = 26
NNZ_LOG = 20
SEED = 1
CPU_SAMPLE_VAR = 22      # bounded sample the CPU arm runs per step: same density, 2^22 domain
CPU_SAMPLE_NNZ_LOG = 16
METRIC = "sumcheck_fr_evals_per_s"
UNIT = "Fr-evals/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--num-var", type=int, default=NUM_VAR, help="smaller domains are for profiling captures only")
    ap.add_argument("--nnz-log", type=int, default=NNZ_LOG)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--device-tail", type=int, default=None, help="override the library's ZK_OPT_DEVICE_TAIL default (0/1)")
    ap.add_argument("--peer-exchange", type=int, default=None, help="override ZK_OPT_PEER_EXCHANGE (0: NCCL all-gather per round)")
    ap.add_argument("--trace", action="store_true", help="print rank 0's per-round host times of one prove to stderr")
    ap.add_argument("--no-msm", action="store_true", help="skip the KZH2 commit (MSM points/s) leg")
    ap.add_argument("--msm-only", action="store_true", help="run the KZH2 commit leg alone and print its JSON (profiling captures)")
    ap.add_argument("--msm-log", type=int, default=24, help="log2 of the committed table (smaller sizes are for profiling captures only)")
    return ap.parse_args()


def workload_config(num_var: int, nnz_log: int, gpus: int, exchange: str = "nccl"):
    lg = gpus.bit_length() - 1
    return {"workload": f"sparse-dense product sumcheck, BN254 Fr, num_var={num_var}, dense 2^{num_var} uniform, "
                        f"sparse 2^{nnz_log} int8 non-zeros, seed {SEED}" +
                        (f" per GPU (one instance of num_var={num_var + lg} sharded on its top {lg} variables)" if lg else ""),
            "parallelism": (f"hypercube sharded over {gpus} GPUs, partial round messages exchanged per round "
                            + ("by peer stores over NVLink inside one kernel" if exchange == "peer memory"
                               else "by an NCCL all-gather")
                            if gpus > 1 else "1 GPU"),
            "l2": "inputs (2 GiB dense table) larger than the 126 MB L2"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------- CPU arm (oracle)
def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sample_inputs(ctx, num_var: int, nnz_log: int):
    """Inputs of the bounded CPU sample, generated by the same device-side generator."""
    import numpy as np
    import torch
    from zkes_b200._lib import check, lib

    dense = torch.empty((1 << num_var, 4), dtype=torch.int64, device="cuda")
    vals = torch.empty((1 << nnz_log, 4), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    check(lib.zk_gen_uniform_fr(ctx.handle, SEED, 0, 0, 1 << num_var, dense.data_ptr()), "gen")
    check(lib.zk_gen_small_fr(ctx.handle, SEED, 2, 0, 1 << nnz_log, 8, vals.data_ptr()), "gen")
    g = torch.Generator(device="cuda")
    g.manual_seed(SEED)
    idx = torch.randperm(1 << num_var, generator=g, device="cuda")[: 1 << nnz_log].sort().values
    return (idx.cpu().numpy().astype(np.uint64), vals.cpu().numpy().view(np.uint64), dense.cpu().numpy().view(np.uint64))


def run_cpu_oracle(inputs, num_var: int, steps: int, warmup: int):
    """Times the CPU restatement of the reference prover on all host threads."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import coracle

    threads = host_threads()
    coracle.set_threads(threads)
    idx, vals, dense = inputs
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        coracle.sparse_dense_prove_mont(b"sumcheck_bench", num_var, idx, vals, dense)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return sum(times) / len(times), threads


def synth_inputs_numpy(num_var: int, nnz_log: int):
    """CPU-only input synthesis for the reference arm when no GPU generator is wanted."""
    import numpy as np

    rng = np.random.default_rng(SEED)
    dense = rng.integers(0, 1 << 61, size=(1 << num_var, 4), dtype=np.uint64)  # top limb < 2^61: value < r
    vals = np.zeros((1 << nnz_log, 4), dtype=np.uint64)
    vals[:, 0] = rng.integers(1, 128, size=1 << nnz_log, dtype=np.uint64)
    idx = np.sort(rng.choice(1 << num_var, size=1 << nnz_log, replace=False)).astype(np.uint64)
    return idx, vals, dense


def reference_arm(args):
    """`--impl reference`: the reference's CPU algorithm (restated in oracle/, kind "port") on a
    bounded sample of the workload per step.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    evals = (1 << CPU_SAMPLE_VAR) + (1 << CPU_SAMPLE_NNZ_LOG)
    inputs = synth_inputs_numpy(CPU_SAMPLE_VAR, CPU_SAMPLE_NNZ_LOG)
    sec, threads = run_cpu_oracle(inputs, CPU_SAMPLE_VAR, args.steps, min(args.warmup, 1))
    value = evals / sec
    sample = (f"per step: one prove on num_var={CPU_SAMPLE_VAR}, nnz=2^{CPU_SAMPLE_NNZ_LOG} (same 1/64 density); "
              "throughput in Fr-evals/s is size-normalised")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u256 (BN254 Fr, Montgomery)", "data": "synthetic",
        "config": workload_config(NUM_VAR, NNZ_LOG, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------- GPU arm
def gpu_arm(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from zkes_b200 import Context
    from zkes_b200._lib import ZK_MEM_DEVICE, ZK_MEM_HOST, check, lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = Context(local_rank)
    if args.device_tail is not None:
        from zkes_b200._lib import ZK_OPT_DEVICE_TAIL
        ctx.set_option(ZK_OPT_DEVICE_TAIL, args.device_tail)
    n, k = args.num_var, args.nnz_log
    comm = None
    if world > 1:
        from zkes_b200.dist import Comm, log2_exact
        comm = Comm(ctx, rank, world)
        if args.peer_exchange is not None:
            from zkes_b200._lib import ZK_OPT_PEER_EXCHANGE
            ctx.set_option(ZK_OPT_PEER_EXCHANGE, args.peer_exchange)
        args.exchange = "peer memory" if comm.peer_exchange and args.peer_exchange != 0 else "nccl"
    total_var = n + (world.bit_length() - 1)  # weak scaling: every rank owns a 2^n chunk of a 2^total_var table

    # ---- inputs, resident in HBM (weak scaling: every rank owns a 2^n chunk of one sharded instance)
    dense = torch.empty((1 << n, 4), dtype=torch.int64, device="cuda")
    vals = torch.empty((1 << k, 4), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    check(lib.zk_gen_uniform_fr(ctx.handle, SEED, rank, 0, 1 << n, dense.data_ptr()), "zk_gen_uniform_fr")
    check(lib.zk_gen_small_fr(ctx.handle, SEED, 1000 + rank, 0, 1 << k, 8, vals.data_ptr()), "zk_gen_small_fr")
    g = torch.Generator(device="cuda")
    g.manual_seed(SEED + rank)
    idx = torch.randperm(1 << n, generator=g, device="cuda")[: 1 << k].sort().values.contiguous()
    torch.cuda.synchronize()

    msgs = np.zeros((total_var, 3, 4), dtype=np.uint64)
    chal = np.zeros((total_var, 4), dtype=np.uint64)
    fin_t = np.zeros((2, 4), dtype=np.uint64)
    fin = np.zeros((1, 4), dtype=np.uint64)
    vp = ctypes.c_void_p

    def prove(idx_p, val_p, dense_p, mem):
        tr = lib.zk_transcript_new(b"sumcheck_bench", 14)
        lib.zk_transcript_append_u64(tr, b"num_var", 7, total_var)
        lib.zk_transcript_append_u64(tr, b"num_poly", 8, 2)
        if comm is None:
            rc = lib.zk_sumcheck_sparse_dense_prove(ctx.handle, n, 1 << k, vp(idx_p), vp(val_p), vp(dense_p), mem, None,
                                                    None, tr, vp(msgs.ctypes.data), vp(chal.ctypes.data),
                                                    vp(fin_t.ctypes.data), vp(fin.ctypes.data))
        else:
            rc = lib.zk_sumcheck_sparse_dense_prove_sharded(ctx.handle, comm.handle, total_var, 1 << k, vp(idx_p),
                                                            vp(val_p), vp(dense_p), mem, None, None, tr,
                                                            vp(msgs.ctypes.data), vp(chal.ctypes.data),
                                                            vp(fin_t.ctypes.data), vp(fin.ctypes.data))
        lib.zk_transcript_free(tr)
        check(rc, "zk_sumcheck_sparse_dense_prove")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ctx.sync()

    stream = torch.cuda.ExternalStream(lib.zk_stream(ctx.handle))
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        e1.synchronize()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- device-resident run (the `value`): the library's per-kernel event timing is off here
    def dev_step():
        prove(idx.data_ptr(), vals.data_ptr(), dense.data_ptr(), ZK_MEM_DEVICE)

    for _ in range(args.warmup):
        dev_step()
    if args.trace:
        buf = (ctypes.c_double * 4096)()
        cnt = ctypes.c_uint32()
        lib.zk_round_times(ctx.handle, buf, 4096, ctypes.byref(cnt))  # clears the warm-up's record
        barrier()
        t0 = time.perf_counter()
        dev_step()
        t1 = time.perf_counter()
        lib.zk_round_times(ctx.handle, buf, 4096, ctypes.byref(cnt))
        if rank == 0:
            ts = [buf[i] for i in range(cnt.value)]
            sys.stderr.write("trace: prove %.1f us; host-stepped rounds at (us): %s\n" % (
                (t1 - t0) * 1e6, " ".join("%.0f" % t for t in ts)))
            sys.stderr.write("trace: per-round gaps (us): %s\n" % " ".join("%.0f" % (b - a) for a, b in zip(ts, ts[1:])))
    l0 = ctx.launch_count
    total_ms = timed(dev_step, args.steps, 0)
    launches = ctx.launch_count - l0
    # ---- the same K steps again with CUDA events around every kernel of the path (roofline figures)
    check(lib.zk_profile_enable(ctx.handle, 1), "zk_profile_enable")
    profiled_ms = timed(dev_step, args.steps, 0)
    prof = {"_profiled_ms_per_step": profiled_ms / args.steps}
    for kind, name in enumerate(["round", "fold", "sparse_msg", "sparse_fold"]):
        nl, ms, by = ctypes.c_uint64(), ctypes.c_double(), ctypes.c_double()
        check(lib.zk_profile_get(ctx.handle, kind, ctypes.byref(nl), ctypes.byref(ms), ctypes.byref(by)), "zk_profile_get")
        prof[name] = {"launches": nl.value, "ms": ms.value, "bytes": by.value}
    check(lib.zk_profile_enable(ctx.handle, 0), "zk_profile_enable")
    ms_per_step = total_ms / args.steps
    evals = ((1 << n) + (1 << k)) * world
    value = evals / (ms_per_step * 1e-3)

    # ---- end to end through the C ABI with pinned host buffers
    e2e = None
    if not args.no_e2e:
        h_dense = torch.empty(dense.shape, dtype=dense.dtype, pin_memory=True).copy_(dense)
        h_vals = torch.empty(vals.shape, dtype=vals.dtype, pin_memory=True).copy_(vals)
        h_idx = torch.empty(idx.shape, dtype=idx.dtype, pin_memory=True).copy_(idx)
        torch.cuda.synchronize()

        def host_step():
            prove(h_idx.data_ptr(), h_vals.data_ptr(), h_dense.data_ptr(), ZK_MEM_HOST)

        e2e_steps = max(1, min(args.steps, 5))
        e2e_ms = timed(host_step, e2e_steps, 1) / e2e_steps
        h2d = h_dense.numel() * 8 + h_vals.numel() * 8 + h_idx.numel() * 8
        d2h = (total_var * 3 + 3) * 32 + 4
        e2e = {"value": evals / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms, "steps": e2e_steps}
        del h_dense, h_vals, h_idx
    clocks = sampler.stop() if rank == 0 else None
    args.msm_sharded = None
    if comm is not None and not args.no_msm:
        del dense, vals, idx
        torch.cuda.empty_cache()
        args.msm_sharded = msm_leg_sharded(ctx, comm, rank, world, timed)
    if comm is not None:
        barrier()
        comm.close()
        dist.destroy_process_group()
    return ctx, rank, world, ms_per_step, value, launches, prof, e2e, clocks


def msm_leg(ctx, n=24, steps=5):
    """Second half of the metric: KZH2 commit of 2^24 int8 evaluations on a 2^12 x 2^12 split
    (BASELINE.json config 3), points/s = 2 * 2^24 / t, with the integer-pipe fraction."""
    import numpy as np
    import torch

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from zkes_b200 import DenseMLPoly, curve, kzh
    from zkes_b200._lib import check, lib
    from zkes_b200.field import from_mont_array

    x_log, y_log = n // 2, n - n // 2

    def uniform(stream, count):
        t = torch.empty((count, 4), dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        check(lib.zk_gen_uniform_fr(ctx.handle, 2, stream, 0, count, t.data_ptr()), "zk_gen_uniform_fr")
        return from_mont_array(t.cpu().numpy().view(np.uint64))

    tau_x, tau_y, alpha = uniform(1, 1 << x_log), uniform(2, 1 << y_log), uniform(3, 1)[0]
    # g = 2 * (1, 2) on y^2 = x^3 + 3, in affine form
    g = (1368015179489954701390400359078579693043519447331113978918064868415326638035,
         9918110051302171585080402603319702774565515993150576347155970296011118125764)
    t0 = time.perf_counter()
    srs = kzh.KZHSRS.setup(ctx, 2, n, g, tau_x, tau_y, alpha=alpha)
    setup_s = time.perf_counter() - t0
    f = torch.empty((1 << n, 4), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    check(lib.zk_gen_small_fr(ctx.handle, 2, 7, 0, 1 << n, 8, f.data_ptr()), "zk_gen_small_fr")
    poly = DenseMLPoly(n, device_ptr=f.data_ptr())
    stream = torch.cuda.ExternalStream(lib.zk_stream(ctx.handle))
    kzh.commit(ctx, srs, poly)  # warm-up (allocates scratch)
    kzh.commit(ctx, srs, poly)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        kzh.commit(ctx, srs, poly)
    e1.record(stream)
    e1.synchronize()
    ms = e0.elapsed_time(e1) / steps
    stats = curve.last_stats(ctx)
    ms_imad, ops = ctypes.c_float(), ctypes.c_double()
    check(lib.zk_microbench(ctx.handle, 0, 148 * 8, 256, 4000, ctypes.byref(ms_imad), ctypes.byref(ops)), "zk_microbench")
    imad_peak = ops.value / (ms_imad.value * 1e-3)
    pairs = 2.0 * (1 << n)
    mac32 = pairs * (255.0 / 256.0) * 1360.0  # one mixed addition (10 products of 136) per non-zero digit
    srs.close()
    return {"metric": "kzh2_commit_msm_points_per_s", "value": pairs / (ms * 1e-3), "unit": "points/s", "ms_per_commit": ms,
            "config": f"KZH2 commit, 2^{n} int8 evaluations, 2^{x_log} x 2^{y_log} split, seed 2 (C over 2^{n} points + 2^{x_log} rows of 2^{y_log})",
            "srs_setup_s": setup_s, "window_bits_last_msm": stats["window_bits"],
            "integer_roofline": {"bound": "imad", "achieved_mac32_per_s": mac32 / (ms * 1e-3), "peak_mac32_per_s": imad_peak,
                                 "frac": mac32 / (ms * 1e-3) / imad_peak,
                                 "note": "algorithmic 32x32+64 multiply-adds (1360 per mixed addition) over the measured "
                                         "32-bit multiply-add rate of this GPU (zk_microbench kind 0)"}}


def msm_leg_sharded(ctx, comm, rank, world, timed):
    """The MSM half of the metric on N GPUs, weak scaling: KZH2 commit of 2^(24 + log2 N) int8 evaluations,
    every rank holding the 2^24 evaluations (and SRS points) of its x-rows.  C is a partial MSM per rank plus
    one exchange of the partial points; the d_x rows are local and gathered.  points/s = 2 * 2^n / t."""
    import numpy as np
    import torch

    from zkes_b200 import dist as zd
    from zkes_b200._lib import ZK_MEM_DEVICE, check, lib
    from zkes_b200.field import from_mont_array

    lg = world.bit_length() - 1
    n = 24 + lg
    x_log, y_log = n // 2, n - n // 2

    def uniform(stream, count):
        t = torch.empty((count, 4), dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        check(lib.zk_gen_uniform_fr(ctx.handle, 2, stream, 0, count, t.data_ptr()), "zk_gen_uniform_fr")
        return from_mont_array(t.cpu().numpy().view(np.uint64))

    tau_x, tau_y, alpha = uniform(1, 1 << x_log), uniform(2, 1 << y_log), uniform(3, 1)[0]
    g = (1368015179489954701390400359078579693043519447331113978918064868415326638035,
         9918110051302171585080402603319702774565515993150576347155970296011118125764)
    srs = zd.sharded_kzh_setup(ctx, comm, 2, n, g, tau_x, tau_y, alpha=alpha)
    local = (1 << n) // world
    f = torch.empty((local, 4), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    check(lib.zk_gen_small_fr(ctx.handle, 2, 7, rank * local, local, 8, f.data_ptr()), "zk_gen_small_fr")
    c = np.zeros((1, 8), dtype=np.uint64)
    dx = np.zeros((1 << x_log, 12), dtype=np.uint64)
    vp = ctypes.c_void_p

    def step():
        check(lib.zk_kzh_commit_sharded(ctx.handle, comm.handle, srs.handle, vp(f.data_ptr()), ZK_MEM_DEVICE,
                                        vp(c.ctypes.data), vp(dx.ctypes.data)), "zk_kzh_commit_sharded")

    steps = 5
    ms = timed(step, steps, 2) / steps
    srs.close()
    pairs = 2.0 * (1 << n)
    return {"metric": "kzh2_commit_msm_points_per_s", "value": pairs / (ms * 1e-3), "unit": "points/s", "ms_per_commit": ms,
            "n_gpus": world, "scaling": "weak",
            "config": f"KZH2 commit, 2^{n} int8 evaluations, 2^{x_log} x 2^{y_log} split, seed 2, x-rows sharded over "
                      f"{world} GPUs (2^24 evaluations and SRS points per GPU)"}


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, burst copy)"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback (earlier measurement on this pool)"


# DRAM bytes per launch of the dominant kernel from an ncu capture, relative to its algorithmic
# bytes (profiles/ holds the capture summary); None until a capture exists.
NCU_TRAFFIC_RATIO = {"fold": 0.977, "round": None}  # profiles/k_fold2_dense_table_fold.md


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    # stdout carries the one JSON line and nothing else: whatever libraries write to file descriptor 1 while
    # the bench runs (NCCL prints a version banner there) is sent to stderr, and the line goes to the real one
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(obj) + "\n").encode())
    if args.msm_only:
        from zkes_b200 import Context

        ctx = Context(0)
        emit(msm_leg(ctx, args.msm_log, max(1, args.steps)))
        return
    ctx, rank, world, ms_per_step, value, launches, prof, e2e, clocks = gpu_arm(args)
    if rank != 0:
        return
    peak, peak_src = measured_peak_gbs()
    profiled_ms_per_step = prof.pop("_profiled_ms_per_step")
    top = max(prof, key=lambda k: prof[k]["ms"])
    t = prof[top]
    per_launch_bytes = t["bytes"] / max(t["launches"], 1)
    achieved = t["bytes"] / (t["ms"] * 1e-3) / 1e9 if t["ms"] > 0 else 0.0
    ratio = NCU_TRAFFIC_RATIO.get(top)
    roofline = {"bound": "hbm", "kernel": {"round": "k_round<2,FOLD>", "fold": "k_fold2 (two folds per pass) + k_fold", "sparse_msg": "k_sparse_msg",
                                            "sparse_fold": "k_sparse_count+k_scan_blocks+k_sparse_fold"}[top],
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                "algorithmic_bytes_per_launch": per_launch_bytes, "launches": t["launches"],
                "avg_launch_ms": t["ms"] / max(t["launches"], 1),
                "traffic": per_launch_bytes * ratio if ratio else None,
                "profiled_ms_per_step": profiled_ms_per_step,
                "share_of_step": {k: v["ms"] / (profiled_ms_per_step * args.steps) for k, v in prof.items()}}
    cpu = None
    if not args.no_cpu_baseline:
        inputs = cpu_sample_inputs(ctx, CPU_SAMPLE_VAR, CPU_SAMPLE_NNZ_LOG)
        sec, threads = run_cpu_oracle(inputs, CPU_SAMPLE_VAR, 2, 1)
        cpu = {"value": ((1 << CPU_SAMPLE_VAR) + (1 << CPU_SAMPLE_NNZ_LOG)) / sec, "unit": UNIT, "cores": threads,
               "kind": "port",
               "sample": f"one prove on num_var={CPU_SAMPLE_VAR}, nnz=2^{CPU_SAMPLE_NNZ_LOG} (same density), mean of 2 "
                         f"runs, {sec:.2f} s each; CPU restatement of the reference prover, not arkworks"}
    msm = None
    if world == 1 and not args.no_msm:
        msm = msm_leg(ctx)
    elif world > 1:
        msm = args.msm_sharded
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u256 (BN254 Fr, Montgomery, 8x32-bit limbs)", "data": "synthetic",
        "config": workload_config(args.num_var, args.nnz_log, world, getattr(args, "exchange", "nccl")),
        "gpu_launches": launches, "clocks": clocks, "e2e": e2e, "roofline": roofline, "cpu_baseline": cpu, "msm": msm,
    }
    emit(out)


if __name__ == "__main__":
    main()
