#!/usr/bin/env python
"""Benchmark of the hot path: dense forward + both backward contractions with the fused
bias+GELU epilogue (M=N=K=8192, fp32 storage, TF32 tensor-core products).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size S]

Prints ONE JSON line.  `value` is whole-job TFLOP/s on algorithmic flops (6*M*N*K per step) with
the operands resident in HBM; `e2e` is the same step driven from pinned host buffers (copies in
the timed region); `roofline` is the tensor-core GEMM kernel against the measured tensor peak;
`cpu_baseline` is the float64 CPU oracle on a bounded sample.  With N > 1 the step is the
data-parallel form of the same layer: every rank holds the weights and its own 8192 rows of the batch
(weak scaling), and the weight and bias gradients are summed over the ranks with one NCCL all-reduce
per step, started right behind the dW product and overlapped with the dA product.  The line also
carries the data-parallel transformer training step (configuration 5) as a sub-record.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)



def ncu_dram_bytes_per_launch(size):
    """dram__bytes_read.sum + dram__bytes_write.sum per gemm_tc_kernel launch (mean of forward, dA, dW) at M=N=K=size,
    from the file the ncu capture step writes next to its summaries; None when no capture covers this size."""
    path = os.path.join(ROOT, "profiles", "gemm_tc_kernel_dram_bytes.json")
    try:
        with open(path) as f:
            return json.load(f)["bytes_per_launch"].get(str(size))
    except (OSError, KeyError, ValueError):
        return None

SWEEP = [(512, 512, 512), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192),
         (16384, 4096, 1024)]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed region runs."""

    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.t0, self.t1 = index, None, None, None

    def start(self):
        """Start sampling (the tool needs a moment to come up, so call this well before the timed region)."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        out, _ = self.proc.communicate()
        import datetime
        sm, pw, mx, reasons = [], [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        self.samples = []          # (timestamp, SM MHz) of every sample, for per-repeat medians
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clk, mx_ = float(f[1]), float(f[2])
            except (ValueError, IndexError):
                continue
            mx = mx_
            self.samples.append((ts, clk))
            if self.t0 is not None and not (self.t0 <= ts <= self.t1 + 0.02):
                continue  # outside the timed region
            sm.append(clk)
            try:
                pw.append(float(f[3]))
            except ValueError:
                pass
            for n, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "samples": len(sm),
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons)}

    def window_mhz(self, t0, t1):
        """Median SM clock of the samples taken between two host times (call after stop())."""
        v = [c for ts, c in getattr(self, "samples", []) if t0 <= ts <= t1 + 0.02]
        return statistics.median(v) if v else None


def make_inputs(M, N, K, seed=1):
    """Config 2 operands: entries N(0,1)/sqrt(K), seed 1 (tensor ids 0..3)."""
    from flutter_ml_b200 import synth
    s = 1.0 / np.sqrt(K)
    return (synth.normal(seed, 0, (M, K), s), synth.normal(seed, 1, (K, N), s), synth.normal(seed, 2, (N,), s),
            synth.normal(seed, 3, (M, N), s))


def cpu_step(M, N, K, omp):
    """One fwd+bwd of config 2 on the CPU oracle; returns seconds."""
    from oracle import oracle
    A, B, bias, dC = (np.ascontiguousarray(x, dtype=np.float64) for x in make_inputs(M, N, K))
    t0 = time.perf_counter()
    oracle.gemm_gelu_fwd_bwd(A, B, bias, dC, omp=omp)
    return time.perf_counter() - t0


def run_reference(args, rank):
    """The reference's CPU algorithm (float64 scalar loops; the Dart original cannot run here, so
    this is the oracle port) with all host threads, on a bounded sample of the same workload."""
    if rank != 0:
        return
    from oracle import oracle
    oracle.build()
    S = args.ref_size
    # launchers such as torchrun export OMP_NUM_THREADS=1; this arm is meant to use every host thread
    oracle.Ops(True).set_threads(os.cpu_count() or 1)
    cores = oracle.Ops(True).threads()
    for _ in range(args.warmup):
        cpu_step(S, S, S, True)
    times = [cpu_step(S, S, S, True) for _ in range(args.steps)]
    total = sum(times)
    tf = 6.0 * S ** 3 * args.steps / total / 1e12
    line = {"impl": "reference", "metric": "gemm_fwd_bwd_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": f"dense fwd+bwd (bias+GELU epilogue, dZ+dbias, dA, dW), fp32, M=N=K={args.size}", "seed": 1,
                       "timed_on": f"a bounded sample: M=N=K={S} per step (6*{S}^3 flop, float64 scalar loops); the RATE is "
                                   f"compared, a full {args.size}^3 step would take about {total / args.steps * (args.size / S) ** 3:.0f} s"},
            "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                             "sample": f"M=N=K={S} fwd+bwd per step (6*{S}^3 flop), OpenMP over {cores} threads"},
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def time_sweep(ctx, reps=5):
    """fwd+bwd TFLOP/s for every size of the config-2 sweep (operands are re-used buffers)."""
    from flutter_ml_b200 import ops
    out = []
    # random operands (all-zero data toggles fewer wires, draws less power and clocks higher)
    pool = np.random.default_rng(1).standard_normal(1 << 22).astype(np.float32)
    for (M, N, K) in SWEEP:
        e = ctx.empty
        A, B, bias, dC = e(M, K), e(K, N), e(N), e(M, N)
        for a in (A, B, bias, dC):
            h = np.resize(pool, a.size) * np.float32(1.0 / np.sqrt(K))
            ctx.upload(h.reshape(a.shape), out=a)
        C, Z, dZ, dA, dB, db = e(M, N), e(M, N), e(M, N), e(M, K), e(K, N), e(N)

        def step():
            ops.dense_forward(ctx, A, B, bias, "gelu", M, N, K, C, Z)
            ctx.zero(db)
            ops.dense_backward(ctx, A, B, Z, dC, "gelu", M, N, K, dZ, dA, dB, db)
        for _ in range(3):
            step()
        ctx.sync()
        ctx.timer_start()
        for _ in range(reps):
            step()
        ms = ctx.timer_stop_ms() / reps
        out.append({"M": M, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(6.0 * M * N * K / ms / 1e9, 1)})
        for a in (A, B, bias, dC, C, Z, dZ, dA, dB, db):
            a.free()
    return out


def cublas_tf32_yardstick(n=8192, reps=10):
    """Library TF32 GEMM (torch.matmul -> cuBLAS) on the same GPU with random operands: a yardstick for
    the tensor-core ceiling beside the driver-measured bf16 figure.  Not on the hot path."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
    a = torch.randn(n, n, device="cuda")
    b = torch.randn(n, n, device="cuda")
    for _ in range(3):
        a @ b
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        a @ b
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    del a, b
    torch.cuda.empty_cache()
    return {"library": "torch.matmul (cuBLAS), allow_tf32", "M=N=K": n, "ms": round(ms, 4),
            "tflops": round(2.0 * n ** 3 / ms / 1e9, 1), "note": "one plain product, no epilogue; for scale only"}


def legacy_roundtrip(n=1024, reps=5):
    """The reference's own micro-benchmark (lib/gpu_benching.dart:25-60): one all-ones n x n x n product through the
    legacy FFI symbol, host buffers in and out, wall clock; c[0] must equal n."""
    from flutter_ml_b200 import _lib
    lib = _lib.load()
    a = np.ones((n, n), dtype=np.float32)
    b = np.ones((n, n), dtype=np.float32)
    c = np.zeros((n, n), dtype=np.float32)
    lib.multiplyMatrices(a.ctypes.data, b.ctypes.data, c.ctypes.data, n, n, n)  # first call creates the cached context
    t = []
    for _ in range(reps):
        t0 = time.perf_counter()
        lib.multiplyMatrices(a.ctypes.data, b.ctypes.data, c.ctypes.data, n, n, n)
        t.append(time.perf_counter() - t0)
    return {"call": "multiplyMatrices(h_a, h_b, h_c, 1024, 1024, 1024), pageable host buffers", "ms": round(1e3 * min(t), 3),
            "c0": float(c[0, 0]), "c0_expected": float(n)}


def time_membound(ctx, hbm_gbs, reps=5, rows=262144, params=1 << 28):
    """Achieved HBM GB/s of the memory-bound kernels on footprints of 1 GiB and more (algorithmic bytes:
    every input read once, every output written once)."""
    pool = np.random.default_rng(2).standard_normal(1 << 22).astype(np.float32)

    def filled(*shape, scale=1.0, positive=False):
        a = ctx.empty(*shape)
        h = np.resize(pool, a.size) * np.float32(scale)
        ctx.upload(np.abs(h) if positive else h, out=a.reshape(a.size))
        return a

    def timed(fn):
        for _ in range(2):
            fn()
        ctx.sync()
        ctx.timer_start()
        for _ in range(reps):
            fn()
        return ctx.timer_stop_ms() / reps

    out = []

    def record(name, ms, nbytes, shape):
        gbs = nbytes / ms / 1e6
        out.append({"kernel": name, "shape": shape, "ms": round(ms, 4), "gbs": round(gbs, 1), "frac_hbm": round(gbs / hbm_gbs, 3)})

    R, C = rows, 1024
    n = R * C
    x, dy = filled(R, C, scale=2.0), filled(R, C)
    y, dx = ctx.empty(R, C), ctx.empty(R, C)
    record("softmax_rows_fwd", timed(lambda: ctx.call("fml_softmax_rows_fwd", x, y, R, C, 0.125, 0)), 8 * n, [R, C])
    record("softmax_rows_bwd", timed(lambda: ctx.call("fml_softmax_rows_bwd", y, dy, dx, R, C, 0.125, 0)), 12 * n, [R, C])
    g, b = filled(C), filled(C)
    xhat, rstd, dg, db = ctx.empty(R, C), ctx.empty(R), ctx.zeros(C), ctx.zeros(C)
    record("layernorm_fwd", timed(lambda: ctx.call("fml_layernorm_fwd", x, None, g, b, y, xhat, rstd, R, C, 1e-5)), 12 * n, [R, C])
    record("layernorm_bwd", timed(lambda: ctx.call("fml_layernorm_bwd", dy, g, xhat, rstd, dx, dg, db, R, C, 0)), 12 * n, [R, C])
    record("act_bwd_gelu+dbias", timed(lambda: ctx.call("fml_act_bwd", 4, x, dy, dx, R, C, 0, dg)), 12 * n, [R, C])
    for a in (y, dx, xhat):
        a.free()
    P = min(params, n)
    w, gr = x.reshape(P), dy.reshape(P)
    m, v = ctx.zeros(P), ctx.zeros(P)
    record("sgd_step", timed(lambda: ctx.call("fml_sgd_step", w, gr, P, 1e-3, 1.0)), 12 * P, [P])
    t = [0]

    def adam():
        t[0] += 1
        ctx.call("fml_adam_step", w, gr, m, v, P, 1e-3, 0.9, 0.999, 1e-8, t[0], 1.0)
    record("adam_step", timed(adam), 28 * P, [P])

    def adam_zero():   # the training step's form: per-slice update with the gradient cleared in the same pass
        t[0] += 1
        ctx.call("fml_adam_step_on", -1, w, gr, m, v, P, 1e-3, 0.9, 0.999, 1e-8, t[0], 1.0, 1)   # lane -1: the timed stream
    record("adam_step+zero_grad", timed(adam_zero), 32 * P, [P])
    return out


def time_attention(ctx, n_seq=32, seq_len=512, heads=16, reps=10):
    """Fused attention at the shape of one config-5 layer (d_head 64, causal): forward and backward, microseconds per
    call and TFLOP/s on the full S x S flop count (2 products forward, 5 backward including the recomputation)."""
    import ctypes
    from flutter_ml_b200 import _lib
    dk = 64
    d = heads * dk
    pool = np.random.default_rng(5).standard_normal(1 << 22).astype(np.float32)
    qkv, G = ctx.empty(n_seq * seq_len, 3 * d), ctx.empty(n_seq * seq_len, d)
    ctx.upload(np.resize(pool, qkv.size), out=qkv.reshape(qkv.size))
    ctx.upload(np.resize(pool[::-1], G.size), out=G.reshape(G.size))
    out, lse, dqkv, scratch = ctx.empty(n_seq * seq_len, d), ctx.empty(n_seq * heads * seq_len), ctx.empty(n_seq * seq_len, 3 * d), ctx.empty(n_seq * heads * seq_len)
    de = _lib.AttentionDesc()
    de.n_seq, de.seq_len, de.heads, de.d_head = n_seq, seq_len, heads, dk
    de.q, de.k, de.v, de.ld_qkv = qkv.ptr, qkv.ptr + 4 * d, qkv.ptr + 8 * d, 3 * d
    de.out, de.ld_out, de.lse, de.scale, de.causal = out.ptr, d, lse.ptr, 0.125, 1

    def timed(fn):
        for _ in range(3):
            fn()
        ctx.sync()
        ctx.timer_start()
        for _ in range(reps):
            fn()
        return ctx.timer_stop_ms() / reps

    f_ms = timed(lambda: ctx.check(ctx.lib.fml_attention_fwd(ctx.h, ctypes.byref(de))))
    b_ms = timed(lambda: ctx.check(ctx.lib.fml_attention_bwd(ctx.h, ctypes.byref(de), G.ptr, d, dqkv.ptr, dqkv.ptr + 4 * d,
                                                            dqkv.ptr + 8 * d, 3 * d, 0, scratch.ptr)))
    unit = 2.0 * n_seq * heads * seq_len * seq_len * dk
    return {"shape": {"n_seq": n_seq, "seq_len": seq_len, "heads": heads, "d_head": dk, "causal": True},
            "fwd_us": round(f_ms * 1e3, 1), "bwd_us": round(b_ms * 1e3, 1),
            "fwd_tflops_full_square": round(2 * unit / f_ms / 1e9, 1), "bwd_tflops_full_square": round(5 * unit / b_ms / 1e9, 1)}




NOMINAL_TF32_TFLOPS = 1125.0   # dense TF32 per B200 (half the 2.25 PFLOP/s bf16 figure)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=8192, help="M=N=K of the timed step (rows per GPU when N > 1)")
    ap.add_argument("--ref-size", type=int, default=1024, help="M=N=K of one CPU sample step")
    ap.add_argument("--repeats", type=int, default=0, help="timed regions of --steps steps each; 0 picks 10, fewer for long regions")
    ap.add_argument("--reserve-sms", type=int, default=20, help="SMs the dA product leaves to the exchange that runs beside it (N > 1)")
    ap.add_argument("--nccl-ctas", type=int, default=16, help="upper limit on the CTAs of the gradient exchange (N > 1; 0: NCCL's choice)")
    ap.add_argument("--overlap-rows", type=int, default=0, help="rows of the dA product computed beside the exchange on the reduced SM set (0: all)")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-train", action="store_true")
    ap.add_argument("--no-membound", action="store_true")
    ap.add_argument("--no-configs", action="store_true")
    ap.add_argument("--membound-only", action="store_true", help="run only the memory-bound kernel sweep (profiling)")
    ap.add_argument("--membound-rows", type=int, default=262144)
    ap.add_argument("--attention-only", action="store_true", help="run only the fused attention kernels (profiling)")
    ap.add_argument("--attention-seqs", type=int, default=32)
    ap.add_argument("--configs-only", action="store_true", help="run only configurations 1, 3, 4 (profiling)")
    ap.add_argument("--config", type=int, default=0, choices=[0, 1, 3, 4], help="with --configs-only: just this one")
    ap.add_argument("--train-only", action="store_true", help="run only the data-parallel training step (profiling)")
    ap.add_argument("--train-steps", type=int, default=20)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from flutter_ml_b200 import _lib, dp, ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    peaks = measured_peaks()
    ctx = _lib.Context(device=local_rank, precision=_lib.PREC_TF32)
    if args.train_only:
        import bench_train
        res = bench_train.run(ctx, rank, world, barrier, max_over_ranks, steps=max(1, args.train_steps), warmup=3)
        if rank == 0:
            print(json.dumps({"train": res}), flush=True)
        ctx.close()
        if world > 1:
            dist.destroy_process_group()
        return
    if args.configs_only:
        import bench_configs
        print(json.dumps({"configs": bench_configs.run(ctx, args.config)}), flush=True)
        ctx.close()
        return
    if args.attention_only:
        print(json.dumps({"attention": time_attention(ctx, n_seq=args.attention_seqs, reps=2)}), flush=True)
        ctx.close()
        return
    if args.membound_only:
        res = time_membound(ctx, peaks["hbm_gbs"], reps=2, rows=args.membound_rows)
        print(json.dumps({"membound": res}), flush=True)
        ctx.close()
        return
    M = N = K = args.size
    flops_step = 6.0 * M * N * K
    # N > 1: the exchange of the weight gradient gets its own communicator (a few CTAs) and the SMs the dA product leaves it
    exchange = None
    if world > 1:
        dp.init_data_parallel(ctx, dist, rank, world, device="cuda", max_ctas=args.nccl_ctas)
        exchange = ops.GradientExchange(ctx, world, lane=2, reserve_sms=args.reserve_sms, overlap_rows=args.overlap_rows)
    host = ops.DenseFwdBwdHost(ctx, M, N, K, act="gelu", exchange=exchange)
    seeds = make_inputs(M, N, K)
    if world > 1:   # every rank has its own rows of the batch (A, dC); weights and bias are replicated
        from flutter_ml_b200 import synth
        sc = 1.0 / np.sqrt(K)
        seeds = (synth.normal(1, 10 + rank, (M, K), sc), seeds[1], seeds[2], synth.normal(1, 30 + rank, (M, N), sc))
    for name, arr in zip(("A", "B", "bias", "dC"), seeds):
        host.h_in[name][...] = arr
    del seeds
    host()  # uploads the operands once; they stay resident for the device-timed loop

    # ---- device-resident loop: R timed regions of K steps each (every region between a barrier and a synchronize on
    # both sides); the headline is the MEDIAN region, and every region carries the SM clock sampled inside it
    repeats = args.repeats or max(1, min(10, int(2000.0 / max(args.steps * 5.5, 1.0))))
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        host.compute()
    barrier()
    sampler.mark_begin()
    launches0 = ctx.launches
    regions, n_ev_steps = [], min(args.steps, 10)
    for rep in range(repeats):
        barrier()
        t_host0 = time.time()
        ev_at = {int(i * args.steps / n_ev_steps): i for i in range(n_ev_steps)} if rep == 0 else {}
        ctx.timer_start()
        for step_i in range(args.steps):
            if step_i in ev_at:
                # per-launch events around the three products of 10 steps spread over the first region
                sl, c = ev_at[step_i], ctx
                c.event_record(6 * sl + 0)
                ops.dense_forward(c, host.A, host.B, host.bias, "gelu", M, N, K, host.C, host.Z)
                c.event_record(6 * sl + 1)
                c.zero(host.dbias)
                c.call("fml_act_bwd", _lib.ACT_GELU, host.Z, host.dC, host.dZ, M, N, 0, host.dbias)
                c.event_record(6 * sl + 2)
                c.gemm(host.A, host.dZ, host.dB, K, N, M, transA=True)
                c.event_record(6 * sl + 3)
                if exchange:
                    exchange.start(host.grads, host.grads.size)
                r1 = exchange.overlap_rows if (exchange and 0 < exchange.overlap_rows < M) else M
                c.gemm(host.dZ, host.B, host.dA, r1, K, N, transB=True)
                if r1 < M:
                    exchange.release_sms()
                    c.gemm(host.dZ.view(r1 * N, (M - r1, N)), host.B, host.dA.view(r1 * K, (M - r1, K)), M - r1, K, N, transB=True)
                c.event_record(6 * sl + 4)
                if exchange:
                    exchange.join()
            else:
                host.compute()
        ms = ctx.timer_stop_ms()
        barrier()
        regions.append({"ms_per_step": max_over_ranks(ms) / args.steps, "t0": t_host0, "t1": time.time()})
    sampler.mark_end()
    clocks = sampler.stop()
    launches = (ctx.launches - launches0) // repeats
    for r in regions:
        r["sm_mhz"] = sampler.window_mhz(r.pop("t0"), r.pop("t1"))
        r["ms_per_step"] = round(r["ms_per_step"], 4)
        r["ms_x_ghz"] = round(r["ms_per_step"] * r["sm_mhz"] / 1e3, 4) if r["sm_mhz"] else None
    ms_step = statistics.median(r["ms_per_step"] for r in regions)
    value = world * flops_step / ms_step / 1e9
    gemm_ms = []
    for sl in range(n_ev_steps):
        gemm_ms += [ctx.event_elapsed_ms(6 * sl, 6 * sl + 1), ctx.event_elapsed_ms(6 * sl + 2, 6 * sl + 3),
                    ctx.event_elapsed_ms(6 * sl + 3, 6 * sl + 4)]
    # with an exchange running beside it the dA product is not a kernel-alone figure: the roofline uses fwd and dW then
    alone = [m for i, m in enumerate(gemm_ms) if world == 1 or i % 3 != 2]
    gemm_avg = sum(alone) / len(alone)
    achieved = 2.0 * M * N * K / gemm_avg / 1e9
    long_run = ms_step * args.steps > 1000.0
    tf32_peak = (peaks["bf16_sustained"] if long_run else peaks["bf16_burst"]) / 2.0
    roofline = {"bound": "tensor", "kernel": "gemm_tc_kernel", "achieved": round(achieved, 1), "peak": round(tf32_peak, 1),
                "unit": "TFLOP/s", "frac": round(achieved / tf32_peak, 4), "traffic": ncu_dram_bytes_per_launch(M),
                "algorithmic_bytes": 4 * (M * K + K * N + M * N),
                "peak_source": f"{peaks['source']}: MEASURED_PEAKS bf16 {'sustained' if long_run else 'burst'} / 2 "
                               "(dense TF32 runs at half the bf16 rate; no TF32 figure is measured by the driver)",
                "frac_of_nominal_tf32": round(achieved / NOMINAL_TF32_TFLOPS, 4),
                "per_gemm_ms": {"fwd": round(statistics.mean(gemm_ms[0::3]), 4), "dW": round(statistics.mean(gemm_ms[1::3]), 4),
                                "dA" + (" (exchange beside it)" if world > 1 else ""): round(statistics.mean(gemm_ms[2::3]), 4)}}

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region.
    # Serial form (upload, kernels, download one after the other) and pipelined form (copies on two
    # side streams, two buffer sets); both move the same bytes every step.
    e2e_steps = max(4, min(args.steps, 10))
    host()
    barrier()
    ctx.timer_start()
    for _ in range(2):
        host()
    serial_ms = max_over_ranks(ctx.timer_stop_ms()) / 2
    host.pipelined(2)
    barrier()
    ctx.timer_start()
    host.pipelined(e2e_steps)
    e2e_ms_rank = ctx.timer_stop_ms() / e2e_steps
    barrier()
    e2e_ms = max_over_ranks(e2e_ms_rank)
    e2e = {"value": round(world * flops_step / e2e_ms / 1e9, 2), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms, 3),
           "h2d_bytes_per_step": host.h2d_bytes, "d2h_bytes_per_step": host.d2h_bytes, "steps": e2e_steps,
           "serial_ms_per_step": round(serial_ms, 3),
           "pcie_gbs_each_way": round(host.h2d_bytes / e2e_ms / 1e6, 1)}
    if world > 1:   # every rank's own figure: the host side (one NUMA node, one memory system) is shared by all ranks
        t = torch.zeros(world, dtype=torch.float64, device="cuda")
        t[rank] = e2e_ms_rank
        dist.all_reduce(t)
        e2e["ms_per_step_by_rank"] = [round(float(x), 2) for x in t.tolist()]
        e2e["note"] = ("all GPUs of the box hang off one NUMA node (nvidia-smi topo: CPU affinity 0-31, NUMA 0 for every GPU), so "
                       "there is no closer memory to bind a rank's staging buffers to; the ranks share the host's copy bandwidth")

    par = (f"data parallel x{world}: {M} rows per GPU, weights replicated, fp32 all-reduce of dW+dbias "
           f"({host.grads.size * 4 // 2 ** 20} MiB) per step on a side stream beside the dA product") if world > 1 else "single GPU"
    line = {"metric": "gemm_fwd_bwd_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
            "config": {"workload": f"dense fwd+bwd (bias+GELU epilogue, dZ+dbias, dA, dW), fp32, M=N=K={M}", "seed": 1,
                       "l2": "operands (3 x %d MB) exceed the 126 MB L2; no flush needed" % (M * K * 4 // 2 ** 20),
                       "parallelism": par,
                       "timed": f"median of {repeats} regions of {args.steps} steps, each between barrier+synchronize"},
            "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "regions": regions,
            "frac_of_tf32_peak": round(value / world / tf32_peak, 4)}
    if world > 1:
        line["exchange"] = {"bytes_per_step": host.grads.size * 4, "nccl_max_ctas": args.nccl_ctas, "reserved_sms": args.reserve_sms,
                            "rows_of_dA_beside_it": args.overlap_rows or M}

    if rank == 0 and not args.no_sweep:
        line["sweep"] = time_sweep(ctx)
        try:
            line["calibration"] = cublas_tf32_yardstick()
            line["roofline"]["frac_of_library_tf32_same_box"] = round(achieved / line["calibration"]["tflops"], 4)
        except Exception as exc:  # the yardstick must never break the benchmark
            line["calibration"] = {"error": str(exc)[:200]}
    if rank == 0 and not args.no_configs:
        import bench_configs
        line["configs"] = bench_configs.run(ctx)
        if local_rank == 0:  # the legacy symbol owns a context on device 0
            line["legacy_roundtrip"] = legacy_roundtrip()
    if rank == 0 and not args.no_membound:
        line["membound"] = time_membound(ctx, peaks["hbm_gbs"], rows=args.membound_rows)
        line["attention"] = time_attention(ctx)
    if rank == 0 and not args.no_cpu:
        from oracle import oracle
        oracle.build()
        S = args.ref_size
        sec = cpu_step(S, S, S, False)
        line["cpu_baseline"] = {"value": 6.0 * S ** 3 / sec / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                                "sample": f"M=N=K={S} fwd+bwd once ({sec:.1f} s), float64 scalar loops, 1 thread"}
    del host
    if not args.no_train:
        if world > 1:
            ctx.check(ctx.lib.fml_dp_shutdown(ctx.h))   # the training step makes its own communicator (NCCL's CTA choice)
            ctx.check(ctx.lib.fml_dp_set_max_ctas(ctx.h, 0))
        import bench_train
        line["train"] = bench_train.run(ctx, rank, world, barrier, max_over_ranks, steps=max(1, args.train_steps))
    if rank == 0:
        print(json.dumps(line), flush=True)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
