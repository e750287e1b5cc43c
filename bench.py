#!/usr/bin/env python
"""Benchmark of the optimizer step: Adam-step params/s and HBM GB/s, 555M-parameter model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over the whole packed arena: gradient norm,
clip / skip decision, AdamW, fp32 master, bf16 moments, bf16 weight twins, gradient
zeroing.  Workload (the headline configuration, "run555m"): 555,762,080 parameters in the
reference's tensor list, bf16 gradients N(0, 5e-4) with 0.1 % entries x100, fp32
master, bf16 m/v, bf16 twins, clip 1.0 (active), weight decay 0.1 on matrices.  All
data are synthetic and seeded; K + W gradient arenas are resident before timing, so no
step reuses (already zeroed) gradients and nothing is copied inside the timed region.
With N > 1 the state is ZeRO-1 sharded (strong scaling: the model stays 555M).

The JSON line carries, besides the contract keys: `roofline` (algorithmic bytes /
kernel time against the measured HBM peak), `cpu_baseline` (the reference's own CPU step
timed on this host, bounded sample), `e2e` (same metric through the C ABI with HOST
gradient buffers: pinned H2D copy + step + D2H status inside the timed region).
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = "run555m"
N_PARAMS = 555_762_080
ALG_BYTES_PER_PARAM = 20     # bf16 grad 2 + fp32 master r/w 8 + bf16 m r/w 4 + bf16 v r/w 4 + bf16 twin 2
# --workload selects another benchmark configuration for side measurements (the default, and the
# only one the contract line is about, is run555m):
#   name -> (shape, gradient dtype, moment dtype, twin kind, algorithmic bytes per parameter)
WORKLOADS = {
    "run555m": ("run555m", "bf16", "bf16", "bf16", 20),          # configuration 3
    "run555m-fp8": ("run555m", "bf16", "bf16", "fp8", 19),       # configuration 5 (e4m3 twins for the block matrices)
    "talk170m-mixed": ("talk170m", "bf16", "f32", "bf16", 28),   # configuration 2
    "talk170m-fp32": ("talk170m", "f32", "f32", "bf16", 30),     # configuration 1 run on the GPU
    "synth3b": ("synth3b", "bf16", "f32", "bf16", 28),           # configuration 4 (8 GPUs)
    # three of run555m's blocks and a small head, about 1 GB on the device: sized for profiler captures
    "blocks3": ("blocks3", "bf16", "bf16", "bf16", 20),
    "blocks3-fp8": ("blocks3", "bf16", "bf16", "fp8", 19),
}
HYPER = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0)
# DRAM bytes per parameter of the fused kernel: dram__bytes_read.sum + dram__bytes_write.sum of one
# 100.7M-parameter launch captured with ncu, divided by the parameter count (traffic grows in
# proportion to it).
NCU_DRAM_BYTES_PER_PARAM = 21.54


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the bench runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], False
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                if self.stop_flag:
                    break
                self.rows.append((time.time(), [c.strip() for c in line.split(",")]))
        except Exception:
            pass

    def finish(self, t0, t1):
        self.stop_flag = True
        if self.proc is not None:
            self.proc.terminate()
        return self.window(t0, t1)

    def window(self, t0, t1):
        rows = [r for ts, r in list(self.rows) if t0 - 0.2 <= ts <= t1 + 0.2] or [r for _, r in list(self.rows)]
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------
# reference arm: the reference's own CPU step (oracle/_ref), bounded sample
# ----------------------------------------------------------------------------------------

def cpu_reference_all_cores(ref, p, gsrc, steps):
    """What every host core together can do with the reference's loop: one independent
    reference optimizer per core, each over its own slice of the sample, stepped at the same
    time (the loop itself is single-threaded; each slice clips by its own norm, which costs
    the same arithmetic).  An upper bound for a parallelised reference, reported beside the
    single-thread figure, not instead of it."""
    import numpy as np
    threads = max(1, os.cpu_count() or 1)
    per = len(p) // threads
    g = gsrc.copy()
    handles = []
    for k in range(threads):
        sl = slice(k * per, (k + 1) * per)
        ps, gs = p[sl], g[sl]
        handles.append(ref.L.ref_adam_bench_create(ps.ctypes.data, gs.ctypes.data, per, HYPER["beta1"],
                                                   HYPER["beta2"], HYPER["eps"], HYPER["wd"], HYPER["clip"], 999))
    assert all(handles)
    times = []
    for i in range(1 + max(1, steps)):
        g[:] = gsrc
        ts = [threading.Thread(target=ref.L.ref_adam_bench_step, args=(h, HYPER["lr"], 1.0)) for h in handles]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        if i >= 1:
            times.append(time.perf_counter() - t0)
    for h in handles:
        ref.L.ref_adam_bench_free(h)
    sec = sum(times) / len(times)
    return dict(value=per * threads / sec, threads=threads,
                note="one independent reference optimizer per host core, stepped concurrently")


def host_mem_available():
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        pass
    return 0


def synthetic_host_arrays(sample):
    """Weights N(0, 0.02) and gradients N(0, 5e-4) with 0.1 % of the entries x100, as fp32 host
    arrays: 16 Mi fresh draws each, repeated to the requested length (the reference's loop does
    the same arithmetic on every element whatever its value, and 64 MB is far beyond any cache)."""
    import numpy as np
    rng = np.random.default_rng(0)
    block = min(sample, 1 << 24)
    pb = rng.standard_normal(block, dtype=np.float32) * np.float32(0.02)
    gb = rng.standard_normal(block, dtype=np.float32) * np.float32(5e-4)
    gb[rng.random(block, dtype=np.float32) < 1e-3] *= 100
    p = np.empty(sample, np.float32)
    g = np.empty(sample, np.float32)
    for lo in range(0, sample, block):
        hi = min(sample, lo + block)
        p[lo:hi] = pb[:hi - lo]
        g[lo:hi] = gb[:hi - lo]
    return p, g


def reference_sample_size(steps, warm, budget_s=None):
    """The largest arena -- the whole 555M one if possible -- that the reference's host loop gets
    through `steps + warm` times within the budget on this host.  Set-up (the reference's slot
    table: 24 bytes per parameter, filled element by element) and step time per parameter are
    measured on a 16 Mi-parameter probe first and taken to grow in proportion."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import RefLib
    small = 32 << 20
    if budget_s is None:        # seconds the whole reference run may take (ANNI_B200_REF_BUDGET_S overrides)
        budget_s = float(os.environ.get("ANNI_B200_REF_BUDGET_S", "200"))
    if not RefLib.available():
        return small
    n0 = 16 << 20
    t0 = time.perf_counter()
    p, g = synthetic_host_arrays(n0)
    ref = RefLib()
    h = ref.L.ref_adam_bench_create(p.ctypes.data, g.ctypes.data, n0, HYPER["beta1"], HYPER["beta2"],
                                    HYPER["eps"], HYPER["wd"], HYPER["clip"], 999)
    t1 = time.perf_counter()
    ref.L.ref_adam_bench_step(h, HYPER["lr"], 1.0)
    t2 = time.perf_counter()
    ref.L.ref_adam_bench_free(h)
    setup_pp, step_pp = (t1 - t0) / n0, (t2 - t1) / n0
    avail = host_mem_available()
    for sample in (N_PARAMS, 256 << 20, 128 << 20, 64 << 20):
        if 48 * sample < avail and 1.5 * setup_pp * sample + (steps + warm) * step_pp * sample <= budget_s:
            return sample
    return small


def cpu_reference_step_rate(sample, steps, warmup, all_cores=True):
    """params/s of lm_adam_step_scaled's host loop (the reference's object code when
    oracle/_ref/libannref.so exists, else this repository's C port), one thread."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import Oracle, RefLib
    p, gsrc = synthetic_host_arrays(sample)
    g = gsrc.copy()
    times = []
    if RefLib.available():
        kind, cores = "reference", 1
        ref = RefLib()
        h = ref.L.ref_adam_bench_create(p.ctypes.data, g.ctypes.data, sample, HYPER["beta1"],
                                        HYPER["beta2"], HYPER["eps"], HYPER["wd"], HYPER["clip"], 999)
        assert h
        for i in range(warmup + steps):
            g[:] = gsrc
            t0 = time.perf_counter()
            ref.L.ref_adam_bench_step(h, HYPER["lr"], 1.0)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
        ref.L.ref_adam_bench_free(h)
    else:
        kind = "port"
        cores = os.cpu_count() or 1
        orc = Oracle()
        m = np.zeros(sample, np.float32)
        v = np.zeros(sample, np.float32)
        for i in range(warmup + steps):
            g[:] = gsrc
            t0 = time.perf_counter()
            orc.step(p, g, m, v, lr=HYPER["lr"], beta1=HYPER["beta1"], beta2=HYPER["beta2"],
                     eps=HYPER["eps"], wd=HYPER["wd"], clip=HYPER["clip"], t_before=999 + i)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    extra = {}
    if kind == "reference" and all_cores:
        extra["all_cores"] = cpu_reference_all_cores(ref, p, gsrc, steps)
    return dict(value=sample / sec, unit="params/s", cores=cores, kind=kind, **extra,
                sample=f"{sample} fp32 parameters of the {WORKLOAD} distribution, {len(times)} timed "
                       f"steps of {sec * 1e3:.0f} ms, clip active, wd {HYPER['wd']}"), sec


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # the whole 555M arena when the host has room for it and K + W steps of it end within a few
    # minutes (about 5 s each on one core, after the set-up); otherwise the largest sample that does
    steps, warm = max(1, args.steps), max(1, min(args.warmup, 5))
    sample = reference_sample_size(steps, warm)
    base, sec = cpu_reference_step_rate(sample, steps, warm, all_cores=False)
    line = {
        "impl": "reference", "metric": "adam_step_params_per_s", "value": base["value"],
        "unit": "params/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "n_params": N_PARAMS, "sample_params": sample,
                   "note": "reference CPU host loop (double math, fp32 storage), single-threaded by "
                           "construction; " + ("every step the whole arena" if sample == N_PARAMS
                                               else "each step a bounded sample")},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "params/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------

def percentiles(xs):
    """p10 / p50 / p90 of the per-step device times (this rank's events), ms."""
    if not xs:
        return None
    xs = sorted(xs)
    pick = lambda q: xs[min(len(xs) - 1, int(round(q * (len(xs) - 1))))]
    return {"p10": pick(0.1), "p50": pick(0.5), "p90": pick(0.9), "n": len(xs)}


def fill_grads(buf, n, seed, device):
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    chunk = 64 * 1024 * 1024
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        g = torch.randn(hi - lo, device=device, generator=gen).mul_(5e-4)
        mask = torch.rand(hi - lo, device=device, generator=gen) < 1e-3
        g[mask] *= 100.0
        buf[lo:hi].copy_(g)


def zero1_parity_check(dev, rank, world, zero1_kwargs):
    """N > 1, before anything is timed: the sharded step against the CPU oracle (the checker, outside
    every timed region).  (1) Three ZeRO-1 steps of the reference's unit-test LM with per-rank
    gradients g / N accumulated into the arenas (N a power of two: the reduced sum is exact), the
    third with an inf in the last rank's shard: decisions, norms, gathered master / moments and
    the all-gathered twins against the oracle on the reduced gradients, and every arena left
    zeroed.  (2) One slice of the 2,773,419,680-parameter arena per rank (ranks spread over it, the
    upper ones above 2^31) through the split form with a handed-in sum of squares, against the
    oracle on the same slice.  Returns the `parity` object of the JSON line; any mismatch makes
    every rank exit non-zero."""
    import math
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from anni_b200.capi import DT_BF16, DT_F32
    from anni_b200.engine import LM_SHAPES, OptStep, lm_segments
    from anni_b200.zero1 import Zero1
    from oracle_lib import Oracle
    from parity_util import bf16_bits_from_f32, check_step, make_inputs, to_dev, to_host, ulp_of

    def ulps(got, want, old):
        # how much of the bar is used: |difference| over (2 ulp of the larger of |p_old|, |p_ref|
        # + 1e-6 of the size of the update), largest over the elements; <= 1 passes
        tol = 2.0 * ulp_of(np.maximum(np.abs(old), np.abs(want))) + 1e-6 * np.abs(old.astype(np.float64) - want)
        return float((np.abs(got.astype(np.float64) - want) / tol).max())

    orc = Oracle()
    problems = []
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    z = Zero1(segs, grad_dtype=DT_BF16, state_dtype=DT_F32, device=dev, **zero1_kwargs)
    rng = np.random.default_rng(321)
    p = rng.normal(0, 0.02, n).astype(np.float32)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    p0 = p.copy()
    z.load_shard_from_full(to_dev(p, dev), to_dev(m, dev), to_dev(v, dev))
    skip_identical = True
    for step in range(3):
        base = rng.normal(0, 1e-3, n).astype(np.float32)
        if step == 2:
            base[n - 7] = np.inf
        gb = torch.from_numpy(base).to(torch.bfloat16)
        z.grad_full[:n] += (gb.float() / world).to(torch.bfloat16).to(dev)
        z.step(OptStep.hyper(lr=3e-4, t=step + 1, beta2=0.95, wd=0.1, clip=1.0, grad_scale=1.0))
        st = z.status()
        info = orc.step(p, orc.bf16_rne(base), m, v, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1,
                        clip=1.0, grad_scale=1.0, t_before=step, check_finite=True,
                        seg_off=segs.offsets, seg_flags=segs.flag_array)
        if bool(st.skipped) != info["skipped"] or st.error != 0:
            skip_identical = False
            problems.append(f"step {step}: skipped {st.skipped} error {st.error}, oracle skipped {info['skipped']}")
        if not info["skipped"] and not abs(st.norm - info["norm"]) <= 1e-9 * info["norm"]:
            problems.append(f"step {step}: norm {st.norm} against {info['norm']}")
        if bool(z.grad_full.any()):
            problems.append(f"step {step}: gradient arena not left zeroed")
    gp, gm, gv = (to_host(z.gather_full(x)) for x in (z.master, z.m, z.v))
    max_ulp = ulps(gp, p, p0)
    try:
        check_step(dict(p=gp, m=gm, v=gv), p, m, v, p0, exact_moments=False)
    except AssertionError as e:
        problems.append(f"sharded state against the oracle: {e}")
    if not np.array_equal(to_host(z.twin_full[:n]), bf16_bits_from_f32(gp)):
        problems.append("all-gathered twins are not the RNE cast of the master")
    z.close()
    del z

    segs4 = lm_segments(**LM_SHAPES["synth3b"], wd="matrices")
    length = 1 << 20
    off = (segs4.n - length) // max(1, world - 1) * rank // 4096 * 4096
    so = segs4.offsets
    first = int(np.searchsorted(so, off, side="right") - 1)
    last = int(np.searchsorted(so, off + length, side="left"))
    loc_off = np.clip(so[first:last + 1] - off, 0, length).astype(np.int64)
    p4, g4, m4, v4 = make_inputs(length, seed=4000 + rank, grad_dtype=DT_BF16, state_dtype=DT_F32, grad_std=3e-4)
    ss = orc.sumsq(g4, 1.0) * (segs4.n / length)
    coef = 1.0 * (1.0 / (math.sqrt(ss) * 1.0 + 1e-12))
    ref = [x.copy() for x in (p4, g4, m4, v4)]
    orc.step(*ref, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=0.0, grad_scale=coef, t_before=41,
             seg_off=loc_off, seg_flags=segs4.flag_array[first:last].copy())
    eng = OptStep(segs4, grad_dtype=DT_BF16, state_dtype=DT_F32, shard_off=off, shard_n=length, device=dev).allocate()
    for t, src in ((eng.master, p4), (eng.grad, g4), (eng.m, m4), (eng.v, v4)):
        t[:length].copy_(to_dev(src, dev))
    eng.reduce_tensor().copy_(torch.tensor([ss, 0.0], dtype=torch.float64))
    eng.update(OptStep.hyper(lr=3e-4, t=42, beta2=0.95, wd=0.1, clip=1.0, grad_scale=1.0))
    st = eng.status()
    out = dict(p=to_host(eng.master[:length]), m=to_host(eng.m[:length]), v=to_host(eng.v[:length]))
    try:
        assert st.error == 0 and st.skipped == 0 and st.eff_scale == coef
        check_step(out, ref[0], ref[2], ref[3], p4, exact_moments=True)
        assert np.array_equal(to_host(eng.twin_bf16[:length]), bf16_bits_from_f32(out["p"]))
    except AssertionError as e:
        problems.append(f"3B-arena slice at offset {off}: {e}")
    max_ulp = max(max_ulp, ulps(out["p"], ref[0], p4))
    eng.close()

    flag = torch.tensor([0.0 if problems else 1.0, max_ulp], dtype=torch.float64, device=dev)
    mins = flag.clone()
    dist.all_reduce(mins, op=dist.ReduceOp.MIN)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    ok = bool(mins[0].item())
    if problems:
        print(f"[bench] rank {rank}: parity check failed: " + "; ".join(problems), file=sys.stderr, flush=True)
    return dict(checked=True, ok=ok, max_master_err_over_bar=round(float(flag[1].item()), 4),
                bar="moments within 1 ulp, master within 2 ulp of the larger of |p_old|, |p_ref| + 1e-6 of the "
                    "update, twins the RNE cast of the master, decisions identical",
                skip_identical=skip_identical and ok,
                steps=3, arena_left_zeroed=ok, slices_of_3b_arena=world,
                against="CPU oracle on the reduced gradients, before the timed region")


def run_ours(args):
    import torch
    import torch.distributed as dist
    from anni_b200.capi import DT_BF16, STEP_REDUCE_CLEARS_OWN
    from anni_b200.engine import LM_SHAPES, OptStep, kernel_launches, lm_segments
    from anni_b200.zero1 import Zero1

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    shape, gdt_name, sdt_name, twin_kind, alg_bytes = WORKLOADS[args.workload]
    from anni_b200.capi import DT_F32
    gdt = DT_BF16 if gdt_name == "bf16" else DT_F32
    sdt = DT_BF16 if sdt_name == "bf16" else DT_F32
    segs = lm_segments(**LM_SHAPES[shape], wd="matrices", twin=twin_kind)
    n = segs.n
    assert args.workload != WORKLOAD or n == N_PARAMS
    mode = os.environ.get("ANNI_B200_ZERO1_MODE", "")          # "", "peer", "copy" or "nccl"
    zero1_kwargs = dict(peer={"": None, "peer": True, "copy": "copy", "nccl": False}[mode],
                        multicast=os.environ.get("ANNI_B200_MULTICAST", "0") == "1")
    parity = None
    if world > 1:
        parity = zero1_parity_check(dev, rank, world, zero1_kwargs)
        if not parity["ok"]:
            dist.destroy_process_group()
            return 3
    z = Zero1(segs, grad_dtype=gdt, state_dtype=sdt, device=dev, **zero1_kwargs)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    z.master.normal_(0, 0.02, generator=gen)
    z.m.copy_(torch.randn(z.per, device=dev, generator=gen).mul_(1e-4))
    z.v.copy_(torch.randn(z.per, device=dev, generator=gen).mul_(1e-6).abs_())

    K, W = args.steps, args.warmup
    # the step consumes (zeroes) the gradient arena it is given -- the whole local arena, on one
    # rank as on several -- so every step gets a fresh one
    pool_n = min(K + W, 48 if n < 1_000_000_000 else 8)
    pool = [z.new_grad_arena() for _ in range(pool_n)]

    def refill():
        for i, (b, _) in enumerate(pool):
            b.zero_()
            fill_grads(b, n, 1000 * rank + i, dev)

    def bind_grads(arena):
        z.use_grad_arena(arena)

    def hyper(t, exact=False, zero_grad=True):
        return OptStep.hyper(lr=HYPER["lr"], t=t, beta1=HYPER["beta1"], beta2=HYPER["beta2"],
                             eps=HYPER["eps"], wd=HYPER["wd"], clip=HYPER["clip"],
                             grad_scale=1.0 / world, check_finite=True, zero_grad=zero_grad, exact=exact)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    refill()
    torch.cuda.synchronize()
    time.sleep(1.0)                 # filling the pool runs at the power cap; let the clocks come back
    t = 1000
    done = 0
    for _ in range(W):
        bind_grads(pool[done % pool_n])
        z.step(hyper(t))
        t += 1
        done += 1
    total_ms, launches0 = 0.0, kernel_launches()
    phase_ms = {}
    step_ms = []
    left = K
    wall0 = time.time()
    while left > 0:
        batch = min(left, pool_n - (done % pool_n)) if done % pool_n else min(left, pool_n)
        if done % pool_n == 0 and done > 0:
            refill()
            torch.cuda.synchronize()
            time.sleep(1.0)
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        marks = []
        e0.record()
        for _ in range(batch):
            bind_grads(pool[done % pool_n])
            if world > 1:
                evs = [torch.cuda.Event(enable_timing=True)]
                evs[0].record()
                if z.driver == "library":
                    # the sequence runs inside the library, which records these events after each phase
                    ph = [torch.cuda.Event(enable_timing=True) for _ in Zero1.PHASES]
                    for e in ph:
                        e.record()
                    z.step(hyper(t), grads_complete=True, phase_events=ph)
                    evs += list(zip(Zero1.PHASES, ph))
                else:
                    def rec(name, evs=evs):
                        e = torch.cuda.Event(enable_timing=True)
                        e.record()
                        evs.append((name, e))
                    z.step(hyper(t), record=rec, grads_complete=True)
                marks.append(evs)
            else:
                z.step(hyper(t))
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append(e)
            t += 1
            done += 1
        e1.record()
        barrier()
        total_ms += e0.elapsed_time(e1)
        if world == 1:
            prev = e0
            for e in marks:
                step_ms.append(prev.elapsed_time(e))
                prev = e
            marks = []
        for evs in marks:
            step_ms.append(evs[0].elapsed_time(evs[-1][1]))
            prev = evs[0]
            for name, e in evs[1:]:
                phase_ms[name] = phase_ms.get(name, 0.0) + prev.elapsed_time(e)
                prev = e
        left -= batch
    wall1 = time.time()
    launches = kernel_launches() - launches0
    st = z.status()
    phases_by_rank = None
    if world > 1:
        tmax = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        total_ms = float(tmax.item())
        # every rank's own view of the phases (a rank that waits for a slower one shows it in the
        # phase that ends with an exchange)
        phases_by_rank = [None] * world
        dist.all_gather_object(phases_by_rank, {k: round(v / K, 4) for k, v in phase_ms.items()})
    ms_per_step = total_ms / K
    value = n / (ms_per_step * 1e-3)
    if args.profile:
        # a run for the profiler: the steps above and nothing else
        if rank == 0:
            print(json.dumps({"metric": "adam_step_params_per_s", "value": value, "unit": "params/s",
                              "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
                              "config": {"workload": args.workload, "n_params": n}, "profile_run": True,
                              "status": {"norm": st.norm, "skipped": int(st.skipped), "error": int(st.error)}}),
                  flush=True)
        z.close()
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- the same step with the parameter update evaluated in double (ANNI_STEP_EXACT_UPDATE) ----
    exact_ms = None
    if world == 1:
        refill()
        torch.cuda.synchronize()
        time.sleep(1.0)             # the refill runs at the power cap; let the clocks come back first
        k_ex = min(10, pool_n - 2)
        for i in range(2):
            bind_grads(pool[i])
            z.step(hyper(t, exact=True))
            t += 1
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(k_ex):
            bind_grads(pool[2 + i])
            z.step(hyper(t, exact=True))
            t += 1
        e1.record()
        barrier()
        exact_ms = e0.elapsed_time(e1) / k_ex

    # ---- the same step without the gradient zeroing (a trainer whose first micro-batch overwrites) ----
    # Not the contract's step: it shows what the 2 bytes per parameter of zeroing stores cost.
    nozero_ms = None
    if world == 1:
        refill()
        torch.cuda.synchronize()
        time.sleep(1.0)
        for i in range(2):
            bind_grads(pool[i])
            z.step(hyper(t, zero_grad=False))
            t += 1
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        k_nz = min(10, pool_n - 2)
        e0.record()
        for i in range(k_nz):
            bind_grads(pool[2 + i])
            z.step(hyper(t, zero_grad=False))
            t += 1
        e1.record()
        barrier()
        nozero_ms = e0.elapsed_time(e1) / k_nz

    # ---- the two phases apart (three-launch form), outside the timed region ------------------
    split_ms = None
    if world == 1:
        refill()
        torch.cuda.synchronize()
        time.sleep(1.0)             # the refill runs at the power cap; let the clocks come back first
        k_sp = min(10, pool_n - 2)
        marks = []
        for i in range(2 + k_sp):
            bind_grads(pool[i])
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            hp_i = hyper(t)
            evs[0].record()
            z.eng.norm(hp_i)
            evs[1].record()
            z.eng.update(hp_i)
            if z.eng.has_fp8:
                z.eng.quantize()
            evs[2].record()
            t += 1
            marks.append(evs)
        barrier()
        marks = marks[2:]
        split_ms = {"norm": sum(a.elapsed_time(b) for a, b, _ in marks) / k_sp,
                    "update": sum(b.elapsed_time(c) for _, b, c in marks) / k_sp}

    # ---- several ranks: this rank's share of the update on its own memory alone ------------------
    # (what falls linearly with N; the step as a whole is bound by the two collectives on the wire)
    hbm_only_ms = hbm_nozero_ms = None
    if world > 1 and hasattr(z.eng, "update_range"):
        evs = []
        barrier()
        for i in range(2 + 5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            hp_i = hyper(t)
            if getattr(z, "reduce_clears_own", False):
                hp_i.flags |= STEP_REDUCE_CLEARS_OWN         # as in the step: the reduce has cleared that part
            z.eng.update_range(hp_i, 0, z.shard_n, first=True, last=True, local_twins=True)
            b.record()
            t += 1
            evs.append((a, b))
        barrier()
        hbm_only_ms = sum(a.elapsed_time(b) for a, b in evs[2:]) / 5
        # ... and the same without clearing the gradient arena, whose size does not shrink with N
        evs = []
        for i in range(2 + 5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            z.eng.update_range(hyper(t, zero_grad=False), 0, z.shard_n, first=True, last=True, local_twins=True)
            b.record()
            t += 1
            evs.append((a, b))
        barrier()
        hbm_nozero_ms = sum(a.elapsed_time(b) for a, b in evs[2:]) / 5
        tmax = torch.tensor([hbm_only_ms, hbm_nozero_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        hbm_only_ms, hbm_nozero_ms = (float(x) for x in tmax.tolist())

    # ---- sustained: 200 steps back to back, no pauses (one rank) ---------------------------------
    # Each step is preceded by an untimed device copy that restores the gradient arena the previous
    # step consumed, so the GPU never idles; the step itself is timed by its own pair of events.
    sustained = None
    if world == 1:
        n_sus = 200
        gsrc = torch.empty(z.padded, dtype=z.grad_full.dtype, device=dev)
        fill_grads(gsrc, n, 4242, dev)
        bind_grads(pool[0])
        arena = pool[0][0]
        evs = []
        torch.cuda.synchronize()
        sus0 = time.time()
        for i in range(n_sus + 10):
            arena.copy_(gsrc)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            z.step(hyper(t))
            b.record()
            t += 1
            evs.append((a, b))
        torch.cuda.synchronize()
        sus1 = time.time()
        ts = sorted(a.elapsed_time(b) for a, b in evs[10:])
        sus_ms = sum(ts) / len(ts)
        sustained = {"steps": n_sus, "ms_per_step": sus_ms, "p50_ms": ts[len(ts) // 2], "value": n / (sus_ms * 1e-3),
                     "roofline_frac": alg_bytes * n / (sus_ms * 1e-3) / 1e9 / measured_peaks()[0],
                     "window_s": sus1 - sus0,
                     "note": "back-to-back steps, each after an untimed device copy that restores the gradient arena"}
        del gsrc

    # ---- e2e: host gradient buffers through the C ABI --------------------------------------
    e2e_steps = max(2, min(5, K))
    host = [torch.empty(z.padded, dtype=z.grad_full.dtype).pin_memory() for _ in range(2)]
    tmp = torch.zeros(z.padded, dtype=z.grad_full.dtype, device=dev)
    for i, hb in enumerate(host):
        fill_grads(tmp, n, 777 + i + 10 * rank, dev)
        hb.copy_(tmp)
    del tmp
    # Two device arenas: while the step of one batch of gradients runs, the copy engine brings the
    # next batch over (what a trainer with host-side gradients does); every copy, every step and
    # every status read lies inside the timed region.
    main = torch.cuda.current_stream(dev)
    copier = torch.cuda.Stream(device=dev)
    arenas = [pool[0], pool[1]]
    copied = [torch.cuda.Event(), torch.cuda.Event()]
    stepped = [None, None]
    barrier()
    w0 = time.perf_counter()
    with torch.cuda.stream(copier):
        arenas[0][0].copy_(host[0], non_blocking=True)       # H2D of the first step's gradients
        copied[0].record(copier)
    for i in range(e2e_steps):
        a = i % 2
        if i + 1 < e2e_steps:
            with torch.cuda.stream(copier):
                if stepped[1 - a] is not None:
                    copier.wait_event(stepped[1 - a])        # the step that last used that arena is done
                arenas[1 - a][0].copy_(host[(i + 1) % 2], non_blocking=True)
                copied[1 - a].record(copier)
        main.wait_event(copied[a])
        bind_grads(arenas[a])
        z.step(hyper(t))
        stepped[a] = torch.cuda.Event()
        stepped[a].record(main)
        t += 1
        st = z.status()                                       # D2H of the step's result (sync)
    barrier()
    e2e_sec = (time.perf_counter() - w0)
    if world > 1:
        tmax = torch.tensor([e2e_sec], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_sec = float(tmax.item())
    e2e_value = n * e2e_steps / e2e_sec

    # ---- e2e through the C optimizer object: host fp32 gradients of configuration 1 -------------
    # anni_lm_adam_step_scaled as a C trainer calls it: uploads the host gradient arrays (pinned),
    # runs the one-launch step, reads the status back, zeroes the host gradients.
    e2e_c = None
    if world == 1 and args.workload == WORKLOAD:
        from anni_b200 import lm_adam
        del pool, host
        torch.cuda.empty_cache()
        segs1 = lm_segments(**LM_SHAPES["talk170m"], wd="matrices")
        n1 = segs1.n
        hw = torch.empty(n1, dtype=torch.float32).pin_memory()
        hg = torch.empty(n1, dtype=torch.float32).pin_memory()
        src = torch.empty(n1, dtype=torch.float32, device=dev)
        fill_grads(src, n1, 99, dev)
        gsrc1 = src.cpu()
        hw.normal_(0, 0.02)
        del src
        L1 = lm_adam.lib()
        opt = lm_adam.create(segs1, hw.data_ptr(), hg.data_ptr())
        o = opt.contents
        o.beta2, o.weight_decay, o.grad_clip = HYPER["beta2"], HYPER["wd"], HYPER["clip"]
        secs, norms1 = [], []
        for i in range(2 + 4):
            hg.copy_(gsrc1)                       # the backward pass's output, untimed
            t0 = time.perf_counter()
            rc = L1.anni_lm_adam_step_scaled(opt, HYPER["lr"], 1.0)
            secs.append(time.perf_counter() - t0)
            assert rc == 0 and o.last_skipped == 0
            # the step left every host gradient zeroed, and saw the same gradients as the first step
            assert not bool(hg.any()), "host gradients not cleared by the step"
            norms1.append(o.last_grad_norm)
            assert abs(norms1[-1] - norms1[0]) <= 1e-9 * norms1[0]
        L1.anni_lm_adam_free(ctypes.byref(opt))
        sec = sum(secs[2:]) / len(secs[2:])
        e2e_c = {"value": n1 / sec, "unit": "params/s", "workload": "talk170m-fp32 (configuration 1)",
                 "n_params": n1, "ms_per_step": sec * 1e3, "h2d_bytes_per_step": 4 * n1,
                 "d2h_bytes_per_step": 48, "steps": len(secs) - 2,
                 "path": "anni_lm_adam_step_scaled: upload of pinned host fp32 gradients (147 tensors), "
                         "one-launch step, status read, host gradients cleared piece by piece by a few threads behind asynchronous uploads"}

    driver_name = z.driver
    z.close()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0
    if sustained is not None and sampler:
        sc = sampler.window(sus0, sus1)
        sustained["sm_mhz"] = sc["sm_mhz"]
        sustained["reasons"] = sc["reasons"]
    clocks = sampler.finish(wall0, wall1) if sampler else None
    peak, peak_kind = measured_peaks()
    # the dominant kernel's share of the step: at N = 1 the step IS one launch of it
    upd_key = "update+all_gather" if "update+all_gather" in phase_ms else "update"
    kern_ms = ms_per_step if world == 1 else phase_ms.get(upd_key, 0.0) / K
    shard_n = z.shard_n
    achieved = alg_bytes * shard_n / (kern_ms * 1e-3) / 1e9 if kern_ms > 0 else None
    line = {
        "metric": "adam_step_params_per_s", "value": value, "unit": "params/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64+f32",
        "data": "synthetic",
        "config": {"workload": args.workload, "n_params": n, "grads": gdt_name, "master": "fp32",
                   "moments": sdt_name, "twins": twin_kind, "clip": HYPER["clip"], "wd": "0.1 on matrices",
                   "alg_bytes_per_param": alg_bytes,
                   "update_arithmetic": "double moments, float update (fast mode)",
                   "zero_grad": True, "zero1_ranks": world,
                   "l2": "inputs larger than L2 (6.7 GB state + a fresh 1.1 GB gradient arena per step)",
                   "grad_arena": ("compressible device memory (anni_arena_alloc)" if getattr(z, "_arenas", None)
                                  else "symmetric memory" if z.peer else "plain device memory"),
                   "hbm_gbs_alg": (alg_bytes * n / (ms_per_step * 1e-3) / 1e9)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak if achieved else None,
                     "traffic": NCU_DRAM_BYTES_PER_PARAM * shard_n if args.workload == WORKLOAD and world == 1 else None,
                     "kernel": f"fused_kernel<{gdt_name},{sdt_name}>" if world == 1 else f"update_kernel<{gdt_name},{sdt_name}>",
                     "kernel_ms": kern_ms, "peak_kind": f"of {peak_kind}",
                     "frac_of_8000": achieved / 8000.0 if achieved else None},
        "e2e": {"value": e2e_value, "unit": "params/s",
                "h2d_bytes_per_step": int(z.padded * z.grad_full.element_size()), "d2h_bytes_per_step": 48,
                "steps": e2e_steps},
        "gpu_launches": int(launches),
        "step_ms": percentiles(step_ms),
        "clocks": clocks,
        "status": {"norm": st.norm, "skipped": int(st.skipped), "error": int(st.error)},
    }
    if parity is not None:
        line["parity"] = parity
    if e2e_c is not None:
        line["e2e_c_api"] = e2e_c
    if sustained is not None:
        line["sustained"] = sustained
    if world > 1:
        line["phases_ms"] = {k: v / K for k, v in phase_ms.items()}
        line["phases_ms_by_rank"] = phases_by_rank
        if hbm_only_ms is not None:
            line["phases_ms"]["update_hbm_only"] = hbm_only_ms
            line["per_rank_update"] = {
                "ms": hbm_only_ms, "shard_params": shard_n,
                "roofline_frac": alg_bytes * shard_n / (hbm_only_ms * 1e-3) / 1e9 / peak,
                "ms_without_arena_zeroing": hbm_nozero_ms,
                "roofline_frac_without_arena_zeroing": alg_bytes * shard_n / (hbm_nozero_ms * 1e-3) / 1e9 / peak,
                "note": "this rank's update on local memory alone (twins stored locally): the part of the step "
                        "that shrinks with N; clearing the other ranks' parts of this rank's gradient arena (2 bytes "
                        "per parameter of (N-1)/N of the WHOLE model; the own part is cleared by the reduce) "
                        "does not, hence the second figure"}
        wire = (world - 1) / world * n * 2 / 1e9            # GB each way per GPU, per collective
        rs_ms = line["phases_ms"].get("reduce_scatter+norm", line["phases_ms"].get("reduce_scatter"))
        ag_ms = line["phases_ms"].get("update+all_gather", line["phases_ms"].get("all_gather"))
        line["nvlink"] = {"driver": driver_name, "mode": ("peer kernels, NVSwitch multicast" if getattr(z, "uses_multicast", False)
                                   else "copy engines + local kernels" if getattr(z, "copy_mode", False)
                                   else "peer kernels" if z.peer else "nccl"), "wire_gb_per_collective": wire,
                          "link_gbs": 770.0, "floor_ms_per_collective": wire / 770.0 * 1e3,
                          "reduce_scatter_frac": (wire / 770.0 * 1e3) / rs_ms if rs_ms else None,
                          "all_gather_frac": (wire / 770.0 * 1e3) / ag_ms if ag_ms else None}
        if z.peer:
            line["roofline"]["kernel"] += " with peer twin stores"
    if world == 1:
        line["exact_update"] = {"ms_per_step": exact_ms, "value": n / (exact_ms * 1e-3),
                                "roofline_frac": alg_bytes * n / (exact_ms * 1e-3) / 1e9 / peak,
                                "note": "same step with ANNI_STEP_EXACT_UPDATE (update term in double)"}
        line["phases_ms"] = dict(split_ms, note="three-launch form of the same step, timed apart: the norm pass "
                                 "(a second read of the gradients) and the update pass; a caller whose "
                                 "gradient producer supplies the sum of squares pays the update pass only")
        line["phases_ms"]["update_only_roofline_frac"] = alg_bytes * n / (split_ms["update"] * 1e-3) / 1e9 / peak
        line["without_zero_grad"] = {"ms_per_step": nozero_ms,
                                     "roofline_frac": alg_bytes * n / (nozero_ms * 1e-3) / 1e9 / peak,
                                     "note": "side measurement, not the contract's step: ANNI_STEP_ZERO_GRAD off "
                                             "(22 instead of 24 bytes per parameter issued)"}
        base, _ = cpu_reference_step_rate(64 * 1024 * 1024, 3, 1)
        line["cpu_baseline"] = base
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--profile", action="store_true",
                    help="warm-up and timed steps only (no side measurements): the command profiler captures run")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
