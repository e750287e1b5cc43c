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
}
HYPER = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0)
# DRAM bytes per parameter of the fused kernel from the ncu capture summarised in
# profiles/fused_kernel_bf16state_100M.md (dram__bytes_read.sum + dram__bytes_write.sum of a
# 100.7M-parameter launch; traffic grows in proportion to the parameter count).
NCU_DRAM_BYTES_PER_PARAM = 21.54   # dram read + write of one fused launch / parameters (ncu, 100.7 M case, profiles/)


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
        rows = [r for ts, r in self.rows if t0 - 0.2 <= ts <= t1 + 0.2] or [r for _, r in self.rows]
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


def cpu_reference_step_rate(sample, steps, warmup):
    """params/s of lm_adam_step_scaled's host loop (the reference's object code when
    oracle/_ref/libannref.so exists, else this repository's C port), one thread."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import Oracle, RefLib
    rng = np.random.default_rng(0)
    p = rng.normal(0, 0.02, sample).astype(np.float32)
    gsrc = rng.normal(0, 5e-4, sample).astype(np.float32)
    gsrc[rng.random(sample) < 1e-3] *= 100
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
    if kind == "reference":
        extra["all_cores"] = cpu_reference_all_cores(ref, p, gsrc, steps)
    return dict(value=sample / sec, unit="params/s", cores=cores, kind=kind, **extra,
                sample=f"{sample} fp32 parameters of the {WORKLOAD} distribution, {len(times)} timed "
                       f"steps of {sec * 1e3:.0f} ms, clip active, wd {HYPER['wd']}"), sec


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    sample = 32 * 1024 * 1024
    base, sec = cpu_reference_step_rate(sample, max(1, args.steps), max(1, min(args.warmup, 3)))
    line = {
        "impl": "reference", "metric": "adam_step_params_per_s", "value": base["value"],
        "unit": "params/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "n_params": N_PARAMS, "sample_params": sample,
                   "note": "reference CPU host loop (double math, fp32 storage), single-threaded "
                           "by construction; each step a bounded sample"},
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


def run_ours(args):
    import torch
    import torch.distributed as dist
    from anni_b200.capi import DT_BF16
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
    z = Zero1(segs, grad_dtype=gdt, state_dtype=sdt, device=dev,
              peer={"": None, "peer": True, "copy": "copy", "nccl": False}[mode],
              multicast=os.environ.get("ANNI_B200_MULTICAST", "0") == "1")
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    z.master.normal_(0, 0.02, generator=gen)
    z.m.copy_(torch.randn(z.per, device=dev, generator=gen).mul_(1e-4))
    z.v.copy_(torch.randn(z.per, device=dev, generator=gen).mul_(1e-6).abs_())

    K, W = args.steps, args.warmup
    # one rank: the step consumes (zeroes) its gradient arena, so every step gets a fresh one;
    # several ranks: the arenas are only read (the reduced shard is what gets zeroed): four, cycled
    pool_n = min(K + W, 48 if n < 1_000_000_000 else 8) if world == 1 else 4
    pool = [z.new_grad_arena() for _ in range(pool_n)]

    def refill():
        for i, (b, _) in enumerate(pool):
            b.zero_()
            fill_grads(b, n, 1000 * rank + i, dev)

    def bind_grads(arena):
        z.use_grad_arena(arena)

    def hyper(t, exact=False):
        return OptStep.hyper(lr=HYPER["lr"], t=t, beta1=HYPER["beta1"], beta2=HYPER["beta2"],
                             eps=HYPER["eps"], wd=HYPER["wd"], clip=HYPER["clip"],
                             grad_scale=1.0 / world, check_finite=True, zero_grad=True, exact=exact)

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
    if world > 1:
        done = 0            # arenas are not consumed: no refills between batches
    total_ms, launches0 = 0.0, kernel_launches()
    phase_ms = {}
    step_ms = []
    left = K
    wall0 = time.time()
    while left > 0:
        if world > 1:
            batch = left
        else:
            batch = min(left, pool_n - (done % pool_n)) if done % pool_n else min(left, pool_n)
        if world == 1 and done % pool_n == 0 and done > 0:
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
    if world > 1:
        tmax = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        total_ms = float(tmax.item())
    ms_per_step = total_ms / K
    value = n / (ms_per_step * 1e-3)

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

    # ---- e2e: host gradient buffers through the C ABI --------------------------------------
    e2e_steps = max(2, min(5, K))
    host = [torch.empty(z.padded, dtype=z.grad_full.dtype).pin_memory() for _ in range(2)]
    tmp = torch.zeros(z.padded, dtype=z.grad_full.dtype, device=dev)
    for i, hb in enumerate(host):
        fill_grads(tmp, n, 777 + i + 10 * rank, dev)
        hb.copy_(tmp)
    del tmp
    dgrad = pool[0][0]
    bind_grads(pool[0])
    barrier()
    w0 = time.perf_counter()
    for i in range(e2e_steps):
        dgrad.copy_(host[i % 2], non_blocking=True)          # H2D of this step's gradients
        z.step(hyper(t))
        t += 1
        st = z.status()                                       # D2H of the step's result (sync)
    barrier()
    e2e_sec = (time.perf_counter() - w0)
    if world > 1:
        tmax = torch.tensor([e2e_sec], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_sec = float(tmax.item())
    e2e_value = n * e2e_steps / e2e_sec

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0
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
    if world > 1:
        line["phases_ms"] = {k: v / K for k, v in phase_ms.items()}
        wire = (world - 1) / world * n * 2 / 1e9            # GB each way per GPU, per collective
        rs_ms = line["phases_ms"].get("reduce_scatter+norm", line["phases_ms"].get("reduce_scatter"))
        ag_ms = line["phases_ms"].get("update+all_gather", line["phases_ms"].get("all_gather"))
        line["nvlink"] = {"mode": ("peer kernels, NVSwitch multicast" if getattr(z, "uses_multicast", False)
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
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
