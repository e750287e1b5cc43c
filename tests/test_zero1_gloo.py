"""ZeRO-1 host logic on CPU: two gloo ranks against the single-process oracle on the reduced
gradients.  Covers shard geometry, the collective sequence, the global skip decision."""
import math
import os
import subprocess
import sys

import numpy as np

from anni_b200.capi import DT_F32
from anni_b200.engine import LM_SHAPES, lm_segments
from anni_b200.zero1 import shard_geometry

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_geometry():
    per, own = shard_geometry(138156, 2)
    assert per % 4096 == 0 and per * 2 >= 138156
    assert own[0] == (0, per) and own[1] == (per, 138156 - per)
    per8, own8 = shard_geometry(555_762_080, 8)
    assert sum(n for _, n in own8) == 555_762_080 and all(n > 0 for _, n in own8)
    per_small, own_small = shard_geometry(5000, 8)          # more ranks than 4096-element shards
    assert sum(n for _, n in own_small) == 5000 and own_small[-1][1] == 0
    _, own1 = shard_geometry(100, 1)
    assert own1 == [(0, 100)]


def test_two_gloo_ranks_match_single_process_oracle(oracle, reflib, tmp_path):
    port = 29500 + (os.getpid() % 400)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "zero1_cpu_worker.py"), str(tmp_path)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    z = np.load(tmp_path / "zero1_out.npz")
    assert int(z["world"]) == 2

    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    rng = np.random.default_rng(123)
    p = rng.normal(0, 0.02, n).astype(np.float32)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    norms, skipped = [], []
    for step in range(3):
        base = rng.normal(0, 1e-3, n).astype(np.float32)
        if step == 2:
            base[n // 2] = np.inf
        g = oracle.bf16_rne(base)                            # 0.5 g + 0.5 g is exact in bf16
        info = oracle.step(p, g, m, v, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0,
                           grad_scale=1.0, t_before=step, check_finite=True,
                           seg_off=segs.offsets, seg_flags=segs.flag_array)
        norms.append(info["norm"])
        skipped.append(info["skipped"])
    assert skipped == [False, False, True] and z["skipped"].tolist() == skipped
    for a, b in zip(z["norms"][:2], norms[:2]):
        assert abs(a - b) <= 1e-12 * b                       # two partial sums instead of one
    assert not math.isfinite(float(z["norms"][2]))
    # the clip factor differs in its last bits (sum order) -> at most 1 ulp, almost always 0
    dp = np.abs(z["p"].view(np.int32).astype(np.int64) - p.view(np.int32).astype(np.int64))
    dm = np.abs(z["m"].view(np.int32).astype(np.int64) - m.view(np.int32).astype(np.int64))
    assert dp.max() <= 1 and dm.max() <= 1 and (dp == 0).mean() > 0.999 and (dm == 0).mean() > 0.999
    assert np.array_equal(z["twin"], oracle.bf16_rne(z["p"]))
    # the checkpoint the two ranks wrote together: reloaded shard-wise by a fresh pair of ranks,
    # byte-identical to the single-process writer, and accepted by the reference's own loader
    from anni_b200 import checkpoint
    assert int(z["ckpt_round_trip"]) == 1
    ck = checkpoint.load_model(str(tmp_path / "zero1.ckpt"))
    assert (ck["info"].t, ck["info"].epoch, ck["info"].step, ck["info"].n) == (3, 1, 3, n)
    assert np.array_equal(ck["w"], z["p"]) and np.array_equal(ck["m"], z["m"]) and np.array_equal(ck["v"], z["v"])
    single = str(tmp_path / "single.ckpt")
    checkpoint.save_model(single, ck["info"], z["p"], z["m"], z["v"], ck["merges"])
    assert open(single, "rb").read() == open(tmp_path / "zero1.ckpt", "rb").read()
    back = reflib.ckpt_load_full(str(tmp_path / "zero1.ckpt"), n)
    assert back["t"] == 3 and np.array_equal(back["w"], z["p"]) and np.array_equal(back["v"], z["v"])
