"""ZeRO-1 on real GPUs (needs at least two): NCCL reduce-scatter / all-reduce / all-gather around
the split kernels, against the single-process oracle on the reduced gradients."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from anni_b200.capi import SEG_TWIN_FP8
from anni_b200.engine import LM_SHAPES, lm_segments
from parity_util import bf16_bits_from_f32, bf16_to_f32, check_step

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _world():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 0


@pytest.mark.parametrize("mode", ["mc", "peer", "nccl"])
@pytest.mark.parametrize("twin,state", [("bf16", "f32"), ("bf16", "bf16"), ("fp8", "f32")])
def test_zero1_matches_oracle_on_reduced_gradients(oracle, tmp_path, twin, state, mode):
    """mc: reduce-scatter and all-gather fused into the kernels through NVSwitch multicast
    (multimem.ld_reduce / multimem.st); peer: the same with plain peer loads / stores;
    nccl: the same step around NCCL reduce-scatter / all-gather."""
    world = _world()
    if world < 2:
        pytest.skip("needs at least two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ANNI_TEST_MODE=mode)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300),
           os.path.join(ROOT, "tests", "zero1_gpu_worker.py"), str(tmp_path), twin, state]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-3000:]
    z = np.load(tmp_path / f"zero1_gpu_{twin}_{state}.npz")
    assert int(z["peer"]) == int(mode != "nccl")
    if mode != "mc":
        assert int(z["multicast"]) == 0
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin=twin)
    n = segs.n
    rng = np.random.default_rng(321)
    p = rng.normal(0, 0.02, n).astype(np.float32)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    if state == "bf16":
        m, v = bf16_bits_from_f32(m), bf16_bits_from_f32(v)
    p0 = p.copy()
    infos = []
    for step in range(3):
        base = rng.normal(0, 1e-3, n).astype(np.float32)
        if step == 2:
            base[n - 7] = np.inf
        g = oracle.bf16_rne(base)
        infos.append(oracle.step(p, g, m, v, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0,
                                 grad_scale=1.0, t_before=step, check_finite=True,
                                 seg_off=segs.offsets, seg_flags=segs.flag_array))
    stats = z["stats"]                                       # [rank, step, (norm, skipped, error)]
    assert stats.shape[0] == int(z["world"])
    for r in range(stats.shape[0]):                          # every rank took the same decisions
        assert stats[r, :, 1].tolist() == [0.0, 0.0, 1.0] and not stats[r, :, 2].any()
        for s in range(2):
            assert abs(stats[r, s, 0] - infos[s]["norm"]) <= 1e-10 * infos[s]["norm"]
        assert not math.isfinite(stats[r, 2, 0])
    out = dict(p=z["p"], m=z["m"], v=z["v"])
    # two updates from p0: per-step bar applied to the pair (moments <= 1 ulp, master <= 2 ulp + 1e-6 |dp|)
    if state == "bf16":
        assert np.abs(z["m"].astype(np.int64) - m.astype(np.int64)).max() <= 1
        assert np.abs(z["v"].astype(np.int64) - v.astype(np.int64)).max() <= 1
        out["m"], out["v"] = bf16_to_f32(z["m"]), bf16_to_f32(z["v"])
        m, v = bf16_to_f32(m), bf16_to_f32(v)
        dp = np.abs(z["p"].astype(np.float64) - p)
        assert (dp <= 4 * np.spacing(np.abs(p)) + 4e-6 * np.abs(p0 - p)).all()
    else:
        check_step(out, p, m, v, p0, exact_moments=False)
    off = segs.offsets
    for i in range(len(segs)):
        sl = slice(int(off[i]), int(off[i + 1]))
        if segs.flags[i] & SEG_TWIN_FP8:                     # per-tensor scale needs the amax all-reduce
            amax, scale, q = oracle.fp8_quant(z["p"][sl])
            assert np.float32(z["scale"][i]) == np.float32(scale)
            assert np.array_equal(z["twin8"][sl], q)
        else:
            assert np.array_equal(z["twin"][sl], bf16_bits_from_f32(z["p"][sl]))
