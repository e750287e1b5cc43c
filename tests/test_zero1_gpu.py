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


@pytest.mark.parametrize("mode", ["mc", "peer", "copy", "nccl", "peer_py", "nccl_py"])
@pytest.mark.parametrize("twin,state", [("bf16", "f32"), ("bf16", "bf16"), ("fp8", "f32")])
def test_zero1_matches_oracle_on_reduced_gradients(oracle, tmp_path, twin, state, mode):
    """mc: reduce-scatter and all-gather fused into the kernels through NVSwitch multicast
    (multimem.ld_reduce / multimem.st); peer: the same with plain peer loads / stores;
    copy: copy engines pull the gradient shards and push the twins, the kernels work on local memory;
    nccl: the same step around NCCL reduce-scatter / all-gather.  mc, peer and nccl run the step
    sequence inside the library (anni_zero1_step, with a communicator of its own); the _py variants
    run the same sequence from Python over torch.distributed.  In every mode the gradients are
    accumulated into the arenas, which the step must therefore leave zeroed."""
    world = _world()
    if world < 2:
        pytest.skip("needs at least two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ANNI_TEST_MODE=mode.split("_")[0],
               ANNI_B200_ZERO1_DRIVER="py" if mode.endswith("_py") else "c")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300),
           os.path.join(ROOT, "tests", "zero1_gpu_worker.py"), str(tmp_path), twin, state]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-3000:]
    z = np.load(tmp_path / f"zero1_gpu_{twin}_{state}.npz")
    assert int(z["peer"]) == int(not mode.startswith("nccl"))
    assert str(z["driver"]) == ("python" if mode.endswith("_py") or mode == "copy" else "library")
    assert int(z["ckpt_round_trip"]) == 1
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


@pytest.mark.parametrize("state", ["f32", "bf16"])
def test_checkpoint_out_of_and_into_the_device_state(reflib, tmp_path, state):
    """One rank: two device steps, lm_save_checkpoint's bytes from the device state, the
    reference's loader reads them back, and a fresh engine resumes with identical bits."""
    from anni_b200 import checkpoint
    from anni_b200.capi import DT_BF16, DT_F32
    from anni_b200.engine import OptStep
    from anni_b200.zero1 import Zero1
    dev = torch.device("cuda", 0)
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    sd = DT_BF16 if state == "bf16" else DT_F32
    z = Zero1(segs, grad_dtype=DT_BF16, state_dtype=sd, device=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    z.master.normal_(0, 0.02, generator=gen)
    for step in range(2):
        z.grad_full[:n].copy_(torch.randn(n, device=dev, generator=gen).mul_(1e-3))
        z.step(OptStep.hyper(lr=3e-4, t=step + 1, beta2=0.95, wd=0.1, clip=1.0))
    k = checkpoint.CkptModel()
    k.kind, k.tied, k.d_model, k.n_heads, k.d_ff, k.max_ctx, k.n_blocks = 1, 0, 64, 4, 256, 2048, 2
    k.vocab, k.n_merges, k.merges_word = 300, 40, 40
    merges = np.array([[4 + (2 * i) % 256, 4 + (2 * i + 1) % 256] for i in range(40)], np.int32)
    path = str(tmp_path / "dev.ckpt")
    z.save_checkpoint(path, k, t=2, epoch=0, step=2, merges=merges)
    back = reflib.ckpt_load_full(path, n)
    assert (back["n"], back["t"], back["step"]) == (n, 2, 2)
    assert np.array_equal(back["w"], z.master[:n].cpu().numpy())
    assert np.array_equal(back["m"], z.m[:n].float().cpu().numpy())
    assert np.array_equal(back["v"], z.v[:n].float().cpu().numpy())
    z2 = Zero1(segs, grad_dtype=DT_BF16, state_dtype=sd, device=dev)
    assert z2.load_checkpoint(path) == (2, 0, 2)
    for a, b in ((z.master, z2.master), (z.m, z2.m), (z.v, z2.v), (z.twin_shard, z2.twin_shard)):
        assert torch.equal(a[:n], b[:n])
    # both continue with the same gradients and stay identical
    g = torch.randn(n, device=dev, generator=gen).mul_(1e-3)
    for zz in (z, z2):
        zz.grad_full[:n].copy_(g)
        zz.step(OptStep.hyper(lr=3e-4, t=3, beta2=0.95, wd=0.1, clip=1.0))
    assert torch.equal(z.master[:n], z2.master[:n]) and torch.equal(z.v[:n], z2.v[:n])
    assert torch.equal(z.twin_shard[:n], z2.twin_shard[:n])
    with pytest.raises(ValueError):
        other = Zero1(lm_segments(**dict(LM_SHAPES["tiny"], vocab=260), wd="matrices"),
                      grad_dtype=DT_BF16, state_dtype=sd, device=dev)
        other.load_checkpoint(path)
