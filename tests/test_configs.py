"""The benchmark configurations as parity cases (GPU): full-size single steps against the oracle,
the 100-step mixed-precision trajectory, and the dynamic loss-scale / skip-step sequence."""
import math

import numpy as np
import pytest
import torch

from anni_b200.capi import DT_BF16, DT_F32
from anni_b200.engine import LM_SHAPES, OptStep, lm_segments
from anni_b200 import schedule
from parity_util import (bf16_bits_from_f32, bf16_to_f32, check_step, check_step_chunked, device_inputs,
                         f32_ulp_dist, make_inputs, to_dev, to_host)

pytestmark = pytest.mark.gpu


def test_config1_full_size_single_step(oracle):
    """Configuration 1 at full size: 184,676,352 fp32 parameters in the reference's 147 tensors,
    weights N(0,0.02), fp32 gradients N(0,1e-3) with 0.1 % x100, m ~ N(0,1e-4), v = |N(0,1e-6)|,
    lr 3e-4, betas 0.9/0.95, eps 1e-8, wd 0.1 on matrices, clip 1.0 (active: norm ~ 45), t = 1000,
    seed 0, exact-update mode.

    (a) As configured.  The clip factor comes from a norm summed in another order than the
    oracle's, so it differs in its last double bits (~1e-13); where beta1*m and (1-beta1)*g nearly
    cancel that shows as more than one ulp OF THE RESULT, so the first moment is held to one ulp
    of the larger operand; v (no cancellation) to one ulp flat.
    (b) Same inputs with the oracle's clip factor handed in as grad_scale (clipping off): the
    multiplier is then bit-identical and so must be m and v.  Master in both: within one ulp of the
    larger of |p_old|, |p_new| everywhere, > 99.99 % bit-identical, > 99.9999 % within one ulp flat."""
    segs = lm_segments(**LM_SHAPES["talk170m"], wd="matrices")
    n = segs.n
    assert n == 184_676_352 and len(segs) == 147
    p, g, m, v = make_inputs(n, seed=0)
    ref = [x.copy() for x in (p, g, m, v)]
    kw = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, seg_off=segs.offsets,
              seg_flags=segs.flag_array, t_before=999, check_finite=True)
    info = oracle.step(*ref, clip=1.0, grad_scale=1.0, **kw)
    assert 40 < info["norm"] < 50 and not info["skipped"]
    eng = OptStep(segs, grad_dtype=DT_F32, state_dtype=DT_F32).allocate()

    def gpu_step(exact=True, **hyper):
        eng.master.copy_(to_dev(p))
        eng.grad.copy_(to_dev(g))
        eng.m.copy_(to_dev(m))
        eng.v.copy_(to_dev(v))
        eng.step(OptStep.hyper(lr=3e-4, t=1000, beta2=0.95, wd=0.1, exact=exact, **hyper))
        st = eng.status()
        assert st.error == 0 and st.skipped == 0
        assert not bool(eng.grad.any())
        return st, to_host(eng.m), to_host(eng.v), to_host(eng.master)

    st, gm, gv, gp = gpu_step(clip=1.0, grad_scale=1.0)
    assert abs(st.norm - info["norm"]) <= 1e-9 * info["norm"]          # far inside the 1e-5 bar
    assert abs(st.eff_scale - info["eff_scale"]) <= 1e-11 * info["eff_scale"]
    tol_m = np.spacing(np.maximum(np.abs(ref[2]), np.float32(0.9) * np.abs(m))).astype(np.float64)
    assert (np.abs(gm.astype(np.float64) - ref[2]) <= tol_m).all()
    tol_p = np.spacing(np.maximum(np.abs(ref[0]), np.abs(p))).astype(np.float64)

    def master_ok(gp):
        # one ulp of the larger of |p_old|, |p_new|: where p_old and the update nearly cancel, the
        # update's own 1e-12 relative error is more than an ulp of the (tiny) result
        return (np.abs(gp.astype(np.float64) - ref[0]) <= tol_p).all()

    dm, dv, dp = f32_ulp_dist(gm, ref[2]), f32_ulp_dist(gv, ref[3]), f32_ulp_dist(gp, ref[0])
    assert dv.max() <= 1 and master_ok(gp)
    assert (dm == 0).mean() > 0.9999 and (dv == 0).mean() > 0.9999 and (dp == 0).mean() > 0.9999
    assert (dp <= 1).mean() > 0.999999
    assert np.array_equal(to_host(eng.twin_bf16), bf16_bits_from_f32(gp))

    st, gm, gv, gp = gpu_step(clip=0.0, grad_scale=info["eff_scale"], check_finite=False)
    assert st.eff_scale == info["eff_scale"]
    assert np.array_equal(gm, ref[2]) and np.array_equal(gv, ref[3])    # bit-identical moments
    dp = f32_ulp_dist(gp, ref[0])
    assert master_ok(gp) and (dp == 0).mean() > 0.9999 and (dp <= 1).mean() > 0.999999

    # (c) the same step in the default (fast) update arithmetic -- the one the benchmark times --
    # held to the stated bar: moments within one ulp, master within 2 ulp of the larger of
    # |p_old|, |p_ref| plus 1e-6 of the update, twins the RNE cast of the GPU master
    st, gm, gv, gp = gpu_step(exact=False, clip=1.0, grad_scale=1.0)
    assert abs(st.norm - info["norm"]) <= 1e-9 * info["norm"]
    stats = check_step_chunked(dict(p=gp, m=gm, v=gv), ref[0], ref[2], ref[3], p, exact_moments=False, m_old=m)
    assert stats["p_exact"] > 0.9          # the bar itself is enforced inside check_step
    assert np.array_equal(to_host(eng.twin_bf16), bf16_bits_from_f32(gp))
    eng.close()


def test_config3_full_size_fast_mode_against_oracle(oracle):
    """Configuration 3 as the benchmark runs it -- 555,762,080 parameters in the reference's 170
    tensors, bf16 gradients N(0,5e-4) with 0.1 % x100, fp32 master, bf16 m/v, bf16 twins, clip 1.0
    (active: norm ~ 39), wd 0.1 on matrices, t = 1000, the default (fast) update arithmetic, one
    fused launch -- compared element by element with the CPU oracle on the same inputs.  Bar:
    norm within 1e-5 relative (here: 1e-9), skip decision equal, v within one bf16 ulp, m within
    one bf16 ulp of the larger operand of its sum, both > 99.9 % identical (the clip factor differs
    in its last double bits), master within 2 ulp of
    the larger of |p_old|, |p_ref| plus 1e-6 of the update, twins bit-exact RNE casts of the GPU
    master, gradients zeroed."""
    segs = lm_segments(**LM_SHAPES["run555m"], wd="matrices")
    n = segs.n
    assert n == 555_762_080 and len(segs) == 170
    p, g, m, v = device_inputs(n, seed=33, grad_dtype=DT_BF16, state_dtype=DT_BF16, grad_std=5e-4)
    ref = [x.copy() for x in (p, g, m, v)]
    info = oracle.step(*ref, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0, grad_scale=1.0,
                       seg_off=segs.offsets, seg_flags=segs.flag_array, t_before=999, check_finite=True)
    assert 30 < info["norm"] < 50 and not info["skipped"] and not ref[1].any()
    eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_BF16).allocate()
    eng.master.copy_(to_dev(p))
    eng.grad.copy_(to_dev(g))
    eng.m.copy_(to_dev(m))
    eng.v.copy_(to_dev(v))
    eng.step(OptStep.hyper(lr=3e-4, t=1000, beta2=0.95, wd=0.1, clip=1.0))
    st = eng.status()
    assert st.error == 0 and st.skipped == 0
    assert abs(st.norm - info["norm"]) <= 1e-9 * info["norm"]
    assert abs(st.eff_scale - info["eff_scale"]) <= 1e-9 * info["eff_scale"]
    assert not bool(eng.grad.any())
    assert torch.equal(eng.twin_bf16, eng.master.to(torch.bfloat16))
    out = dict(p=to_host(eng.master), m=to_host(eng.m), v=to_host(eng.v))
    twin_head = to_host(eng.twin_bf16[:1 << 24])
    eng.close()
    assert np.array_equal(twin_head, bf16_bits_from_f32(out["p"][:1 << 24]))   # numpy's RNE, not torch's
    stats = check_step_chunked(out, ref[0], ref[2], ref[3], p, exact_moments=False, m_old=m)
    assert stats["p_exact"] > 0.9          # the bar itself is enforced inside check_step


def test_config3_full_size_properties():
    """Configuration 3 at full size (555,762,080 parameters, bf16 gradients, bf16 m/v, bf16 twins):
    size-independent properties -- the norm equals an independent float64 reduction, the single
    launch and the three-launch form give identical bits, twins are the RNE cast of the master,
    gradients end zeroed, a second step (now on zero gradients) reports norm 0 and only decays v."""
    segs = lm_segments(**LM_SHAPES["run555m"], wd="matrices")
    n = segs.n
    assert n == 555_762_080 and len(segs) == 170
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    outs = []
    for split in (False, True):
        gen.manual_seed(3)
        eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_BF16).allocate()
        eng.master.normal_(0, 0.02, generator=gen)
        eng.m.copy_(torch.randn(n, device="cuda", generator=gen).mul_(1e-4))
        eng.v.copy_(torch.randn(n, device="cuda", generator=gen).mul_(1e-6).abs_())
        g = torch.randn(n, device="cuda", generator=gen).mul_(5e-4)
        g[torch.rand(n, device="cuda", generator=gen) < 1e-3] *= 100
        eng.grad.copy_(g)
        want_norm = float(eng.grad.double().square().sum().sqrt())
        del g
        hp = OptStep.hyper(lr=3e-4, t=1000, beta2=0.95, wd=0.1, clip=1.0)
        (eng.step_split if split else eng.step)(hp)
        st = eng.status()
        assert st.error == 0 and st.skipped == 0
        assert abs(st.norm - want_norm) <= 1e-9 * want_norm and st.norm > 1.0
        assert not bool(eng.grad.any())
        assert torch.equal(eng.twin_bf16, eng.master.to(torch.bfloat16))          # RNE cast of the master
        outs.append((eng.master.clone(), eng.m.clone(), eng.v.clone()))
        if split:
            v_before = eng.v.clone()
            eng.step(OptStep.hyper(lr=3e-4, t=1001, beta2=0.95, wd=0.1, clip=1.0))   # zero gradients now
            st2 = eng.status()
            assert st2.norm == 0.0 and st2.skipped == 0
            assert bool((eng.v.float() <= v_before.float()).all())                 # v only decays
        eng.close()
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)


def test_config2_hundred_step_trajectory(oracle):
    """Configuration 2 on the reference's unit-test shapes: bf16 gradients pre-multiplied by a
    static loss scale of 1024, fp32 master and moments, bf16 twins, fresh seeded gradients every
    step, cosine LR from 3e-4 over 1000 steps with 100 warm-up, 100 consecutive steps.  Compared
    step-wise: each GPU step starts from the oracle's state of the previous step."""
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    p, _, m, v = make_inputs(n, seed=90)
    m[:] = 0
    v[:] = 0
    eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_F32).allocate()
    rng = np.random.default_rng(91)
    worst = 0
    for t in range(100):
        g = bf16_bits_from_f32((rng.normal(0, 1e-3, n) * 1024).astype(np.float32))
        lr = schedule.lr_at(3e-4, t, 100, 1000, "cosine")
        assert lr == oracle.lr_schedule(3e-4, t, 100, 1000)
        eng.master.copy_(to_dev(p))
        eng.m.copy_(to_dev(m))
        eng.v.copy_(to_dev(v))
        eng.grad.copy_(to_dev(g))
        eng.step(OptStep.hyper(lr=lr, t=t + 1, beta2=0.95, wd=0.1, clip=1.0, grad_scale=1.0 / 1024, exact=True))
        p_old = p.copy()
        info = oracle.step(p, g, m, v, lr=lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0,
                           grad_scale=1.0 / 1024, t_before=t, check_finite=True,
                           seg_off=segs.offsets, seg_flags=segs.flag_array)
        st = eng.status()
        assert st.skipped == 0 and abs(st.norm - info["norm"]) <= 1e-9 * info["norm"]
        out = dict(p=to_host(eng.master), m=to_host(eng.m), v=to_host(eng.v))
        check_step(out, p, m, v, p_old, exact_moments=not info["norm"] > 1.0)
        worst = max(worst, int(f32_ulp_dist(out["p"], p).max()))
        assert np.array_equal(to_host(eng.twin_bf16), bf16_bits_from_f32(out["p"]))
    assert worst <= 1
    eng.close()


def test_config5_dynamic_loss_scale_and_skip_sequence(oracle):
    """Configuration 5 in small: dynamic loss scale starting at 65536, x2 after 200 clean steps
    (here: 5, to see growth in a short run), /2 on overflow; one gradient tensor gets an inf every
    7th step; e4m3 twins for the block matrices, bf16 twins elsewhere.  The device-resident state
    machine, the skip decisions and the state after 30 steps match the oracle's."""
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin="fp8")
    n = segs.n
    p, _, m, v = make_inputs(n, seed=95, state_dtype=DT_BF16)
    eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_BF16).allocate()
    eng.master.copy_(to_dev(p))
    eng.m.copy_(to_dev(m))
    eng.v.copy_(to_dev(v))
    eng.loss_scale_init(scale=65536.0, growth_interval=5, growth=2.0, backoff=0.5)
    ls = oracle.loss_scaler(scale=65536.0, growth_interval=5)
    rng = np.random.default_rng(96)
    scales, skips = [], []
    for t in range(30):
        base = rng.normal(0, 5e-4, n).astype(np.float32) * np.float32(ls.scale)   # grads carry the current scale
        if t % 7 == 3:
            sl = segs.slice_of(f"blk{t % 2}.w1")
            base[sl.start + 11] = np.inf
        g = bf16_bits_from_f32(base)
        eng.grad.copy_(to_dev(g))
        eng.step(OptStep.hyper(lr=3e-4, t=t + 1, beta2=0.95, wd=0.1, clip=1.0, grad_scale=1.0,
                               dev_loss_scale=True))
        info = oracle.step(p, g, m, v, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0,
                           grad_scale=1.0 / ls.scale, t_before=t, check_finite=True,
                           seg_off=segs.offsets, seg_flags=segs.flag_array)
        oracle.loss_scale_update(ls, info["skipped"])
        st = eng.status()
        assert bool(st.skipped) == info["skipped"], t                      # skip decision bit-exact
        assert st.loss_scale == ls.scale and st.good_steps == ls.good_steps, t
        scales.append(st.loss_scale)
        skips.append(int(st.skipped))
        # keep the two trajectories glued: next step starts from the oracle's state
        eng.master.copy_(to_dev(p))
        eng.m.copy_(to_dev(m))
        eng.v.copy_(to_dev(v))
    grew = sum(b > a for a, b in zip(scales, scales[1:]))
    shrank = sum(b < a for a, b in zip(scales, scales[1:]))
    assert sum(skips) == 4 and grew >= 2 and shrank >= 3 and scales[3] == 32768.0
    # after the last clean step the twins describe the GPU master (fp8 per tensor, bf16 elsewhere)
    g = bf16_bits_from_f32(rng.normal(0, 5e-4, n).astype(np.float32) * np.float32(ls.scale))
    eng.grad.copy_(to_dev(g))
    eng.step(OptStep.hyper(lr=3e-4, t=31, beta2=0.95, wd=0.1, clip=1.0, grad_scale=1.0, dev_loss_scale=True))
    gp = to_host(eng.master)
    t8, t16, sc = to_host(eng.twin_fp8), to_host(eng.twin_bf16), eng.scale_tensor().cpu().numpy()
    from anni_b200.capi import SEG_TWIN_FP8
    off = segs.offsets
    for i in range(len(segs)):
        sl = slice(int(off[i]), int(off[i + 1]))
        if segs.flags[i] & SEG_TWIN_FP8:
            amax, scale, q = oracle.fp8_quant(gp[sl])
            assert np.float32(sc[i]) == np.float32(scale) and np.array_equal(t8[sl], q)
        else:
            assert np.array_equal(t16[sl], bf16_bits_from_f32(gp[sl]))
    eng.close()


def test_config2_full_size_two_steps_with_static_loss_scale(oracle):
    """Configuration 2 at its own size: the 184,676,352-parameter shapes, bf16 gradients that carry
    a static loss scale of 1024 (grad_scale = 1/1024), fp32 master and moments, bf16 twins, LR from
    the warm-up / cosine schedule, the default (fast) update arithmetic.  Two consecutive steps
    with fresh gradients; after each, the device state against the oracle's step from the same
    previous state (the device state is then carried on, so the second step starts from what the
    first one really left)."""
    segs = lm_segments(**LM_SHAPES["talk170m"], wd="matrices")
    n = segs.n
    p, g, m, v = device_inputs(n, seed=21, grad_dtype=DT_BF16, state_dtype=DT_F32)
    eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_F32).allocate()
    eng.master.copy_(to_dev(p))
    eng.m.copy_(to_dev(m))
    eng.v.copy_(to_dev(v))
    for t in (150, 151):
        # gradients as the backward pass leaves them: multiplied by the loss scale, rounded to bf16
        gs = to_host((to_dev(g).float() * (1024.0 if t == 150 else 768.0)).to(torch.bfloat16))
        lr = schedule.lr_at(3e-4, t, 100, 1000, "cosine")
        eng.grad.copy_(to_dev(gs))
        eng.step(OptStep.hyper(lr=lr, t=t + 1, beta2=0.95, wd=0.1, clip=1.0, grad_scale=1.0 / 1024))
        st = eng.status()
        ref = [x.copy() for x in (p, gs, m, v)]
        info = oracle.step(*ref, lr=lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0,
                           grad_scale=1.0 / 1024, t_before=t, check_finite=True,
                           seg_off=segs.offsets, seg_flags=segs.flag_array)
        assert st.error == 0 and st.skipped == 0 and not info["skipped"]
        assert abs(st.norm - info["norm"]) <= 1e-9 * info["norm"] and st.norm > 1.0
        out = dict(p=to_host(eng.master), m=to_host(eng.m), v=to_host(eng.v))
        check_step_chunked(out, ref[0], ref[2], ref[3], p, exact_moments=False, m_old=m)
        assert torch.equal(eng.twin_bf16, eng.master.to(torch.bfloat16))
        assert not bool(eng.grad.any())
        p, m, v = out["p"], out["m"], out["v"]          # carry the DEVICE state on
    eng.close()


def test_config5_full_size_fp8_twins_and_skip(oracle):
    """Configuration 5 at its own size: 555,762,080 parameters, bf16 gradients carrying the dynamic
    loss scale (65536), bf16 m/v, e4m3 twins with a per-tensor scale for the block matrices and bf16
    twins elsewhere, one launch per step.  Step 1 is clean: state against the oracle, every e4m3
    tensor against the oracle's quantiser applied to the GPU master (scale and codes bit for bit),
    bf16 twins the RNE cast.  Step 2 carries an inf in one tensor: skipped, loss scale halved,
    master, moments and twins untouched, gradients zeroed."""
    segs = lm_segments(**LM_SHAPES["run555m"], wd="matrices", twin="fp8")
    n = segs.n
    p, g, m, v = device_inputs(n, seed=55, grad_dtype=DT_BF16, state_dtype=DT_BF16, grad_std=5e-4)
    gs = to_host((to_dev(g).float() * 65536.0).to(torch.bfloat16))
    del g
    eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_BF16).allocate()
    eng.master.copy_(to_dev(p))
    eng.m.copy_(to_dev(m))
    eng.v.copy_(to_dev(v))
    eng.grad.copy_(to_dev(gs))
    eng.loss_scale_init(scale=65536.0, growth_interval=200)
    hp = OptStep.hyper(lr=3e-4, t=1000, beta2=0.95, wd=0.1, clip=1.0, grad_scale=1.0, dev_loss_scale=True)
    eng.step(hp)
    st = eng.status()
    ref = [x.copy() for x in (p, gs, m, v)]
    info = oracle.step(*ref, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0,
                       grad_scale=1.0 / 65536.0, t_before=999, check_finite=True,
                       seg_off=segs.offsets, seg_flags=segs.flag_array)
    assert st.error == 0 and st.skipped == 0 and not info["skipped"]
    assert abs(st.norm - info["norm"]) <= 1e-9 * info["norm"] and st.loss_scale == 65536.0 and st.good_steps == 1
    out = dict(p=to_host(eng.master), m=to_host(eng.m), v=to_host(eng.v))
    check_step_chunked(out, ref[0], ref[2], ref[3], p, exact_moments=False, m_old=m)
    del ref
    t8, t16, sc = to_host(eng.twin_fp8), to_host(eng.twin_bf16), eng.scale_tensor().cpu().numpy()
    from anni_b200.capi import SEG_TWIN_FP8
    off = segs.offsets
    n8 = 0
    for i in range(len(segs)):
        sl = slice(int(off[i]), int(off[i + 1]))
        if segs.flags[i] & SEG_TWIN_FP8:
            amax, scale, q = oracle.fp8_quant(out["p"][sl])
            assert np.float32(sc[i]) == np.float32(scale), segs.names[i]
            assert np.array_equal(t8[sl], q), segs.names[i]
            n8 += 1
        else:
            assert np.array_equal(t16[sl], bf16_bits_from_f32(out["p"][sl])), segs.names[i]
    assert n8 == 6 * 14
    # step 2: one tensor's gradient holds an inf
    eng.grad.copy_(to_dev(gs))
    eng.grad[segs.slice_of("blk7.w1").start + 12345] = float("inf")
    before = [x.clone() for x in (eng.master, eng.m, eng.v, eng.twin_fp8, eng.twin_bf16)]
    eng.step(OptStep.hyper(lr=3e-4, t=1001, beta2=0.95, wd=0.1, clip=1.0, grad_scale=1.0, dev_loss_scale=True))
    st = eng.status()
    assert st.error == 0 and st.skipped == 1 and st.loss_scale == 32768.0 and st.good_steps == 0
    for a, b in zip(before, (eng.master, eng.m, eng.v, eng.twin_fp8, eng.twin_bf16)):
        assert torch.equal(a, b)
    assert not bool(eng.grad.any())
    eng.close()
