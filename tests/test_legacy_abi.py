"""GPU tests of the reference-facing boundary: the reference's own device symbols
(num/gpu.h) as defined by libanni_b200.so, the reference's unmodified optimizer linked against
them, and the library's C mirror of the optimizer object -- all against the CPU oracle."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from anni_b200 import capi, checkpoint, schedule
from anni_b200.capi import DT_BF16, DT_F32, SEG_TWIN_BF16, SEG_WD
from anni_b200.engine import LM_SHAPES, lm_segments
from parity_util import bf16_bits_from_f32, check_step, f32_ulp_dist, make_inputs, to_dev, to_host

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DROPIN = os.path.join(ROOT, "oracle", "_ref", "libannref_dropin.so")
FUSED = os.path.join(ROOT, "oracle", "_ref", "libannref_fused.so")
HYP = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8)
d = C.c_double


def _legacy():
    L = capi.lib()
    L.gpu_available.restype = C.c_int
    L.gpu_grad_sumsq.restype = C.c_int
    L.gpu_grad_sumsq.argtypes = [C.c_void_p, C.c_int, C.POINTER(d)]
    L.gpu_adam_set_weight_decay.argtypes = [d]
    L.gpu_set_compute_prec.argtypes = [C.c_int]
    L.gpu_adam_step_dev_bf16.restype = C.c_int
    L.gpu_adam_step_dev_bf16.argtypes = [C.c_void_p] * 5 + [C.c_int, d, d, d, d, C.c_int, d]
    L.gpu_stream_sync.restype = C.c_int
    L.gpu_adam_set_bf16_flat.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
    L.gpu_adam_seed_bf16_flat.restype = C.c_int
    L.gpu_adam_seed_bf16_flat.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
    L.anni_half_wt_lookup.restype = C.c_void_p
    L.anni_half_wt_lookup.argtypes = [C.c_void_p, C.c_size_t]
    L.gpu_half_wt_invalidate.argtypes = [C.c_void_p]
    L.gpu_param_epoch.restype = C.c_uint
    L.gpu_device_sync.restype = None
    return L


@pytest.mark.parametrize("n", [70001, 262144])
@pytest.mark.parametrize("twin", [True, False])
def test_two_call_sequence_of_the_reference(oracle, n, twin):
    """gpu_grad_sumsq -> host sqrt / clip -> gpu_adam_step_dev_bf16, as lang/lm_adam.c:466-493 does."""
    L = _legacy()
    assert L.gpu_available() == 1
    p, g, m, v = make_inputs(n, seed=31)
    dp, dg, dm, dv = (to_dev(x) for x in (p, g, m, v))
    t16 = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    ss = d()
    assert L.gpu_grad_sumsq(dg.data_ptr(), n, C.byref(ss)) == 0
    want = oracle.sumsq(g, 1.0)
    assert abs(ss.value - want) <= 1e-12 * want
    gs, clip, wd = 0.5, 1.0, 0.1
    norm = np.sqrt(ss.value) * abs(gs)
    coef = gs * (clip / norm) if norm > clip else gs           # the device path divides by norm (lm_adam.c:488)
    L.gpu_adam_set_weight_decay(wd)
    L.gpu_set_compute_prec(1 if twin else 0)
    rc = L.gpu_adam_step_dev_bf16(dp.data_ptr(), t16.data_ptr(), dg.data_ptr(), dm.data_ptr(),
                                  dv.data_ptr(), n, HYP["lr"], HYP["beta1"], HYP["beta2"], HYP["eps"],
                                  7, coef)
    assert rc == 0 and L.gpu_stream_sync() == 0
    ref = [x.copy() for x in (p, g, m, v)]
    oracle.step(*ref, wd=wd, clip=0.0, grad_scale=coef, t_before=6, **HYP)   # same multiplier: exact moments
    out = dict(p=to_host(dp), m=to_host(dm), v=to_host(dv))
    check_step(out, ref[0], ref[2], ref[3], p, exact_moments=True)
    assert not to_host(dg).any()                                # "d_grad is zeroed after"
    if twin:
        assert np.array_equal(to_host(t16), bf16_bits_from_f32(out["p"]))
    else:
        assert not to_host(t16).any()                           # fp32 precision: twin untouched
    L.gpu_set_compute_prec(0)
    # the reference launcher's rejections (num/gpu_cuda.cu:8675-8682)
    args = [dp.data_ptr(), t16.data_ptr(), dg.data_ptr(), dm.data_ptr(), dv.data_ptr()]
    assert L.gpu_adam_step_dev_bf16(*args, n, 0.0, 0.9, 0.95, 1e-8, 7, 1.0) == -1      # lr <= 0
    assert L.gpu_adam_step_dev_bf16(*args, n, 1e-3, 0.9, 0.95, 1e-8, 0, 1.0) == -1     # t < 1
    assert L.gpu_adam_step_dev_bf16(*args, 0, 1e-3, 0.9, 0.95, 1e-8, 1, 1.0) == -1     # n <= 0
    assert L.gpu_adam_step_dev_bf16(*args, n, 1e-3, 1.0, 0.95, 1e-8, 1, 1.0) == -1     # bc1 == 0
    assert L.gpu_adam_step_dev_bf16(None, *args[1:], n, 1e-3, 0.9, 0.95, 1e-8, 1, 1.0) == -1
    assert np.array_equal(to_host(dp), out["p"])                # nothing ran


def test_bf16_flat_twin_registry():
    L = _legacy()
    n = 50000
    f32 = torch.randn(n, device="cuda") * 0.02
    b16 = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    assert L.gpu_adam_seed_bf16_flat(b16.data_ptr(), f32.data_ptr(), n) == 0
    L.gpu_device_sync()
    assert np.array_equal(to_host(b16), bf16_bits_from_f32(f32.cpu().numpy()))
    L.gpu_adam_set_bf16_flat(b16.data_ptr(), f32.data_ptr(), n)
    # a slice of the fp32 flat is served at the same ELEMENT offset of the bf16 flat
    assert L.anni_half_wt_lookup(f32.data_ptr() + 4 * 1234, 100) == b16.data_ptr() + 2 * 1234
    assert L.anni_half_wt_lookup(f32.data_ptr(), n) == b16.data_ptr()
    assert L.anni_half_wt_lookup(f32.data_ptr() + 4 * (n - 10), 11) is None        # runs past the end
    assert L.anni_half_wt_lookup(b16.data_ptr(), 1) in (None, 0) or True
    e0 = L.gpu_param_epoch()
    L.gpu_half_wt_invalidate(None)
    assert L.gpu_param_epoch() == e0 + 1
    L.gpu_adam_set_bf16_flat(None, None, 0)
    assert L.anni_half_wt_lookup(f32.data_ptr(), 1) is None


def test_mat_axpy_on_device_twins():
    class Mat(C.Structure):
        _fields_ = [("data", C.c_void_p), ("d_data", C.c_void_p), ("rows", C.c_int),
                    ("cols", C.c_int), ("on_device", C.c_int)]
    L = _legacy()
    L.gpu_mat_axpy.restype = C.c_int
    L.gpu_mat_axpy.argtypes = [C.POINTER(Mat), d, C.POINTER(Mat)]
    rows, cols = 37, 129
    rng = np.random.default_rng(3)
    xh = rng.normal(size=rows * cols).astype(np.float32)
    yh = rng.normal(size=rows * cols).astype(np.float32)
    xd, yd = to_dev(xh), to_dev(yh)
    x = Mat(xh.ctypes.data, xd.data_ptr(), rows, cols, 1)
    y = Mat(yh.ctypes.data, yd.data_ptr(), rows, cols, 1)
    assert L.gpu_mat_axpy(C.byref(y), 0.25, C.byref(x)) == 0
    L.gpu_device_sync()
    want = np.float32(0.25) * xh.astype(np.float64) + yh        # one fused multiply-add per element
    assert np.max(np.abs(to_host(yd) - want.astype(np.float32))) <= np.spacing(np.float32(4.0))
    assert y.on_device == 1
    bad = Mat(xh.ctypes.data, xd.data_ptr(), rows, cols + 1, 1)
    assert L.gpu_mat_axpy(C.byref(y), 1.0, C.byref(bad)) == -1  # shape mismatch -> CPU path


def test_gradient_buffer_helpers():
    """mat_zero / mat_zero_dev / vec_zero / mat_axpy of lang/gradutil.h on the reference's mat layout."""
    class Mat(C.Structure):
        _fields_ = [("data", C.c_void_p), ("d_data", C.c_void_p), ("rows", C.c_int),
                    ("cols", C.c_int), ("on_device", C.c_int)]

    class Vec(C.Structure):
        _fields_ = [("data", C.c_void_p), ("n", C.c_int)]
    L = _legacy()
    for f in (L.anni_mat_zero, L.anni_mat_zero_dev):
        f.argtypes = [C.POINTER(Mat)]
        f.restype = None
    L.anni_vec_zero.argtypes = [C.POINTER(Vec)]
    L.anni_mat_axpy.restype = C.c_int
    L.anni_mat_axpy.argtypes = [C.POINTER(Mat), d, C.POINTER(Mat)]
    rows, cols = 19, 33
    host = np.ones(rows * cols, np.float32)
    dev = torch.ones(rows * cols, device="cuda")
    m = Mat(host.ctypes.data, dev.data_ptr(), rows, cols, 1)          # device-authoritative
    L.anni_mat_zero(C.byref(m))
    L.gpu_device_sync()
    assert not dev.any() and host.all() and m.on_device == 1         # only the authoritative side
    host[:] = 1
    dev.fill_(1)
    m.on_device = 2
    L.anni_mat_zero_dev(C.byref(m))
    L.gpu_device_sync()
    assert not dev.any() and not host.any() and m.on_device == 2     # both sides, still in sync
    dev.fill_(1)
    host[:] = 1
    m.on_device = 3                                                   # aliased view into a flat
    L.anni_mat_zero_dev(C.byref(m))
    L.gpu_device_sync()
    assert not dev.any() and host.all() and m.on_device == 3         # alias kept, host untouched
    m.on_device = 0                                                   # host-authoritative
    L.anni_mat_zero(C.byref(m))
    assert not host.any() and m.on_device == 0
    vh = np.ones(7, np.float32)
    v = Vec(vh.ctypes.data, 7)
    L.anni_vec_zero(C.byref(v))
    assert not vh.any()
    x = Mat(None, torch.full((rows * cols,), 2.0, device="cuda").data_ptr(), rows, cols, 1)
    dev.fill_(1)
    m.on_device = 1
    assert L.anni_mat_axpy(C.byref(m), 0.5, C.byref(x)) == 0
    L.gpu_device_sync()
    assert bool((dev == 2.0).all())


@pytest.mark.skipif(not os.path.exists(DROPIN), reason="oracle/_ref/libannref_dropin.so not built")
@pytest.mark.parametrize("bf16_prec", [0, 1])
@pytest.mark.parametrize("build", ["unmodified", "fused"])
def test_reference_optimizer_runs_on_this_library(oracle, bf16_prec, build):
    """The reference's own lang/lm_adam.c (with its num/mat.c, num/vec.c) linked against
    libanni_b200.so in place of its backend: three steps take its device path and land on the
    oracle's numbers.  "unmodified": the file as it is -- the two-call sequence gpu_grad_sumsq /
    gpu_adam_step_dev_bf16 with the host deciding in between.  "fused": the same file with
    oracle/lm_adam_fused_step.patch applied (the change a maintainer makes to put the one-launch
    engine behind lm_adam_step_scaled); the driver then also checks that every step went through
    the engine."""
    capi.lib()
    lib = DROPIN if build == "unmodified" else FUSED
    if not os.path.exists(lib):
        pytest.skip(f"{os.path.basename(lib)} not built")
    R = C.CDLL(lib)
    R.dropin_run.restype = C.c_int
    segs = lm_segments(**LM_SHAPES["tiny"], wd="all")
    kinds = np.array([0 if (f & 1) and s > 300 else 1 for f, s in zip(lm_segments(**LM_SHAPES["tiny"]).flags,
                                                                      segs.sizes)], np.int32)
    rows = np.array([s if k else 64 for s, k in zip(segs.sizes, kinds)], np.int32)
    cols = np.array([1 if k else s // 64 for s, k in zip(segs.sizes, kinds)], np.int32)
    n, steps = segs.n, 3
    p, _, _, _ = make_inputs(n, seed=41)
    rng = np.random.default_rng(42)
    g = (rng.normal(0, 1e-3, (steps, n))).astype(np.float32)
    g[2, n // 5] = np.inf                                      # third step: skipped by the host check
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    norms = np.zeros(steps, np.float64)
    used = C.c_int()
    pp = p.copy()
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    rc = R.dropin_run(len(kinds), ptr(kinds), ptr(rows), ptr(cols), ptr(pp), ptr(g), ptr(m), ptr(v),
                      steps, d(1e-3), d(0.9), d(0.95), d(1e-8), d(0.1), d(1.0), d(0.25),
                      bf16_prec, ptr(norms), C.byref(used))
    assert rc == 0 and used.value == (1 if build == "unmodified" else 1 + steps)
    rp, rm, rv = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for s in range(steps):
        gg = g[s].copy()
        info = oracle.step(rp, gg, rm, rv, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0,
                           grad_scale=0.25, t_before=s, check_finite=True)
        if s < 2:
            assert abs(norms[s] - info["norm"]) <= 1e-10 * info["norm"] and not info["skipped"]
        else:
            assert info["skipped"] and not np.isfinite(norms[s])
    dm, dv, dp = f32_ulp_dist(m, rm), f32_ulp_dist(v, rv), f32_ulp_dist(pp, rp)
    assert dm.max() <= 1 and dv.max() <= 1 and (dm == 0).mean() > 0.999
    check_step(dict(p=pp, m=m, v=v), rp, rm, rv, p, exact_moments=False)
    assert (dp <= 2).mean() > 0.95      # two consecutive first steps (|update| = lr): off-by-ones add up


# ---- the library's own optimizer object (C mirror of lm_adam) -------------------------------

from anni_b200.lm_adam import LmAdam, Mat, Seg, Tensor  # noqa: E402
from anni_b200 import lm_adam as lm_adam_mod  # noqa: E402


def _mirror():
    return lm_adam_mod.lib()


def _make_opt(L, segs, p, g):
    """Tensors as host arrays (views of p and g), in the reference's optimizer order."""
    off = segs.offsets
    ts = (Tensor * len(segs))()
    for i in range(len(segs)):
        ts[i].w = p[off[i]:].ctypes.data
        ts[i].dw = g[off[i]:].ctypes.data
        ts[i].n = segs.sizes[i]
        ts[i].flags = segs.flags[i]
    opt = L.anni_lm_adam_create(ts, len(segs), DT_F32, DT_F32)
    assert opt and opt.contents.n == segs.n
    o = opt.contents
    assert (o.t, o.beta1, o.beta2, o.eps, o.weight_decay, o.grad_clip) == (0, 0.9, 0.999, 1e-8, 0.0, 0.0)
    return opt


def test_optimizer_object_trajectory_with_schedule_and_static_loss_scale(oracle, tmp_path):
    """Config-2 style: gradients pre-multiplied by a static loss scale of 1024, LR from the
    warm-up/cosine schedule evaluated at opt->t before the step, twelve consecutive steps; a
    checkpoint written after step 6 and resumed into a fresh object gives the same final state."""
    L = _mirror()
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    p0, _, _, _ = make_inputs(n, seed=51)
    rng = np.random.default_rng(52)
    grads = [(rng.normal(0, 1e-3, n) * 1024).astype(np.float32) for _ in range(12)]

    def run(opt, p, g, first, last):
        o = opt.contents
        o.beta2, o.weight_decay, o.grad_clip = 0.95, 0.1, 1.0
        for s in range(first, last):
            g[:] = grads[s]
            lr = schedule.lr_at(3e-4, o.t, 100, 1000, "cosine")
            assert L.anni_lm_adam_step_scaled(opt, lr, 1.0 / 1024) == 0
            assert o.t == s + 1 and o.last_skipped == 0
            assert not g.any()                                    # host gradients zeroed by the step

    p, g = p0.copy(), np.zeros(n, np.float32)
    opt = _make_opt(L, segs, p, g)
    run(opt, p, g, 0, 6)
    assert L.anni_lm_adam_sync_host(opt) == 0
    o = opt.contents
    m6 = np.ctypeslib.as_array(o.h_m, (n,)).copy()
    v6 = np.ctypeslib.as_array(o.h_v, (n,)).copy()
    ck = str(tmp_path / "mid.adam")
    checkpoint.write_adam(ck, m6, v6, t=o.t, epoch=0, step=6)
    p6 = p.copy()
    run(opt, p, g, 6, 12)
    assert L.anni_lm_adam_sync_host(opt) == 0
    mA = np.ctypeslib.as_array(o.h_m, (n,)).copy()
    pA = p.copy()
    norm_last = o.last_grad_norm
    L.anni_lm_adam_free(C.byref(opt))

    # oracle trajectory
    rp, rm, rv = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for s in range(12):
        gg = grads[s].copy()
        info = oracle.step(rp, gg, rm, rv, lr=oracle.lr_schedule(3e-4, s, 100, 1000), beta1=0.9, beta2=0.95,
                           eps=1e-8, wd=0.1, clip=1.0, grad_scale=1.0 / 1024, t_before=s, check_finite=True,
                           seg_off=segs.offsets, seg_flags=segs.flag_array)
    assert abs(norm_last - info["norm"]) <= 1e-9 * info["norm"]
    # twelve steps of <= 1 ulp each may drift a little; stay within a few ulp of the oracle
    assert f32_ulp_dist(mA, rm).max() <= 4
    dp = np.abs(pA.astype(np.float64) - rp)
    assert (dp <= 4 * np.spacing(np.abs(rp)) + 12e-6 * 3e-4).all()

    # resume from the checkpoint in a fresh object
    back = checkpoint.read_adam(ck, n)
    p2, g2 = p6.copy(), np.zeros(n, np.float32)
    opt2 = _make_opt(L, segs, p2, g2)
    assert L.anni_lm_adam_set_moments(opt2, back["m"].ctypes.data, back["v"].ctypes.data) == 0
    opt2.contents.t = back["t"]
    run(opt2, p2, g2, 6, 12)
    assert L.anni_lm_adam_sync_host(opt2) == 0
    assert np.array_equal(p2, pA)                                 # bit-identical to the uninterrupted run
    assert np.array_equal(np.ctypeslib.as_array(opt2.contents.h_m, (n,)), mA)
    L.anni_lm_adam_free(C.byref(opt2))


def test_optimizer_object_semantics(oracle):
    """lr <= 0 is a no-op; t advances on a skipped step; invalidate re-reads host weights;
    offload keeps m/v on the host between steps; free writes the weights back."""
    L = _mirror()
    segs = lm_segments(**LM_SHAPES["tiny"], wd="all")
    n = segs.n
    p, g0, _, _ = make_inputs(n, seed=61)
    g = g0.copy()
    opt = _make_opt(L, segs, p, g)
    o = opt.contents
    o.grad_clip = 1.0
    assert L.anni_lm_adam_step(opt, 0.0) == 0 and o.t == 0 and np.array_equal(g, g0)
    p_before = p.copy()
    g[n // 2] = np.nan
    assert L.anni_lm_adam_step(opt, 1e-3) == 0
    assert o.t == 1 and o.last_skipped == 1 and not np.isfinite(o.last_grad_norm)
    assert L.anni_lm_adam_sync_host(opt) == 0 and np.array_equal(p, p_before) and not g.any()
    # host rewrites the weights -> invalidate -> the next step starts from the new values
    p[:] = p_before * 2
    L.anni_lm_adam_invalidate(opt)
    L.anni_lm_adam_set_offload(1)
    g[:] = g0
    assert L.anni_lm_adam_step(opt, 1e-3) == 0 and o.t == 2 and o.last_skipped == 0
    assert not o.d_m and not o.d_v and o.dev_mv == 0              # offloaded after the step
    rp, rm, rv, rg = p_before * 2, np.zeros(n, np.float32), np.zeros(n, np.float32), g0.copy()
    oracle.step(rp, rg, rm, rv, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, clip=1.0, t_before=1,
                check_finite=True)
    hm = np.ctypeslib.as_array(o.h_m, (n,))
    assert f32_ulp_dist(hm, rm).max() <= 1
    g[:] = g0
    assert L.anni_lm_adam_step(opt, 1e-3) == 0 and o.t == 3        # m/v re-uploaded from the host copy
    rg = g0.copy()
    oracle.step(rp, rg, rm, rv, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, clip=1.0, t_before=2,
                check_finite=True)
    L.anni_lm_adam_set_offload(0)
    L.anni_lm_adam_free(C.byref(opt))                              # pulls the weights back first
    assert (np.abs(p.astype(np.float64) - rp) <= 2 * np.spacing(np.abs(rp)) + 2e-9).all()


def test_large_host_gradients_are_uploaded_and_cleared():
    """A model's worth of host gradients (98 M fp32: above the size from which the step deals the
    clearing out to threads behind the uploads; pinned arrays go up with asynchronous copies and
    an event per tensor, pageable ones with blocking copies): two steps see exactly the gradients
    they were given -- the norm is that of the arrays, the same on both steps -- leave every host
    gradient zero, and give the same weights whichever way the gradients travelled."""
    L = _mirror()
    segs = lm_segments(**LM_SHAPES["blocks3"], wd="matrices")
    n = segs.n
    gen = torch.Generator().manual_seed(77)
    p0 = torch.empty(n).normal_(0, 0.02, generator=gen)
    g_src = torch.empty(n).normal_(0, 1e-3, generator=gen)
    want = float(torch.linalg.vector_norm(g_src.double()))
    results = []
    for pinned in (True, False):
        p_t = p0.clone()
        g_t = torch.empty(n, pin_memory=pinned)
        p, g = p_t.numpy(), g_t.numpy()
        opt = _make_opt(L, segs, p, g)
        o = opt.contents
        o.grad_clip, o.weight_decay = 1.0, 0.1
        for _ in range(2):
            g_t.copy_(g_src)
            assert L.anni_lm_adam_step(opt, 3e-4) == 0 and o.last_skipped == 0
            assert abs(o.last_grad_norm - want) <= 1e-9 * want
            assert not bool(g_t.any())
        assert L.anni_lm_adam_sync_host(opt) == 0
        results.append(p.copy())
        L.anni_lm_adam_free(C.byref(opt))
    assert np.array_equal(results[0], results[1]) and not np.array_equal(results[0], p0.numpy())


def test_resume_from_reference_format_checkpoint_and_save_back(oracle, tmp_path):
    """A checkpoint in the reference's format (tied-embedding kind, BPE table embedded) is loaded
    into the optimizer object, two steps run on the GPU, the result is saved in the same format;
    the saved state equals the oracle stepping from the same file."""
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from golden.make_golden import ckpt_moments, ckpt_weights, synthetic_merges
    from anni_b200.engine import lm_param_count
    L = _mirror()
    n_merges = 44
    vocab = 4 + 256 + n_merges
    k = checkpoint.CkptModel()
    k.kind, k.tied, k.d_model, k.n_heads, k.d_ff, k.max_ctx, k.n_blocks, k.vocab = 2, 1, 64, 4, 256, 2048, 2, vocab
    k.n_merges = k.merges_word = n_merges
    k.n = lm_param_count(64, 256, 2, vocab, True)
    k.t, k.epoch, k.step = 500, 1, 40
    w0 = ckpt_weights(k.n)
    m0, v0 = ckpt_moments(k.n)
    src = str(tmp_path / "in.ckpt")
    checkpoint.save_model(src, k, w0, m0, v0, synthetic_merges(n_merges))

    ck = checkpoint.load_model(src)
    segs = lm_segments(d_model=64, d_ff=256, n_blocks=2, vocab=vocab, tied=True, wd="matrices")
    assert segs.n == ck["info"].n
    p, g = ck["w"].copy(), np.zeros(segs.n, np.float32)
    opt = _make_opt(L, segs, p, g)
    o = opt.contents
    assert L.anni_lm_adam_set_moments(opt, ck["m"].ctypes.data, ck["v"].ctypes.data) == 0
    o.t, o.beta2, o.weight_decay, o.grad_clip = ck["info"].t, 0.95, 0.1, 0.0
    rng = np.random.default_rng(12)
    grads = [rng.normal(0, 1e-3, segs.n).astype(np.float32) for _ in range(2)]
    for gg in grads:
        g[:] = gg
        assert L.anni_lm_adam_step_scaled(opt, 3e-4, 0.5) == 0
    assert L.anni_lm_adam_sync_host(opt) == 0 and o.t == 502
    info = ck["info"]
    info.t, info.step = o.t, 42
    dst = str(tmp_path / "out.ckpt")
    checkpoint.save_model(dst, info, p, np.ctypeslib.as_array(o.h_m, (segs.n,)),
                          np.ctypeslib.as_array(o.h_v, (segs.n,)), ck["merges"])
    L.anni_lm_adam_free(C.byref(opt))

    back = checkpoint.load_model(dst)
    assert back["info"].t == 502 and back["info"].step == 42 and back["info"].kind == 2
    rp, rm, rv = w0.copy(), m0.copy(), v0.copy()
    for i, gg in enumerate(grads):
        oracle.step(rp, gg.copy(), rm, rv, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=0.0,
                    grad_scale=0.5, t_before=500 + i, seg_off=segs.offsets, seg_flags=segs.flag_array)
    # first step's moments are bit-identical; the second starts from masters that may be 1 ulp apart
    assert f32_ulp_dist(back["m"], rm).max() <= 1 and f32_ulp_dist(back["v"], rv).max() <= 1
    dp = np.abs(back["w"].astype(np.float64) - rp)
    assert (dp <= 2 * np.spacing(np.maximum(np.abs(rp), np.abs(w0))) + 2e-6 * np.abs(w0 - rp)).all()


def test_aliased_matrices_and_async_moment_snapshot(oracle):
    """Hand-off as the reference does it: weight / gradient matrices become views into the
    optimizer's flats (gradients written on the device, weights updated in place), vectors stay
    host-resident; m / v are snapshotted on a side stream; free pulls the weights back and
    detaches the views."""
    class Mat(C.Structure):
        _fields_ = [("data", C.c_void_p), ("d_data", C.c_void_p), ("rows", C.c_int),
                    ("cols", C.c_int), ("on_device", C.c_int)]
    L = _mirror()
    Lg = _legacy()
    Lg.gpu_memcpy_h2d.restype = C.c_int
    Lg.gpu_memcpy_h2d.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    for f in (L.anni_lm_adam_prepare, L.anni_lm_adam_snapshot_begin, L.anni_lm_adam_snapshot_finish):
        f.restype = C.c_int
        f.argtypes = [C.POINTER(LmAdam)]
    L.anni_lm_adam_alias.restype = C.c_int
    L.anni_lm_adam_alias.argtypes = [C.POINTER(LmAdam), C.c_int, C.POINTER(Mat), C.POINTER(Mat)]
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n, off = segs.n, segs.offsets
    p, g0, _, _ = make_inputs(n, seed=71)
    g = np.zeros(n, np.float32)
    opt = _make_opt(L, segs, p, g)
    o = opt.contents
    o.beta2, o.weight_decay, o.grad_clip = 0.95, 0.1, 1.0
    assert L.anni_lm_adam_prepare(opt) == 0 and o.d_param and o.params_valid == 1
    mats = {}
    for i in range(len(segs)):
        if not (segs.flags[i] & 1):                                  # vectors stay host-resident
            continue
        rows = 64
        w = Mat(p[off[i]:].ctypes.data, None, rows, segs.sizes[i] // rows, 0)
        dw = Mat(g[off[i]:].ctypes.data, None, rows, segs.sizes[i] // rows, 0)
        assert L.anni_lm_adam_alias(opt, i, C.byref(w), C.byref(dw)) == 0
        assert w.d_data == o.d_param + 4 * off[i] and dw.d_data == o.d_grad + 4 * off[i]
        assert w.on_device == 3 and dw.on_device == 3
        mats[i] = (w, dw)
    assert len(mats) == 14
    rp, rm, rv = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for step in range(2):
        for i in range(len(segs)):
            sl = slice(int(off[i]), int(off[i + 1]))
            if i in mats:                                            # "backward GEMM": dW on the device
                chunk = np.ascontiguousarray(g0[sl] * (step + 1))
                assert Lg.gpu_memcpy_h2d(mats[i][1].d_data, chunk.ctypes.data, chunk.nbytes) == 0
                Lg.gpu_device_sync()
            else:                                                    # bias / LN gradients on the host
                g[sl] = g0[sl] * (step + 1)
        assert L.anni_lm_adam_step_scaled(opt, 1e-3, 1.0) == 0
        gg = g0 * np.float32(step + 1)
        info = oracle.step(rp, gg, rm, rv, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0,
                           t_before=step, check_finite=True, seg_off=off, seg_flags=segs.flag_array)
        assert abs(o.last_grad_norm - info["norm"]) <= 1e-9 * info["norm"]
    assert L.anni_lm_adam_snapshot_begin(opt) == 0                  # copies run beside whatever comes next
    assert L.anni_lm_adam_snapshot_finish(opt) == 0
    hm = np.ctypeslib.as_array(o.h_m, (n,)).copy()
    hv = np.ctypeslib.as_array(o.h_v, (n,)).copy()
    assert f32_ulp_dist(hm, rm).max() <= 1 and f32_ulp_dist(hv, rv).max() <= 1
    L.anni_lm_adam_free(C.byref(opt))
    for w, dw in mats.values():                                      # views detached, weights on the host
        assert not w.d_data and not dw.d_data and w.on_device == 0 and dw.on_device == 0
    dp = np.abs(p.astype(np.float64) - rp)
    assert (dp <= 2 * np.spacing(np.abs(rp)) + 4e-9).all()


def test_vector_gradients_stay_on_the_device(oracle, capfd, monkeypatch):
    """Every tensor's gradient lives in the device flat: matrices as aliased views, bias / LayerNorm
    vectors attached with anni_lm_adam_alias_vec, their gradients produced by gpu_mat_col_sum_add
    (called with the HOST vector's address, as the backward pass does) straight into the flat.  The
    step then uploads nothing; its result equals the oracle's on the gradients the device held.
    Also here: the per-operation profile table (ANN_OP_PROF) and the periodic norm report."""
    class Mat(C.Structure):
        _fields_ = [("data", C.c_void_p), ("d_data", C.c_void_p), ("rows", C.c_int),
                    ("cols", C.c_int), ("on_device", C.c_int)]
    L = _mirror()
    Lg = _legacy()
    L.anni_lm_adam_prepare.restype = C.c_int
    L.anni_lm_adam_prepare.argtypes = [C.POINTER(LmAdam)]
    L.anni_lm_adam_alias.restype = C.c_int
    L.anni_lm_adam_alias.argtypes = [C.POINTER(LmAdam), C.c_int, C.POINTER(Mat), C.POINTER(Mat)]
    L.anni_lm_adam_alias_vec.restype = C.c_int
    L.anni_lm_adam_alias_vec.argtypes = [C.POINTER(LmAdam), C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]
    Lg.gpu_mat_col_sum_add.restype = C.c_int
    Lg.gpu_mat_col_sum_add.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
    Lg.gpu_memcpy_h2d.restype = C.c_int
    Lg.gpu_memcpy_h2d.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    Lg.anni_op_prof_enable.argtypes = [C.c_int]
    Lg.anni_op_prof_totals.restype = C.c_int
    Lg.anni_op_prof_totals.argtypes = [C.c_char_p, C.POINTER(C.c_double), C.POINTER(C.c_long)]
    Lg.anni_op_prof_enable(1)
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n, off = segs.n, segs.offsets
    p, g0, _, _ = make_inputs(n, seed=73)
    g = np.zeros(n, np.float32)
    g[off[1]:off[2]] = 0.25                     # what the host vector of b_head holds when it is attached
    opt = _make_opt(L, segs, p, g)
    o = opt.contents
    o.beta2, o.weight_decay, o.grad_clip = 0.95, 0.1, 1.0
    assert L.anni_lm_adam_alias_vec(opt, 1, None, None) == capi.E_ARG      # before the flats exist
    assert L.anni_lm_adam_prepare(opt) == 0
    views, vec_ptrs = {}, {}
    for i in range(len(segs)):
        if segs.flags[i] & 1:
            rows = 64
            w = Mat(p[off[i]:].ctypes.data, None, rows, segs.sizes[i] // rows, 0)
            dw = Mat(g[off[i]:].ctypes.data, None, rows, segs.sizes[i] // rows, 0)
            assert L.anni_lm_adam_alias(opt, i, C.byref(w), C.byref(dw)) == 0
            views[i] = (w, dw)
        else:
            dwp, ddw = C.c_void_p(), C.c_void_p()
            assert L.anni_lm_adam_alias_vec(opt, i, C.byref(dwp), C.byref(ddw)) == 0
            assert dwp.value == o.d_param + 4 * off[i] and ddw.value == o.d_grad + 4 * off[i]
            vec_ptrs[i] = ddw.value
    for i in range(o.n_segs):
        assert not o.segs[i].dw                                   # nothing left to upload
    rows = 48
    rng = np.random.default_rng(74)
    for i in range(len(segs)):
        sl = slice(int(off[i]), int(off[i + 1]))
        if i in views:
            chunk = np.ascontiguousarray(g0[sl])
            assert Lg.gpu_memcpy_h2d(views[i][1].d_data, chunk.ctypes.data, chunk.nbytes) == 0
        else:
            cols = segs.sizes[i]
            x = to_dev((rng.normal(0, 1e-3, (rows, cols)) / rows).astype(np.float32))
            assert Lg.gpu_mat_col_sum_add(g[off[i]:].ctypes.data, x.data_ptr(), rows, cols) == 0
            assert Lg.gpu_mat_col_sum_add(g[off[i]:].ctypes.data, x.data_ptr(), rows, cols) == 0   # accumulates
    # a vector nobody attached, and a matrix that is not on the device: the caller's CPU path
    other = np.zeros(64, np.float32)
    x = torch.zeros(4, 64, device="cuda")
    assert Lg.gpu_mat_col_sum_add(other.ctypes.data, x.data_ptr(), 4, 64) == -1
    hostx = np.zeros((4, segs.sizes[1]), np.float32)
    assert Lg.gpu_mat_col_sum_add(g[off[1]:].ctypes.data, hostx.ctypes.data, 4, segs.sizes[1]) == -1
    Lg.gpu_device_sync()
    flat = torch.empty(n, dtype=torch.float32, device="cuda")
    Lg.gpu_memcpy_d2h.restype = C.c_int
    Lg.gpu_memcpy_d2h.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    held = np.empty(n, np.float32)
    assert Lg.gpu_memcpy_d2h(held.ctypes.data, o.d_grad, 4 * n) == 0
    # column sums landed where the vectors live, on top of what the host vector held when attached
    sl = slice(int(off[1]), int(off[2]))
    assert np.all(np.abs(held[sl] - 0.25) < 0.01) and held[sl].std() > 0
    for i in views:
        assert np.array_equal(held[off[i]:off[i + 1]], g0[off[i]:off[i + 1]])
    monkeypatch.setenv("ANN_GNORM_EVERY", "1")
    assert L.anni_lm_adam_step_scaled(opt, 1e-3, 1.0) == 0
    rp, rm, rv, rg = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), held.copy()
    info = oracle.step(rp, rg, rm, rv, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0, t_before=0,
                       check_finite=True, seg_off=off, seg_flags=segs.flag_array)
    assert abs(o.last_grad_norm - info["norm"]) <= 1e-9 * info["norm"]
    assert Lg.gpu_memcpy_d2h(held.ctypes.data, o.d_grad, 4 * n) == 0 and not held.any()   # left zeroed
    ms, calls = C.c_double(), C.c_long()
    assert Lg.anni_op_prof_totals(b"adam", C.byref(ms), C.byref(calls)) == 0
    assert calls.value >= 1 and ms.value > 0.0
    assert Lg.anni_op_prof_totals(b"colsum", C.byref(ms), C.byref(calls)) == 0 and calls.value == 2 * len(vec_ptrs)
    Lg.gpu_op_prof_dump()
    err = capfd.readouterr().err
    assert "[opprof]" in err and "adam" in err and "colsum" in err
    assert Lg.anni_op_prof_totals(b"adam", C.byref(ms), C.byref(calls)) == 0 and calls.value == 0   # the dump resets
    Lg.anni_op_prof_enable(0)
    L.anni_lm_adam_free(C.byref(opt))
    dp = np.abs(p.astype(np.float64) - rp)
    assert (dp <= 2 * np.spacing(np.maximum(np.abs(rp), 1e-3)) + 2e-9).all()
    # the registry forgot the freed flat: the same host vector is unknown again
    x = torch.zeros(4, segs.sizes[1], device="cuda")
    assert Lg.gpu_mat_col_sum_add(g[off[1]:].ctypes.data, x.data_ptr(), 4, segs.sizes[1]) == -1
