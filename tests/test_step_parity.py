"""GPU parity: the CUDA step (through the C ABI) against the CPU oracle, same seeded inputs."""
import numpy as np
import pytest

from anni_b200.capi import DT_BF16, DT_F32, SEG_TWIN_BF16, SEG_WD
import torch

from anni_b200.engine import OptStep, Segments, lm_segments, LM_SHAPES
from parity_util import (bf16_bits_from_f32, check_step, make_inputs, run_gpu, to_dev, to_host)

pytestmark = pytest.mark.gpu

HYP = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8)


def _oracle_step(oracle, segs, p, g, m, v, **kw):
    a = [x.copy() for x in (p, g, m, v)]
    info = oracle.step(*a, seg_off=segs.offsets if segs is not None else None,
                       seg_flags=segs.flag_array if segs is not None else None, **kw)
    return a, info


@pytest.mark.parametrize("grad_dtype,state_dtype", [(DT_F32, DT_F32), (DT_BF16, DT_F32),
                                                    (DT_BF16, DT_BF16), (DT_F32, DT_BF16)])
@pytest.mark.parametrize("clip", [0.0, 1.0])
@pytest.mark.parametrize("split", [False, True])
def test_tiny_lm_step(oracle, grad_dtype, state_dtype, clip, split):
    """The reference's unit-test LM (138,156 scalars, 27 tensors), wd on matrices only."""
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    p, g, m, v = make_inputs(n, seed=1, grad_dtype=grad_dtype, state_dtype=state_dtype)
    kw = dict(HYP, wd=0.1, clip=clip, grad_scale=1.0, t_before=999)
    (rp, rg, rm, rv), info = _oracle_step(oracle, segs, p, g, m, v, check_finite=True, **kw)
    out = run_gpu(segs, p, g, m, v, dict(HYP, wd=0.1, clip=clip, grad_scale=1.0, t=1000), split=split)
    st = out["status"]
    assert st.error == 0 and st.skipped == 0 and not info["skipped"]
    assert abs(st.norm - info["norm"]) <= 1e-5 * info["norm"] + 1e-300
    clipped = clip > 0 and info["norm"] > clip
    res = check_step(out, rp, rm, rv, p, exact_moments=not clipped)
    assert np.array_equal(out["twin"], bf16_bits_from_f32(out["p"]))      # twin = RNE(GPU master)
    assert not out["g"].any()                                             # grads zeroed by the step
    assert res["p_exact"] > 0.9


def test_all_params_decay_matches_reference_layout(oracle):
    """n_seg = 0: one implicit segment with decay everywhere, the reference kernels' behaviour."""
    n = 70001          # odd size: exercises the element-wise tail
    p, g, m, v = make_inputs(n, seed=2)
    kw = dict(HYP, wd=0.1, clip=1.0, grad_scale=0.5, t_before=0)
    (rp, rg, rm, rv), info = _oracle_step(oracle, None, p, g, m, v, check_finite=True, **kw)
    out = run_gpu(None, p, g, m, v, dict(HYP, wd=0.1, clip=1.0, grad_scale=0.5, t=1), n_arena=n)
    assert abs(out["status"].norm - info["norm"]) <= 1e-5 * info["norm"]
    check_step(out, rp, rm, rv, p, exact_moments=not (info["norm"] > 1.0))
    assert np.array_equal(out["twin"], bf16_bits_from_f32(out["p"]))


def test_unaligned_segment_boundaries(oracle):
    """Tensor sizes that are not multiples of the vector width: boundaries fall inside vectors."""
    segs = Segments()
    for i, sz in enumerate([5, 4099, 1, 2048, 7777, 3, 12289]):
        segs.add(f"t{i}", sz, (SEG_WD if i % 2 == 0 else 0) | SEG_TWIN_BF16)
    n = segs.n
    p, g, m, v = make_inputs(n, seed=3, grad_dtype=DT_BF16)
    kw = dict(HYP, wd=0.1, clip=0.0, grad_scale=1.0 / 1024, t_before=10)
    (rp, rg, rm, rv), info = _oracle_step(oracle, segs, p, g, m, v, check_finite=True, **kw)
    out = run_gpu(segs, p, g, m, v, dict(HYP, wd=0.1, clip=0.0, grad_scale=1.0 / 1024, t=11))
    check_step(out, rp, rm, rv, p, exact_moments=True)
    assert np.array_equal(out["twin"], bf16_bits_from_f32(out["p"]))


@pytest.mark.parametrize("bad", [np.inf, -np.inf, np.nan])
@pytest.mark.parametrize("split", [False, True])
def test_skip_step_on_nonfinite(oracle, bad, split):
    """A single non-finite gradient: parameters, moments and twins untouched, grads zeroed."""
    segs = lm_segments(**LM_SHAPES["tiny"])
    n = segs.n
    p, g, m, v = make_inputs(n, seed=4, grad_dtype=DT_BF16)
    gf = (g.astype(np.uint32) << 16).view(np.float32).copy()
    gf[n // 3] = bad
    g = bf16_bits_from_f32(gf) if not np.isnan(bad) else g.copy()
    if np.isnan(bad):
        g[n // 3] = 0x7fc0
    kw = dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0, t_before=5)
    (rp, rg, rm, rv), info = _oracle_step(oracle, segs, p, g, m, v, check_finite=True, **kw)
    assert info["skipped"]
    out = run_gpu(segs, p, g, m, v, dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0, t=6), split=split)
    assert out["status"].skipped == 1
    assert np.array_equal(out["p"], p) and np.array_equal(out["m"], m) and np.array_equal(out["v"], v)
    assert not out["g"].any() and not out["twin"].any()      # twin buffer never written


@pytest.mark.parametrize("split", [False, True])
def test_fp8_twins_per_tensor_scale(oracle, split):
    """e4m3 twins of the block matrices: amax, scale and codes are those of the oracle's
    restatement of the reference quantiser applied to the GPU master (bit-exact); vectors,
    head and embedding keep bf16 twins."""
    from anni_b200.capi import SEG_TWIN_FP8
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin="fp8")
    n = segs.n
    p, g, m, v = make_inputs(n, seed=5, grad_dtype=DT_BF16)
    p[segs.slice_of("blk0.wq")] *= 37.0            # tensors with different ranges
    p[segs.slice_of("blk1.w2")] *= 1e-3
    kw = dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0, t_before=99)
    (rp, rg, rm, rv), info = _oracle_step(oracle, segs, p, g, m, v, check_finite=True, **kw)
    out = run_gpu(segs, p, g, m, v, dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0, t=100), split=split)
    check_step(out, rp, rm, rv, p, exact_moments=not info["norm"] > 1.0)
    off = segs.offsets
    n_fp8 = 0
    for i, name in enumerate(segs.names):
        sl = slice(int(off[i]), int(off[i + 1]))
        if segs.flags[i] & SEG_TWIN_FP8:
            amax, scale, q = oracle.fp8_quant(out["p"][sl])
            assert np.float32(out["amax"][i]) == np.float32(amax), name
            assert np.float32(out["scale"][i]) == np.float32(scale), name
            assert np.array_equal(out["twin8"][sl], q), name
            assert not out["twin"][sl].any()
            n_fp8 += 1
        else:
            assert np.array_equal(out["twin"][sl], bf16_bits_from_f32(out["p"][sl])), name
            assert not out["twin8"][sl].any()
    assert n_fp8 == 12


@pytest.mark.parametrize("grad_dtype,state_dtype", [(DT_F32, DT_F32), (DT_BF16, DT_F32), (DT_BF16, DT_BF16)])
@pytest.mark.parametrize("t", [1, 1000])
def test_exact_update_mode_is_bit_faithful(oracle, grad_dtype, state_dtype, t):
    """ANNI_STEP_EXACT_UPDATE: the master equals the oracle's float bit for bit except for a
    vanishing fraction one ulp off -- also where the parameter is as small as its update
    (the cancellation case the fast float path cannot resolve) and at step 1, where
    |update| = lr.  Flat bar here: at most 1 ulp anywhere, at least 99.999 % identical."""
    from parity_util import f32_ulp_dist
    n = 1 << 20
    p, g, m, v = make_inputs(n, seed=70 + t, grad_dtype=grad_dtype, state_dtype=state_dtype)
    if t == 1:
        m[:] = 0
        v[:] = 0
    p[::3] *= np.float32(1e-2)                     # a third of the weights of the size of the update
    p[1::97] = 0.0
    kw = dict(HYP, wd=0.1, clip=0.0, grad_scale=1.0, t_before=t - 1)
    (rp, rg, rm, rv), info = _oracle_step(oracle, None, p, g, m, v, check_finite=True, **kw)
    out = run_gpu(None, p, g, m, v, dict(HYP, wd=0.1, clip=0.0, grad_scale=1.0, t=t, exact=True), n_arena=n)
    assert np.array_equal(out["m"], rm) and np.array_equal(out["v"], rv)
    d = f32_ulp_dist(out["p"], rp)
    assert d.max() <= 1, int(d.max())
    assert (d == 0).mean() >= 0.99999, float((d == 0).mean())
    assert np.array_equal(out["twin"], bf16_bits_from_f32(out["p"]))


def test_bounded_wait_runs_out_and_engine_recovers(oracle):
    """Failure detection without a fault: a barrier that cannot complete (it expects one block
    more than the grid has) makes every block's bounded wait run out after a few milliseconds;
    the host reads ANNI_E_BARRIER_TIMEOUT, the engine is re-armed, and the next real step is
    correct."""
    import ctypes as C
    from anni_b200 import capi
    from anni_b200.engine import OptStep
    from parity_util import to_dev, to_host
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    p, g, m, v = make_inputs(n, seed=8)
    eng = OptStep(segs, grad_dtype=DT_F32, state_dtype=DT_F32).allocate()
    for t_, a_ in ((eng.master, p), (eng.grad, g), (eng.m, m), (eng.v, v)):
        t_.copy_(to_dev(a_))
    rc = eng.L.anni_optstep_selftest_barrier_timeout(eng.h, 1 << 16, eng._stream(None))
    assert rc == capi.OK
    st = eng.status()
    assert st.error == capi.E_BARRIER_TIMEOUT
    assert np.array_equal(to_host(eng.master), p)              # nothing was touched
    assert eng.status().error == 0                             # reading the status re-armed the engine
    kw = dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0, t_before=3)
    (rp, rg, rm, rv), info = _oracle_step(oracle, segs, p, g, m, v, check_finite=True, **kw)
    eng.step(OptStep.hyper(**dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0, t=4)))
    st = eng.status()
    assert st.error == 0 and st.skipped == 0
    out = dict(p=to_host(eng.master), m=to_host(eng.m), v=to_host(eng.v))
    check_step(out, rp, rm, rv, p, exact_moments=not info["norm"] > 1.0)
    eng.close()


@pytest.mark.parametrize("split", [False, True])
def test_derived_twins_packed_qkv_and_transposed_fp8(oracle, split):
    """Twin consumers fed by the step itself: per layer the packed [Wq|Wk|Wv] bf16 matrix (here the
    attention matrices keep bf16 twins), and e4m3 twins of the FFN / output matrices in the
    transposed [cols][rows] layout -- both equal to what the reference's separate kernels would
    build from the GPU master (num/gpu_cuda.cu:6456, :898-924)."""
    import torch
    from anni_b200.capi import SEG_TWIN_BF16, SEG_TWIN_FP8, SEG_WD
    from anni_b200.engine import OptStep, lm_derived
    from parity_util import to_dev, to_host
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin="fp8")
    for i, name in enumerate(segs.names):                       # attention inputs stay bf16 for the packed matrix
        if name.endswith((".wq", ".wk", ".wv")):
            segs.flags[i] = SEG_WD | SEG_TWIN_BF16
    D, FF, n = 64, 256, segs.n
    p, g, m, v = make_inputs(n, seed=13, grad_dtype=DT_BF16)
    eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_F32).allocate()
    for t_, a_ in ((eng.master, p), (eng.grad, g), (eng.m, m), (eng.v, v)):
        t_.copy_(to_dev(a_))
    aux, n_packed, t_bytes = lm_derived(segs, D, FF)
    assert n_packed == 2 * 3 * D * D and t_bytes == 2 * (D * D + 2 * D * FF)
    packed = torch.zeros(n_packed, dtype=torch.bfloat16, device="cuda")
    fp8_t = torch.zeros(t_bytes, dtype=torch.uint8, device="cuda")
    eng.set_derived(aux, packed, fp8_t)
    hp = OptStep.hyper(**dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0, t=50))
    (eng.step_split if split else eng.step)(hp)
    assert eng.status().error == 0
    gp, t16, t8 = to_host(eng.master), to_host(eng.twin_bf16), to_host(eng.twin_fp8)
    pk, ft, sc = to_host(packed), to_host(fp8_t), eng.scale_tensor().cpu().numpy()
    assert np.array_equal(t16[segs.slice_of("blk0.wq")], bf16_bits_from_f32(gp[segs.slice_of("blk0.wq")]))
    for layer in range(2):
        want = np.concatenate([bf16_bits_from_f32(gp[segs.slice_of(f"blk{layer}.{w}")]).reshape(D, D)
                               for w in ("wq", "wk", "wv")], axis=1)
        assert np.array_equal(pk[layer * 3 * D * D:(layer + 1) * 3 * D * D].reshape(D, 3 * D), want)
    seen = 0
    for i, name in enumerate(segs.names):
        if not (segs.flags[i] & SEG_TWIN_FP8):
            continue
        sl = segs.slice_of(name)
        amax, scale, q = oracle.fp8_quant(gp[sl])
        a = aux[i]
        assert np.float32(sc[i]) == np.float32(scale)
        got = ft[a.fp8_t_off:a.fp8_t_off + a.rows * a.cols].reshape(a.cols, a.rows)
        assert np.array_equal(got, q.reshape(a.rows, a.cols).T), name
        assert not t8[sl].any()                                   # the row-major twin of these is not written
        seen += 1
    assert seen == 6
    # bad tables are refused
    aux[0].rows, aux[0].cols, aux[0].pack_ld = 3, 5, 8
    with pytest.raises(Exception):
        eng.set_derived(aux, packed, fp8_t)
    eng.close()


@pytest.mark.parametrize("n", [1, 3, 1023, 1025])
def test_tiny_and_ragged_sizes(oracle, n):
    """Sizes below and around one chunk (1024 elements): everything goes through the element-wise path."""
    p, g, m, v = make_inputs(n, seed=100 + n, grad_dtype=DT_BF16, state_dtype=DT_BF16)
    kw = dict(HYP, wd=0.1, clip=0.5, grad_scale=1.0, t_before=9)
    (rp, rg, rm, rv), info = _oracle_step(oracle, None, p, g, m, v, check_finite=True, **kw)
    out = run_gpu(None, p, g, m, v, dict(HYP, wd=0.1, clip=0.5, grad_scale=1.0, t=10), n_arena=n)
    assert abs(out["status"].norm - info["norm"]) <= 1e-12 * info["norm"] + 1e-300
    clipped = info["norm"] > 0.5
    assert np.abs(out["m"].astype(np.int64) - rm.astype(np.int64)).max() <= (1 if clipped else 0)
    assert np.abs(out["v"].astype(np.int64) - rv.astype(np.int64)).max() <= (1 if clipped else 0)
    from parity_util import bf16_to_f32
    check_step(dict(p=out["p"], m=bf16_to_f32(out["m"]), v=bf16_to_f32(out["v"])), rp, bf16_to_f32(rm),
               bf16_to_f32(rv), p, exact_moments=False)
    assert np.array_equal(out["twin"], bf16_bits_from_f32(out["p"])) and not out["g"].any()


def test_empty_shard_and_misaligned_buffers(oracle):
    """An engine that owns nothing still launches (an empty ZeRO rank); buffers that are not
    16-byte aligned take the element-wise path everywhere and give the same numbers."""
    import torch
    from anni_b200.engine import OptStep
    from parity_util import to_dev, to_host
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    eng = OptStep(segs, grad_dtype=DT_F32, state_dtype=DT_F32, shard_off=n, shard_n=0).allocate()
    eng.step_split(OptStep.hyper(**dict(HYP, wd=0.1, clip=1.0, t=3)))
    st = eng.status()
    assert st.error == 0 and st.norm == 0.0 and st.skipped == 0
    eng.close()
    p, g, m, v = make_inputs(n, seed=14)
    kw = dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0, t_before=2)
    (rp, rg, rm, rv), info = _oracle_step(oracle, segs, p, g, m, v, check_finite=True, **kw)
    eng = OptStep(segs, grad_dtype=DT_F32, state_dtype=DT_F32)
    bufs = [torch.zeros(n + 4, dtype=torch.float32, device="cuda")[1:n + 1] for _ in range(4)]   # 4 bytes off
    twin = torch.zeros(n + 8, dtype=torch.bfloat16, device="cuda")[1:n + 1]                       # 2 bytes off
    assert all(b.data_ptr() % 16 != 0 for b in bufs)
    eng.bind(*bufs, twin)
    for b, a in zip(bufs, (p, m, v, g)):
        b.copy_(to_dev(a))
    eng.step(OptStep.hyper(**dict(HYP, wd=0.1, clip=1.0, t=3)))
    st = eng.status()
    assert st.error == 0 and abs(st.norm - info["norm"]) <= 1e-12 * info["norm"]
    out = dict(p=to_host(bufs[0]), m=to_host(bufs[1]), v=to_host(bufs[2]))
    check_step(out, rp, rm, rv, p, exact_moments=not info["norm"] > 1.0)
    assert np.array_equal(to_host(twin), bf16_bits_from_f32(out["p"])) and not to_host(bufs[3]).any()
    eng.close()


def test_transposed_fp8_twins_whole_and_edge_tiles(oracle):
    """The transposed e4m3 twins for shapes that exercise the tiled path (whole 128 x 64 tiles,
    128-bit accesses), the element-wise path (edge tiles, odd shapes) and both inside one tensor."""
    import torch
    from anni_b200 import capi
    from anni_b200.capi import SEG_TWIN_FP8, SEG_WD
    from anni_b200.engine import OptStep, Segments
    from parity_util import to_dev, to_host
    shapes = [(256, 128), (128, 64), (384, 192), (200, 100), (256, 96), (160, 64), (16, 4), (1536, 64)]
    segs = Segments()
    for i, (r, c) in enumerate(shapes):
        segs.add(f"w{i}", r * c, SEG_WD | SEG_TWIN_FP8)
    n = segs.n
    p, g, m, v = make_inputs(n, seed=21, grad_dtype=DT_BF16)
    eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_F32).allocate()
    for t_, a_ in ((eng.master, p), (eng.grad, g), (eng.m, m), (eng.v, v)):
        t_.copy_(to_dev(a_))
    aux, off = [], 0
    for r, c in shapes:
        aux.append(capi.SegDerived(r, c, 0, 0, 0, off))
        off += r * c
    fp8_t = torch.full((off,), 0xAA, dtype=torch.uint8, device="cuda")
    eng.set_derived(aux, None, fp8_t)
    eng.step(OptStep.hyper(**dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0, t=9)))
    assert eng.status().error == 0
    gp, ft, sc = to_host(eng.master), to_host(fp8_t), eng.scale_tensor().cpu().numpy()
    for i, (r, c) in enumerate(shapes):
        amax, scale, q = oracle.fp8_quant(gp[segs.slice_of(f"w{i}")])
        assert np.float32(sc[i]) == np.float32(scale)
        got = ft[aux[i].fp8_t_off:aux[i].fp8_t_off + r * c].reshape(c, r)
        assert np.array_equal(got, q.reshape(r, c).T), (r, c)
    eng.close()


def test_step_with_sumsq_from_the_producer(oracle):
    """anni_optstep_step_with_sumsq: the gradient producer hands over {sum of squares, non-finite
    count} on the device, the step reads the gradients once.  Same bits as the one-launch step
    that computes the norm itself; a non-finite count skips the step."""
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin="fp8")
    n = segs.n
    p, g, m, v = make_inputs(n, seed=66, grad_dtype=DT_BF16, state_dtype=DT_BF16)
    hp = OptStep.hyper(lr=3e-4, t=9, beta2=0.95, wd=0.1, clip=1.0)
    outs = []
    for handed in (False, True):
        eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_BF16).allocate()
        for t, src in ((eng.master, p), (eng.grad, g), (eng.m, m), (eng.v, v)):
            t.copy_(to_dev(src))
        if handed:
            ss = torch.stack([eng.grad.double().square().sum(), torch.zeros((), dtype=torch.float64, device="cuda")])
            eng.step_with_sumsq(hp, ss)
        else:
            eng.step(hp)
        st = eng.status()
        assert st.error == 0 and st.skipped == 0
        outs.append((st.norm, [to_host(x).copy() for x in (eng.master, eng.m, eng.v, eng.twin_bf16, eng.twin_fp8, eng.grad)]))
        if handed:
            eng.grad.copy_(to_dev(g))
            before = eng.master.clone()
            eng.step_with_sumsq(hp, torch.tensor([1.0, 3.0], dtype=torch.float64, device="cuda"))
            st = eng.status()
            assert st.skipped == 1 and torch.equal(eng.master, before) and not bool(eng.grad.any())
        eng.close()
    # the producer's sum (torch, another order) differs from the kernel's in the last bits only
    assert abs(outs[0][0] - outs[1][0]) <= 1e-12 * outs[0][0]
    for a, b in zip(outs[0][1], outs[1][1]):
        same = (a == b).mean()
        assert same > 0.999, same
