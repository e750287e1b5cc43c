"""The part-wise forms of the split step (anni_optstep_update_range / _reduce_norm_range):
the same bits as the whole-shard launches, one step counted, one loss-scale transition."""
import numpy as np
import pytest
import torch

from anni_b200.capi import DT_BF16, DT_F32, AnniError
from anni_b200.engine import LM_SHAPES, OptStep, lm_segments
from parity_util import make_inputs, to_dev, to_host

pytestmark = pytest.mark.gpu

PARTS = [(0, 8192), (8192, 4096), (12288, None)]       # offsets are multiples of 4096


def _engine(segs, gd, sd, p, g, m, v):
    eng = OptStep(segs, grad_dtype=gd, state_dtype=sd).allocate()
    eng.master.copy_(to_dev(p))
    eng.grad.copy_(to_dev(g))
    eng.m.copy_(to_dev(m))
    eng.v.copy_(to_dev(v))
    return eng


@pytest.mark.parametrize("twin", ["bf16", "fp8"])
@pytest.mark.parametrize("gd,sd", [(DT_BF16, DT_BF16), (DT_F32, DT_F32)])
def test_update_in_parts_equals_update_of_the_whole_shard(gd, sd, twin):
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin=twin)
    n = segs.n
    p, g, m, v = make_inputs(n, seed=3, grad_dtype=gd, state_dtype=sd)
    hp = OptStep.hyper(lr=3e-4, t=7, beta2=0.95, wd=0.1, clip=1.0, check_finite=True, dev_loss_scale=True)
    whole = _engine(segs, gd, sd, p, g, m, v)
    parts = _engine(segs, gd, sd, p, g, m, v)
    for eng in (whole, parts):
        eng.loss_scale_init(scale=1.0, growth_interval=1)       # every clean step doubles the scale
    whole.step_split(hp)
    parts.norm(hp)
    cuts = [(o, (n - o) if ln is None else ln) for o, ln in PARTS]
    for i, (o, ln) in enumerate(cuts):
        parts.update_range(hp, o, ln, first=i == 0, last=i == len(cuts) - 1, local_twins=False)
    if parts.has_fp8:
        parts.quantize()
    a, b = whole.status(), parts.status()
    assert (a.norm, a.skipped, a.steps_done, a.loss_scale) == (b.norm, b.skipped, b.steps_done, b.loss_scale)
    assert b.steps_done == 1 and b.loss_scale == 2.0             # the epilogue ran once, at the last part
    for name in ("master", "m", "v", "grad", "twin_bf16", "twin_fp8"):
        x, y = getattr(whole, name), getattr(parts, name)
        if x is not None:
            assert torch.equal(x, y), name
    assert torch.equal(whole.scale_tensor(), parts.scale_tensor())
    with pytest.raises(AnniError):
        parts.update_range(hp, 100, 50, first=True, last=True)    # offset not a multiple of 4096
    with pytest.raises(AnniError):
        parts.update_range(hp, 4096, n, first=True, last=True)    # runs past the shard
    whole.close()
    parts.close()


def test_reduce_norm_in_parts_accumulates_the_sum_of_squares():
    """One rank standing for all: the "peer" arena is a second local buffer.  Part-wise
    launches leave the same reduced gradients and the same sum of squares (to the last bits:
    the partial sums are grouped differently) as one launch."""
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    p, g, m, v = make_inputs(n, seed=4, grad_dtype=DT_BF16, state_dtype=DT_F32)
    hp = OptStep.hyper(lr=3e-4, t=1, clip=1.0)
    src = to_dev(g).clone()
    twin_arena = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    out = []
    for cuts in ([(0, n)], [(o, (n - o) if ln is None else ln) for o, ln in PARTS]):
        eng = _engine(segs, DT_BF16, DT_F32, p, g, m, v)
        eng.grad.zero_()
        eng.set_peers([src.data_ptr()], [twin_arena.data_ptr()], None, 0)
        for i, (o, ln) in enumerate(cuts):
            eng.reduce_norm_range(hp, o, ln, accumulate=i > 0)
        torch.cuda.synchronize()
        out.append((to_host(eng.grad).copy(), eng.reduce_tensor().cpu().numpy().copy()))
        eng.close()
    assert np.array_equal(out[0][0], out[1][0]) and np.array_equal(out[0][0], to_host(src))
    assert out[0][1][1] == out[1][1][1] == 0.0
    assert abs(out[0][1][0] - out[1][1][0]) <= 1e-14 * out[0][1][0]
    ref = float((to_host(src).astype(np.uint32) << 16).view(np.float32).astype(np.float64).__pow__(2).sum())
    assert abs(out[1][1][0] - ref) <= 1e-12 * ref


@pytest.mark.parametrize("sc", [0, 1, 3])
def test_other_super_chunk_sizes_give_the_same_bits(sc, monkeypatch):
    """The tuning knob ANNI_B200_SUPERCHUNK moves chunks between blocks and switches the
    per-super-chunk short cuts off or on; without clipping the result does not depend on it."""
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin="fp8")
    n = segs.n
    p, g, m, v = make_inputs(n, seed=8, grad_dtype=DT_BF16, state_dtype=DT_BF16)
    hp = OptStep.hyper(lr=3e-4, t=3, beta2=0.95, wd=0.1, clip=0.0, check_finite=True)
    ref = _engine(segs, DT_BF16, DT_BF16, p, g, m, v)
    ref.step(hp)
    monkeypatch.setenv("ANNI_B200_SUPERCHUNK", str(sc))
    for split in (False, True):
        eng = _engine(segs, DT_BF16, DT_BF16, p, g, m, v)
        (eng.step_split if split else eng.step)(hp)
        assert eng.status().error == 0 and eng.status().skipped == 0
        for name in ("master", "m", "v", "grad", "twin_bf16", "twin_fp8"):
            assert torch.equal(getattr(ref, name), getattr(eng, name)), (name, split)
        assert torch.equal(ref.scale_tensor(), eng.scale_tensor())
        eng.close()
    ref.close()


def test_update_clears_the_named_gradient_arena():
    """ZeRO-1 on one GPU's worth of memory: an engine that owns the SECOND, shorter half of the arena
    is told where the rank's full gradient arena lies (two parts); its update must leave that whole
    arena zeroed -- both parts, and the ends of the parts beyond this shard's length -- while the
    step's results are those of an engine that clears its bound buffer."""
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    stride = -(-(-(-n // 2)) // 4096) * 4096
    off, cnt = stride, n - stride
    assert 0 < cnt < stride
    p, g, m, v = make_inputs(n, seed=8, grad_dtype=DT_BF16, state_dtype=DT_F32)
    outs = []
    for named in (False, True):
        eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_F32, shard_off=off, shard_n=cnt).allocate()
        eng.master[:cnt].copy_(to_dev(p[off:]))
        eng.grad[:cnt].copy_(to_dev(g[off:]))
        eng.m[:cnt].copy_(to_dev(m[off:]))
        eng.v[:cnt].copy_(to_dev(v[off:]))
        arena = torch.ones(2 * stride, dtype=torch.bfloat16, device="cuda")
        if named:
            eng.set_grad_arena(arena, stride, 2)
        for skip in (False, True):
            if skip:
                arena.fill_(1.0)
                eng.grad[:cnt].copy_(to_dev(g[off:]))
                eng.grad[5] = float("inf")
            hp = OptStep.hyper(lr=3e-4, t=3, beta2=0.95, wd=0.1, clip=1.0)
            eng.norm(hp)
            eng.update(hp)
            st = eng.status()
            assert st.error == 0 and bool(st.skipped) == skip
            if named:
                assert not bool(arena.any())                   # every element of both parts
                assert bool(eng.grad[:cnt].any())              # the reduced shard is scratch: left alone
            else:
                assert bool((arena == 1).all()) and not bool(eng.grad[:cnt].any())
        outs.append([to_host(x[:cnt]).copy() for x in (eng.master, eng.m, eng.v, eng.twin_bf16)])
        with pytest.raises(AnniError):
            eng.set_grad_arena(arena, cnt - 8, 2)              # parts shorter than the shard
        eng.close()
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


def test_fp8_step_in_one_launch_equals_the_other_forms(monkeypatch):
    """e4m3 twins, one launch: the optional form whose quantiser follows the update tensor by
    tensor (ANNI_B200_FP8_PIPE=1) must give the same bits as the default one (a quantise phase
    after a second grid barrier) and as the three-launch form.  Shapes with tensors of several million elements, so that blocks wait for,
    report and quantise tensors many rounds apart; two steps in a row reuse the counters."""
    segs = lm_segments(d_model=512, d_ff=6144, n_blocks=2, vocab=1000, tied=True, wd="matrices", twin="fp8")
    n = segs.n
    p, g, m, v = make_inputs(n, seed=9, grad_dtype=DT_BF16, state_dtype=DT_BF16)
    _, g2, _, _ = make_inputs(n, seed=10, grad_dtype=DT_BF16, state_dtype=DT_BF16)
    outs = []
    for form in ("pipe", "barrier", "split"):
        monkeypatch.setenv("ANNI_B200_FP8_PIPE", "1" if form == "pipe" else "0")
        eng = _engine(segs, DT_BF16, DT_BF16, p, g, m, v)
        for t, grads in ((5, g), (6, g2)):
            eng.grad.copy_(to_dev(grads))
            hp = OptStep.hyper(lr=3e-4, t=t, beta2=0.95, wd=0.1, clip=1.0)
            (eng.step_split if form == "split" else eng.step)(hp)
            st = eng.status()
            assert st.error == 0 and st.skipped == 0
        assert bool(eng.twin_fp8.any())
        outs.append([to_host(x).copy() for x in (eng.master, eng.m, eng.v, eng.twin_bf16, eng.twin_fp8)]
                    + [eng.scale_tensor().cpu().numpy().copy(), eng.amax_tensor().cpu().numpy().copy()])
        eng.close()
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert np.array_equal(a, b)


def test_rotated_peer_order_on_local_arenas():
    """anni_optstep_rotate_peers with three "ranks" standing on one GPU (their arenas are local
    buffers): whatever peer comes first, the reduced gradients (an exact sum here), the sum of
    squares and the twins stored into every arena are the same; a bad start index is refused."""
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    p, g, m, v = make_inputs(n, seed=5, grad_dtype=DT_BF16, state_dtype=DT_F32)
    hp = OptStep.hyper(lr=3e-4, t=2, beta2=0.95, wd=0.1, clip=1.0)
    base = to_dev(g).float()
    parts = [(base * w).to(torch.bfloat16) for w in (0.5, 0.25, 0.25)]      # sums exactly to g
    outs = []
    for first in (0, 1, 2):
        eng = _engine(segs, DT_BF16, DT_F32, p, g, m, v)
        eng.grad.zero_()
        twins = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
        eng.set_peers([x.data_ptr() for x in parts], [t.data_ptr() for t in twins], None, 0)
        eng.rotate_peers(first)
        eng.reduce_norm(hp)
        eng.update(hp)
        st = eng.status()
        assert st.error == 0 and st.skipped == 0
        assert all(torch.equal(t, twins[0]) for t in twins) and bool(twins[0].any())
        outs.append((st.norm, to_host(eng.master).copy(), to_host(twins[2]).copy()))
        with pytest.raises(AnniError):
            eng.rotate_peers(3)
        eng.close()
    for o in outs[1:]:
        assert o[0] == outs[0][0] and np.array_equal(o[1], outs[0][1]) and np.array_equal(o[2], outs[0][2])


@pytest.mark.parametrize("ranged", [False, True], ids=["whole", "parts"])
@pytest.mark.parametrize("gd", [DT_BF16, DT_F32])
def test_reduce_clears_own_part_of_the_arena(gd, ranged):
    """ANNI_STEP_REDUCE_CLEARS_OWN with two "ranks" on one GPU: the engine of rank 1 (the shorter
    half) reads its shard out of both arenas; with the flag the reduce leaves rank 1's own part of
    ITS arena zeroed (and touches nothing else), the update clears the rest of that arena and
    leaves the other rank's alone; results equal the step without the flag, also when both kernels
    run part by part (the parts of the own part already reduced are zero, the others not yet).
    The flag is refused where no arena was named."""
    from anni_b200.capi import STEP_REDUCE_CLEARS_OWN
    tdt = torch.bfloat16 if gd == DT_BF16 else torch.float32
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    stride = -(-(-(-n // 2)) // 4096) * 4096
    off, cnt = stride, n - stride
    p, g, m, v = make_inputs(n, seed=11, grad_dtype=gd, state_dtype=DT_F32)
    half = (to_dev(g).float() * 0.5).to(tdt)               # both ranks hold g/2: the sum is g exactly
    outs = []
    for flag in (0, STEP_REDUCE_CLEARS_OWN):
        eng = OptStep(segs, grad_dtype=gd, state_dtype=DT_F32, shard_off=off, shard_n=cnt).allocate()
        eng.master[:cnt].copy_(to_dev(p[off:]))
        eng.m[:cnt].copy_(to_dev(m[off:]))
        eng.v[:cnt].copy_(to_dev(v[off:]))
        arenas = [torch.zeros(2 * stride, dtype=tdt, device="cuda") for _ in range(2)]
        for a in arenas:
            a[:n].copy_(half)
        theirs = arenas[0].clone()
        twins = [torch.zeros(2 * stride, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        eng.set_peers([a.data_ptr() for a in arenas], [t.data_ptr() for t in twins], None, off)
        eng.rotate_peers(0)
        hp = OptStep.hyper(lr=3e-4, t=3, beta2=0.95, wd=0.1, clip=1.0)
        hp.flags |= flag
        if flag:
            with pytest.raises(AnniError):
                eng.reduce_norm(hp)                             # no arena named yet
        eng.set_grad_arena(arenas[1], stride, 2)
        own = arenas[1]
        cuts = [(o, (cnt - o) if ln is None else ln) for o, ln in PARTS] if ranged else [(0, cnt)]
        for i, (o, ln) in enumerate(cuts):
            if ranged:
                eng.reduce_norm_range(hp, o, ln, accumulate=i > 0)
                if flag and i == 0:
                    assert not bool(own[stride:stride + ln].any()) and bool(own[stride + ln:stride + cnt].any())
            else:
                eng.reduce_norm(hp)
        assert torch.equal(arenas[0], theirs)
        assert torch.equal(own[:stride], theirs[:stride])       # the part another rank reads: untouched
        assert bool(own[stride:stride + cnt].any()) == (flag == 0)
        for i, (o, ln) in enumerate(cuts):
            if ranged:
                eng.update_range(hp, o, ln, first=i == 0, last=i == len(cuts) - 1, local_twins=False)
            else:
                eng.update(hp)
        st = eng.status()
        assert st.error == 0 and st.skipped == 0
        assert not bool(own.any()) and torch.equal(arenas[0], theirs)
        outs.append([st.norm] + [to_host(x[:cnt]).copy() for x in (eng.master, eng.m, eng.v, eng.grad)]
                    + [to_host(twins[0][off:off + cnt]).copy()])
        eng.close()
    assert outs[0][0] == outs[1][0]
    for a, b in zip(outs[0][1:], outs[1][1:]):
        assert np.array_equal(a, b)
