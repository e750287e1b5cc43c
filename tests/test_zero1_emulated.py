"""The sharded step with ALL its ranks standing on one GPU: every "rank" is an engine of its own
over its shard, the peers' arenas are local buffers, the small all-reduce is a sum on the
device.  The kernels of the peer-memory form never wait for one another (the exchanges
between them are the caller's), so the ranks can simply run one after the other; what this
covers is the code that depends on the NUMBER of ranks -- eight peers' loads in flight per
thread, the element-wise reduce for fp32 gradients beyond four peers, twin stores into eight
arenas, clearing seven parts of the arena beside the own one, a rank whose shard is empty --
on a machine with a single GPU, against the CPU oracle on the reduced gradients."""
import numpy as np
import pytest
import torch

from anni_b200.capi import DT_BF16, DT_F32, STEP_REDUCE_CLEARS_OWN
from anni_b200.engine import LM_SHAPES, OptStep, lm_segments
from parity_util import bf16_bits_from_f32, check_step, make_inputs, to_dev, to_host

pytestmark = pytest.mark.gpu

HYP = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8)


@pytest.mark.parametrize("own_clear", [True, False], ids=["reduce_clears_own", "update_clears_all"])
@pytest.mark.parametrize("gd", [DT_BF16, DT_F32], ids=["bf16", "f32"])
@pytest.mark.parametrize("world", [8, 4, 2])
def test_all_ranks_on_one_gpu_match_the_oracle(oracle, world, gd, own_clear):
    tdt = torch.bfloat16 if gd == DT_BF16 else torch.float32
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    per = -(-(-(-n // world)) // 4096) * 4096
    padded = per * world
    p, g, m, v = make_inputs(n, seed=21 + world, grad_dtype=gd, state_dtype=DT_F32)
    if gd == DT_F32:        # keep 20 mantissa bits: the partial sums k * g / world then stay exact in float
        g = (g.view(np.uint32) & np.uint32(0xFFFFFFF0)).view(np.float32)
    kw = dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0)
    ref = [x.copy() for x in (p, g, m, v)]
    info = oracle.step(*ref, seg_off=segs.offsets, seg_flags=segs.flag_array, check_finite=True,
                       t_before=999, **kw)
    rp, _, rm, rv = ref
    share = (to_dev(g).float() / world).to(tdt)            # exact: the ranks' sum is g again
    arenas = [torch.zeros(padded, dtype=tdt, device="cuda") for _ in range(world)]
    for a in arenas:
        a[:n].copy_(share)
        a[n:].fill_(1.0)                                    # padding: must come back zeroed too
    twins = [torch.zeros(padded, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    engines = []
    for r in range(world):
        off = r * per
        cnt = max(0, min(per, n - off))
        eng = OptStep(segs, grad_dtype=gd, state_dtype=DT_F32, shard_off=min(off, n), shard_n=cnt).allocate()
        if cnt:
            eng.master[:cnt].copy_(to_dev(p[off:off + cnt]))
            eng.m[:cnt].copy_(to_dev(m[off:off + cnt]))
            eng.v[:cnt].copy_(to_dev(v[off:off + cnt]))
        eng.set_peers([a.data_ptr() for a in arenas], [t.data_ptr() for t in twins], None, off)
        eng.rotate_peers((r + 1) % world)
        eng.set_grad_arena(arenas[r], per, world)
        engines.append((eng, off, cnt))
    assert any(cnt == 0 for _, _, cnt in engines) == (world == 8)      # the empty shard is part of the case
    hp = OptStep.hyper(t=1000, check_finite=True, **kw)
    if own_clear:
        hp.flags |= STEP_REDUCE_CLEARS_OWN
    for eng, _, _ in engines:
        eng.reduce_norm(hp)
    if own_clear:                                           # own parts cleared, the others still to be read
        for r, (eng, off, cnt) in enumerate(engines):
            assert not bool(arenas[r][off:off + cnt].any())
            if r + 1 < world and engines[r + 1][2]:
                o2, c2 = engines[r + 1][1], engines[r + 1][2]
                assert bool(arenas[r][o2:o2 + c2].any())
    total = torch.stack([eng.reduce_tensor() for eng, _, _ in engines]).sum(0)
    for eng, _, _ in engines:
        eng.reduce_tensor().copy_(total)                    # the two-double all-reduce
    for eng, _, _ in engines:
        eng.update(hp)
    out = {k: np.empty(n, dtype=np.float32) for k in ("p", "m", "v")}
    for eng, off, cnt in engines:
        st = eng.status()
        assert st.error == 0 and st.skipped == 0 and not info["skipped"]
        assert abs(st.norm - info["norm"]) <= 1e-5 * info["norm"]
        if cnt:
            out["p"][off:off + cnt] = to_host(eng.master[:cnt])
            out["m"][off:off + cnt] = to_host(eng.m[:cnt])
            out["v"][off:off + cnt] = to_host(eng.v[:cnt])
    check_step(out, rp, rm, rv, p, exact_moments=False, m_old=m)
    want = bf16_bits_from_f32(out["p"])
    for r in range(world):
        assert np.array_equal(to_host(twins[r][:n]), want), r          # every arena holds every shard's twins
        assert not bool(arenas[r].any()), r                             # whole arena, padding included
    for eng, _, _ in engines:
        eng.close()


@pytest.mark.parametrize("world", [8, 2])
def test_all_ranks_on_one_gpu_fp8_twins_and_bf16_moments(oracle, world):
    """The same with e4m3 twins and bf16 moments: a tensor cut by a shard boundary gets its amax
    from both owners (the max all-reduce, emulated on the device) before either quantises its
    part; every rank's e4m3 arena then holds the codes of the oracle's quantiser applied to the
    gathered masters, and the scales agree on all ranks."""
    from anni_b200.capi import SEG_TWIN_FP8
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin="fp8")
    n = segs.n
    per = -(-(-(-n // world)) // 4096) * 4096
    padded = per * world
    p, g, m, v = make_inputs(n, seed=40 + world, grad_dtype=DT_BF16, state_dtype=DT_BF16)
    p[segs.slice_of("blk0.wq")] *= 37.0
    kw = dict(HYP, wd=0.1, clip=1.0, grad_scale=1.0)
    ref = [x.copy() for x in (p, g, m, v)]
    info = oracle.step(*ref, seg_off=segs.offsets, seg_flags=segs.flag_array, check_finite=True,
                       t_before=999, **kw)
    rp, _, rm, rv = ref
    share = (to_dev(g).float() / world).to(torch.bfloat16)
    arenas = [torch.zeros(padded, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for a in arenas:
        a[:n].copy_(share)
    twins = [torch.zeros(padded, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    twins8 = [torch.zeros(padded, dtype=torch.uint8, device="cuda") for _ in range(world)]
    engines = []
    for r in range(world):
        off = r * per
        cnt = max(0, min(per, n - off))
        eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_BF16, shard_off=min(off, n), shard_n=cnt).allocate()
        if cnt:
            eng.master[:cnt].copy_(to_dev(p[off:off + cnt]))
            eng.m[:cnt].copy_(to_dev(m[off:off + cnt]))
            eng.v[:cnt].copy_(to_dev(v[off:off + cnt]))
        eng.set_peers([a.data_ptr() for a in arenas], [t.data_ptr() for t in twins],
                      [t.data_ptr() for t in twins8], off)
        eng.rotate_peers((r + 1) % world)
        eng.set_grad_arena(arenas[r], per, world)
        engines.append((eng, off, cnt))
    hp = OptStep.hyper(t=1000, check_finite=True, **kw)
    hp.flags |= STEP_REDUCE_CLEARS_OWN
    for eng, _, _ in engines:
        eng.reduce_norm(hp)
    total = torch.stack([eng.reduce_tensor() for eng, _, _ in engines]).sum(0)
    for eng, _, _ in engines:
        eng.reduce_tensor().copy_(total)
    for eng, _, _ in engines:
        eng.update(hp)
    amax = torch.stack([eng.amax_tensor() for eng, _, _ in engines]).max(0).values
    for eng, _, _ in engines:
        eng.amax_tensor().copy_(amax)                       # the max all-reduce
        eng.quantize()
    out = {"p": np.empty(n, dtype=np.float32), "m": np.empty(n, dtype=np.uint16), "v": np.empty(n, dtype=np.uint16)}
    for eng, off, cnt in engines:
        st = eng.status()
        assert st.error == 0 and st.skipped == 0 and not info["skipped"]
        if cnt:
            out["p"][off:off + cnt] = to_host(eng.master[:cnt])
            out["m"][off:off + cnt] = to_host(eng.m[:cnt])
            out["v"][off:off + cnt] = to_host(eng.v[:cnt])
    check_step(out, rp, rm, rv, p, exact_moments=False, m_old=m)
    scales = [to_host(eng.scale_tensor()) for eng, _, _ in engines]
    off_t = segs.offsets
    for i, name in enumerate(segs.names):
        sl = slice(int(off_t[i]), int(off_t[i + 1]))
        if segs.flags[i] & SEG_TWIN_FP8:
            a_ref, s_ref, q = oracle.fp8_quant(out["p"][sl])
            assert np.float32(amax[i].item()) == np.float32(a_ref), name
            owners = [r for r, (_, o, c) in enumerate(engines) if c and o < sl.stop and o + c > sl.start]
            assert owners and all(np.float32(scales[r][i]) == np.float32(s_ref) for r in owners), name
            for r in range(world):
                assert np.array_equal(to_host(twins8[r][sl]), q), (name, r)
        else:
            want = bf16_bits_from_f32(out["p"][sl])
            for r in range(world):
                assert np.array_equal(to_host(twins[r][sl]), want), (name, r)
    for r in range(world):
        assert not bool(arenas[r].any()), r
    for eng, _, _ in engines:
        eng.close()
