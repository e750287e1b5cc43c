"""Pins the CPU oracle: against the committed golden vectors (generated from the reference's
own object code by tests/golden/make_golden.py) and, where it was built, against that object
code itself, bit for bit.  CPU only."""
import hashlib
import json
import os

import numpy as np
import pytest

from golden.make_golden import CASES, ckpt_moments, inputs

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("case", [c[0] for c in CASES])
def test_step_matches_golden(oracle, case):
    z = np.load(os.path.join(GOLD, "adam_steps.npz"))
    lr, b1, b2, eps, wd, clip, gs, t0 = z[f"{case}/hyper"]
    a = [z[f"{case}/in_{k}"].copy() for k in "pgmv"]
    info = oracle.step(*a, lr=lr, beta1=b1, beta2=b2, eps=eps, wd=wd, clip=clip, grad_scale=gs,
                       t_before=int(t0))
    assert info["t_after"] == int(t0) + 1 and not info["skipped"]
    for k, got in zip("pgmv", a):
        assert np.array_equal(_bits(got), _bits(z[f"{case}/out_{k}"])), (case, k)
    assert not a[1].any()                                   # gradients zeroed (lm_adam.c:597)


def test_golden_inputs_are_reproducible():
    """The committed inputs are the ones the generator draws (guards the fixture itself)."""
    z = np.load(os.path.join(GOLD, "adam_steps.npz"))
    name, n, seed, kw = CASES[0]
    p, g, m, v = inputs(n, seed)
    assert np.array_equal(z[f"{name}/in_p"], p) and np.array_equal(z[f"{name}/in_g"], g)


def test_lr_schedule_matches_golden(oracle):
    with open(os.path.join(GOLD, "lr_schedule.json")) as f:
        pts = json.load(f)
    assert len(pts) > 100
    for q in pts:
        got = oracle.lr_schedule(q["base"], q["step"], q["warmup"], q["decay"], q["kind"], q["start"])
        assert got == q["lr"], q


def test_lr_schedule_reference_known_answers(oracle):
    """The reference's own unit test of the schedule (tests/test_ann.c:866-879)."""
    f = lambda step, start: oracle.lr_schedule(1.0, step, 100, 1000, "cosine", start)
    assert abs(f(29000, 0) - 0.0) < 1e-12
    assert abs(f(29000, 29000) - 0.01) < 1e-12
    assert abs(f(29099, 29000) - 1.0) < 1e-12
    assert abs(f(29600, 29000) - 0.5) < 1e-12
    assert abs(f(31000, 29000) - 0.0) < 1e-12
    assert abs(f(10, 29000) - 0.01) < 1e-12


def test_checkpoint_trailer_matches_golden(oracle, tmp_path):
    with open(os.path.join(GOLD, "segments_tiny.json")) as f:
        meta = json.load(f)
    m, v = ckpt_moments(meta["n"])
    path = str(tmp_path / "adam.bin")
    oracle.ckpt_write_adam(path, m, v, t=meta["t"], epoch=meta["epoch"], step=meta["step"])
    data = open(path, "rb").read()
    assert len(data) == 20 + 8 * meta["n"]                  # the size rule run555m_checks.py relies on
    assert data[:36].hex() == meta["trailer_head_hex"]
    assert hashlib.sha256(data).hexdigest() == meta["trailer_sha256"]


def test_segment_order_matches_golden():
    from anni_b200.engine import LM_SHAPES, lm_param_count, lm_segments
    with open(os.path.join(GOLD, "segments_tiny.json")) as f:
        meta = json.load(f)
    segs = lm_segments(**LM_SHAPES["tiny"])
    assert segs.n == meta["n"] == lm_param_count(**LM_SHAPES["tiny"])
    assert segs.offsets[:-1].tolist() == meta["off"]
    assert segs.sizes == meta["n_per"]
    # vectors are exactly the tensors without weight decay in the "matrices" setting
    assert [int(not (f & 1)) for f in segs.flags] == meta["is_vec"]


def test_param_counts_of_the_benchmark_shapes():
    from anni_b200.engine import LM_SHAPES, lm_param_count, lm_segments
    assert lm_param_count(**LM_SHAPES["talk170m"]) == 184_676_352
    assert lm_param_count(**LM_SHAPES["run555m"]) == 555_762_080
    assert lm_param_count(**LM_SHAPES["synth3b"]) == 2_773_419_680
    assert len(lm_segments(**LM_SHAPES["talk170m"])) == 147
    assert len(lm_segments(**LM_SHAPES["run555m"])) == 170
    assert len(lm_segments(**LM_SHAPES["synth3b"])) == 386


# ---- against the reference's object code itself (skipped where oracle/_ref is absent) ----------

@pytest.mark.parametrize("clip,wd,gs,t0,n", [(1.0, 0.1, 1.0, 999, 100003), (0.0, 0.0, 1 / 252., 0, 4097),
                                             (1.0, 0.0, 1 / 1024., 5, 65536), (5.0, 0.01, 1.0, 10000, 33333)])
def test_step_matches_compiled_reference(oracle, reflib, clip, wd, gs, t0, n):
    rng = np.random.default_rng(n)
    p = rng.normal(0, 0.02, n).astype(np.float32)
    g = rng.normal(0, 1e-3, n).astype(np.float32)
    g[rng.random(n) < 1e-3] *= 100
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    a = [x.copy() for x in (p, g, m, v)]
    b = [x.copy() for x in (p, g, m, v)]
    kw = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=wd, clip=clip, grad_scale=gs, t_before=t0)
    oracle.step(*a, **kw)
    reflib.step(*b, **kw)
    for x, y in zip(a, b):
        assert np.array_equal(_bits(x), _bits(y))


def test_multi_step_trajectory_matches_compiled_reference(oracle, reflib):
    """Ten consecutive steps with fresh gradients and the cosine schedule (config-2 style)."""
    n = 20011
    rng = np.random.default_rng(77)
    p = rng.normal(0, 0.02, n).astype(np.float32)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    a = [p.copy(), None, m.copy(), v.copy()]
    b = [p.copy(), None, m.copy(), v.copy()]
    for t in range(10):
        g = (rng.normal(0, 1e-3, n) * 1024).astype(np.float32)
        lr = oracle.lr_schedule(3e-4, t, 100, 1000)
        assert lr == reflib.lr_schedule(3e-4, t, 100, 1000)
        a[1], b[1] = g.copy(), g.copy()
        kw = dict(lr=lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0, grad_scale=1 / 1024., t_before=t)
        oracle.step(*a, **kw)
        reflib.step(*b, **kw)
    for x, y in zip(a, b):
        assert np.array_equal(_bits(x), _bits(y))


def test_checkpoint_roundtrip_with_compiled_reference(oracle, reflib, tmp_path):
    """Reference writes, we read; we write the trailer bytes, they equal the reference's."""
    from anni_b200 import checkpoint
    vocab = 256             # the reference's loader rebuilds a byte-level model (no BPE table) only at 256
    n = reflib.slot_count(vocab)
    m, v = ckpt_moments(n)
    ref_path = str(tmp_path / "ref.ckpt")
    reflib.ckpt_save(ref_path, vocab, m, v, t=55, epoch=2, step=9)
    got = checkpoint.read_adam(ref_path, n)                 # product reader on the reference's file
    assert (got["t"], got["epoch"], got["step"]) == (55, 2, 9)
    assert np.array_equal(got["m"], m) and np.array_equal(got["v"], v)
    size = os.path.getsize(ref_path)
    with open(ref_path, "rb") as f:
        f.seek(size - (20 + 8 * n))
        tail = f.read()
    ours = str(tmp_path / "ours.bin")
    checkpoint.write_adam(ours, m, v, t=55, epoch=2, step=9)   # product writer
    assert open(ours, "rb").read() == tail
    assert not os.path.exists(ours + ".tmp")                # tmp + rename leaves nothing behind
    # append our trailer to the reference's weight section: the reference loads it back
    spliced = str(tmp_path / "spliced.ckpt")
    with open(ref_path, "rb") as f:
        head = f.read(size - (20 + 8 * n))
    with open(spliced, "wb") as f:
        f.write(head)
    checkpoint.write_adam(spliced, m * 2, v * 3, t=56, epoch=4, step=1, append=True)
    back = reflib.ckpt_load(spliced, n)
    assert (back["n"], back["t"], back["epoch"], back["step"]) == (n, 56, 4, 1)
    assert np.array_equal(back["m"], m * 2) and np.array_equal(back["v"], v * 3)


def test_segment_order_matches_compiled_reference(reflib):
    from anni_b200.engine import LM_SHAPES, lm_segments
    off, cnt, isv = reflib.seg_list(300)
    segs = lm_segments(**LM_SHAPES["tiny"])
    assert segs.offsets[:-1].tolist() == off.tolist() and segs.sizes == cnt.tolist()
