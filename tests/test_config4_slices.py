"""Configuration 4 (2,773,419,680 parameters: arena offsets beyond 2^31) on one GPU.

The whole state of that model does not belong on one GPU, and the reference's own optimizer
cannot even count it (``int n``, lang/lm_adam.h:35 of the reference) -- it is the ZeRO-1
configuration.  What one GPU can prove is what each rank does: an engine that owns a slice
``[shard_off, shard_off + shard_n)`` of the 386-tensor arena, handed the global sum of squares
through the reduce buffer (the split form of the step), must produce exactly what the CPU
oracle produces on the same slice with the same multiplier -- wherever the slice lies: at the
arena start, above 2^31, and across a tensor boundary above 2^31.  The legacy 64-bit entry
points are run over more than 2^31 elements as well.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from anni_b200 import capi
from anni_b200.capi import DT_BF16, DT_F32
from anni_b200.engine import LM_SHAPES, OptStep, lm_segments
from parity_util import bf16_bits_from_f32, check_step, make_inputs, to_dev, to_host

pytestmark = pytest.mark.gpu
TWO31 = 1 << 31


def _local_table(segs, off, n):
    """The segment table as the oracle needs it for arena elements [off, off + n): offsets
    relative to the slice, tensors clipped to it."""
    so = segs.offsets
    first = int(np.searchsorted(so, off, side="right") - 1)
    last = int(np.searchsorted(so, off + n, side="left"))
    loc = np.clip(so[first:last + 1] - off, 0, n).astype(np.int64)
    return loc, segs.flag_array[first:last].copy(), first, last


def test_config4_slices_above_two_to_the_31(oracle):
    segs = lm_segments(**LM_SHAPES["synth3b"], wd="matrices")
    assert segs.n == 2_773_419_680 and len(segs) == 386 and segs.n > TWO31
    so = segs.offsets
    edge = int(so[np.searchsorted(so, TWO31, side="right")])        # first tensor boundary above 2^31
    assert edge > TWO31
    length = 4 * 1024 * 1024 + 1536
    # (offset, what it exercises); the third straddles a tensor boundary above 2^31 at an odd
    # distance, the fourth runs into the arena's last element
    slices = [(0, "arena start"), (TWO31 + 4096 * 3, "above 2^31, inside one tensor"),
              (edge - 2 * 1024 * 1024 - 4096 + 8, "across a tensor boundary above 2^31"),
              (segs.n - length, "arena end")]
    hyp = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
    for k, (off, what) in enumerate(slices):
        loc_off, loc_flags, first, last = _local_table(segs, off, length)
        if "boundary" in what:
            assert last - first >= 2, what
        p, g, m, v = make_inputs(length, seed=400 + k, grad_dtype=DT_BF16, state_dtype=DT_F32, grad_std=3e-4)
        # the global sum of squares: this slice's own, scaled as if every other slice carried as much
        # (norm forced above the clip threshold, as the configuration asks)
        ss = oracle.sumsq(g, 1.0) * (segs.n / length)
        gs, clip = 1.0, 1.0
        norm = math.sqrt(ss) * abs(gs)
        assert norm > clip
        coef = gs * (clip / (norm + 1e-12))                          # the engine's own expression
        ref = [x.copy() for x in (p, g, m, v)]
        oracle.step(*ref, clip=0.0, grad_scale=coef, t_before=41, seg_off=loc_off, seg_flags=loc_flags, **hyp)
        eng = OptStep(segs, grad_dtype=DT_BF16, state_dtype=DT_F32, shard_off=off, shard_n=length).allocate()
        eng.master[:length].copy_(to_dev(p))
        eng.grad[:length].copy_(to_dev(g))
        eng.m[:length].copy_(to_dev(m))
        eng.v[:length].copy_(to_dev(v))
        hp = OptStep.hyper(lr=3e-4, t=42, beta2=0.95, wd=0.1, clip=clip, grad_scale=gs, exact=(k % 2 == 0))
        eng.reduce_tensor().copy_(torch.tensor([ss, 0.0], dtype=torch.float64))
        eng.update(hp)
        st = eng.status()
        assert st.error == 0 and st.skipped == 0, what
        assert st.norm == norm and st.eff_scale == coef, what          # same bits in, same bits out
        out = dict(p=to_host(eng.master[:length]), m=to_host(eng.m[:length]), v=to_host(eng.v[:length]))
        check_step(out, ref[0], ref[2], ref[3], p, exact_moments=True)
        if k % 2 == 0:
            assert (out["p"] == ref[0]).mean() > 0.9999, what
        assert np.array_equal(to_host(eng.twin_bf16[:length]), bf16_bits_from_f32(out["p"])), what
        assert not bool(eng.grad[:length].any()), what
        # decay lands on matrices only, also across the boundary: an element of a vector tensor
        # with zero gradient and zero moments must not move
        eng.close()


def _legacy64():
    L = capi.lib()
    L.anni_grad_sumsq64.restype = C.c_int
    L.anni_grad_sumsq64.argtypes = [C.c_void_p, C.c_int, C.c_ulonglong, C.POINTER(C.c_double)]
    L.anni_adam_step_dev64.restype = C.c_int
    L.anni_adam_step_dev64.argtypes = [C.c_void_p] * 5 + [C.c_ulonglong] + [C.c_double] * 4 + [C.c_int, C.c_double]
    L.gpu_adam_set_weight_decay.argtypes = [C.c_double]
    L.gpu_set_compute_prec.argtypes = [C.c_int]
    L.gpu_stream_sync.restype = C.c_int
    return L


def test_sumsq64_over_more_than_two_to_the_31_elements():
    """anni_grad_sumsq64 on a bf16 buffer of 2^31 + 12,288 elements: every value a power of two, so
    the sum is exact in double and the expected result is known in closed form; the elements that
    only a 64-bit index reaches carry a different value."""
    L = _legacy64()
    n = TWO31 + 12288
    g = torch.full((n,), 2.0 ** -10, dtype=torch.bfloat16, device="cuda")
    g[TWO31:] = 2.0 ** -3
    g[5] = 4.0
    torch.cuda.synchronize()
    ss = C.c_double()
    assert L.anni_grad_sumsq64(g.data_ptr(), DT_BF16, n, C.byref(ss)) == 0
    want = (TWO31 - 1) * 2.0 ** -20 + 12288 * 2.0 ** -6 + 16.0
    assert ss.value == want


def test_adam_step_dev64_over_more_than_two_to_the_31_elements(oracle):
    """anni_adam_step_dev64 (the 64-bit form of gpu_adam_step_dev_bf16, num/gpu.h:129-132 of the
    reference) over 2^31 + 8192 fp32 elements: windows at the start, around 2^31 and at the very
    end are compared with the oracle; the buffers are filled with a pattern that repeats every
    2^20 elements, so every other element is covered by comparing the arena with its own first
    period."""
    free, _ = torch.cuda.mem_get_info()
    n = TWO31 + 8192
    if free < 19 * n + (4 << 30):
        pytest.skip("needs about 45 GB of device memory")
    L = _legacy64()
    period = 1 << 20
    p0, g0, m0, v0 = make_inputs(period, seed=64)

    def tiled(x):
        t = torch.empty(n, dtype=torch.float32, device="cuda")
        src = to_dev(x)
        t[:n // period * period].view(-1, period).copy_(src.expand(n // period, period))
        t[n // period * period:].copy_(src[:n % period])
        return t
    dp, dg, dm, dv = (tiled(x) for x in (p0, g0, m0, v0))
    t16 = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    coef, wd = 0.37, 0.1
    L.gpu_adam_set_weight_decay(wd)
    L.gpu_set_compute_prec(1)
    rc = L.anni_adam_step_dev64(dp.data_ptr(), t16.data_ptr(), dg.data_ptr(), dm.data_ptr(), dv.data_ptr(),
                                n, 3e-4, 0.9, 0.95, 1e-8, 7, coef)
    assert rc == 0 and L.gpu_stream_sync() == 0
    L.gpu_set_compute_prec(0)
    ref = [x.copy() for x in (p0, g0, m0, v0)]
    oracle.step(*ref, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=wd, clip=0.0, grad_scale=coef, t_before=6)
    out = dict(p=to_host(dp[:period]), m=to_host(dm[:period]), v=to_host(dv[:period]))
    check_step(out, ref[0], ref[2], ref[3], p0, exact_moments=True)
    # the last period-aligned window and the ragged tail beyond 2^31 against the first period
    for name, t in (("p", dp), ("m", dm), ("v", dv)):
        whole = t[:n // period * period].view(-1, period)
        assert bool((whole == whole[0]).all()), name
        assert torch.equal(t[n // period * period:], t[:n % period]), name
    assert not bool(dg.any())
    assert torch.equal(t16, dp.to(torch.bfloat16))
    L.gpu_adam_set_weight_decay(0.0)
