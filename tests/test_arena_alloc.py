"""Compressible device memory for the gradient arena (anni_arena_alloc): same results, the
buffer behaves like any other device memory."""
import numpy as np
import pytest
import torch

from anni_b200 import capi
from anni_b200.capi import DT_BF16, DT_F32
from anni_b200.engine import LM_SHAPES, CompressibleArena, OptStep, lm_segments
from parity_util import make_inputs, to_dev

pytestmark = pytest.mark.gpu


def _arena(n, dtype):
    try:
        return CompressibleArena(n, dtype)
    except capi.AnniError as e:
        if e.code == capi.E_LIMIT:
            pytest.skip("no compressible memory on this device / driver")
        raise


def test_arena_is_zeroed_writable_and_freed():
    a = _arena(3_000_001, torch.float32)
    assert a.compressed and a.mapped_bytes >= 4 * 3_000_001
    t = a.tensor
    assert t.is_cuda and t.numel() == 3_000_001 and not t.any()
    t.copy_(torch.arange(t.numel(), device="cuda", dtype=torch.float32))
    assert float(t[-1]) == 3_000_000.0 and float(t.sum(dtype=torch.float64)) == 3_000_000 * 3_000_001 / 2
    a.close()
    a.close()                                             # idempotent
    assert capi.lib().anni_arena_free(None, 0) == 0


@pytest.mark.parametrize("gd", [DT_BF16, DT_F32])
def test_step_on_a_compressible_gradient_arena_gives_the_same_bits(gd):
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    p, g, m, v = make_inputs(n, seed=5, grad_dtype=gd, state_dtype=DT_BF16)
    hp = OptStep.hyper(lr=3e-4, t=4, beta2=0.95, wd=0.1, clip=1.0)
    outs = []
    for compressible in (False, True):
        eng = OptStep(segs, grad_dtype=gd, state_dtype=DT_BF16).allocate()
        arena = None
        if compressible:
            arena = _arena(n, torch.bfloat16 if gd == DT_BF16 else torch.float32)
            eng.bind(eng.master, eng.m, eng.v, arena.tensor, eng.twin_bf16, None)
        for t_, a_ in ((eng.master, p), (eng.grad, g), (eng.m, m), (eng.v, v)):
            t_.copy_(to_dev(a_))
        for _ in range(2):
            eng.step(hp)
        st = eng.status()
        outs.append((eng.master.clone(), eng.m.clone(), eng.v.clone(), eng.twin_bf16.clone(), eng.grad.clone(),
                     st.norm, st.skipped))
        eng.close()
        if arena is not None:
            arena.close()
    for a, b in zip(outs[0][:5], outs[1][:5]):
        assert torch.equal(a, b)
    assert outs[0][5:] == outs[1][5:] and not outs[1][4].any()


def test_large_gpu_malloc_blocks_are_compressible_and_behave():
    """The reference-facing allocator (num/gpu.h:40-41): a large block comes from compressible
    memory, works with the other gpu_* calls, and gpu_free knows how to release it."""
    import ctypes as C
    L = capi.lib()
    L.gpu_malloc.restype = C.c_void_p
    L.gpu_malloc.argtypes = [C.c_size_t]
    L.gpu_free.argtypes = [C.c_void_p]
    L.gpu_memcpy_h2d.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    L.gpu_grad_sumsq.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_double)]
    L.gpu_mem_info.argtypes = [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
    assert L.gpu_available() == 1
    n = 8 * 1024 * 1024                                    # 32 MB of floats: above the threshold
    free0, tot = C.c_size_t(), C.c_size_t()
    L.gpu_mem_info(C.byref(free0), C.byref(tot))
    big, small = L.gpu_malloc(4 * n), L.gpu_malloc(4096)
    assert big and small
    host = np.random.default_rng(0).normal(0, 1e-3, n).astype(np.float32)
    assert L.gpu_memcpy_h2d(big, host.ctypes.data, host.nbytes) == 0
    ss = C.c_double()
    assert L.gpu_grad_sumsq(big, n, C.byref(ss)) == 0
    want = float((host.astype(np.float64) ** 2).sum())
    assert abs(ss.value - want) <= 1e-12 * want
    L.gpu_free(big)
    L.gpu_free(small)
    free1 = C.c_size_t()
    L.gpu_mem_info(C.byref(free1), C.byref(tot))
    assert free1.value >= free0.value - (4 << 20)          # the block went back
