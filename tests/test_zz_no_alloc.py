"""The allocation-free entry point against the regular engine (collected last on purpose).

``anni_optstep_step_noalloc`` is for callers that may not allocate device memory once
they are running -- a trainer whose own arena owns the whole GPU, or code inside a region
where the CUDA allocator must not be entered.  Its working memory is an array built into
the library instead of a block from cudaMalloc, so every call on a device shares it and
must clear it first.  The test therefore runs TWO steps in a row through the C ABI (the
second one meets whatever the first left in that array) and compares parameters, moments,
twins, gradients and the reported norm with the engine-based ``anni_optstep_step`` on the
same inputs.  Both paths launch the same kernel with the same grid, so the comparison is
bit for bit, tighter than the ulp tolerances of the oracle tests.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from anni_b200 import capi
from anni_b200.capi import DT_BF16, DT_F32, SEG_TWIN_BF16, SEG_TWIN_FP8, SEG_WD
from anni_b200.engine import LM_SHAPES, OptStep, Segments, lm_segments
from parity_util import make_inputs, to_dev, to_host

pytestmark = pytest.mark.gpu


def _noalloc_steps(segs, p, g_list, m, v, grad_dtype, state_dtype, hypers):
    L = capi.lib()
    n = segs.n
    off = np.ascontiguousarray(segs.offsets)
    flg = np.ascontiguousarray(segs.flag_array)
    cfg = capi.Config()
    cfg.n_arena, cfg.shard_off, cfg.shard_n = n, 0, n
    cfg.grad_dtype, cfg.state_dtype, cfg.n_seg = grad_dtype, state_dtype, len(segs)
    cfg.seg_off, cfg.seg_flags = off.ctypes.data, flg.ctypes.data
    has_fp8 = bool((flg & SEG_TWIN_FP8).any())
    # every buffer is the caller's; the library allocates nothing
    d = dict(p=to_dev(p), m=to_dev(m), v=to_dev(v), g=to_dev(g_list[0]),
             t16=torch.zeros(n, dtype=torch.bfloat16, device="cuda"),
             t8=torch.zeros(n, dtype=torch.uint8, device="cuda") if has_fp8 else None,
             sc=torch.zeros(len(segs), dtype=torch.float32, device="cuda"))
    buf = capi.Buffers()
    buf.master, buf.m, buf.v, buf.grad = (d["p"].data_ptr(), d["m"].data_ptr(), d["v"].data_ptr(),
                                          d["g"].data_ptr())
    buf.twin_bf16 = d["t16"].data_ptr()
    buf.twin_fp8 = d["t8"].data_ptr() if has_fp8 else None
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    norms = []
    for g, hp in zip(g_list, hypers):
        d["g"].copy_(to_dev(g))
        rc = L.anni_optstep_step_noalloc(C.byref(cfg), C.byref(buf), C.byref(hp),
                                         C.c_void_p(d["sc"].data_ptr()), stream)
        assert rc == capi.OK, rc
        st = capi.Status()
        assert L.anni_optstep_status_noalloc(C.byref(st), stream) == capi.OK
        assert st.error == 0
        norms.append((st.norm, st.skipped))
    out = {k: (to_host(t) if t is not None else None) for k, t in d.items()}
    out["norms"] = norms
    return out


def _engine_steps(segs, p, g_list, m, v, grad_dtype, state_dtype, hypers):
    eng = OptStep(segs, grad_dtype=grad_dtype, state_dtype=state_dtype).allocate()
    n = segs.n
    eng.master.copy_(to_dev(p))
    eng.m.copy_(to_dev(m))
    eng.v.copy_(to_dev(v))
    norms = []
    for g, hp in zip(g_list, hypers):
        eng.grad.copy_(to_dev(g))
        eng.step(hp)
        st = eng.status()
        norms.append((st.norm, st.skipped))
    out = dict(p=to_host(eng.master[:n]), m=to_host(eng.m[:n]), v=to_host(eng.v[:n]),
               g=to_host(eng.grad[:n]), t16=to_host(eng.twin_bf16[:n]),
               t8=to_host(eng.twin_fp8[:n]) if eng.twin_fp8 is not None else None,
               sc=eng.scale_tensor().cpu().numpy(), norms=norms)
    eng.close()
    return out


@pytest.mark.parametrize("grad_dtype,state_dtype,twin", [(DT_BF16, DT_BF16, "bf16"),
                                                         (DT_F32, DT_F32, "bf16"),
                                                         (DT_BF16, DT_F32, "fp8")])
def test_noalloc_matches_engine_two_steps_in_a_row(grad_dtype, state_dtype, twin):
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin=twin)
    p, g0, m, v = make_inputs(segs.n, seed=21, grad_dtype=grad_dtype, state_dtype=state_dtype)
    _, g1, _, _ = make_inputs(segs.n, seed=22, grad_dtype=grad_dtype, state_dtype=state_dtype,
                              grad_std=1e-5)        # second step: small norm, no clipping
    hypers = [OptStep.hyper(lr=3e-4, t=1000 + i, beta2=0.95, wd=0.1, clip=1.0) for i in range(2)]
    a = _noalloc_steps(segs, p, [g0, g1], m, v, grad_dtype, state_dtype, hypers)
    b = _engine_steps(segs, p, [g0, g1], m, v, grad_dtype, state_dtype, hypers)
    assert a["norms"] == b["norms"]
    assert a["norms"][0][0] > 1.0 > a["norms"][1][0] > 0.0      # step 1 clipped, step 2 not
    for key in ("p", "m", "v", "g", "t16"):
        assert np.array_equal(a[key], b[key]), key
    if twin == "fp8":
        assert np.array_equal(a["t8"], b["t8"]) and a["t8"].any()
        assert np.array_equal(a["sc"], b["sc"])


def test_noalloc_rejects_oversized_tensor_table():
    n_seg = capi.NOALLOC_MAX_SEG + 1
    segs = Segments()
    for i in range(n_seg):
        segs.add(f"t{i}", 8, SEG_WD | SEG_TWIN_BF16)
    off = np.ascontiguousarray(segs.offsets)
    flg = np.ascontiguousarray(segs.flag_array)
    cfg = capi.Config()
    cfg.n_arena, cfg.shard_off, cfg.shard_n = segs.n, 0, segs.n
    cfg.grad_dtype, cfg.state_dtype, cfg.n_seg = DT_F32, DT_F32, n_seg
    cfg.seg_off, cfg.seg_flags = off.ctypes.data, flg.ctypes.data
    t = torch.zeros(segs.n, device="cuda")
    buf = capi.Buffers()
    buf.master = buf.m = buf.v = buf.grad = t.data_ptr()
    hp = OptStep.hyper(lr=1e-3, t=1)
    rc = capi.lib().anni_optstep_step_noalloc(C.byref(cfg), C.byref(buf), C.byref(hp), None, None)
    assert rc == capi.E_LIMIT
    assert not t.any()
