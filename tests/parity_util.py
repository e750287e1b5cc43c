"""Shared helpers of the parity tests: seeded inputs, ulp distances, GPU-vs-oracle runs."""
import numpy as np
import torch

from anni_b200.capi import DT_BF16, DT_F32
from anni_b200.engine import OptStep


def f32_ulp_dist(a, b):
    """Distance in units in the last place between two float32 arrays (finite values)."""
    def key(x):
        i = np.ascontiguousarray(x, dtype=np.float32).view(np.int32).astype(np.int64)
        return np.where(i < 0, -(i & 0x7fffffff), i)
    return np.abs(key(a) - key(b))


def ulp_of(x):
    x = np.abs(np.asarray(x, dtype=np.float32))
    return np.spacing(np.maximum(x, np.float32(1.2e-38))).astype(np.float64)


def bf16_bits_from_f32(x):
    """Round-to-nearest-even bf16 bit patterns of a float32 array (numpy, independent of the oracle)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7fff + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_to_f32(h):
    return (np.asarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def make_inputs(n, seed=0, *, grad_dtype=DT_F32, state_dtype=DT_F32, grad_std=1e-3, outlier=1e-3,
                loss_scale=1.0):
    """Seeded inputs with the benchmark configurations' distributions: weights N(0,0.02),
    gradients N(0,grad_std) with a fraction `outlier` multiplied by 100, m ~ N(0,1e-4),
    v = |N(0,1e-6)|.  bf16 arrays are returned as uint16 bit patterns."""
    rng = np.random.default_rng(seed)
    p = rng.normal(0, 0.02, n).astype(np.float32)
    g = rng.normal(0, grad_std, n).astype(np.float32)
    g[rng.random(n) < outlier] *= 100.0
    g *= np.float32(loss_scale)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    if grad_dtype == DT_BF16:
        g = bf16_bits_from_f32(g)
    if state_dtype == DT_BF16:
        m, v = bf16_bits_from_f32(m), bf16_bits_from_f32(v)
    return p, g, m, v


def to_dev(a, device="cuda"):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if a.dtype == np.uint16:
        t = t.view(torch.bfloat16)
    return t.to(device)


def to_host(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def run_gpu(segs, p, g, m, v, hyper_kw, *, n_arena=None, split=False, shard=None, steps=1):
    """One step on the device through the C ABI; returns host copies and the status."""
    grad_dtype = DT_BF16 if g.dtype == np.uint16 else DT_F32
    state_dtype = DT_BF16 if m.dtype == np.uint16 else DT_F32
    so, sn = (0, None) if shard is None else shard
    eng = OptStep(segs, n_arena=n_arena if segs is None else None, grad_dtype=grad_dtype,
                  state_dtype=state_dtype, shard_off=so, shard_n=sn)
    n = eng.shard_n
    sl = slice(so, so + n)
    eng.allocate()
    eng.master[:n].copy_(to_dev(p[sl]))
    eng.grad[:n].copy_(to_dev(g[sl]))
    eng.m[:n].copy_(to_dev(m[sl]))
    eng.v[:n].copy_(to_dev(v[sl]))
    hp = OptStep.hyper(**hyper_kw)
    for _ in range(steps):
        (eng.step_split if split else eng.step)(hp)
    st = eng.status()
    out = dict(p=to_host(eng.master[:n]), g=to_host(eng.grad[:n]), m=to_host(eng.m[:n]),
               v=to_host(eng.v[:n]), twin=to_host(eng.twin_bf16[:n]),
               twin8=to_host(eng.twin_fp8[:n]) if eng.twin_fp8 is not None else None,
               status=st, scale=eng.scale_tensor().cpu().numpy(),
               amax=eng.amax_tensor().cpu().numpy())
    eng.close()
    return out


def check_step(out, ref_p, ref_m, ref_v, p_old, *, exact_moments, m_old=None, beta1=0.9):
    """The parity bar of one step.

    m, v: bit-identical when the gradient multiplier is bit-identical (clipping inactive);
    otherwise at most 1 ulp apart (the multiplier then differs in its last double bits
    because the norm is summed in a different order).  With ``m_old`` (the first moment before
    the step) the bar for m is one ulp of the LARGER OPERAND of beta1*m + (1-beta1)*g instead of
    one ulp of the result: where the two nearly cancel, a last-bit difference of the multiplier is
    more than an ulp of the small result -- among hundreds of millions of elements that happens.
    fp32 master: within 2 ulp of the larger of |p_old|, |p_ref| plus 1e-6 of the size of the update."""
    half = ref_m.dtype == np.uint16
    if half:
        dm = np.abs(out["m"].astype(np.int64) - ref_m.astype(np.int64))
        dv = np.abs(out["v"].astype(np.int64) - ref_v.astype(np.int64))
    else:
        dm = f32_ulp_dist(out["m"], ref_m)
        dv = f32_ulp_dist(out["v"], ref_v)
    if exact_moments:
        assert dm.max() == 0 and dv.max() == 0, (dm.max(), dv.max())
    else:
        if m_old is None:
            assert dm.max() <= 1, dm.max()
        else:
            f = (lambda a: bf16_to_f32(a)) if half else (lambda a: a)
            big = np.maximum(np.abs(f(ref_m)), np.float32(beta1) * np.abs(f(m_old)))
            tol = ulp_of(big) * (65536.0 if half else 1.0)
            err = np.abs(f(out["m"]).astype(np.float64) - f(ref_m).astype(np.float64))
            assert (err <= tol).all(), float((err / tol).max())
        assert dv.max() <= 1, dv.max()
        assert (dm == 0).mean() > 0.999 and (dv == 0).mean() > 0.999
    dp = np.abs(out["p"].astype(np.float64) - ref_p.astype(np.float64))
    tol = 2.0 * ulp_of(np.maximum(np.abs(p_old), np.abs(ref_p))) \
        + 1e-6 * np.abs(p_old.astype(np.float64) - ref_p.astype(np.float64))
    bad = dp > tol
    assert not bad.any(), (int(bad.sum()), float((dp / tol).max()))
    return dict(p_exact=float((dp == 0).mean()), p_max_ulp=int(f32_ulp_dist(out["p"], ref_p).max()))


def check_step_chunked(out, ref_p, ref_m, ref_v, p_old, *, exact_moments, m_old=None, chunk=1 << 25):
    """check_step over slices, so that a full-size arena (hundreds of millions of elements) is
    compared without float64 temporaries of the whole arena; returns the merged statistics."""
    n = ref_p.size
    exact = 0
    worst = 0
    for lo in range(0, n, chunk):
        sl = slice(lo, min(n, lo + chunk))
        part = {k: out[k][sl] for k in ("p", "m", "v")}
        st = check_step(part, ref_p[sl], ref_m[sl], ref_v[sl], p_old[sl], exact_moments=exact_moments,
                        m_old=None if m_old is None else m_old[sl])
        exact += st["p_exact"] * (sl.stop - sl.start)
        worst = max(worst, st["p_max_ulp"])
    return dict(p_exact=exact / n, p_max_ulp=worst)


def device_inputs(n, seed, *, grad_dtype=DT_F32, state_dtype=DT_F32, grad_std=1e-3, device="cuda"):
    """make_inputs' distributions drawn on the device (seconds instead of minutes at 555 M
    elements), returned as host arrays in the same conventions (bf16 as uint16 bit patterns)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    p = torch.empty(n, device=device).normal_(0, 0.02, generator=gen)
    g = torch.empty(n, device=device).normal_(0, grad_std, generator=gen)
    chunk = 1 << 27
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        g[lo:hi][torch.rand(hi - lo, device=device, generator=gen) < 1e-3] *= 100.0
    m = torch.empty(n, device=device).normal_(0, 1e-4, generator=gen)
    v = torch.empty(n, device=device).normal_(0, 1e-6, generator=gen).abs_()
    if grad_dtype == DT_BF16:
        g = g.to(torch.bfloat16)
    if state_dtype == DT_BF16:
        m, v = m.to(torch.bfloat16), v.to(torch.bfloat16)
    out = tuple(to_host(x) for x in (p, g, m, v))
    del p, g, m, v
    torch.cuda.empty_cache()
    return out
