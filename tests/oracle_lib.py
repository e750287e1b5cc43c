"""ctypes bindings of the two CPU checkers (test infrastructure only).

``Oracle`` wraps ``oracle/liboracle.so`` (this repository's C restatement of the
reference step).  ``RefLib`` wraps ``oracle/_ref/libannref.so`` (the reference's own
CPU sources compiled by ``oracle/Makefile``); it exists only where that file was
built, so everything that needs it is skipped when it is absent.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libannref.so")

DT_F32, DT_BF16 = 0, 1
SEG_WD, SEG_TWIN_BF16, SEG_TWIN_FP8 = 1, 2, 4


def build_oracle():
    """Compile the checkers (liboracle.so always, _ref when the reference is present)."""
    subprocess.run(["make", "-s", "-C", ORACLE_DIR, "all"], check=True)


class StepArgs(C.Structure):
    _fields_ = [
        ("n", C.c_int64), ("param", C.c_void_p), ("grad", C.c_void_p),
        ("m", C.c_void_p), ("v", C.c_void_p),
        ("grad_dtype", C.c_int), ("state_dtype", C.c_int),
        ("n_seg", C.c_int), ("seg_off", C.c_void_p), ("seg_flags", C.c_void_p),
        ("lr", C.c_double), ("beta1", C.c_double), ("beta2", C.c_double),
        ("eps", C.c_double), ("weight_decay", C.c_double), ("grad_clip", C.c_double),
        ("grad_scale", C.c_double), ("t_before", C.c_int), ("check_finite", C.c_int),
        ("zero_grad", C.c_int),
        ("norm", C.c_double), ("eff_scale", C.c_double), ("skipped", C.c_int),
        ("t_after", C.c_int),
    ]


class LossScaler(C.Structure):
    _fields_ = [("scale", C.c_double), ("good_steps", C.c_int),
                ("growth_interval", C.c_int), ("growth", C.c_double),
                ("backoff", C.c_double), ("min_scale", C.c_double),
                ("max_scale", C.c_double)]


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build_oracle()
        L = C.CDLL(ORACLE_SO)
        L.oracle_bf16_rne.restype = C.c_uint16
        L.oracle_bf16_rne.argtypes = [C.c_float]
        L.oracle_fp8_e4m3_satfinite.restype = C.c_uint8
        L.oracle_fp8_e4m3_satfinite.argtypes = [C.c_float]
        L.oracle_fp8_e4m3_to_f32.restype = C.c_float
        L.oracle_fp8_e4m3_to_f32.argtypes = [C.c_uint8]
        L.oracle_sumsq.restype = C.c_double
        L.oracle_sumsq.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_double]
        L.oracle_adam_step.restype = C.c_int
        L.oracle_adam_step.argtypes = [C.POINTER(StepArgs)]
        L.oracle_twin_bf16.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        L.oracle_fp8_tensor_quant.argtypes = [C.c_void_p, C.c_int64, C.c_void_p,
                                              C.c_void_p, C.c_void_p]
        L.oracle_lr_schedule.restype = C.c_double
        L.oracle_lr_schedule.argtypes = [C.c_double, C.c_int, C.c_int, C.c_int,
                                         C.c_char_p, C.c_int]
        L.oracle_loss_scale_update.argtypes = [C.POINTER(LossScaler), C.c_int]
        L.oracle_ckpt_write_adam.restype = C.c_int
        L.oracle_ckpt_write_adam.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int,
                                             C.c_int, C.c_int64, C.c_void_p, C.c_void_p]
        L.oracle_ckpt_read_adam.restype = C.c_int
        L.oracle_ckpt_read_adam.argtypes = [C.c_char_p, C.c_int64] + [C.c_void_p] * 6 + [C.c_int64]
        self.L = L

    # -- formats -------------------------------------------------------------
    def bf16_rne(self, x):
        """fp32 array -> uint16 array of bf16 bit patterns (round to nearest even)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.uint16)
        self.L.oracle_twin_bf16(_ptr(x), x.size, _ptr(out))
        return out

    @staticmethod
    def bf16_to_f32(h):
        return (np.asarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)

    def fp8_quant(self, p):
        p = np.ascontiguousarray(p, dtype=np.float32)
        amax = np.zeros(1, np.float32)
        scale = np.zeros(1, np.float32)
        q = np.empty(p.size, np.uint8)
        self.L.oracle_fp8_tensor_quant(_ptr(p), p.size, _ptr(amax), _ptr(scale), _ptr(q))
        return float(amax[0]), float(scale[0]), q

    def sumsq(self, g, scale=1.0):
        dt = DT_BF16 if g.dtype == np.uint16 else DT_F32
        return self.L.oracle_sumsq(_ptr(g), dt, g.size, scale)

    # -- the step --------------------------------------------------------------
    def step(self, p, g, m, v, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0,
             clip=0.0, grad_scale=1.0, t_before=0, check_finite=False, zero_grad=True,
             seg_off=None, seg_flags=None):
        """In-place step on numpy arrays.  g / m / v may be float32 or uint16 (bf16 bits).

        Returns a dict(norm, eff_scale, skipped, t_after)."""
        assert p.dtype == np.float32 and p.flags.c_contiguous
        a = StepArgs()
        a.n = p.size
        a.param, a.grad, a.m, a.v = _ptr(p), _ptr(g), _ptr(m), _ptr(v)
        a.grad_dtype = DT_BF16 if g.dtype == np.uint16 else DT_F32
        assert m.dtype == v.dtype
        a.state_dtype = DT_BF16 if m.dtype == np.uint16 else DT_F32
        if seg_off is not None:
            so = np.ascontiguousarray(seg_off, dtype=np.int64)
            sf = np.ascontiguousarray(seg_flags, dtype=np.uint32)
            assert so.size == sf.size + 1
            a.n_seg, a.seg_off, a.seg_flags = sf.size, _ptr(so), _ptr(sf)
        a.lr, a.beta1, a.beta2, a.eps = lr, beta1, beta2, eps
        a.weight_decay, a.grad_clip, a.grad_scale = wd, clip, grad_scale
        a.t_before, a.check_finite, a.zero_grad = t_before, int(check_finite), int(zero_grad)
        rc = self.L.oracle_adam_step(C.byref(a))
        assert rc == 0
        return dict(norm=a.norm, eff_scale=a.eff_scale, skipped=bool(a.skipped),
                    t_after=a.t_after)

    def lr_schedule(self, base, step, warmup, decay, kind="cosine", start=0):
        return self.L.oracle_lr_schedule(base, step, warmup, decay, kind.encode(), start)

    def loss_scaler(self, scale=65536.0, growth_interval=200, growth=2.0, backoff=0.5,
                    min_scale=1.0, max_scale=2.0 ** 24):
        return LossScaler(scale, 0, growth_interval, growth, backoff, min_scale, max_scale)

    def loss_scale_update(self, s, skipped):
        self.L.oracle_loss_scale_update(C.byref(s), int(skipped))

    def ckpt_write_adam(self, path, m, v, *, t, epoch=0, step=0, append=False):
        m = np.ascontiguousarray(m, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        rc = self.L.oracle_ckpt_write_adam(path.encode(), int(append), epoch, step, t,
                                           m.size, _ptr(m), _ptr(v))
        assert rc == 0


class RefLib:
    """The reference's own CPU object code.  ``available()`` is False on machines where
    ``oracle/_ref/libannref.so`` was never built."""

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def __init__(self):
        L = C.CDLL(REF_SO)
        d = C.c_double
        L.ref_adam_step.restype = C.c_int
        L.ref_adam_step.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_int] + [d] * 7
        L.ref_adam_bench_create.restype = C.c_void_p
        L.ref_adam_bench_create.argtypes = [C.c_void_p, C.c_void_p, C.c_int, d, d, d, d, d, C.c_int]
        L.ref_adam_bench_step.argtypes = [C.c_void_p, d, d]
        L.ref_adam_bench_free.argtypes = [C.c_void_p]
        L.ref_step_lr.restype = d
        L.ref_step_lr.argtypes = [d, C.c_int, C.c_int, C.c_int, C.c_char_p, C.c_int]
        L.ref_ckpt_save.restype = C.c_int
        L.ref_ckpt_save.argtypes = [C.c_char_p, C.c_int, C.c_void_p, C.c_void_p,
                                    C.POINTER(C.c_int), C.c_int, C.c_int, C.c_int]
        L.ref_ckpt_load.restype = C.c_int
        L.ref_ckpt_load.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_int] + \
            [C.POINTER(C.c_int)] * 4
        L.ref_ckpt_save_full.restype = C.c_int
        L.ref_ckpt_save_full.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.POINTER(C.c_int), C.c_int, C.c_int, C.c_int]
        L.ref_ckpt_load_full.restype = C.c_int
        L.ref_ckpt_load_full.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int] + \
            [C.POINTER(C.c_int)] * 6
        L.ref_seg_list.restype = C.c_int
        L.ref_seg_list.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        self.L = L

    def step(self, p, g, m, v, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, clip=0.0,
             grad_scale=1.0, t_before=0):
        for a in (p, g, m, v):
            assert a.dtype == np.float32 and a.flags.c_contiguous
        rc = self.L.ref_adam_step(_ptr(p), _ptr(g), _ptr(m), _ptr(v), p.size, t_before,
                                  lr, beta1, beta2, eps, wd, clip, grad_scale)
        assert rc == 0, rc

    def lr_schedule(self, base, step, warmup, decay, kind="cosine", start=0):
        return self.L.ref_step_lr(base, step, warmup, decay, kind.encode(), start)

    def slot_count(self, vocab):
        n = C.c_int(0)
        rc = self.L.ref_ckpt_save(b"", vocab, None, None, C.byref(n), 0, 0, 0)
        assert rc == 0
        return n.value

    def ckpt_save(self, path, vocab, m, v, *, t, epoch, step):
        n = C.c_int(m.size)
        rc = self.L.ref_ckpt_save(path.encode(), vocab, _ptr(m), _ptr(v), C.byref(n),
                                  t, epoch, step)
        assert rc == 0, rc

    def ckpt_load(self, path, n):
        m = np.zeros(n, np.float32)
        v = np.zeros(n, np.float32)
        no, t, ep, st = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        rc = self.L.ref_ckpt_load(path.encode(), _ptr(m), _ptr(v), n, C.byref(no),
                                  C.byref(t), C.byref(ep), C.byref(st))
        assert rc == 0, rc
        return dict(n=no.value, t=t.value, epoch=ep.value, step=st.value, m=m, v=v)

    def full_slot_count(self, mode, n_merges):
        n = C.c_int(0)
        assert self.L.ref_ckpt_save_full(b"", mode, n_merges, None, None, None, C.byref(n), 0, 0, 0) == 0
        return n.value

    def ckpt_save_full(self, path, mode, n_merges, w, m, v, *, t, epoch, step):
        """mode 0: byte-level model (LMCF); 1: BPE embedded (LMCV); 2: BPE + tied embedding (LMCT)."""
        n = C.c_int(w.size)
        rc = self.L.ref_ckpt_save_full(path.encode(), mode, n_merges, _ptr(w), _ptr(m), _ptr(v),
                                       C.byref(n), t, epoch, step)
        assert rc == 0, rc

    def ckpt_load_full(self, path, n):
        w, m, v = (np.zeros(n, np.float32) for _ in range(3))
        out = [C.c_int() for _ in range(6)]
        rc = self.L.ref_ckpt_load_full(path.encode(), _ptr(w), _ptr(m), _ptr(v), n, *[C.byref(o) for o in out])
        assert rc == 0, rc
        no, t, ep, st, vocab, tied = (o.value for o in out)
        return dict(n=no, t=t, epoch=ep, step=st, vocab=vocab, tied=tied, w=w, m=m, v=v)

    def seg_list(self, vocab, cap=512):
        off = np.zeros(cap, np.int32)
        n = np.zeros(cap, np.int32)
        isv = np.zeros(cap, np.int32)
        ns = self.L.ref_seg_list(vocab, _ptr(off), _ptr(n), _ptr(isv), cap)
        assert ns > 0
        return off[:ns].copy(), n[:ns].copy(), isv[:ns].copy()
