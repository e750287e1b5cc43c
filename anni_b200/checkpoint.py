"""Adam section of the reference checkpoint (``lang/lm_serialize.c:263-331``).

Layout: int32 ``{1, epoch, step, t, n}`` then ``n`` interleaved ``(m, v)`` fp32 pairs in
optimizer (arena) order -- 20 + 8 n bytes at the end of the file.  m and v are always fp32
on disk, whatever the device keeps them in.  The byte work is done by the library
(``anni_ckpt_write_adam`` / ``anni_ckpt_read_adam``).
"""
import ctypes as C

import numpy as np

from . import capi


def _lib():
    L = capi.lib()
    L.anni_ckpt_write_adam.restype = C.c_int
    L.anni_ckpt_write_adam.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64,
                                       C.c_void_p, C.c_void_p]
    L.anni_ckpt_read_adam.restype = C.c_int
    L.anni_ckpt_read_adam.argtypes = [C.c_char_p, C.c_int64, C.c_int64, C.POINTER(C.c_int),
                                      C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_void_p, C.c_void_p]
    return L


def write_adam(path, m, v, *, t, epoch=0, step=0, append=False):
    """Write (or append after a weight section) the Adam trailer for fp32 arrays m, v."""
    m = np.ascontiguousarray(m, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    assert m.shape == v.shape and m.ndim == 1
    capi.check("anni_ckpt_write_adam",
               _lib().anni_ckpt_write_adam(path.encode(), int(append), epoch, step, t, m.size,
                                           m.ctypes.data, v.ctypes.data))


def read_adam(path, n, offset=-1):
    """Read the trailer of a checkpoint whose optimizer has n slots; returns dict(t, epoch, step, m, v)."""
    m = np.empty(n, np.float32)
    v = np.empty(n, np.float32)
    ep, st, t = C.c_int(), C.c_int(), C.c_int()
    capi.check("anni_ckpt_read_adam",
               _lib().anni_ckpt_read_adam(path.encode(), offset, n, C.byref(ep), C.byref(st),
                                          C.byref(t), m.ctypes.data, v.ctypes.data))
    return dict(t=t.value, epoch=ep.value, step=st.value, m=m, v=v)


# ---- whole checkpoints (weight section + Adam section) -------------------------------------

class CkptModel(C.Structure):
    """Mirror of anni_ckpt_model (include/anni_lm_adam.h)."""
    _fields_ = [("kind", C.c_int), ("d_model", C.c_int), ("n_heads", C.c_int), ("d_ff", C.c_int),
                ("max_ctx", C.c_int), ("n_blocks", C.c_int), ("vocab", C.c_int), ("tied", C.c_int),
                ("n_merges", C.c_int), ("merges_word", C.c_int), ("n", C.c_int64),
                ("has_adam", C.c_int), ("epoch", C.c_int), ("step", C.c_int), ("t", C.c_int)]


def _lib_full():
    L = _lib()
    L.anni_ckpt_probe.restype = C.c_int
    L.anni_ckpt_probe.argtypes = [C.c_char_p, C.POINTER(CkptModel)]
    L.anni_ckpt_load.restype = C.c_int
    L.anni_ckpt_load.argtypes = [C.c_char_p, C.POINTER(CkptModel)] + [C.c_void_p] * 4
    L.anni_ckpt_save.restype = C.c_int
    L.anni_ckpt_save.argtypes = [C.c_char_p, C.POINTER(CkptModel)] + [C.c_void_p] * 4
    return L


def probe(path):
    """Header of a reference-format checkpoint (dimensions, kind, slot count, Adam header)."""
    k = CkptModel()
    capi.check("anni_ckpt_probe", _lib_full().anni_ckpt_probe(path.encode(), C.byref(k)))
    return k


def load_model(path):
    """Whole checkpoint: weights, m, v as fp32 arrays in optimizer (arena) order, merge pairs."""
    L = _lib_full()
    k = probe(path)
    w = np.empty(k.n, np.float32)
    m = np.zeros(k.n, np.float32)
    v = np.zeros(k.n, np.float32)
    merges = np.zeros((max(k.n_merges, 1), 2), np.int32)
    capi.check("anni_ckpt_load", L.anni_ckpt_load(path.encode(), C.byref(k), w.ctypes.data,
                                                  m.ctypes.data, v.ctypes.data, merges.ctypes.data))
    return dict(info=k, w=w, m=m if k.has_adam else None, v=v if k.has_adam else None,
                merges=merges[:k.n_merges])


def save_model(path, info, w, m=None, v=None, merges=None):
    """Write a checkpoint the reference trainer loads (lm_save_checkpoint's bytes); m = v = None
    writes the weights-only form (lm_save)."""
    L = _lib_full()
    w = np.ascontiguousarray(w, np.float32)
    assert w.size == info.n
    if m is not None:
        m = np.ascontiguousarray(m, np.float32)
        v = np.ascontiguousarray(v, np.float32)
    mg = np.ascontiguousarray(merges, np.int32) if merges is not None and len(merges) else None
    capi.check("anni_ckpt_save",
               L.anni_ckpt_save(path.encode(), C.byref(info), mg.ctypes.data if mg is not None else None,
                                w.ctypes.data, m.ctypes.data if m is not None else None,
                                v.ctypes.data if v is not None else None))
