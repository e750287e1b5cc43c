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
