"""ctypes mirror of the library's optimizer object (``include/anni_lm_adam.h``), the C-side
counterpart of the reference's ``lm_adam`` (``lang/lm_adam.h``): same field names, same calls
(``create / step / step_scaled / zero_grad / invalidate / sync_host / set_offload / free``).
What a C trainer does with the struct, Python does through ``opt.contents``."""
import ctypes as C

from . import capi

d = C.c_double


class Tensor(C.Structure):
    """anni_lm_tensor: host weights, host gradients (or NULL), element count, ANNI_SEG_* flags."""
    _fields_ = [("w", C.c_void_p), ("dw", C.c_void_p), ("n", C.c_int64), ("flags", C.c_uint32)]


class Seg(C.Structure):
    _fields_ = [("w", C.c_void_p), ("dw", C.c_void_p), ("off", C.c_int64), ("n", C.c_int64),
                ("flags", C.c_uint32), ("w_mat", C.c_void_p), ("dw_mat", C.c_void_p)]


class LmAdam(C.Structure):
    _fields_ = [("segs", C.POINTER(Seg)), ("n_segs", C.c_int), ("n", C.c_int64), ("t", C.c_int),
                ("beta1", d), ("beta2", d), ("eps", d), ("h_m", C.POINTER(C.c_float)),
                ("h_v", C.POINTER(C.c_float)), ("d_param", C.c_void_p), ("d_param_bf16", C.c_void_p),
                ("d_param_fp8", C.c_void_p), ("d_grad", C.c_void_p), ("d_m", C.c_void_p),
                ("d_v", C.c_void_p), ("dev_mv", C.c_int), ("params_valid", C.c_int),
                ("offload_mv", C.c_int), ("weight_decay", d), ("grad_clip", d), ("last_grad_norm", d),
                ("grad_dtype", C.c_int), ("state_dtype", C.c_int), ("last_skipped", C.c_int),
                ("last_error", C.c_int), ("loss_scale", d), ("exact_update", C.c_int),
                ("snap_m", C.c_void_p), ("snap_v", C.c_void_p), ("snap_stream", C.c_void_p),
                ("snap_event", C.c_void_p), ("grad_arena_bytes", C.c_size_t), ("engine", C.c_void_p)]


class Mat(C.Structure):
    """anni_mat, the reference's ``mat`` (num/mat.h:12-18)."""
    _fields_ = [("data", C.c_void_p), ("d_data", C.c_void_p), ("rows", C.c_int),
                ("cols", C.c_int), ("on_device", C.c_int)]


def lib():
    """The library with the optimizer object's entry points typed."""
    L = capi.lib()
    P = C.POINTER(LmAdam)
    L.anni_lm_adam_create.restype = P
    L.anni_lm_adam_create.argtypes = [C.POINTER(Tensor), C.c_int, C.c_int, C.c_int]
    L.anni_lm_adam_free.argtypes = [C.POINTER(P)]
    L.anni_lm_adam_step_scaled.restype = C.c_int
    L.anni_lm_adam_step_scaled.argtypes = [P, d, d]
    L.anni_lm_adam_step.restype = C.c_int
    L.anni_lm_adam_step.argtypes = [P, d]
    for name in ("anni_lm_adam_sync_host", "anni_lm_adam_prepare", "anni_lm_adam_upload_grads",
                 "anni_lm_adam_snapshot_begin", "anni_lm_adam_snapshot_finish"):
        f = getattr(L, name)
        f.restype = C.c_int
        f.argtypes = [P]
    L.anni_lm_adam_invalidate.argtypes = [P]
    L.anni_lm_adam_zero_grad.argtypes = [P]
    L.anni_lm_adam_set_offload.argtypes = [C.c_int]
    L.anni_lm_adam_set_moments.restype = C.c_int
    L.anni_lm_adam_set_moments.argtypes = [P, C.c_void_p, C.c_void_p]
    L.anni_lm_adam_alias.restype = C.c_int
    L.anni_lm_adam_alias.argtypes = [P, C.c_int, C.POINTER(Mat), C.POINTER(Mat)]
    L.anni_lm_adam_alias_vec.restype = C.c_int
    L.anni_lm_adam_alias_vec.argtypes = [P, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]
    return L


def create(segments, w_ptr, dw_ptr, grad_dtype=capi.DT_F32, state_dtype=capi.DT_F32):
    """lm_adam_create over host arrays: ``w_ptr`` / ``dw_ptr`` are the addresses of fp32 host
    arrays holding all weights / gradients back to back in ``segments`` order (``dw_ptr`` 0:
    gradients are produced on the device)."""
    L = lib()
    off = segments.offsets
    ts = (Tensor * len(segments))()
    for i in range(len(segments)):
        ts[i].w = w_ptr + 4 * int(off[i])
        ts[i].dw = dw_ptr + 4 * int(off[i]) if dw_ptr else None
        ts[i].n = segments.sizes[i]
        ts[i].flags = segments.flags[i]
    opt = L.anni_lm_adam_create(ts, len(segments), grad_dtype, state_dtype)
    if not opt:
        raise capi.AnniError("anni_lm_adam_create", capi.E_ARG)
    return opt
