"""ctypes binding of ``libanni_b200.so`` -- the only way Python reaches the kernels.

Loading fails loudly when the library is missing or cannot be built: there is no
Python or CPU implementation of the step to fall back on.
"""
import ctypes as C
import os

from . import build as _build

_LIB = None

DT_F32, DT_BF16 = 0, 1
SEG_WD, SEG_TWIN_BF16, SEG_TWIN_FP8 = 1, 2, 4
STEP_CHECK_FINITE, STEP_ZERO_GRAD, STEP_DEV_LOSS_SCALE, STEP_EXACT_UPDATE = 1, 2, 4, 8
STEP_REDUCE_CLEARS_OWN = 16     # peer-memory ZeRO-1: the reduce clears this rank's own arena part
OK, E_ARG, E_CUDA, E_BARRIER_TIMEOUT, E_NOMEM, E_LIMIT = 0, -1, -2, -3, -4, -5
NOALLOC_MAX_SEG = 1024
RANGE_ACCUMULATE, RANGE_LAST, RANGE_LOCAL_TWINS, RANGE_FIRST = 1, 2, 4, 8


class Config(C.Structure):
    _fields_ = [("n_arena", C.c_uint64), ("shard_off", C.c_uint64), ("shard_n", C.c_uint64),
                ("grad_dtype", C.c_int), ("state_dtype", C.c_int), ("n_seg", C.c_int),
                ("seg_off", C.c_void_p), ("seg_flags", C.c_void_p)]


class Buffers(C.Structure):
    _fields_ = [("master", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
                ("grad", C.c_void_p), ("twin_bf16", C.c_void_p), ("twin_fp8", C.c_void_p)]


class Hyper(C.Structure):
    _fields_ = [("lr", C.c_double), ("beta1", C.c_double), ("beta2", C.c_double),
                ("eps", C.c_double), ("weight_decay", C.c_double), ("grad_clip", C.c_double),
                ("grad_scale", C.c_double), ("t", C.c_int), ("flags", C.c_int)]


class SegDerived(C.Structure):
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("pack_off", C.c_int64),
                ("pack_ld", C.c_int32), ("reserved", C.c_int32), ("fp8_t_off", C.c_int64)]


class Status(C.Structure):
    _fields_ = [("sumsq", C.c_double), ("norm", C.c_double), ("eff_scale", C.c_double),
                ("loss_scale", C.c_double), ("skipped", C.c_int32), ("error", C.c_int32),
                ("good_steps", C.c_int32), ("steps_done", C.c_int32)]


class Zero1Config(C.Structure):
    """anni_zero1_config (include/anni_zero1.h)."""
    _fields_ = [("n_arena", C.c_uint64), ("grad_dtype", C.c_int), ("state_dtype", C.c_int),
                ("n_seg", C.c_int), ("seg_off", C.c_void_p), ("seg_flags", C.c_void_p),
                ("rank", C.c_int), ("world", C.c_int), ("nccl_comm", C.c_void_p),
                ("grad_arena", C.c_void_p), ("twin_arena", C.c_void_p), ("twin_fp8_arena", C.c_void_p),
                ("peer_grad", C.c_void_p), ("peer_twin", C.c_void_p), ("peer_twin_fp8", C.c_void_p),
                ("mc_grad", C.c_void_p), ("mc_twin", C.c_void_p), ("mc_twin_fp8", C.c_void_p)]


ZERO1_GRADS_COMPLETE = 1
ZERO1_UNIQUE_ID_BYTES = 128


def lib():
    """The loaded library (built on first use when nvcc is available)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _build.LIB
    if not os.path.exists(path) or (_build.needs_build() and _build.shutil.which("nvcc")):
        path = _build.build()
    # RTLD_LOCAL on purpose: the library defines the reference's gpu_* symbol set, which must not
    # interpose the same names inside other libraries of the process (e.g. the CPU checker).
    L = C.CDLL(path, mode=C.RTLD_LOCAL)
    vp, i, d = C.c_void_p, C.c_int, C.c_double
    L.anni_optstep_create.restype = i
    L.anni_optstep_create.argtypes = [C.POINTER(Config), C.POINTER(vp)]
    L.anni_optstep_destroy.restype = None
    L.anni_optstep_destroy.argtypes = [vp]
    L.anni_optstep_bind.restype = i
    L.anni_optstep_bind.argtypes = [vp, C.POINTER(Buffers)]
    for name in ("anni_optstep_step", "anni_optstep_norm", "anni_optstep_update"):
        f = getattr(L, name)
        f.restype = i
        f.argtypes = [vp, C.POINTER(Hyper), vp]
    L.anni_optstep_step_with_sumsq.restype = i
    L.anni_optstep_step_with_sumsq.argtypes = [vp, C.POINTER(Hyper), vp, vp]
    L.anni_optstep_set_derived.restype = i
    L.anni_optstep_set_derived.argtypes = [vp, vp, vp, vp]
    L.anni_optstep_set_peers.restype = i
    L.anni_optstep_set_peers.argtypes = [vp, vp, vp, vp, i, C.c_uint64]
    L.anni_optstep_set_multicast.restype = i
    L.anni_optstep_set_multicast.argtypes = [vp, vp, vp, vp, C.c_uint64]
    L.anni_optstep_rotate_peers.restype = i
    L.anni_optstep_rotate_peers.argtypes = [vp, i]
    L.anni_optstep_set_grad_arena.restype = i
    L.anni_optstep_set_grad_arena.argtypes = [vp, vp, C.c_uint64, i]
    L.anni_optstep_reduce_norm.restype = i
    L.anni_optstep_reduce_norm.argtypes = [vp, C.POINTER(Hyper), vp]
    L.anni_optstep_reduce_norm_range.restype = i
    L.anni_optstep_reduce_norm_range.argtypes = [vp, C.POINTER(Hyper), C.c_uint64, C.c_uint64, i, vp]
    L.anni_optstep_update_range.restype = i
    L.anni_optstep_update_range.argtypes = [vp, C.POINTER(Hyper), C.c_uint64, C.c_uint64, i, vp]
    L.anni_optstep_quantize_ex.restype = i
    L.anni_optstep_quantize_ex.argtypes = [vp, i, vp]
    L.anni_peer_copy.restype = i
    L.anni_peer_copy.argtypes = [vp, vp, C.c_size_t, vp]
    L.anni_arena_alloc.restype = i
    L.anni_arena_alloc.argtypes = [C.c_size_t, C.POINTER(vp), C.POINTER(C.c_size_t), C.POINTER(i)]
    L.anni_arena_free.restype = i
    L.anni_arena_free.argtypes = [vp, C.c_size_t]
    L.anni_optstep_selftest_barrier_timeout.restype = i
    L.anni_optstep_selftest_barrier_timeout.argtypes = [vp, C.c_uint, vp]
    L.anni_optstep_quantize.restype = i
    L.anni_optstep_quantize.argtypes = [vp, vp]
    for name in ("anni_optstep_reduce_buffer", "anni_optstep_amax_buffer",
                 "anni_optstep_scale_buffer"):
        f = getattr(L, name)
        f.restype = vp
        f.argtypes = [vp]
    L.anni_optstep_status_read.restype = i
    L.anni_optstep_status_read.argtypes = [vp, C.POINTER(Status), vp]
    L.anni_optstep_loss_scale_init.restype = i
    L.anni_optstep_loss_scale_init.argtypes = [vp, d, i, d, d, d, d]
    L.anni_optstep_grid.restype = i
    L.anni_optstep_grid.argtypes = [vp, C.POINTER(i), C.POINTER(i)]
    L.anni_optstep_step_noalloc.restype = i
    L.anni_optstep_step_noalloc.argtypes = [C.POINTER(Config), C.POINTER(Buffers), C.POINTER(Hyper), vp, vp]
    L.anni_optstep_status_noalloc.restype = i
    L.anni_optstep_status_noalloc.argtypes = [C.POINTER(Status), vp]
    L.anni_zero1_geometry.restype = i
    L.anni_zero1_geometry.argtypes = [C.c_uint64, i, i] + [C.POINTER(C.c_uint64)] * 3
    L.anni_zero1_nccl_available.restype = i
    L.anni_zero1_unique_id.restype = i
    L.anni_zero1_unique_id.argtypes = [vp]
    L.anni_zero1_comm_init.restype = i
    L.anni_zero1_comm_init.argtypes = [vp, i, i, C.POINTER(vp)]
    L.anni_zero1_comm_free.restype = None
    L.anni_zero1_comm_free.argtypes = [vp]
    L.anni_zero1_create.restype = i
    L.anni_zero1_create.argtypes = [C.POINTER(Zero1Config), C.POINTER(vp)]
    L.anni_zero1_bind.restype = i
    L.anni_zero1_bind.argtypes = [vp, vp, vp, vp, vp]
    L.anni_zero1_set_grad_arena.restype = i
    L.anni_zero1_set_grad_arena.argtypes = [vp, vp, vp, vp]
    L.anni_zero1_step.restype = i
    L.anni_zero1_step.argtypes = [vp, C.POINTER(Hyper), i, vp, vp]
    L.anni_zero1_engine.restype = vp
    L.anni_zero1_engine.argtypes = [vp]
    L.anni_zero1_destroy.restype = None
    L.anni_zero1_destroy.argtypes = [vp]
    L.anni_kernel_launches.restype = C.c_uint64
    L.anni_kernel_launches.argtypes = []
    _LIB = L
    return L


class AnniError(RuntimeError):
    def __init__(self, what, code):
        names = {E_ARG: "bad argument", E_CUDA: "CUDA call failed",
                 E_BARRIER_TIMEOUT: "bounded device wait timed out",
                 E_NOMEM: "out of memory", E_LIMIT: "size beyond the stated maximum"}
        super().__init__(f"{what}: {names.get(code, 'error')} ({code})")
        self.code = code


def check(what, code):
    if code != OK:
        raise AnniError(what, code)
