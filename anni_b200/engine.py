"""Host-side mirror of the reference optimizer's interface over the packed arena.

Names follow the reference (``lang/lm_adam.h``): an optimizer owns flat device
buffers ``d_param / d_grad / d_m / d_v / d_param_bf16`` indexed by one running element
offset per tensor ("segment"), in the order ``lm_adam_create`` walks the model
(``lang/lm_adam.c:117-136``).  Here torch only provides device memory and streams; all
arithmetic happens inside ``libanni_b200.so``.
"""
import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch

from . import capi
from .capi import (DT_BF16, DT_F32, SEG_TWIN_BF16, SEG_TWIN_FP8, SEG_WD, STEP_CHECK_FINITE,
                   STEP_DEV_LOSS_SCALE, STEP_ZERO_GRAD, check)


# ---------------------------------------------------------------------------------
# segment tables
# ---------------------------------------------------------------------------------

@dataclass
class Segments:
    """Packed-arena layout: per tensor a name, an element count and ANNI_SEG_* flags."""
    names: List[str] = field(default_factory=list)
    sizes: List[int] = field(default_factory=list)
    flags: List[int] = field(default_factory=list)

    def add(self, name, n, flags):
        self.names.append(name)
        self.sizes.append(int(n))
        self.flags.append(int(flags))

    @property
    def n(self):
        return int(sum(self.sizes))

    @property
    def offsets(self):
        return np.concatenate([[0], np.cumsum(np.asarray(self.sizes, dtype=np.int64))]).astype(np.int64)

    @property
    def flag_array(self):
        return np.asarray(self.flags, dtype=np.uint32)

    def __len__(self):
        return len(self.sizes)

    def index(self, name):
        return self.names.index(name)

    def slice_of(self, name):
        i = self.index(name)
        off = self.offsets
        return slice(int(off[i]), int(off[i + 1]))


def lm_segments(d_model, d_ff, n_blocks, vocab, tied, *, wd="matrices", twin="bf16",
                attn_bias=False):
    """Segment list of a decoder-only LM in the reference's optimizer order.

    Order and shapes: ``lang/lm_adam.c:117-136`` -- ``w_head`` (D x V), ``b_head`` (V),
    the embedding table (V x D) when untied, then per block ``wq wk wv wo`` (D x D),
    ``w1`` (D x FF), ``b1``, ``w2`` (FF x D), ``b2``, ``ln1.gamma ln1.beta ln2.gamma
    ln2.beta``.  ``wd`` selects where decoupled decay applies: "matrices" (the benchmark
    configuration's wording) or "all" (what the reference kernels do,
    ``num/gpu_cuda.cu:8553``).  ``twin``: "bf16" for every tensor, or "fp8" = e4m3 for the
    block matrices with bf16 kept for vectors, the head and the embedding.
    ``attn_bias`` adds the four per-block attention bias vectors the benchmark wording
    mentions and the reference model does not have.
    """
    s = Segments()
    D, FF, V = d_model, d_ff, vocab

    def mat(name, n, fp8_ok=True):
        f = SEG_WD if wd in ("matrices", "all") else 0
        if twin == "fp8" and fp8_ok:
            f |= SEG_TWIN_FP8
        elif twin in ("bf16", "fp8"):
            f |= SEG_TWIN_BF16
        s.add(name, n, f)

    def vec(name, n):
        f = SEG_WD if wd == "all" else 0
        if twin in ("bf16", "fp8"):
            f |= SEG_TWIN_BF16
        s.add(name, n, f)

    mat("w_head", D * V, fp8_ok=False)
    vec("b_head", V)
    if not tied:
        mat("embed", V * D, fp8_ok=False)
    for b in range(n_blocks):
        for w in ("wq", "wk", "wv", "wo"):
            mat(f"blk{b}.{w}", D * D)
            if attn_bias:
                vec(f"blk{b}.b{w[1]}", D)
        mat(f"blk{b}.w1", D * FF)
        vec(f"blk{b}.b1", FF)
        mat(f"blk{b}.w2", FF * D)
        vec(f"blk{b}.b2", D)
        for v_ in ("ln1.gamma", "ln1.beta", "ln2.gamma", "ln2.beta"):
            vec(f"blk{b}.{v_}", D)
    return s


def lm_derived(segs, d_model, d_ff, *, pack_qkv=True, fp8_transposed=True):
    """Derived-twin table of an LM segment list: per layer one packed [Wq|Wk|Wv] (D x 3D) bf16
    matrix, and the e4m3 twins of the block matrices in the transposed [cols][rows] layout.
    Returns (aux list, elements of the packed buffer, bytes of the transposed buffer)."""
    D, FF = d_model, d_ff
    shapes = {"wq": (D, D), "wk": (D, D), "wv": (D, D), "wo": (D, D), "w1": (D, FF), "w2": (FF, D)}
    aux, packed, t_bytes = [], 0, 0
    for name, n, flags in zip(segs.names, segs.sizes, segs.flags):
        a = capi.SegDerived(0, 0, 0, 0, 0, -1)
        kind = name.split(".")[-1]
        if name.startswith("blk") and kind in shapes:
            a.rows, a.cols = shapes[kind]
            if pack_qkv and kind in ("wq", "wk", "wv") and (flags & SEG_TWIN_BF16):
                layer = int(name[3:name.index(".")])
                a.pack_ld = 3 * D
                a.pack_off = layer * 3 * D * D + ("wq", "wk", "wv").index(kind) * D
                packed = max(packed, (layer + 1) * 3 * D * D)
            if fp8_transposed and (flags & SEG_TWIN_FP8):
                a.fp8_t_off = t_bytes
                t_bytes += n
        aux.append(a)
    return aux, packed, t_bytes


# the benchmark configurations' shapes (element counts follow lm_param_count, lang/lm_adam.c:59-77)
LM_SHAPES = {
    "talk170m": dict(d_model=1024, d_ff=4096, n_blocks=12, vocab=16384, tied=False),   # 184,676,352
    "run555m": dict(d_model=1536, d_ff=6272, n_blocks=14, vocab=100000, tied=True),    # 555,762,080
    "synth3b": dict(d_model=2560, d_ff=10240, n_blocks=32, vocab=100000, tied=True),   # 2,773,419,680
    "tiny": dict(d_model=64, d_ff=256, n_blocks=2, vocab=300, tied=False),             # 138,156 (the reference's unit-test LM)
    "blocks3": dict(d_model=1536, d_ff=6272, n_blocks=3, vocab=8000, tied=True),       # 98,452,160: run555m's blocks, a case sized for profiler captures
}


def lm_param_count(d_model, d_ff, n_blocks, vocab, tied):
    n = d_model * vocab + vocab
    if not tied:
        n += vocab * d_model
    n += n_blocks * (4 * d_model * d_model + 2 * d_model * d_ff + d_ff + d_model + 4 * d_model)
    return n


# ---------------------------------------------------------------------------------
# the engine
# ---------------------------------------------------------------------------------

_TORCH_DT = {DT_F32: torch.float32, DT_BF16: torch.bfloat16}


class OptStep:
    """One shard of the packed arena and the kernels that step it.

    ``shard_off`` / ``shard_n`` select the arena elements this engine owns (the whole
    arena by default).  Buffers are torch tensors on ``device``; pass your own with
    ``bind`` or let ``allocate`` create zeroed ones.
    """

    def __init__(self, segments: Optional[Segments], *, n_arena=None, grad_dtype=DT_BF16,
                 state_dtype=DT_F32, shard_off=0, shard_n=None, device="cuda", handle=None):
        if not torch.cuda.is_available():
            raise RuntimeError("anni_b200 needs a CUDA device: there is no CPU path")
        self.L = capi.lib()
        self.device = torch.device(device)
        self.segments = segments
        self.n_arena = int(segments.n if segments is not None else n_arena)
        self.shard_off = int(shard_off)
        self.shard_n = int(self.n_arena - self.shard_off if shard_n is None else shard_n)
        self.grad_dtype, self.state_dtype = grad_dtype, state_dtype
        self.master = self.m = self.v = self.grad = self.twin_bf16 = self.twin_fp8 = None
        self.owned = handle is None
        if handle is not None:
            # an engine that something else created and will destroy (the C ZeRO-1 driver's)
            self.h = C.c_void_p(handle)
            self.n_seg = len(segments) if segments is not None and len(segments) > 0 else 1
            self.has_fp8 = bool(segments is not None and (segments.flag_array & SEG_TWIN_FP8).any())
            return
        cfg = capi.Config()
        cfg.n_arena, cfg.shard_off, cfg.shard_n = self.n_arena, self.shard_off, self.shard_n
        cfg.grad_dtype, cfg.state_dtype = grad_dtype, state_dtype
        if segments is not None and len(segments) > 0:
            self._off = np.ascontiguousarray(segments.offsets)
            self._flg = np.ascontiguousarray(segments.flag_array)
            cfg.n_seg = len(segments)
            cfg.seg_off = self._off.ctypes.data
            cfg.seg_flags = self._flg.ctypes.data
            self.n_seg = len(segments)
            self.has_fp8 = bool((self._flg & SEG_TWIN_FP8).any())
        else:
            cfg.n_seg = 0
            self.n_seg = 1
            self.has_fp8 = False
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            check("anni_optstep_create", self.L.anni_optstep_create(C.byref(cfg), C.byref(h)))
        self.h = h

    # -- memory -----------------------------------------------------------------------
    def allocate(self, twin_bf16=True, pad_to=None):
        n = max(self.shard_n, 1) if pad_to is None else int(pad_to)
        dev = self.device
        master = torch.zeros(n, dtype=torch.float32, device=dev)
        m = torch.zeros(n, dtype=_TORCH_DT[self.state_dtype], device=dev)
        v = torch.zeros(n, dtype=_TORCH_DT[self.state_dtype], device=dev)
        grad = torch.zeros(n, dtype=_TORCH_DT[self.grad_dtype], device=dev)
        t16 = torch.zeros(n, dtype=torch.bfloat16, device=dev) if twin_bf16 else None
        t8 = torch.zeros(n, dtype=torch.uint8, device=dev) if self.has_fp8 else None
        self.bind(master, m, v, grad, t16, t8)
        return self

    def bind(self, master, m, v, grad, twin_bf16=None, twin_fp8=None):
        for t in (master, m, v, grad, twin_bf16, twin_fp8):
            if t is not None:
                assert t.is_cuda and t.is_contiguous() and t.numel() >= self.shard_n
        assert master.dtype == torch.float32
        assert m.dtype == v.dtype == _TORCH_DT[self.state_dtype]
        assert grad.dtype == _TORCH_DT[self.grad_dtype]
        b = capi.Buffers()
        b.master, b.m, b.v, b.grad = master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr()
        b.twin_bf16 = twin_bf16.data_ptr() if twin_bf16 is not None else None
        b.twin_fp8 = twin_fp8.data_ptr() if twin_fp8 is not None else None
        check("anni_optstep_bind", self.L.anni_optstep_bind(self.h, C.byref(b)))
        self.master, self.m, self.v, self.grad = master, m, v, grad
        self.twin_bf16, self.twin_fp8 = twin_bf16, twin_fp8
        return self

    # -- stepping ---------------------------------------------------------------------
    @staticmethod
    def hyper(*, lr, t, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, clip=0.0, grad_scale=1.0,
              check_finite=True, zero_grad=True, dev_loss_scale=False, exact=False):
        hp = capi.Hyper()
        hp.lr, hp.beta1, hp.beta2, hp.eps = lr, beta1, beta2, eps
        hp.weight_decay, hp.grad_clip, hp.grad_scale, hp.t = wd, clip, grad_scale, int(t)
        hp.flags = ((STEP_CHECK_FINITE if check_finite else 0) | (STEP_ZERO_GRAD if zero_grad else 0)
                    | (STEP_DEV_LOSS_SCALE if dev_loss_scale else 0)
                    | (capi.STEP_EXACT_UPDATE if exact else 0))
        return hp

    def _stream(self, stream):
        s = torch.cuda.current_stream(self.device) if stream is None else stream
        return C.c_void_p(s.cuda_stream)

    def step(self, hp, stream=None):
        """The whole step in one cooperative launch (single-GPU form)."""
        check("anni_optstep_step", self.L.anni_optstep_step(self.h, C.byref(hp), self._stream(stream)))

    def norm(self, hp, stream=None):
        check("anni_optstep_norm", self.L.anni_optstep_norm(self.h, C.byref(hp), self._stream(stream)))

    def update(self, hp, stream=None):
        check("anni_optstep_update", self.L.anni_optstep_update(self.h, C.byref(hp), self._stream(stream)))

    def step_with_sumsq(self, hp, sumsq, stream=None):
        """The step without its norm pass: ``sumsq`` is a device float64 tensor {sum of squares of
        the raw gradients, non-finite count} supplied by whoever produced the gradients."""
        assert sumsq.is_cuda and sumsq.dtype == torch.float64 and sumsq.numel() >= 2
        check("anni_optstep_step_with_sumsq",
              self.L.anni_optstep_step_with_sumsq(self.h, C.byref(hp), sumsq.data_ptr(), self._stream(stream)))

    def set_derived(self, aux, qkv_packed=None, fp8_t=None):
        """Derived twins emitted by the step: ``aux`` is a list of capi.SegDerived (one per tensor),
        ``qkv_packed`` a bf16 tensor for the packed [Wq|Wk|Wv] matrices, ``fp8_t`` a uint8 tensor
        for the transposed e4m3 twins (see anni_optstep_set_derived)."""
        arr = (capi.SegDerived * len(aux))(*aux) if aux else None
        self._derived = (arr, qkv_packed, fp8_t)        # keep the buffers alive
        check("anni_optstep_set_derived",
              self.L.anni_optstep_set_derived(self.h, arr,
                                              qkv_packed.data_ptr() if qkv_packed is not None else None,
                                              fp8_t.data_ptr() if fp8_t is not None else None))

    def set_peers(self, peer_grad, peer_twin, peer_twin_fp8, arena_off_padded):
        """Peer-accessible device pointers (ints) of every rank's full gradient / twin arenas."""
        n = len(peer_grad)
        arr = lambda xs: (C.c_void_p * n)(*[C.c_void_p(int(x)) for x in xs]) if xs else None
        check("anni_optstep_set_peers",
              self.L.anni_optstep_set_peers(self.h, arr(peer_grad), arr(peer_twin), arr(peer_twin_fp8),
                                            n, int(arena_off_padded)))

    def set_multicast(self, mc_grad, mc_twin, mc_twin_fp8, arena_off_padded):
        """NVSwitch multicast addresses (ints, 0 = none) of the same arenas; call after set_peers."""
        v = lambda x: C.c_void_p(int(x)) if x else None
        check("anni_optstep_set_multicast",
              self.L.anni_optstep_set_multicast(self.h, v(mc_grad), v(mc_twin), v(mc_twin_fp8),
                                                int(arena_off_padded)))

    def rotate_peers(self, first):
        """Visit the peers starting at index ``first`` (see anni_optstep_rotate_peers)."""
        check("anni_optstep_rotate_peers", self.L.anni_optstep_rotate_peers(self.h, int(first)))

    def set_grad_arena(self, arena, stride, parts):
        """ZeRO-1: the rank's full gradient arena (a tensor, or None) that ``update`` clears in
        place of the bound shard buffer (see anni_optstep_set_grad_arena)."""
        self._grad_arena = arena
        check("anni_optstep_set_grad_arena",
              self.L.anni_optstep_set_grad_arena(self.h, arena.data_ptr() if arena is not None else None,
                                                 int(stride), int(parts)))

    def reduce_norm(self, hp, stream=None):
        check("anni_optstep_reduce_norm",
              self.L.anni_optstep_reduce_norm(self.h, C.byref(hp), self._stream(stream)))

    def quantize(self, stream=None, local_twins=False):
        check("anni_optstep_quantize",
              self.L.anni_optstep_quantize_ex(self.h, capi.RANGE_LOCAL_TWINS if local_twins else 0,
                                              self._stream(stream)))

    def reduce_norm_range(self, hp, off, n, accumulate, stream=None):
        """reduce_norm over elements [off, off + n) of the shard; accumulate: add to the running sum."""
        check("anni_optstep_reduce_norm_range",
              self.L.anni_optstep_reduce_norm_range(self.h, C.byref(hp), int(off), int(n),
                                                    capi.RANGE_ACCUMULATE if accumulate else 0,
                                                    self._stream(stream)))

    def update_range(self, hp, off, n, *, first, last, local_twins=True, stream=None):
        """update over elements [off, off + n) of the shard (see anni_optstep_update_range)."""
        flags = ((capi.RANGE_FIRST if first else 0) | (capi.RANGE_LAST if last else 0)
                 | (capi.RANGE_LOCAL_TWINS if local_twins else 0))
        check("anni_optstep_update_range",
              self.L.anni_optstep_update_range(self.h, C.byref(hp), int(off), int(n), flags,
                                               self._stream(stream)))

    def peer_copy(self, dst_ptr, src_ptr, nbytes, stream=None):
        """One asynchronous device copy between raw addresses (peer memory included)."""
        check("anni_peer_copy", self.L.anni_peer_copy(C.c_void_p(int(dst_ptr)), C.c_void_p(int(src_ptr)),
                                                      int(nbytes), self._stream(stream)))

    def step_split(self, hp, stream=None):
        """Same result through the three-launch form (what ZeRO-1 interleaves with collectives)."""
        self.norm(hp, stream)
        self.update(hp, stream)
        if self.has_fp8:
            self.quantize(stream)

    # -- small device buffers as tensors (for collectives) -----------------------------------
    def _as_tensor(self, ptr, n, dtype):
        """A torch view of library-owned device memory (no copy, not owned by torch)."""
        class _Holder:
            pass
        hold = _Holder()
        hold.__cuda_array_interface__ = {
            "shape": (n,), "typestr": {torch.float64: "<f8", torch.float32: "<f4"}[dtype],
            "data": (int(ptr), False), "version": 3, "strides": None}
        return torch.as_tensor(hold, device=self.device)

    def reduce_tensor(self):
        return self._as_tensor(self.L.anni_optstep_reduce_buffer(self.h), 2, torch.float64)

    def amax_tensor(self):
        return self._as_tensor(self.L.anni_optstep_amax_buffer(self.h), self.n_seg, torch.float32)

    def scale_tensor(self):
        return self._as_tensor(self.L.anni_optstep_scale_buffer(self.h), self.n_seg, torch.float32)

    # -- status -------------------------------------------------------------------------
    def status(self, stream=None):
        st = capi.Status()
        check("anni_optstep_status_read",
              self.L.anni_optstep_status_read(self.h, C.byref(st), self._stream(stream)))
        return st

    def loss_scale_init(self, scale=65536.0, growth_interval=200, growth=2.0, backoff=0.5,
                        min_scale=1.0, max_scale=2.0 ** 24):
        check("anni_optstep_loss_scale_init",
              self.L.anni_optstep_loss_scale_init(self.h, scale, growth_interval, growth, backoff,
                                                  min_scale, max_scale))

    def grid(self):
        b, t = C.c_int(), C.c_int()
        check("anni_optstep_grid", self.L.anni_optstep_grid(self.h, C.byref(b), C.byref(t)))
        return b.value, t.value

    def close(self):
        if getattr(self, "h", None):
            if self.owned:
                self.L.anni_optstep_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CompressibleArena:
    """A zeroed device buffer in compressible memory (anni_arena_alloc) seen as a torch tensor.
    Meant for the gradient arena, which every step leaves zeroed: the L2 writes zero lines back
    at a fraction of their size.  Raises capi.AnniError(E_LIMIT) where the device has no such
    memory.  The mapping is released by ``close()`` only -- never behind the back of a tensor or
    slice that may still point into it; an arena that is never closed lives until the process ends."""

    def __init__(self, n, dtype, device="cuda"):
        self.L = capi.lib()
        esz = torch.empty((), dtype=dtype).element_size()
        p, size, comp = C.c_void_p(), C.c_size_t(), C.c_int()
        with torch.cuda.device(torch.device(device)):
            check("anni_arena_alloc", self.L.anni_arena_alloc(int(n) * esz, C.byref(p), C.byref(size),
                                                              C.byref(comp)))
        self.ptr, self.mapped_bytes, self.compressed = p, size.value, bool(comp.value)

        class _Holder:
            pass
        hold = _Holder()
        hold.__cuda_array_interface__ = {"shape": (int(n),), "typestr": {1: "|u1", 2: "<i2", 4: "<f4"}[esz],
                                         "data": (int(p.value), False), "version": 3, "strides": None}
        t = torch.as_tensor(hold, device=torch.device(device))
        self.tensor = t if t.dtype == dtype else t.view(dtype)

    def close(self):
        """Unmaps the arena (synchronises the device first).  The caller vouches that no tensor or
        slice of it is used afterwards."""
        if getattr(self, "ptr", None):
            self.tensor = None
            self.L.anni_arena_free(self.ptr, self.mapped_bytes)
            self.ptr = None


def kernel_launches():
    return int(capi.lib().anni_kernel_launches())
