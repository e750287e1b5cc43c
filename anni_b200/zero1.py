"""ZeRO-1 partitioning of the optimizer step over the GPUs of one node.

The reference trainer is single-GPU (its README lists multi-GPU as an open item), so
this layer has no counterpart there; parity is defined against the single-device CPU
step applied to the REDUCED gradients.

Layout: the packed arena (``lang/lm_adam.c:217-311`` of the reference: one running
element offset per tensor) is padded to ``world * shard`` elements and cut into
``world`` equal contiguous shards irrespective of tensor boundaries.  Every rank holds
the full gradient arena (input of the reduce-scatter) and the full twin arena (output of
the all-gather); rank r owns master / m / v of shard r only.  Per step::

    reduce_scatter(sum)  bf16 or fp32 gradients      -> this rank's gradient shard
    norm kernel          local sum of squares        -> {sumsq, nonfinite}
    all_reduce(sum)      2 doubles                   -> global norm and skip flag
    update kernel        decision + AdamW + bf16 twin + per-tensor amax
    [all_reduce(max) of amax[n_seg]; quantise kernel]       (fp8 twins only)
    all_gather           twins, in place inside the full twin arena

``torch.distributed`` (NCCL over NVLink / NVSwitch) is the plumbing; the arithmetic is
in ``libanni_b200.so``.  The collectives see only this process's own device memory.

Peer mode (``peer=True``, the default on GPUs when symmetric memory is available): the
two big collectives disappear into the kernels.  The gradient and twin arenas live in
symmetric memory (``torch.distributed._symmetric_memory``); ``reduce_norm`` reads this
rank's shard out of every peer's gradient arena over NVLink, reduces it and computes the
norm in one pass, and the update kernel stores its twins straight into every peer's twin
arena.  What is left for NCCL is the two-double all-reduce (which doubles as the "my arena
has been read" barrier) and one small barrier at the end of the step::

    [barrier: every rank's gradients are complete]
    reduce_norm kernel   peer loads + sum + round + local store + sum of squares
    all_reduce(sum)      2 doubles
    update kernel        decision + AdamW + twins stored into all ranks' arenas
    [all_reduce(max) of amax; quantise kernel with peer stores]      (fp8 twins only)
    barrier              every rank's twins have landed

Copy mode (``peer="copy"``, opt-in): the same arenas, but the data crosses NVLink on the copy
engines and the kernels work on local memory, part by part::

    [barrier]
    copy streams: pull part p of this rank's shard out of every peer's gradient arena
    main stream:  reduce_norm over part p of the local copies         (overlaps pulls of p + 1)
    all_reduce(sum)      2 doubles
    main stream:  update part p, twins stored locally
    copy streams: push part p of the twins into every peer's arena    (overlaps update of p + 1)
    barrier

Between two B200s with both directions busy a copy engine carries 771 GB/s per direction against
640 GB/s for loads and 700 GB/s for stores issued by SMs, but with every rank copying from / to
all others at once the engines reach 685-705 GB/s, and the extra pass over local memory and the
hand-offs between streams use that up: 2.40 ms against 2.09 ms per step at N = 2 (where the step
is bound by local memory), 2.78 against 2.69 ms at N = 4.  The fused kernels stay the default.

``multicast=True`` makes the same two kernels go through the NVSwitch multicast address of the
arenas instead (``multimem.ld_reduce`` adds all ranks' copies in the switch, ``multimem.st``
replicates a store into all of them).  It is off by default: a multicast group always includes
the issuing GPU, so its own shard travels out and back over its link -- the busy direction
carries the whole arena instead of (N-1)/N of it.  Measured at N = 2: 3.46 ms per step against
2.09 ms with plain peer loads / stores.
"""
import os

import torch
import torch.distributed as dist

from .capi import DT_BF16, DT_F32, STEP_REDUCE_CLEARS_OWN, STEP_ZERO_GRAD

_TORCH_DT = {DT_F32: torch.float32, DT_BF16: torch.bfloat16}
SHARD_ALIGN = 4096      # elements: keeps every shard base 16-byte aligned for all dtypes


def shard_geometry(n_arena, world, align=SHARD_ALIGN):
    """(shard elements incl. padding, [(offset, owned elements) per rank])."""
    per = -(-int(n_arena) // world)
    per = -(-per // align) * align
    own = []
    for r in range(world):
        off = min(r * per, n_arena)
        own.append((r * per, max(0, min(per, n_arena - off)) if r * per < n_arena else 0))
    return per, own


class Zero1:
    """Host-side driver of the sharded step.

    ``make_stepper(shard_off, shard_n)`` builds the object that steps one shard; by
    default that is the CUDA engine (:class:`anni_b200.engine.OptStep`).  The object must
    offer ``allocate / bind``-style buffers (see ``_Buffers``) and the calls ``norm``,
    ``update``, ``quantize``, ``reduce_tensor``, ``amax_tensor``, ``has_fp8``.
    """

    def __init__(self, segments, *, grad_dtype=DT_BF16, state_dtype=DT_F32, group=None,
                 device=None, make_stepper=None, peer=None, multicast=False, copy_parts=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.segments = segments
        self.n_arena = segments.n
        self.per, own = shard_geometry(self.n_arena, self.world)
        self.shard_off, self.shard_n = own[self.rank]
        self.padded = self.per * self.world
        self._c = None
        self._comm = None
        self._shard_n_real = self.shard_n
        has_fp8 = bool((segments.flag_array & 4).any()) if len(segments) else False
        default_stepper = make_stepper is None
        if default_stepper:
            from .engine import OptStep
            dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device

            def make_stepper(off, n):
                return OptStep(segments, grad_dtype=grad_dtype, state_dtype=state_dtype,
                               shard_off=off, shard_n=n, device=dev)
            self.device = dev
        else:
            self.device = torch.device("cpu") if device is None else device
        gdt, sdt, dev = _TORCH_DT[grad_dtype], _TORCH_DT[state_dtype], self.device
        self._gdt = gdt
        self._arenas = []
        if peer is None:
            peer = self.world > 1 and dev.type == "cuda" and default_stepper
        self.copy_mode = peer == "copy" and self.world > 1
        self.peer = bool(peer) and self.world > 1
        self.multicast = bool(multicast)        # use NVSwitch multicast addresses when the arenas have them
        # several ranks on GPUs: the step sequence itself runs in the library (anni_zero1_step, the
        # call a C trainer makes); this class then only owns the memory.  ANNI_B200_ZERO1_DRIVER=py
        # keeps the sequence below in Python (what copy mode and the CPU stand-in always use).
        use_c = (default_stepper and dev.type == "cuda" and self.world > 1 and not self.copy_mode
                 and os.environ.get("ANNI_B200_ZERO1_DRIVER", "c") != "py")
        if use_c:
            from . import capi
            use_c = bool(capi.lib().anni_zero1_nccl_available())
        self._tiny = torch.zeros(1, dtype=torch.float32, device=dev)
        if self.peer:
            self.grad_full, self._peer_grad = self._symm(self.padded, gdt)
            self.twin_full, self._peer_twin = self._symm(self.padded, torch.bfloat16)
            if has_fp8:
                self.twin8_full, self._peer_twin8 = self._symm(self.padded, torch.uint8)
            else:
                self.twin8_full, self._peer_twin8 = None, None
        else:
            self.grad_full = self._local_grad_arena()
            self.twin_full = torch.zeros(self.padded, dtype=torch.bfloat16, device=dev)
            self.twin8_full = torch.zeros(self.padded, dtype=torch.uint8, device=dev) if has_fp8 else None
        lo, hi = self.rank * self.per, (self.rank + 1) * self.per
        self.master = torch.zeros(self.per, dtype=torch.float32, device=dev)
        self.m = torch.zeros(self.per, dtype=sdt, device=dev)
        self.v = torch.zeros(self.per, dtype=sdt, device=dev)
        # with one rank the reduce-scatter is the identity: step the arena in place
        self.grad_shard = (self.grad_full[lo:hi] if self.world == 1
                           else torch.zeros(self.per, dtype=gdt, device=dev))
        self.twin_shard = self.twin_full[lo:hi]
        self.twin8_shard = self.twin8_full[lo:hi] if self.twin8_full is not None else None
        if use_c:
            self._create_c_driver(grad_dtype, state_dtype)
        else:
            # an empty shard still takes part in every collective; it sits at the arena end
            self.eng = make_stepper(min(self.shard_off, self.n_arena), self.shard_n)
            if self.peer:
                if self.copy_mode:
                    # local landing area for the peers' copies of this shard, and a stream for the copies
                    self._stage = torch.zeros(self.world, self.per, dtype=gdt, device=dev)
                    # one stream per peer, so that the copies to / from all peers run at the same time
                    self._copy_streams = [torch.cuda.Stream(device=dev) for _ in range(self.world - 1)]
                    n_parts = copy_parts if copy_parts else (4 if self.shard_n >= (4 << 20) else 1)
                    step = -(-max(self.shard_n, 1) // n_parts)
                    step = -(-step // SHARD_ALIGN) * SHARD_ALIGN
                    self._parts = [(o, min(step, self.shard_n - o)) for o in range(0, max(self.shard_n, 1), step)]
                    if self.shard_n == 0:
                        self._parts = [(0, 0)]
                self._attach_peers()
            self.eng.bind(self.master, self.m, self.v, self.grad_shard, self.twin_shard,
                          self.twin8_shard)
            self._name_grad_arena()
        self.timing = None

    # -- the library's own driver of the sequence (include/anni_zero1.h) -------------------------
    def _ptr_array(self, ptrs):
        import ctypes as C
        return (C.c_void_p * len(ptrs))(*[C.c_void_p(int(p)) for p in ptrs])

    def _create_c_driver(self, grad_dtype, state_dtype):
        import ctypes as C
        import numpy as np
        from . import capi
        from .engine import OptStep
        L = capi.lib()
        # a communicator of the library's own: rank 0 draws the id, the process group carries it
        box = [None]
        if self.rank == 0:
            raw = (C.c_char * capi.ZERO1_UNIQUE_ID_BYTES)()
            capi.check("anni_zero1_unique_id", L.anni_zero1_unique_id(raw))
            box[0] = bytes(raw)
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                                   group=self.group)
        comm = C.c_void_p()
        with torch.cuda.device(self.device):
            capi.check("anni_zero1_comm_init", L.anni_zero1_comm_init(box[0], self.rank, self.world, C.byref(comm)))
        self._comm = comm
        cfg = capi.Zero1Config()
        self._c_off = np.ascontiguousarray(self.segments.offsets)
        self._c_flg = np.ascontiguousarray(self.segments.flag_array)
        cfg.n_arena, cfg.grad_dtype, cfg.state_dtype = self.n_arena, grad_dtype, state_dtype
        cfg.n_seg, cfg.seg_off, cfg.seg_flags = len(self.segments), self._c_off.ctypes.data, self._c_flg.ctypes.data
        cfg.rank, cfg.world, cfg.nccl_comm = self.rank, self.world, comm
        cfg.grad_arena, cfg.twin_arena = self.grad_full.data_ptr(), self.twin_full.data_ptr()
        cfg.twin_fp8_arena = self.twin8_full.data_ptr() if self.twin8_full is not None else None
        keep = []
        self.uses_multicast = False
        if self.peer:
            pg, pt, p8 = self._peer_grad, self._peer_twin, self._peer_twin8
            keep = [self._ptr_array(pg[0]), self._ptr_array(pt[0]), self._ptr_array(p8[0]) if p8 else None]
            cfg.peer_grad = C.cast(keep[0], C.c_void_p)
            cfg.peer_twin = C.cast(keep[1], C.c_void_p)
            cfg.peer_twin_fp8 = C.cast(keep[2], C.c_void_p) if p8 else None
            self.uses_multicast = bool(pg[1] and pt[1] and (p8 is None or p8[1]))
            if self.uses_multicast:
                cfg.mc_grad, cfg.mc_twin = pg[1], pt[1]
                cfg.mc_twin_fp8 = p8[1] if p8 else None
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            capi.check("anni_zero1_create", L.anni_zero1_create(C.byref(cfg), C.byref(h)))
        self._c, self._c_keep = h, keep
        capi.check("anni_zero1_bind", L.anni_zero1_bind(h, self.master.data_ptr(), self.m.data_ptr(),
                                                        self.v.data_ptr(), self.grad_shard.data_ptr()))
        self.eng = OptStep(self.segments, grad_dtype=grad_dtype, state_dtype=state_dtype,
                           shard_off=min(self.shard_off, self.n_arena), shard_n=self.shard_n,
                           device=self.device, handle=L.anni_zero1_engine(h))
        self.eng.master, self.eng.m, self.eng.v, self.eng.grad = self.master, self.m, self.v, self.grad_shard
        self.eng.twin_bf16, self.eng.twin_fp8 = self.twin_shard, self.twin8_shard
        self._arena_by_engine = True

    def close(self):
        """Releases the library-side driver and its communicator (collective when there is one)."""
        if self._c is not None:
            from . import capi
            torch.cuda.synchronize(self.device)
            self.eng.close()
            capi.lib().anni_zero1_destroy(self._c)
            capi.lib().anni_zero1_comm_free(self._comm)
            self._c = self._comm = None

    # -- peer memory ----------------------------------------------------------------------
    def _symm(self, n, dtype):
        """A zeroed arena in symmetric memory and every rank's device pointer to its copy."""
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(n, dtype=dtype, device=self.device)
        t.zero_()
        hdl = symm_mem.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0) if self.multicast else 0
        return t, ([int(p) for p in hdl.buffer_ptrs], mc)

    def _attach_peers(self):
        off = self.rank * self.per
        pg, pt = self._peer_grad, self._peer_twin
        p8 = self._peer_twin8
        if self.copy_mode:
            # the reduce kernel reads LOCAL copies: row k of the landing area stands for rank k's
            # arena (the engine adds this shard's offset to every base), this rank's own arena for itself
            gsz = self.grad_full.element_size()
            bases = [self._stage[k].data_ptr() - off * gsz for k in range(self.world)]
            bases[self.rank] = pg[0][self.rank]
            self.eng.set_peers(bases, pt[0], p8[0] if p8 else None, off)
            self.uses_multicast = False
            return
        self.eng.set_peers(pg[0], pt[0], p8[0] if p8 else None, off)
        if os.environ.get("ANNI_B200_PEER_ROTATE", "1") != "0":
            # remote copies first, each rank starting at another peer; this rank's own copy last
            self.eng.rotate_peers((self.rank + 1) % self.world)
        self.uses_multicast = bool(pg[1] and pt[1] and (p8 is None or p8[1]))
        if self.uses_multicast:
            self.eng.set_multicast(pg[1], pt[1], p8[1] if p8 else 0, off)

    def _name_grad_arena(self):
        """Several ranks: the buffer the backward pass accumulates into is the FULL arena, of which
        the update only sees the reduced shard -- tell the engine, so that "the step leaves the
        gradients zeroed" (lang/lm_adam.c:597 of the reference) holds for it: the update kernel
        clears the whole local arena once every peer has read it.  A stepper without that call
        (the CPU stand-in of the tests) gets the arena cleared after its update."""
        self._arena_by_engine = False
        if self.world > 1 and hasattr(self.eng, "set_grad_arena"):
            self.eng.set_grad_arena(self.grad_full, self.per, self.world)
            self._arena_by_engine = True

    def _zero_arena_after_update(self, hp):
        if self.world > 1 and not self._arena_by_engine and (getattr(hp, "flags", 2) & 2):
            self.grad_full.zero_()

    def _local_grad_arena(self):
        """A zeroed gradient arena in this GPU's memory: on one GPU compressible memory where the
        device has it (every step leaves the arena zeroed, and zero lines then cost a fraction of
        their size on the way to HBM), plain memory otherwise."""
        if self.device.type == "cuda" and self.world == 1:      # several ranks: NCCL reads this arena; plain memory
            from . import capi
            from .engine import CompressibleArena
            try:
                arena = CompressibleArena(self.padded, self._gdt, self.device)
            except capi.AnniError:
                pass                # no such memory here, or none left: plain memory does the same job
            else:
                self._arenas.append(arena)          # keeps the mapping alive as long as this object
                return arena.tensor
        return torch.zeros(self.padded, dtype=self._gdt, device=self.device)

    def new_grad_arena(self):
        """Another full gradient arena (e.g. one per micro-step buffer); see use_grad_arena."""
        if self.peer:
            return self._symm(self.padded, self._gdt)
        return self._local_grad_arena(), None

    def use_grad_arena(self, arena):
        """Make (tensor, peer pointers) from new_grad_arena the input of the next steps."""
        t, ptrs = arena
        self.grad_full = t
        if self._c is not None:
            from . import capi
            if self.peer:
                self._peer_grad = ptrs
                self._c_keep[0] = self._ptr_array(ptrs[0])
                arr, mc = self._c_keep[0], (ptrs[1] if self.uses_multicast else None)
            else:
                arr, mc = None, None
            capi.check("anni_zero1_set_grad_arena",
                       capi.lib().anni_zero1_set_grad_arena(self._c, t.data_ptr(), arr, mc))
            return
        if self.world > 1:
            self._name_grad_arena()
        if self.peer:
            self._peer_grad = ptrs
            self._attach_peers()
        elif self.world == 1:
            self.grad_shard = t[:self.per]
            self.eng.bind(self.master, self.m, self.v, self.grad_shard, self.twin_shard, self.twin8_shard)

    def _barrier(self):
        """Stream-ordered barrier across the ranks (a one-float all-reduce)."""
        dist.all_reduce(self._tiny, group=self.group)

    # -- state in / out (arena order, full arrays; used by tests and checkpoints) -------
    def load_shard_from_full(self, master_full, m_full, v_full):
        lo, n = self.shard_off, self.shard_n
        if n:
            self.master[:n].copy_(master_full[lo:lo + n])
            self.m[:n].copy_(m_full[lo:lo + n])
            self.v[:n].copy_(v_full[lo:lo + n])

    def gather_full(self, shard):
        """All ranks' shards of a per-rank buffer, concatenated in arena order (unpadded)."""
        if self.world == 1:
            return shard[:self.n_arena].clone()
        out = torch.empty(self.padded, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(out, shard.contiguous(), group=self.group)
        return out[:self.n_arena]

    # -- checkpoints in the reference trainer's format, from / to the sharded state ------
    def _shards_to_rank0(self, shard):
        """This buffer's shards as one fp32 host array in arena order on rank 0 (None elsewhere):
        one shard at a time travels to rank 0, so no rank ever holds a second full copy on its device."""
        import numpy as np
        own = shard_geometry(self.n_arena, self.world)[1]
        full = np.empty(self.n_arena, np.float32) if self.rank == 0 else None
        mine = shard[:self.per].float()
        for r, (off, cnt) in enumerate(own):
            if cnt == 0:
                continue
            if r == 0:
                if self.rank == 0:
                    full[off:off + cnt] = mine[:cnt].cpu().numpy()
            elif self.rank == r:
                dist.send(mine[:cnt].contiguous(), dst=dist.get_global_rank(self.group, 0)
                          if self.group is not None else 0, group=self.group)
            elif self.rank == 0:
                tmp = torch.empty(cnt, dtype=torch.float32, device=self.device)
                dist.recv(tmp, src=dist.get_global_rank(self.group, r) if self.group is not None else r,
                          group=self.group)
                full[off:off + cnt] = tmp.cpu().numpy()
        return full

    def _shards_from_rank0(self, full, shard):
        """The inverse: rank 0 hands every rank its slice of a full fp32 host array."""
        own = shard_geometry(self.n_arena, self.world)[1]
        for r, (off, cnt) in enumerate(own):
            if cnt == 0:
                continue
            if self.rank == 0:
                piece = torch.from_numpy(full[off:off + cnt]).to(self.device)
                if r == 0:
                    shard[:cnt].copy_(piece)
                else:
                    dist.send(piece, dst=dist.get_global_rank(self.group, r) if self.group is not None else r,
                              group=self.group)
            elif self.rank == r:
                tmp = torch.empty(cnt, dtype=torch.float32, device=self.device)
                dist.recv(tmp, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                          group=self.group)
                shard[:cnt].copy_(tmp)

    def save_checkpoint(self, path, info, *, t, epoch=0, step=0, merges=None):
        """lm_save_checkpoint (lang/lm_serialize.c:302-331 of the reference) from the sharded
        state: weights, m and v of all ranks in optimizer order, written by rank 0 in the
        reference's byte layout (``info``: an anni_b200.checkpoint.CkptModel with the model's
        dimensions and kind).  Collective: every rank calls it."""
        from . import checkpoint
        w = self._shards_to_rank0(self.master)
        m = self._shards_to_rank0(self.m)
        v = self._shards_to_rank0(self.v)
        if self.rank == 0:
            info.n, info.has_adam, info.t, info.epoch, info.step = self.n_arena, 1, int(t), int(epoch), int(step)
            checkpoint.save_model(path, info, w, m, v, merges)
        if self.world > 1:
            dist.barrier(group=self.group)

    def load_checkpoint(self, path):
        """lm_load_checkpoint (lang/lm_serialize.c:526-587) into the sharded state: rank 0 reads
        the file, every rank receives its slice of the weights, m and v (rounded to the moment
        dtype) and rebuilds its bf16 twins.  Returns (t, epoch, step).  Collective."""
        from . import checkpoint
        head = torch.zeros(4, dtype=torch.int64, device=self.device)
        ck = None
        if self.rank == 0:
            ck = checkpoint.load_model(path)
            k = ck["info"]
            ok = k.n == self.n_arena and bool(k.has_adam)
            head.copy_(torch.tensor([1 if ok else 0, k.t, k.epoch, k.step], dtype=torch.int64))
        if self.world > 1:
            dist.broadcast(head, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                           group=self.group)
        ok, t, epoch, step = (int(x) for x in head.tolist())
        if not ok:
            raise ValueError(f"{path}: slot count or Adam section does not match this arena "
                             f"({self.n_arena} parameters)")
        for key, dst in (("w", self.master), ("m", self.m), ("v", self.v)):
            self._shards_from_rank0(ck[key] if ck is not None else None, dst)
        self.twin_shard.copy_(self.master.to(torch.bfloat16))
        if self.world > 1:
            dist.all_gather_into_tensor(self.twin_full, self.twin_shard.contiguous(), group=self.group)
        return t, epoch, step

    # -- the step ------------------------------------------------------------------------
    PHASES = ("reduce_scatter+norm", "all_reduce", "update+all_gather", "barrier")

    def step(self, hp, record=None, grads_complete=False, phase_events=None):
        """One sharded step.  ``grads_complete``: every rank's gradient arena was complete before
        the previous step's closing barrier (peer mode then skips the opening barrier).
        Timing hooks: ``phase_events``, four ``torch.cuda.Event`` (timing enabled and recorded
        once before, so that they exist) which the library records after the phases named in
        ``PHASES`` when the sequence runs there (``driver == "library"``); ``record``, a callable
        given a phase name after each phase has been queued, when it runs in Python."""
        if self._c is not None:
            from . import capi
            import ctypes as C
            evs = None
            if phase_events is not None:
                evs = (C.c_void_p * 4)(*[C.c_void_p(int(e.cuda_event)) for e in phase_events])
            st = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            capi.check("anni_zero1_step",
                       capi.lib().anni_zero1_step(self._c, C.byref(hp),
                                                  capi.ZERO1_GRADS_COMPLETE if grads_complete else 0, st, evs))
            return
        mark = record if record is not None else (lambda name: None)
        if self.world == 1 and hasattr(self.eng, "step"):
            self.eng.step(hp)           # nothing to exchange: the single cooperative launch
            mark("step")
            return
        if self.copy_mode:
            self._step_copy(hp, mark, grads_complete)
            return
        if self.peer:
            if not grads_complete:
                self._barrier()
            if self.reduce_clears_own and (hp.flags & STEP_ZERO_GRAD):
                # nobody else reads this rank's own part of its arena: the reduce clears it
                own = type(hp).from_buffer_copy(hp)
                own.flags |= STEP_REDUCE_CLEARS_OWN
                hp = own
            self.eng.reduce_norm(hp)
            mark("reduce_scatter+norm")
            dist.all_reduce(self.eng.reduce_tensor(), op=dist.ReduceOp.SUM, group=self.group)
            mark("all_reduce")
            self.eng.update(hp)         # also clears this rank's gradient arena: every peer has read it
            self._zero_arena_after_update(hp)
            if self.eng.has_fp8:
                dist.all_reduce(self.eng.amax_tensor(), op=dist.ReduceOp.MAX, group=self.group)
                self.eng.quantize()
            mark("update+all_gather")
            self._barrier()
            mark("barrier")
            return
        if self.world > 1:
            dist.reduce_scatter_tensor(self.grad_shard, self.grad_full, op=dist.ReduceOp.SUM,
                                       group=self.group)
        mark("reduce_scatter")
        self.eng.norm(hp)
        if self.world > 1:
            dist.all_reduce(self.eng.reduce_tensor(), op=dist.ReduceOp.SUM, group=self.group)
        mark("norm")
        self.eng.update(hp)             # several ranks: clears the full arena the reduce-scatter has consumed
        self._zero_arena_after_update(hp)
        if self.eng.has_fp8:
            if self.world > 1:
                dist.all_reduce(self.eng.amax_tensor(), op=dist.ReduceOp.MAX, group=self.group)
            self.eng.quantize()
        mark("update")
        if self.world > 1:
            dist.all_gather_into_tensor(self.twin_full, self.twin_shard, group=self.group)
            if self.twin8_full is not None:
                dist.all_gather_into_tensor(self.twin8_full, self.twin8_shard, group=self.group)
        mark("all_gather")

    def _step_copy(self, hp, mark, grads_complete):
        """The step with the copy engines moving the data (see the module text)."""
        eng, streams = self.eng, self._copy_streams
        main = torch.cuda.current_stream(self.device)
        gsz = self.grad_full.element_size()
        base = self.rank * self.per                     # this shard inside every padded arena
        # rank r starts with peer r + 1: at any moment every GPU serves a different peer
        others = [(self.rank + j) % self.world for j in range(1, self.world)]
        pg, pt, p8 = self._peer_grad[0], self._peer_twin[0], self._peer_twin8

        def after(src, dst):
            ev = torch.cuda.Event()
            ev.record(src)
            dst.wait_event(ev)

        if not grads_complete:
            self._barrier()
        for cs in streams:
            after(main, cs)
        for i, (o, n) in enumerate(self._parts):
            for k, cs in zip(others, streams):
                eng.peer_copy(self._stage[k].data_ptr() + o * gsz, pg[k] + (base + o) * gsz, n * gsz, cs)
                after(cs, main)
            eng.reduce_norm_range(hp, o, n, accumulate=i > 0)
        mark("reduce_scatter+norm")
        dist.all_reduce(eng.reduce_tensor(), op=dist.ReduceOp.SUM, group=self.group)
        mark("all_reduce")
        last = len(self._parts) - 1
        for i, (o, n) in enumerate(self._parts):
            eng.update_range(hp, o, n, first=i == 0, last=i == last, local_twins=True)   # + clears the arena part
            for k, cs in zip(others, streams):
                after(main, cs)
                eng.peer_copy(pt[k] + (base + o) * 2, self.twin_full.data_ptr() + (base + o) * 2, n * 2, cs)
        if eng.has_fp8:
            dist.all_reduce(eng.amax_tensor(), op=dist.ReduceOp.MAX, group=self.group)
            eng.quantize(local_twins=True)
            for k, cs in zip(others, streams):
                after(main, cs)
                eng.peer_copy(p8[0][k] + base, self.twin8_full.data_ptr() + base, self.shard_n, cs)
        for cs in streams:
            after(cs, main)
        mark("update+all_gather")
        self._barrier()
        mark("barrier")

    @property
    def reduce_clears_own(self):
        """Peer-memory form without multicast: the reduce kernel clears this rank's own part of its
        gradient arena as it reads it, and the update clears the other parts only
        (ANNI_STEP_REDUCE_CLEARS_OWN; ``ANNI_B200_REDUCE_CLEARS_OWN=0`` turns it off)."""
        return bool(self.world > 1 and self.peer and not self.copy_mode and not self.uses_multicast
                    and getattr(self, "_arena_by_engine", False)
                    and os.environ.get("ANNI_B200_REDUCE_CLEARS_OWN", "1") != "0")

    @property
    def driver(self):
        """Where the step sequence runs: "library" (anni_zero1_step) or "python"."""
        return "library" if self._c is not None else "python"

    def status(self):
        return self.eng.status()
