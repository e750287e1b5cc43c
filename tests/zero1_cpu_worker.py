"""Worker of the world-size-2 gloo test: the ZeRO-1 host logic with the CPU oracle as the
shard stepper (test infrastructure; the product stepper is the CUDA engine)."""
import math
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from anni_b200.capi import DT_BF16, DT_F32, SEG_TWIN_FP8  # noqa: E402
from anni_b200.engine import LM_SHAPES, lm_segments  # noqa: E402
from anni_b200.zero1 import Zero1  # noqa: E402
from oracle_lib import Oracle  # noqa: E402


def _np(t):
    return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()


class OracleStepper:
    """Same calls as the CUDA engine, arithmetic by the oracle on this rank's shard."""

    def __init__(self, segs, off, n):
        self.o, self.segs, self.off, self.n = Oracle(), segs, off, n
        self.has_fp8 = bool((segs.flag_array & SEG_TWIN_FP8).any())
        self._reduce = torch.zeros(2, dtype=torch.float64)
        self._amax = torch.zeros(len(segs), dtype=torch.float32)
        self.skipped = False
        self.norm_value = 0.0
        # this shard's view of the segment table (offsets relative to the shard, clipped)
        so = np.clip(segs.offsets - off, 0, n).astype(np.int64)
        self.seg_off, self.seg_flags = so, segs.flag_array

    def bind(self, master, m, v, grad, twin16, twin8):
        self.master, self.m, self.v, self.grad, self.twin16 = master, m, v, grad, twin16

    def reduce_tensor(self):
        return self._reduce

    def amax_tensor(self):
        return self._amax

    def norm(self, hp):
        g = _np(self.grad)[:self.n]
        ss = self.o.sumsq(g, 1.0)
        self._reduce[0] = ss
        self._reduce[1] = 0.0 if math.isfinite(ss) else 1.0

    def update(self, hp):
        n = self.n
        ss = float(self._reduce[0])
        norm = math.sqrt(ss) * abs(hp.grad_scale) if math.isfinite(ss) else float("nan")
        self.norm_value = norm
        self.skipped = not math.isfinite(norm)
        g = _np(self.grad)[:n]
        if self.skipped:
            g[:] = 0
            return
        coef = hp.grad_scale
        if hp.grad_clip > 0 and norm > hp.grad_clip:
            coef *= hp.grad_clip / (norm + 1e-12)
        # clip = 0 here: the global decision was taken above from the reduced sum
        self.o.step(_np(self.master)[:n], g, _np(self.m)[:n], _np(self.v)[:n], lr=hp.lr, beta1=hp.beta1,
                    beta2=hp.beta2, eps=hp.eps, wd=hp.weight_decay, clip=0.0, grad_scale=coef,
                    t_before=hp.t - 1, seg_off=self.seg_off, seg_flags=self.seg_flags)
        _np(self.twin16)[:n] = self.o.bf16_rne(_np(self.master)[:n])

    def quantize(self):
        pass

    def status(self):
        return dict(norm=self.norm_value, skipped=self.skipped)


class Hyper:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def main():
    out_dir = sys.argv[1]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices")
    n = segs.n
    z = Zero1(segs, grad_dtype=DT_BF16, state_dtype=DT_F32, device=torch.device("cpu"),
              make_stepper=lambda off, cnt: OracleStepper(segs, off, cnt))
    rng = np.random.default_rng(123)                      # same stream on every rank
    p = rng.normal(0, 0.02, n).astype(np.float32)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    z.load_shard_from_full(torch.from_numpy(p), torch.from_numpy(m), torch.from_numpy(v))
    results = []
    for step in range(3):
        # per-rank gradients whose sum is exact in bf16: rank r holds G * 2^-(r+1) twice over
        base = rng.normal(0, 1e-3, n).astype(np.float32)
        if step == 2:
            base[n // 2] = np.inf                           # third step must be skipped on every rank
        gb = torch.from_numpy(base).to(torch.bfloat16)
        assert not bool(z.grad_full.any())                  # the previous step left the whole arena zeroed
        z.grad_full[:n] += (gb.float() * (0.5 if world > 1 else 1.0)).to(torch.bfloat16)
        hp = Hyper(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, grad_clip=1.0,
                   grad_scale=1.0, t=step + 1)
        z.step(hp)
        results.append(z.status())
    full_p = z.gather_full(z.master)
    full_m = z.gather_full(z.m)
    full_v = z.gather_full(z.v)
    # checkpoint out of the sharded state, and back into a fresh one
    from anni_b200 import checkpoint
    k = checkpoint.CkptModel()
    k.kind, k.tied, k.d_model, k.n_heads, k.d_ff, k.max_ctx, k.n_blocks = 1, 0, 64, 4, 256, 2048, 2
    k.vocab, k.n_merges, k.merges_word = 300, 40, 40
    merges = np.array([[4 + (2 * i) % 256, 4 + (2 * i + 1) % 256] for i in range(40)], np.int32)
    path = os.path.join(out_dir, "zero1.ckpt")
    z.save_checkpoint(path, k, t=3, epoch=1, step=3, merges=merges)
    z2 = Zero1(segs, grad_dtype=DT_BF16, state_dtype=DT_F32, device=torch.device("cpu"),
               make_stepper=lambda off, cnt: OracleStepper(segs, off, cnt))
    counters = z2.load_checkpoint(path)
    same = all(torch.equal(a[:z.shard_n], b[:z.shard_n]) for a, b in
               ((z.master, z2.master), (z.m, z2.m), (z.v, z2.v), (z.twin_shard, z2.twin_shard)))
    flags = torch.tensor([1 if same and counters == (3, 1, 3) else 0])
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    full_twin = z.twin_full[:n].clone()
    if rank == 0:
        np.savez(os.path.join(out_dir, "zero1_out.npz"), p=full_p.numpy(), m=full_m.numpy(),
                 v=full_v.numpy(), ckpt_round_trip=int(flags.item()),
                 twin=_np(full_twin), norms=np.array([r["norm"] for r in results]),
                 skipped=np.array([r["skipped"] for r in results]), per=z.per, world=world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
