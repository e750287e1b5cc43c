"""Worker of the multi-GPU ZeRO-1 test: one process per GPU, NCCL, the CUDA engine."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from anni_b200.capi import DT_BF16, DT_F32  # noqa: E402
from anni_b200.engine import LM_SHAPES, OptStep, lm_segments  # noqa: E402
from anni_b200.zero1 import Zero1  # noqa: E402
from parity_util import bf16_bits_from_f32, to_dev, to_host  # noqa: E402


def main():
    out_dir, twin, state = sys.argv[1], sys.argv[2], sys.argv[3]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    segs = lm_segments(**LM_SHAPES["tiny"], wd="matrices", twin=twin)
    n = segs.n
    sd = DT_BF16 if state == "bf16" else DT_F32
    mode = os.environ.get("ANNI_TEST_MODE", "mc")
    z = Zero1(segs, grad_dtype=DT_BF16, state_dtype=sd, device=dev,
              peer="copy" if mode == "copy" else mode != "nccl", multicast=mode == "mc",
              copy_parts=3)
    rng = np.random.default_rng(321)
    p = rng.normal(0, 0.02, n).astype(np.float32)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    if sd == DT_BF16:
        m_in, v_in = bf16_bits_from_f32(m), bf16_bits_from_f32(v)
    else:
        m_in, v_in = m, v
    z.load_shard_from_full(to_dev(p, dev), to_dev(m_in, dev), to_dev(v_in, dev))
    stats = []
    for step in range(3):
        base = rng.normal(0, 1e-3, n).astype(np.float32)
        if step == 2:
            base[n - 7] = np.inf                                # lands in the LAST rank's shard only
        gb = torch.from_numpy(base).to(torch.bfloat16)
        # every rank contributes g / world with world a power of two: the bf16 sum is exact.  The
        # gradients are ACCUMULATED into the arena, as a backward pass does (beta = 1 GEMMs): right
        # only if the previous step left the whole arena zeroed, padding included.
        z.grad_full[:n] += (gb.float() / world).to(torch.bfloat16).to(dev)
        hp = OptStep.hyper(lr=3e-4, t=step + 1, beta2=0.95, wd=0.1, clip=1.0, grad_scale=1.0)
        z.step(hp)
        st = z.status()
        arena_clean = not bool(z.grad_full.any())            # also after the skipped step
        stats.append((st.norm, st.skipped, st.error if arena_clean else -99))
    full_p = z.gather_full(z.master)
    full_m = z.gather_full(z.m)
    full_v = z.gather_full(z.v)
    # checkpoint written by all ranks together and read back shard-wise into a fresh engine
    from anni_b200 import checkpoint
    k = checkpoint.CkptModel()
    k.kind, k.tied, k.d_model, k.n_heads, k.d_ff, k.max_ctx, k.n_blocks = 1, 0, 64, 4, 256, 2048, 2
    k.vocab, k.n_merges, k.merges_word = 300, 40, 40
    merges = np.array([[4 + (2 * i) % 256, 4 + (2 * i + 1) % 256] for i in range(40)], np.int32)
    path = os.path.join(out_dir, f"zero1_gpu_{twin}_{state}.ckpt")
    z.save_checkpoint(path, k, t=3, epoch=0, step=3, merges=merges)
    z2 = Zero1(segs, grad_dtype=DT_BF16, state_dtype=sd, device=dev, peer=False)
    counters = z2.load_checkpoint(path)
    same = counters == (3, 0, 3) and all(torch.equal(a[:z.shard_n], b[:z.shard_n]) for a, b in
                                         ((z.master, z2.master), (z.m, z2.m), (z.v, z2.v)))
    ck_ok = torch.tensor([1 if same else 0], device=dev)
    dist.all_reduce(ck_ok, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    all_stats = [None] * world
    dist.all_gather_object(all_stats, stats)
    if rank == 0:
        np.savez(os.path.join(out_dir, f"zero1_gpu_{twin}_{state}.npz"), peer=int(z.peer), driver=z.driver, multicast=int(getattr(z, "uses_multicast", False)), p=to_host(full_p), m=to_host(full_m),
                 v=to_host(full_v), twin=to_host(z.twin_full[:n]),
                 twin8=to_host(z.twin8_full[:n]) if z.twin8_full is not None else np.zeros(1, np.uint8),
                 scale=z.eng.scale_tensor().cpu().numpy(), stats=np.array(all_stats, dtype=np.float64),
                 world=world, ckpt_round_trip=int(ck_ok.item()))
    z.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
