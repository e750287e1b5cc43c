"""Generates the golden vectors of this folder from the reference's own object code.

Run where the reference checkout is present (``make -C oracle`` has built
``oracle/_ref/libannref.so`` from the reference's CPU sources):

    python tests/golden/make_golden.py

Writes ``adam_steps.npz`` (inputs and outputs of lm_adam_step_scaled's host loop on small
seeded cases), ``lr_schedule.json`` (lm_train_step_lr values), the SHA-256 of the Adam trailer of a checkpoint
written by lm_save_checkpoint for the reference's unit-test LM with known m/v and
``segments_tiny.json`` (the optimizer's tensor order for that LM).  The files are small and
committed, so the oracle stays pinned on machines without the reference.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle_lib import RefLib  # noqa: E402

CASES = [
    # name, n, seed, kwargs
    ("clip_decay_t1000", 4099, 0, dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0, grad_scale=1.0, t_before=999)),
    ("first_step_no_clip", 2048, 1, dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, clip=0.0, grad_scale=1.0 / 252, t_before=0)),
    ("unscale_1024", 3001, 2, dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0, grad_scale=1.0 / 1024, t_before=41)),
    ("clip_inactive", 1537, 3, dict(lr=2e-4, beta1=0.8, beta2=0.99, eps=1e-6, wd=0.01, clip=50.0, grad_scale=1.0, t_before=7)),
]


def inputs(n, seed, loss_scale=1.0):
    rng = np.random.default_rng(seed)
    p = rng.normal(0, 0.02, n).astype(np.float32)
    g = rng.normal(0, 1e-3, n).astype(np.float32)
    g[rng.random(n) < 1e-2] *= 100.0
    g *= np.float32(loss_scale)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    return p, g, m, v


def ckpt_moments(n):
    """m and v of the checkpoint fixture from integer arithmetic only (no RNG stream involved)."""
    i = np.arange(n, dtype=np.uint64)
    a = ((i * np.uint64(2654435761)) % np.uint64(1 << 32)).astype(np.float64) / float(1 << 32)
    b = ((i * np.uint64(40503) + np.uint64(12345)) % np.uint64(1 << 24)).astype(np.float64) / float(1 << 24)
    return ((a - 0.5) * 2e-4).astype(np.float32), (b * 3e-6).astype(np.float32)


FULL_CKPT_CASES = [(0, 0), (1, 44), (2, 44)]      # (kind, BPE merges): LMCF, LMCV, LMCT


def ckpt_weights(n):
    i = np.arange(n, dtype=np.uint64)
    a = ((i * np.uint64(2246822519) + np.uint64(7)) % np.uint64(1 << 32)).astype(np.float64) / float(1 << 32)
    return ((a - 0.5) * 0.08).astype(np.float32)


def synthetic_merges(n_merges):
    """The merge table the reference driver builds: merge i joins tokens 4 + 2i and 4 + 2i + 1 (mod 256)."""
    i = np.arange(n_merges, dtype=np.int32)
    return np.stack([4 + (2 * i) % 256, 4 + (2 * i + 1) % 256], axis=1).astype(np.int32)


def main():
    ref = RefLib()
    out = {}
    for name, n, seed, kw in CASES:
        ls = 1024.0 if "unscale" in name else 1.0
        p, g, m, v = inputs(n, seed, ls)
        if kw["t_before"] == 0:
            m[:] = 0
            v[:] = 0
        q = [x.copy() for x in (p, g, m, v)]
        ref.step(*q, **kw)
        for k, a in zip("pgmv", (p, g, m, v)):
            out[f"{name}/in_{k}"] = a
        for k, a in zip("pgmv", q):
            out[f"{name}/out_{k}"] = a
        out[f"{name}/hyper"] = np.array([kw[k] for k in ("lr", "beta1", "beta2", "eps", "wd", "clip",
                                                         "grad_scale", "t_before")], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "adam_steps.npz"), **out)

    sched = []
    for base, warm, dec, kind, frm in [(1.0, 100, 1000, "cosine", 0), (1.0, 100, 1000, "cosine", 29000),
                                       (3e-4, 100, 1000, "cosine", 0), (2e-3, 0, 500, "linear", 0),
                                       (1e-3, 50, 0, "none", 0), (1e-3, 10, 100, "linear", 5)]:
        for step in [0, 1, 9, 10, 49, 50, 99, 100, 101, 350, 600, 1099, 1100, 5000, 29000, 29099, 29600, 31000]:
            sched.append(dict(base=base, warmup=warm, decay=dec, kind=kind, start=frm, step=step,
                              lr=ref.lr_schedule(base, step, warm, dec, kind, frm)))
    with open(os.path.join(HERE, "lr_schedule.json"), "w") as f:
        json.dump(sched, f, indent=0)

    vocab = 300
    n = ref.slot_count(vocab)
    m, v = ckpt_moments(n)
    path = os.path.join(HERE, "ckpt_tiny.bin")
    ref.ckpt_save(path, vocab, m, v, t=1234, epoch=3, step=77)
    size = os.path.getsize(path)
    # keep only the Adam trailer (20 + 8 n bytes): the weight section is random-initialised
    with open(path, "rb") as f:
        f.seek(size - (20 + 8 * n))
        tail = f.read()
    os.remove(path)
    import hashlib
    digest = hashlib.sha256(tail).hexdigest()
    off, cnt, isv = ref.seg_list(vocab)
    with open(os.path.join(HERE, "segments_tiny.json"), "w") as f:
        json.dump(dict(vocab=vocab, d_model=64, d_ff=256, n_blocks=2, n=n, file_size_full=size,
                       trailer_sha256=digest, trailer_head_hex=tail[:36].hex(), t=1234, epoch=3, step=77, off=off.tolist(), n_per=cnt.tolist(),
                       is_vec=isv.tolist()), f)
    # whole checkpoints of the three kinds, weights and moments from integer formulas: only hashes
    import hashlib
    full = []
    for mode, n_merges in FULL_CKPT_CASES:
        nn = ref.full_slot_count(mode, n_merges)
        w, mm, vv = ckpt_weights(nn), *ckpt_moments(nn)
        fpath = os.path.join(HERE, f"_full{mode}.bin")
        ref.ckpt_save_full(fpath, mode, n_merges, w, mm, vv, t=4321, epoch=5, step=66)
        data = open(fpath, "rb").read()
        os.remove(fpath)
        full.append(dict(mode=mode, n_merges=n_merges, n=nn, size=len(data),
                         sha256=hashlib.sha256(data).hexdigest(), head_hex=data[:40].hex()))
    with open(os.path.join(HERE, "ckpt_full.json"), "w") as f:
        json.dump(full, f, indent=0)
    print("golden vectors written:", n, "slots;", len(sched), "schedule points;", len(CASES), "steps")


if __name__ == "__main__":
    main()
