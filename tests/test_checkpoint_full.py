"""Whole checkpoints in the reference's format (weight section + Adam section), CPU side:
the product reader/writer against golden hashes of files the reference wrote, and against the
reference's own object code where it was built."""
import hashlib
import json
import os

import numpy as np
import pytest

from anni_b200 import capi, checkpoint
from anni_b200.engine import lm_param_count
from golden.make_golden import FULL_CKPT_CASES, ckpt_moments, ckpt_weights, synthetic_merges

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TINY = dict(d_model=64, n_heads=4, d_ff=256, max_ctx=2048, n_blocks=2)


def _info(kind, n_merges, **adam):
    k = checkpoint.CkptModel()
    k.kind, k.tied = kind, int(kind == 2)
    k.d_model, k.n_heads, k.d_ff, k.max_ctx, k.n_blocks = (TINY[x] for x in
                                                           ("d_model", "n_heads", "d_ff", "max_ctx", "n_blocks"))
    k.vocab = 4 + 256 + n_merges
    k.n_merges = k.merges_word = n_merges
    k.n = lm_param_count(TINY["d_model"], TINY["d_ff"], TINY["n_blocks"], k.vocab, bool(k.tied))
    k.epoch, k.step, k.t = adam.get("epoch", 0), adam.get("step", 0), adam.get("t", 0)
    return k


@pytest.mark.parametrize("case", range(len(FULL_CKPT_CASES)))
def test_writer_reproduces_the_reference_files(case, tmp_path):
    """Same weights, moments and counters -> the very bytes lm_save_checkpoint wrote (golden hash)."""
    with open(os.path.join(GOLD, "ckpt_full.json")) as f:
        gold = json.load(f)[case]
    kind, n_merges = FULL_CKPT_CASES[case]
    k = _info(kind, n_merges, t=4321, epoch=5, step=66)
    assert k.n == gold["n"]
    w = ckpt_weights(k.n)
    m, v = ckpt_moments(k.n)
    path = str(tmp_path / "full.ckpt")
    checkpoint.save_model(path, k, w, m, v, synthetic_merges(n_merges))
    data = open(path, "rb").read()
    assert len(data) == gold["size"] and data[:40].hex() == gold["head_hex"]
    assert hashlib.sha256(data).hexdigest() == gold["sha256"]
    assert not os.path.exists(path + ".tmp")
    # and back: the reader returns what went in, in optimizer order
    back = checkpoint.load_model(path)
    bi = back["info"]
    assert (bi.kind, bi.vocab, bi.tied, bi.n, bi.t, bi.epoch, bi.step, bi.has_adam) == \
        (kind, k.vocab, k.tied, k.n, 4321, 5, 66, 1)
    assert np.array_equal(back["w"], w) and np.array_equal(back["m"], m) and np.array_equal(back["v"], v)
    assert np.array_equal(back["merges"], synthetic_merges(n_merges))
    # the trailer alone is what the Adam-section reader sees (20 + 8 n bytes at the end)
    tail = checkpoint.read_adam(path, k.n)
    assert tail["t"] == 4321 and np.array_equal(tail["m"], m)


def test_weights_only_file_and_bad_files(tmp_path):
    k = _info(0, 0)
    w = ckpt_weights(k.n)
    path = str(tmp_path / "w.bin")
    checkpoint.save_model(path, k, w)                       # lm_save form: has_adam = 0
    back = checkpoint.load_model(path)
    assert back["info"].has_adam == 0 and back["m"] is None and np.array_equal(back["w"], w)
    assert os.path.getsize(path) == 32 + 4 * k.n + 8 * 14 + 4 * 13 + 4   # header, data, 14 matrices, 13 vectors, flag
    data = bytearray(open(path, "rb").read())
    bad = str(tmp_path / "bad.bin")
    for patch in ((0, b"LMCK"),                             # legacy double-precision magic
                  (4, (8).to_bytes(4, "little")),           # real size 8
                  (32, (65).to_bytes(4, "little"))):        # first tensor's row count off by one
        d2 = bytearray(data)
        d2[patch[0]:patch[0] + 4] = patch[1]
        open(bad, "wb").write(d2)
        with pytest.raises(capi.AnniError):
            checkpoint.load_model(bad)
    open(bad, "wb").write(data[:len(data) // 2])            # truncated
    with pytest.raises(capi.AnniError):
        checkpoint.load_model(bad)


@pytest.mark.parametrize("kind,n_merges", FULL_CKPT_CASES)
def test_round_trip_with_the_compiled_reference(reflib, tmp_path, kind, n_merges):
    """Reference writes -> product reads -> product writes identical bytes -> reference loads it."""
    n = reflib.full_slot_count(kind, n_merges)
    rng = np.random.default_rng(kind)
    w = rng.normal(0, 0.02, n).astype(np.float32)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = np.abs(rng.normal(0, 1e-6, n)).astype(np.float32)
    ref_path = str(tmp_path / "ref.ckpt")
    reflib.ckpt_save_full(ref_path, kind, n_merges, w, m, v, t=99, epoch=2, step=7)
    got = checkpoint.load_model(ref_path)
    assert got["info"].n == n and got["info"].t == 99 and got["info"].kind == kind
    assert np.array_equal(got["w"], w) and np.array_equal(got["m"], m) and np.array_equal(got["v"], v)
    ours = str(tmp_path / "ours.ckpt")
    checkpoint.save_model(ours, got["info"], got["w"], got["m"], got["v"], got["merges"])
    assert open(ours, "rb").read() == open(ref_path, "rb").read()
    # continue "training" on our side, save, and let the reference resume from it
    got["info"].t, got["info"].step = 100, 8
    checkpoint.save_model(ours, got["info"], w * 0.5, m * 2, v * 3, got["merges"])
    back = reflib.ckpt_load_full(ours, n)
    assert (back["n"], back["t"], back["epoch"], back["step"], back["tied"]) == (n, 100, 2, 8, int(kind == 2))
    assert np.array_equal(back["w"], w * 0.5) and np.array_equal(back["m"], m * 2) \
        and np.array_equal(back["v"], v * 3)
