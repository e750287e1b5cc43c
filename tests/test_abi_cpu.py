"""CPU-only checks of the C ABI: the library loads, exports every symbol the headers declare,
and its pure-host entry points (schedule, checkpoint, parameter count, argument checks) behave."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

from anni_b200 import capi, checkpoint, schedule

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden")


def _declared_symbols(header):
    src = open(os.path.join(ROOT, "include", header)).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    src = re.sub(r"#.*", "", src)
    names = set()
    for decl in src.split(";"):
        if "(" not in decl or "typedef" in decl:
            continue
        m = re.search(r"\b((?:anni|gpu)_\w+)\s*\(", decl)
        if m:
            names.add(m.group(1))
    return names


@pytest.mark.parametrize("header", ["anni_b200.h", "anni_gpu_compat.h", "anni_lm_adam.h", "anni_zero1.h"])
def test_every_declared_symbol_is_exported(header):
    L = capi.lib()
    names = _declared_symbols(header)
    assert len(names) >= 10
    missing = [n for n in sorted(names) if not hasattr(L, n)]
    assert not missing, missing


def test_reference_device_api_symbols_all_link():
    """Every gpu_* symbol of the reference's num/gpu.h (99 of them) resolves in the library,
    so the reference trainer links it in place of its own backend object."""
    L = capi.lib()
    names = """gpu_available gpu_mem_info gpu_sync_mode gpu_fp8 gpu_memcpy_h2d gpu_memcpy_d2h gpu_host_pin
    gpu_memcpy_d2h_async gpu_stream_sync gpu_memcpy_d2d gpu_memset gpu_adam_seed_bf16_flat gpu_ce_fetch_mean
    gpu_mat_mul gpu_mat_mul_bias gpu_mat_mul_res gpu_mat_mul_bias_relu gpu_mat_mul_bt gpu_mat_mul_bt_acc
    gpu_mat_mul_bt_twin gpu_mat_mul_at gpu_mat_outer_add gpu_layernorm_backward gpu_layernorm_backward_acc
    gpu_layernorm_backward_x gpu_layernorm_xhat gpu_grad_sumsq gpu_adam_step_dev_bf16 gpu_softmax_rows
    gpu_softmax_bwd_rows gpu_layernorm_forward_ex gpu_bias_row_add gpu_ce_delta_from_softmax
    gpu_ce_softmax_delta_bf16 gpu_ce_bias_fused gpu_ce_bf16_delta_done gpu_ce_nll_rows gpu_posenc_add_packed
    gpu_mat_col_sum_add gpu_relu_backward gpu_ffn_relu_bwd_fused gpu_act_bf16_only gpu_attn_causal_fwd
    gpu_attn_flash_fwd gpu_attn_fa_fwd gpu_attn_fa_usable gpu_attn_fa_bwd gpu_attn_qkv_bwd gpu_attn_tiled_bwd
    gpu_attn_causal_bwd gpu_attn_tc_fwd gpu_attn_tc_bwd gpu_attn_qkv_fused gpu_pack_seq_rows gpu_unpack_seq_rows
    gpu_ffn_w1_finish gpu_mat_copy gpu_mat_add gpu_mat_add2 gpu_mat_axpy gpu_embed_lookup gpu_embed_scatter
    gpu_graph_begin gpu_graph_end gpu_graph_replay gpu_graph_replayable gpu_graph_supported gpu_ids_stage
    gpu_dec_set_layer gpu_dec_set_io gpu_dec_kv_load gpu_dec_step gpu_backend_name gpu_debug_last_error
    gpu_set_sync_mode gpu_set_compute_prec gpu_set_fp8 gpu_set_fp8_dgrad gpu_device_sync gpu_free
    gpu_half_wt_invalidate gpu_host_forget gpu_op_prof_dump gpu_adam_set_bf16_flat gpu_grad_twins_clear
    gpu_adam_set_weight_decay gpu_attn_qkv_bf16_hint gpu_attn_set_seqlens gpu_host_free gpu_graph_destroy
    gpu_graph_set_mode gpu_ids_unstage gpu_dec_free gpu_malloc gpu_host_alloc gpu_copy_stream gpu_param_epoch
    gpu_ce_targets_staged gpu_dec_create""".split()
    assert len(names) == 99
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing
    # forward/backward entry points answer like the reference's stub backend
    for n in ("gpu_mat_mul", "gpu_attn_flash_fwd", "gpu_graph_begin", "gpu_dec_step"):
        f = getattr(L, n)
        f.restype = C.c_int
        assert f() == -1
    for n in ("gpu_graph_supported", "gpu_attn_fa_usable", "gpu_act_bf16_only"):
        f = getattr(L, n)
        f.restype = C.c_int
        assert f() == 0


def test_lr_schedule_product_equals_golden():
    with open(os.path.join(GOLD, "lr_schedule.json")) as f:
        pts = json.load(f)
    for q in pts:
        assert schedule.lr_at(q["base"], q["step"], q["warmup"], q["decay"], q["kind"], q["start"]) == q["lr"]


def test_checkpoint_trailer_product_equals_golden(tmp_path):
    import hashlib
    from golden.make_golden import ckpt_moments
    with open(os.path.join(GOLD, "segments_tiny.json")) as f:
        meta = json.load(f)
    m, v = ckpt_moments(meta["n"])
    path = str(tmp_path / "adam.bin")
    checkpoint.write_adam(path, m, v, t=meta["t"], epoch=meta["epoch"], step=meta["step"])
    data = open(path, "rb").read()
    assert hashlib.sha256(data).hexdigest() == meta["trailer_sha256"]
    back = checkpoint.read_adam(path, meta["n"])
    assert back["t"] == meta["t"] and np.array_equal(back["m"], m) and np.array_equal(back["v"], v)
    with pytest.raises(capi.AnniError):                       # wrong slot count is refused, like the loader
        checkpoint.read_adam(path, meta["n"] - 1, offset=0)


def test_param_count_entry_point():
    L = capi.lib()
    L.anni_lm_param_count.restype = C.c_int64
    L.anni_lm_param_count.argtypes = [C.c_int] * 5
    assert L.anni_lm_param_count(1024, 4096, 12, 16384, 0) == 184_676_352
    assert L.anni_lm_param_count(1536, 6272, 14, 100000, 1) == 555_762_080
    assert L.anni_lm_param_count(2560, 10240, 32, 100000, 1) == 2_773_419_680


def test_bad_arguments_are_refused_before_any_launch():
    L = capi.lib()
    h = C.c_void_p()
    cfg = capi.Config()
    cfg.n_arena, cfg.shard_off, cfg.shard_n = 100, 50, 51          # shard sticks out of the arena
    assert L.anni_optstep_create(C.byref(cfg), C.byref(h)) == capi.E_ARG
    cfg.shard_n, cfg.grad_dtype = 50, 7
    assert L.anni_optstep_create(C.byref(cfg), C.byref(h)) == capi.E_ARG
    off = np.array([0, 60, 40, 100], np.int64)                     # offsets not ascending
    flg = np.zeros(3, np.uint32)
    cfg.grad_dtype, cfg.n_seg, cfg.seg_off, cfg.seg_flags = 0, 3, off.ctypes.data, flg.ctypes.data
    assert L.anni_optstep_create(C.byref(cfg), C.byref(h)) == capi.E_ARG
    assert L.anni_optstep_step(None, None, None) == capi.E_ARG
    big = capi.Config()
    big.n_seg = capi.NOALLOC_MAX_SEG + 1
    assert L.anni_optstep_step_noalloc(C.byref(big), C.byref(capi.Buffers()), C.byref(capi.Hyper()),
                                       None, None) == capi.E_LIMIT


def test_part_wise_calls_and_helpers_refuse_bad_arguments():
    L = capi.lib()
    hp = capi.Hyper()
    assert L.anni_optstep_update_range(None, C.byref(hp), 0, 0, 0, None) == capi.E_ARG
    assert L.anni_optstep_reduce_norm_range(None, C.byref(hp), 0, 0, 0, None) == capi.E_ARG
    assert L.anni_optstep_quantize_ex(None, 0, None) == capi.E_ARG
    assert L.anni_peer_copy(None, None, 16, None) == capi.E_ARG
    p, size, comp = C.c_void_p(), C.c_size_t(), C.c_int()
    assert L.anni_arena_alloc(0, C.byref(p), C.byref(size), C.byref(comp)) == capi.E_ARG
    assert L.anni_arena_alloc(1 << 20, None, C.byref(size), None) == capi.E_ARG
    assert L.anni_arena_free(None, 0) == capi.OK
    import torch
    if not torch.cuda.is_available():                       # without a device the allocator says so
        assert L.anni_arena_alloc(1 << 20, C.byref(p), C.byref(size), C.byref(comp)) in (capi.E_CUDA, capi.E_LIMIT)
        assert not p.value and size.value == 0


def test_zero1_driver_geometry_and_argument_checks():
    """anni_zero1_*: the shard geometry equals the Python driver's, and create judges its
    arguments before it touches a device or the communicator -- checked here with made-up
    arena addresses and a made-up communicator handle, none of which is ever dereferenced."""
    from anni_b200.capi import DT_BF16, DT_F32, E_ARG, OK, Zero1Config
    from anni_b200.zero1 import shard_geometry
    L = capi.lib()
    u64 = C.c_uint64
    for n, world in ((138156, 2), (555_762_080, 8), (2_773_419_680, 8), (5000, 8), (100, 1)):
        per, own = shard_geometry(n, world)
        for rank in range(world):
            a, b, c = u64(), u64(), u64()
            assert L.anni_zero1_geometry(n, world, rank, C.byref(a), C.byref(b), C.byref(c)) == OK
            assert a.value == per and c.value == own[rank][1]
            assert b.value == min(own[rank][0], n)
    assert L.anni_zero1_geometry(100, 9, 0, None, None, None) == E_ARG         # more ranks than one NVSwitch domain
    assert L.anni_zero1_geometry(100, 2, 2, None, None, None) == E_ARG

    off = np.array([0, 600, 1000], np.int64)
    flg = np.array([3, 2], np.uint32)
    fake = 0x7f0000001000                                                      # never dereferenced

    def cfg(**kw):
        c = Zero1Config()
        c.n_arena, c.grad_dtype, c.state_dtype = 1000, DT_BF16, DT_F32
        c.n_seg, c.seg_off, c.seg_flags = 2, off.ctypes.data, flg.ctypes.data
        c.rank, c.world, c.nccl_comm = 0, 2, fake
        c.grad_arena, c.twin_arena = fake + 0x1000, fake + 0x2000
        for k, v in kw.items():
            setattr(c, k, v)
        return c
    h = C.c_void_p()
    for bad in (dict(world=0), dict(world=9), dict(rank=2), dict(rank=-1), dict(grad_dtype=7),
                dict(nccl_comm=None), dict(grad_arena=None), dict(twin_arena=None), dict(n_seg=-1),
                dict(seg_off=None)):
        assert L.anni_zero1_create(C.byref(cfg(**bad)), C.byref(h)) == E_ARG, bad
        assert not h.value
    # e4m3 twins asked for, but no arena for them
    flg8 = np.array([5, 2], np.uint32)
    assert L.anni_zero1_create(C.byref(cfg(seg_flags=flg8.ctypes.data)), C.byref(h)) == E_ARG
    # peer mode: this rank's entry must be its own arena
    arr = (C.c_void_p * 2)(fake + 0x9000, fake + 0xa000)
    tw = (C.c_void_p * 2)(fake + 0x2000, fake + 0xb000)
    assert L.anni_zero1_create(C.byref(cfg(peer_grad=C.cast(arr, C.c_void_p), peer_twin=C.cast(tw, C.c_void_p))),
                               C.byref(h)) == E_ARG
    assert L.anni_zero1_create(None, C.byref(h)) == E_ARG and L.anni_zero1_create(C.byref(cfg()), None) == E_ARG
    assert L.anni_zero1_step(None, None, 0, None, None) == E_ARG
    assert L.anni_zero1_unique_id(None) == E_ARG
    assert L.anni_zero1_comm_init(None, 0, 2, C.byref(h)) == E_ARG
    assert L.anni_zero1_nccl_available() in (0, 1)


def test_shard_geometry_properties():
    """Shard geometry of the C driver over many arena sizes and world sizes: shards are whole
    multiples of 4096 elements, cover the arena exactly once in rank order, and agree with the
    Python driver's."""
    from hypothesis import given, settings, strategies as st
    from anni_b200.zero1 import shard_geometry
    L = capi.lib()
    u64 = C.c_uint64

    @settings(max_examples=200, deadline=None)
    @given(n=st.integers(min_value=1, max_value=3_000_000_000), world=st.integers(min_value=1, max_value=8))
    def check(n, world):
        per, own = shard_geometry(n, world)
        covered = 0
        for rank in range(world):
            a, b, c = u64(), u64(), u64()
            assert L.anni_zero1_geometry(n, world, rank, C.byref(a), C.byref(b), C.byref(c)) == capi.OK
            assert a.value == per and a.value % 4096 == 0 and a.value * world >= n
            assert c.value == own[rank][1] and c.value <= a.value
            if c.value:
                assert b.value == covered == rank * a.value
            covered += c.value
        assert covered == n
    check()


def test_binding_constants_equal_the_header():
    """The Python binding's flag and type constants are the header's (a drifted copy would pass
    wrong flags silently)."""
    import re
    from anni_b200 import capi
    text = open(os.path.join(ROOT, "include", "anni_b200.h")).read()
    text += open(os.path.join(ROOT, "include", "anni_zero1.h")).read()
    defs = {m.group(1): int(m.group(2), 0)
            for m in re.finditer(r"^#define\s+(ANNI_[A-Z0-9_]+)\s+\(?(-?(?:0x[0-9a-fA-F]+|\d+))u?\)?\s", text, re.M)}
    pairs = {"ANNI_STEP_CHECK_FINITE": capi.STEP_CHECK_FINITE, "ANNI_STEP_ZERO_GRAD": capi.STEP_ZERO_GRAD,
             "ANNI_STEP_DEV_LOSS_SCALE": capi.STEP_DEV_LOSS_SCALE, "ANNI_STEP_EXACT_UPDATE": capi.STEP_EXACT_UPDATE,
             "ANNI_STEP_REDUCE_CLEARS_OWN": capi.STEP_REDUCE_CLEARS_OWN, "ANNI_DT_F32": capi.DT_F32,
             "ANNI_DT_BF16": capi.DT_BF16, "ANNI_SEG_WD": capi.SEG_WD, "ANNI_SEG_TWIN_BF16": capi.SEG_TWIN_BF16,
             "ANNI_SEG_TWIN_FP8": capi.SEG_TWIN_FP8, "ANNI_ZERO1_GRADS_COMPLETE": capi.ZERO1_GRADS_COMPLETE,
             "ANNI_ZERO1_UNIQUE_ID_BYTES": capi.ZERO1_UNIQUE_ID_BYTES}
    for name, value in pairs.items():
        assert defs.get(name) == value, (name, defs.get(name), value)
