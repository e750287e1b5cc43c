"""anni_b200: B200-native optimizer-step engine behind the AnnI trainer's C host API.

The product is ``libanni_b200.so`` (CUDA C++ for sm_100a, C ABI declared in
``include/``).  This package is the thin host-side mirror used by the tests and the
benchmark: ctypes bindings, the reference's segment order and schedules, and the
ZeRO-1 plumbing over ``torch.distributed``.
"""
from .capi import (DT_BF16, DT_F32, SEG_TWIN_BF16, SEG_TWIN_FP8, SEG_WD,  # noqa: F401
                   STEP_CHECK_FINITE, STEP_DEV_LOSS_SCALE, STEP_ZERO_GRAD, AnniError)
