"""The LR schedule the trainer evaluates before each step (host side).

``lr_at`` is the reference trainer's ``lm_train_step_lr`` (``lang/lm_train.c:98-124``),
evaluated by the library's C function ``anni_lr_schedule`` so that Python and C callers get
the same doubles.  The trainer calls it with ``opt->t`` BEFORE the step increments it
(``lang/lm_train.c:1336``).  (The dynamic loss scale is not kept here: it lives on the device,
``anni_optstep_loss_scale_init`` / ``OptStep.loss_scale_init``.)
"""
import ctypes as C

from . import capi


def lr_at(base_lr, step, warmup_steps=0, decay_steps=0, decay_kind="cosine", sched_from=0):
    L = capi.lib()
    L.anni_lr_schedule.restype = C.c_double
    L.anni_lr_schedule.argtypes = [C.c_double, C.c_int, C.c_int, C.c_int, C.c_char_p, C.c_int]
    return L.anni_lr_schedule(base_lr, int(step), int(warmup_steps), int(decay_steps),
                              decay_kind.encode(), int(sched_from))
