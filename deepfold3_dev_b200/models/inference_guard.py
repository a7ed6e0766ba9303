"""Kernels that say no.

Two ways an op can decline a call, both loud: ``NotActive`` ("this kernel does not take this call", with the name of
the switch and the reason, so that the kernel census can report why a requested path did not run), and the
``inference_only`` decorator for entry points that have no backward (they must never be reached while autograd is
recording; reference: model/inference_guard.py:48-75).
"""

from __future__ import annotations

from functools import wraps

import torch


class InferenceOnlyKernelError(RuntimeError):
    """Autograd was recording when an entry point without a backward was called."""


class NotActive(Exception):
    """``lever`` (the configuration switch of a kernel) cannot serve the call, for ``reason``."""

    def __init__(self, lever: str, reason: str):
        super().__init__(f"NOT ACTIVE: {lever}: {reason}")
        self.lever = lever
        self.reason = reason


def inference_only(lever: str):
    """Decorator: the wrapped function raises ``InferenceOnlyKernelError`` when called with grad mode on."""

    def wrap(fn):
        message = (f"{lever} has no backward pass; it may only run under torch.no_grad() or torch.inference_mode() "
                   "(grad mode was on)")  # fmt: skip

        @wraps(fn)
        def guarded(*args, **kwargs):
            if torch.is_grad_enabled():
                raise InferenceOnlyKernelError(message)
            return fn(*args, **kwargs)

        return guarded

    return wrap
