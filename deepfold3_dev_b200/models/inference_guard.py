"""Refusals by name: an op that cannot serve a call says so instead of falling back silently.

Same contract as the reference (model/inference_guard.py:48-75): an
inference-only entry point raises as soon as autograd could record through it.
"""

from __future__ import annotations

import functools

import torch


class InferenceOnlyKernelError(RuntimeError):
    """An inference-only kernel was reached with grad enabled."""


class NotActive(Exception):
    """A kernel cannot serve this call; ``lever`` names it and ``reason`` says why."""

    def __init__(self, lever: str, reason: str):
        self.lever, self.reason = lever, reason
        super().__init__(f"NOT ACTIVE: {lever}: {reason}")


def inference_only(lever: str):
    def decorate(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            if torch.is_grad_enabled():
                raise InferenceOnlyKernelError(
                    f"{lever} is inference-only and has no backward: call it under torch.no_grad() "
                    "or torch.inference_mode()."
                )
            return fn(*args, **kwargs)

        return wrapper

    return decorate
