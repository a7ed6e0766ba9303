"""Lifecycle hooks of the trainer (reference: training/callbacks/__init__.py:33-112).

Every rank constructs the same callbacks in the same order, and a hook that issues a collective must do so
on every rank in the same call: hooks run inside the step loop, where a rank-dependent branch would
desynchronise the ranks.
"""

from __future__ import annotations


class Callback:
    def on_train_start(self, trainer) -> None: ...
    def on_step_start(self, trainer, features: dict) -> None: ...
    def on_step_end(self, trainer, result) -> None: ...
    def on_skip_step(self, trainer, result) -> None: ...
    def on_eval_start(self, trainer) -> None: ...
    def on_eval_end(self, trainer, metrics: dict) -> None: ...
    def on_checkpoint_save(self, trainer, path) -> None: ...
    def on_train_end(self, trainer) -> None: ...


class CallbackList:
    def __init__(self, callbacks=()):
        self.callbacks = list(callbacks)

    def fire(self, hook: str, *args) -> None:
        for cb in self.callbacks:
            getattr(cb, hook)(*args)


class EMACallback(Callback):
    """The shadow update is fused into the optimizer kernel; this hook only exposes its counters to the log."""

    def on_step_end(self, trainer, result) -> None:
        if result.advanced and trainer.optimizer.shadow is not None:
            trainer.state.ema_updates = trainer.optimizer.ema_updates


class ActivationMeterCallback(Callback):
    """Logs the residual-branch RMS values collected by ``ActivationRMSMeter`` every ``interval`` steps."""

    def __init__(self, meter, interval: int = 100):
        self.meter, self.interval = meter, interval

    def on_step_start(self, trainer, features) -> None:
        self.meter.enabled = (trainer.state.effective_step + 1) % self.interval == 0

    def on_step_end(self, trainer, result) -> None:
        if self.meter.enabled:
            trainer._log(self.meter.flush_to_dict())
            self.meter.enabled = False
