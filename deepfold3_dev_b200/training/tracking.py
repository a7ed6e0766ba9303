"""Metric sinks (reference: training/tracking.py:18-128).

A tracker has ``log(values: dict, step: int)`` and ``close()``. ``JsonlTracker`` appends one JSON object
per call to ``{output}/logs/metrics.jsonl``; ``StdoutTracker`` prints a compact line; ``WandbTracker`` is
used only when the ``wandb`` package is importable and ``--wandb`` was given.
"""

from __future__ import annotations

import json
import logging
import os
import time

logger = logging.getLogger(__name__)


class StdoutTracker:
    def __init__(self, keys=("train/total", "train/diffusion", "lr", "grad_norm", "time/step_s")):
        self.keys = keys

    def log(self, values: dict, step: int) -> None:
        shown = [f"{k}={values[k]:.4g}" for k in self.keys if isinstance(values.get(k), (int, float))]
        others = len(values) - len(shown)
        print(f"[step {step}] " + " ".join(shown) + (f"  (+{others} more)" if others > 0 else ""), flush=True)

    def close(self) -> None:
        pass


class JsonlTracker:
    def __init__(self, output_dir: str):
        os.makedirs(os.path.join(output_dir, "logs"), exist_ok=True)
        self.path = os.path.join(output_dir, "logs", "metrics.jsonl")
        self._f = open(self.path, "a")

    def log(self, values: dict, step: int) -> None:
        row = {"step": step, "time": time.time()}
        row.update({k: v for k, v in values.items() if isinstance(v, (int, float, str, bool))})
        self._f.write(json.dumps(row) + "\n")
        self._f.flush()

    def close(self) -> None:
        self._f.close()


class WandbTracker:
    def __init__(self, project: str, entity: str | None = None, name: str | None = None, config: dict | None = None):
        import wandb  # gated: raises ImportError where the package is absent

        self._wandb = wandb
        self._run = wandb.init(project=project, entity=entity, name=name, config=config or {}, resume="allow")

    def log(self, values: dict, step: int) -> None:
        self._wandb.log({k: v for k, v in values.items() if isinstance(v, (int, float))}, step=step)

    def close(self) -> None:
        self._run.finish()


def build_trackers(output_dir: str, is_main: bool, wandb_project: str | None = None, wandb_entity: str | None = None,
                   config: dict | None = None) -> list:  # fmt: skip
    if not is_main:
        return []
    out = [StdoutTracker(), JsonlTracker(output_dir)]
    if wandb_project:
        try:
            out.append(WandbTracker(wandb_project, wandb_entity, os.path.basename(os.path.normpath(output_dir)), config))
        except ImportError:
            logger.warning("--wandb given but the wandb package is not installed; logging to files only")
    return out
