"""``.pt`` checkpoints (model + EMA + optimizer) and weight loading.

Blob layout follows the reference (training/checkpointing.py:246-536) key for
key so checkpoints interchange (schedule-free runs are written under eval mode:
``model`` = the averaged iterate, ``snapshot_kind`` "x", ``train_mode`` False): ``model`` (no ``module.`` prefix),
``optimizer`` (``torch.optim.AdamW`` layout), ``optimizer_param_names``,
``scheduler``, ``global_step``, ``effective_step``, ``epoch``,
``best_eval_loss``, ``rng_states`` (one per rank), ``model_cfg`` / ``train_cfg``
(pickled dataclasses), ``snapshot_kind``, ``ema{decay,num_updates,shadow}``,
``scaler``, ``sampler``. Rank 0 writes; a single background thread fsyncs,
drops the page cache for the file, publishes it with an atomic rename and
rotates old files.
"""

from __future__ import annotations

import logging
import os
import queue
import random
import re
import shutil
import threading

import numpy as np
import torch

from ..compat import torch_load_compat
import torch.distributed as dist

from ..parallel.dist import DistInfo

logger = logging.getLogger(__name__)
CKPT_RE = re.compile(r"checkpoint_(\d+)\.pt$")


# --------------------------------------------------------------------------- weights
def load_safetensors(path: str):
    """``(state_dict, ModelConfig or None)`` from a safetensors file with embedded ``model_cfg_json``."""
    from safetensors import safe_open

    from ..config.schema import model_cfg_from_metadata

    state = {}
    with safe_open(path, framework="pt", device="cpu") as f:
        meta = f.metadata()
        for k in f.keys():
            state[k] = f.get_tensor(k)
    return state, model_cfg_from_metadata(meta)


def save_safetensors(path: str, state_dict: dict, model_cfg=None) -> None:
    from safetensors.torch import save_file

    from ..config.schema import model_cfg_to_metadata

    tensors = {k: v.detach().cpu().contiguous() for k, v in state_dict.items()}
    save_file(tensors, path, metadata=model_cfg_to_metadata(model_cfg) if model_cfg is not None else None)


def strip_module_prefix(state: dict) -> dict:
    out = {}
    for k, v in state.items():
        for prefix in ("module.df3.", "module.", "df3."):
            if k.startswith(prefix):
                k = k[len(prefix) :]
                break
        out[k] = v
    return out


def load_pretrained_weights(model, path: str, strict: bool = True) -> None:
    """Initialise ``model`` from ``.safetensors`` or from the ``model`` entry of a ``.pt`` checkpoint."""
    if path.endswith(".safetensors"):
        state, _ = load_safetensors(path)
    else:
        blob = torch_load_compat(path, map_location="cpu", weights_only=False, mmap=True)
        state = blob["model"] if isinstance(blob, dict) and "model" in blob else blob
    missing = model.load_state_dict(strip_module_prefix(state), strict=strict)
    if not strict and (missing.missing_keys or missing.unexpected_keys):
        logger.warning("load_pretrained_weights: %d missing, %d unexpected keys", len(missing.missing_keys),
                       len(missing.unexpected_keys))  # fmt: skip


# --------------------------------------------------------------------------- RNG
def local_rng_state() -> dict:
    state = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        state["cuda"] = torch.cuda.get_rng_state()
    return state


def restore_rng_state(state: dict | None) -> None:
    if not state:
        return
    random.setstate(state["python"])
    np.random.set_state(state["numpy"])
    torch.set_rng_state(state["torch"])
    if "cuda" in state and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["cuda"])


def gather_rng_states(info: DistInfo) -> list:
    """Every rank's RNG state, on every rank (an all-rank collective)."""
    mine = local_rng_state()
    if not info.is_distributed:
        return [mine]
    out = [None] * info.world_size
    dist.all_gather_object(out, mine)
    return out


# --------------------------------------------------------------------------- manager
class CheckpointManager:
    def __init__(self, output_dir: str, info: DistInfo, max_checkpoints: int = 0, staging_dir: str = ""):
        self.dir, self.info = output_dir, info
        self.max_checkpoints, self.staging_dir = max_checkpoints, staging_dir
        self._queue: queue.Queue = queue.Queue()
        self._error: BaseException | None = None
        self._thread: threading.Thread | None = None
        if info.is_main:
            os.makedirs(output_dir, exist_ok=True)
            if staging_dir:
                os.makedirs(staging_dir, exist_ok=True)

    # ---- background publish ----
    def _worker(self):
        while True:
            job = self._queue.get()
            if job is None:
                self._queue.task_done()
                return
            tmp, final = job
            try:
                with open(tmp, "rb") as fh:
                    os.fsync(fh.fileno())
                    if hasattr(os, "posix_fadvise"):
                        os.posix_fadvise(fh.fileno(), 0, 0, os.POSIX_FADV_DONTNEED)
                if os.path.dirname(tmp) != os.path.dirname(final):
                    part = final + ".part"
                    shutil.copyfile(tmp, part)
                    os.replace(part, final)
                    os.remove(tmp)
                else:
                    os.replace(tmp, final)
                self._rotate()
            except BaseException as exc:  # noqa: BLE001 - surfaced by wait_for_io / next save
                self._error = exc
            finally:
                self._queue.task_done()

    def _ensure_thread(self):
        if self._thread is None or not self._thread.is_alive():
            self._thread = threading.Thread(target=self._worker, name="ckpt-publish", daemon=True)
            self._thread.start()

    def wait_for_io(self) -> None:
        self._queue.join()
        if self._error is not None:
            err, self._error = self._error, None
            raise RuntimeError(f"checkpoint publish failed: {err!r}") from err

    def _rotate(self) -> None:
        if self.max_checkpoints <= 0:
            return
        found = sorted((int(m.group(1)), f) for f in os.listdir(self.dir) if (m := CKPT_RE.search(f)))
        for _, name in found[: -self.max_checkpoints]:
            try:
                os.remove(os.path.join(self.dir, name))
            except OSError:
                pass

    # ---- save / load ----
    def save(self, name: str, *, model, optimizer, scheduler, state, model_cfg, train_cfg, sampler=None,
             snapshot_kind: str = "live", scaler_state: dict | None = None, background: bool = True) -> str | None:  # fmt: skip
        """All ranks call this (the RNG gather is collective); rank 0 writes ``{dir}/{name}``."""
        from .schedule_free import FlatAdamWScheduleFree, optimizer_eval_mode

        rng_states = gather_rng_states(self.info)
        if not self.info.is_main:
            return None
        if self._error is not None:
            self.wait_for_io()
        if isinstance(optimizer, FlatAdamWScheduleFree):
            snapshot_kind = "x"  # written under eval mode: ``model`` holds the averaged iterate, train_mode False
        with optimizer_eval_mode(optimizer):
            model_state = {k: v.detach().cpu().clone() for k, v in strip_module_prefix(model.state_dict()).items()}
            optimizer_state = optimizer.state_dict()
        blob = {
            "model": model_state,
            "optimizer": optimizer_state,
            "optimizer_param_names": optimizer.param_names_by_index(),
            "scheduler": scheduler.state_dict(),
            "global_step": state.global_step,
            "effective_step": state.effective_step,
            "epoch": state.epoch,
            "best_eval_loss": state.best_eval_loss,
            "rng_states": rng_states,
            "model_cfg": model_cfg,
            "train_cfg": train_cfg,
            "snapshot_kind": snapshot_kind,
            "ema": optimizer.ema_state_dict() if optimizer.shadow is not None else None,
            "scaler": scaler_state or {},
            "sampler": sampler.state_dict() if sampler is not None and hasattr(sampler, "state_dict") else None,
        }
        final = os.path.join(self.dir, name)
        tmp = os.path.join(self.staging_dir or self.dir, name + ".tmp")
        torch.save(blob, tmp)
        self._ensure_thread()
        self._queue.put((tmp, final))
        if not background:
            self.wait_for_io()
        return final

    def load(self, path: str, *, model, optimizer=None, scheduler=None, state=None, sampler=None, strict=True,
             skip_optimizer=False, skip_scheduler=False, skip_step=False) -> dict:  # fmt: skip
        """Restore from ``path`` on every rank; returns the blob (minus tensors already consumed)."""
        blob = torch_load_compat(path, map_location="cpu", weights_only=False, mmap=True)
        model.load_state_dict(strip_module_prefix(blob["model"]), strict=strict)
        if optimizer is not None:
            # parameters are views into the flat buffer, load_state_dict copied into them in place
            if not skip_optimizer and blob.get("optimizer"):
                optimizer.load_state_dict(blob["optimizer"])
            from .schedule_free import FlatAdamWScheduleFree

            if isinstance(optimizer, FlatAdamWScheduleFree):
                groups = (blob.get("optimizer") or {}).get("param_groups") or [{}]
                if not skip_optimizer and blob.get("optimizer"):
                    if groups[0].get("train_mode", False):
                        raise RuntimeError(f"Schedule-Free checkpoint at {path} was saved with train_mode=True; expected False "
                                           "(checkpoints are written under optimizer_eval_mode)")
                    if blob["optimizer"].get("state"):
                        optimizer.train()  # parameters were loaded as x; back to y for training
                    else:
                        optimizer.reseed_z()  # saved before the first step: x = y = z
                else:
                    optimizer.reseed_z()  # no optimizer state: both sequences start from the loaded weights
            ema = blob.get("ema")
            if optimizer.shadow is not None:
                if ema and ema.get("shadow"):
                    optimizer.load_ema_state_dict(ema)
                else:
                    optimizer.ema_reseed()
        if scheduler is not None and not skip_scheduler and blob.get("scheduler"):
            scheduler.load_state_dict(blob["scheduler"])
        if state is not None and not skip_step:
            state.global_step = blob.get("global_step", 0)
            state.effective_step = blob.get("effective_step", state.global_step)
            state.epoch = blob.get("epoch", 0)
            state.best_eval_loss = blob.get("best_eval_loss", float("inf"))
        if sampler is not None and blob.get("sampler") is not None and hasattr(sampler, "load_state_dict"):
            sampler.load_state_dict(blob["sampler"])
        rng = blob.get("rng_states")
        if rng and not skip_step:
            restore_rng_state(rng[self.info.rank] if self.info.rank < len(rng) else rng[0])
        return blob

    def find_latest(self) -> str | None:
        if not os.path.isdir(self.dir):
            return None
        found = sorted((int(m.group(1)), f) for f in os.listdir(self.dir) if (m := CKPT_RE.search(f)))
        return os.path.join(self.dir, found[-1][1]) if found else None

    def close(self) -> None:
        if self._thread is not None and self._thread.is_alive():
            self._queue.put(None)
            self._thread.join()
