"""Training loop: ``Trainer(train_cfg, model_cfg, ...).run(resume)`` (reference: training/trainer.py:144-1375).

One process per GPU. The model is not wrapped in DDP: parameters and gradients
live in the flat buffers of ``FlatAdamW`` and ``GradSync`` reduces them. The
loop keeps the reference's contracts: every rank runs the skip consensus on
every sync step, the shutdown flag is agreed on every micro-step, checkpoints
are written by rank 0 after an all-rank RNG gather, auto-resume picks the newest
``checkpoint_{step}.pt`` of the run directory.
"""

from __future__ import annotations

import dataclasses
import gc
import logging
import os
import time
from contextlib import nullcontext

import torch
import yaml

from ..config.schema import ModelConfig, TrainingConfig
from ..models.model import DeepFold3
from ..parallel.dist import (
    CheckpointRequestHandler,
    DistInfo,
    ShutdownCoordinator,
    destroy_process_group_safely,
    init_process_group,
)
from ..parallel.grad_sync import GradSync
from .checkpointing import CheckpointManager, load_pretrained_weights
from .engine import OptimizerEngine, training_step
from .flat_optimizer import FlatAdamW
from .meters import DistributedAverageMeters, StepTimeMeter
from .scheduler import build_scheduler
from .state import TrainState, seed_everything

logger = logging.getLogger(__name__)


def freeze_for_confidence(model) -> None:
    for name, p in model.named_parameters():
        if "confidence" not in name:
            p.requires_grad_(False)


def freeze_modules(model, names: list[str]) -> None:
    children = dict(model.named_children())
    unknown = [n for n in names if n not in children]
    if unknown:
        raise ValueError(f"freeze_modules: no top-level module {unknown}; have {sorted(children)}")
    for n in names:
        children[n].requires_grad_(False)


class Trainer:
    def __init__(self, train_cfg: TrainingConfig, model_cfg: ModelConfig | None = None, *, train_loader=None,
                 eval_loader=None, sampler=None, dist_info: DistInfo | None = None, device: str | None = None,
                 trackers=None, callbacks=None):  # fmt: skip
        self.cfg = train_cfg
        self.model_cfg = model_cfg or ModelConfig()
        self.dist = dist_info or init_process_group(train_cfg.collective_timeout_s, device)
        self.device = self.dist.device
        seed_everything(train_cfg.seed, self.dist.rank, deterministic=train_cfg.deterministic)
        if train_cfg.accumulate_grad_batches > 1 and self.model_cfg.precision.grad_acc_dtype != "fp32":
            raise ValueError("accumulate_grad_batches > 1 needs precision.grad_acc_dtype = 'fp32'")
        self.model = DeepFold3(self.model_cfg).to(self.device)
        if train_cfg.params_path:
            load_pretrained_weights(self.model, train_cfg.params_path, strict=train_cfg.load_strict)
        if train_cfg.train_confidence_only:
            freeze_for_confidence(self.model)
        if train_cfg.freeze_modules:
            freeze_modules(self.model, list(train_cfg.freeze_modules))
        self.model.train()
        if train_cfg.optimizer_type == "schedule_free":
            from .schedule_free import FlatAdamWScheduleFree as Opt

            self.optimizer = Opt(
                self.model, lr=train_cfg.lr, betas=train_cfg.betas, eps=train_cfg.eps,
                weight_decay=train_cfg.weight_decay, warmup_steps=train_cfg.warmup_steps,
                decoupling_parameter=train_cfg.decoupling_parameter, strong_decay=train_cfg.strong_decay,
                ema_decay=train_cfg.ema_decay,
            )  # fmt: skip
        elif train_cfg.optimizer_type == "adamw":
            self.optimizer = FlatAdamW(
                self.model, lr=train_cfg.lr, betas=train_cfg.betas, eps=train_cfg.eps,
                weight_decay=train_cfg.weight_decay, strong_decay=train_cfg.strong_decay,
                ema_decay=train_cfg.ema_decay,
            )  # fmt: skip
        else:
            raise ValueError(f"optimizer_type must be 'adamw' or 'schedule_free', got {train_cfg.optimizer_type!r}")
        self.scheduler = build_scheduler(self.optimizer, train_cfg)
        self.grad_sync = GradSync(self.dist)
        self.grad_sync.broadcast_parameters(self.optimizer)
        self.grad_sync.attach(self.optimizer)
        # the one-kernel optimizer step adopts the gradient buffer; do it now so that nothing captured later (CUDA graphs
        # of the training pass write into the gradient views) points at a buffer that is about to be replaced
        self.grad_sync.fused_step_engine(self.optimizer)
        self.engine = OptimizerEngine(self.optimizer, self.scheduler, self.dist, train_cfg, self.grad_sync)
        self.state = TrainState()
        self.ckpt = CheckpointManager(train_cfg.output_dir, self.dist, train_cfg.max_checkpoints,
                                      train_cfg.checkpoint_staging_dir)  # fmt: skip
        self.meters = DistributedAverageMeters(self.dist)
        self.timer = StepTimeMeter()
        self.train_loader, self.eval_loader, self.sampler = train_loader, eval_loader, sampler
        self.trackers = trackers or []
        from .callbacks import CallbackList

        self.callbacks = CallbackList(callbacks or [])
        self._pinned: dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ one optimizer step
    def _autocast(self):
        dtype = self.cfg.torch_dtype
        if dtype == torch.float32:
            return nullcontext()
        return torch.autocast(device_type=self.device.type, dtype=dtype)

    def stage_batch(self, features: dict) -> dict:
        """Host batch → device through reusable pinned buffers (asynchronous copies on the current stream)."""
        if self.device.type != "cuda":
            return features
        out = {}
        for k, v in features.items():
            if not isinstance(v, torch.Tensor):
                out[k] = v
                continue
            if v.is_cuda:
                out[k] = v
                continue
            buf = self._pinned.get(k)
            if buf is None or buf.shape != v.shape or buf.dtype != v.dtype:
                buf = torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
                self._pinned[k] = buf
            buf.copy_(v)
            out[k] = buf.to(self.device, non_blocking=True)
        return out

    def micro_step(self, features: dict, record_ids=None, num_recycles: int | None = None):
        """Forward, loss and backward of one micro-batch. Returns ``(loss, loss_dict, counts)``."""
        cfg = self.cfg
        features = self.stage_batch(features)
        with self._autocast():
            loss, loss_dict, counts, nrec = training_step(
                self.model, features, cfg=cfg, model_cfg=self.model_cfg, global_step=self.state.global_step,
                device=self.device, num_recycles=num_recycles,
            )  # fmt: skip
        self.state.last_num_recycles = nrec
        (loss / cfg.accumulate_grad_batches).backward()
        self.engine.add_microstep_loss(loss, record_ids)
        self.state.global_step += 1
        return loss.detach(), loss_dict, counts

    def train_step(self, features: dict, num_recycles: int | None = None) -> dict:
        """One full optimizer step on one batch (accumulation 1): the unit the throughput benchmark times.

        Copies the batch from host memory, runs forward / backward / gradient
        reduction / AdamW / EMA, and returns host floats (``loss``, ``grad_norm``, ``advanced``).
        """
        loss, _, _ = self.micro_step(features, num_recycles=num_recycles)
        result = self.engine.step_or_skip(self.state)
        loss_value = float(loss.item())  # the one host read of the step; the fused step's verdict has landed by then
        result = self.engine.resolve(self.state) or result
        norm = result.grad_norm
        return {
            "loss": loss_value,
            "grad_norm": float(norm.item()) if norm is not None else float("nan"),
            "advanced": result.advanced,
        }

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, name: str | None = None, background: bool = True):
        name = name or f"checkpoint_{self.state.effective_step}.pt"
        self.callbacks.fire("on_checkpoint_save", self, name)
        return self.ckpt.save(
            name, model=self.model, optimizer=self.optimizer, scheduler=self.scheduler, state=self.state,
            model_cfg=self.model_cfg, train_cfg=self.cfg, sampler=self.sampler, background=background,
        )  # fmt: skip

    def load_checkpoint(self, path: str, own_run: bool = False) -> None:
        """``own_run`` (auto-resume from this run's directory) ignores the ``skip_load_*`` switches."""
        cfg = self.cfg
        self.ckpt.load(
            path, model=self.model, optimizer=self.optimizer, scheduler=self.scheduler, state=self.state,
            sampler=self.sampler, strict=cfg.load_strict,
            skip_optimizer=cfg.skip_load_optimizer and not own_run,
            skip_scheduler=cfg.skip_load_scheduler and not own_run,
            skip_step=cfg.skip_load_step and not own_run,
        )  # fmt: skip
        if self.dist.is_main:
            logger.info("resumed from %s at step %d", path, self.state.effective_step)
        # the YAML learning rate wins over the checkpoint's
        self.scheduler.base_lrs = [cfg.lr for _ in self.scheduler.base_lrs]
        self.scheduler._apply()

    def _dump_run_files(self) -> None:
        if not self.dist.is_main:
            return
        os.makedirs(self.cfg.output_dir, exist_ok=True)
        with open(os.path.join(self.cfg.output_dir, "config.yaml"), "w") as fh:
            yaml.safe_dump({"training": _plain(self.cfg), "model": _plain(self.model_cfg)}, fh, sort_keys=False)
        from ..utils.provenance import provenance

        with open(os.path.join(self.cfg.output_dir, "provenance.yaml"), "w") as fh:
            yaml.safe_dump(provenance(), fh, sort_keys=False)

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def evaluate(self) -> dict[str, float]:
        """Mean losses over ``eval_loader`` with the EMA weights swapped in (``eval_snapshot='shadow'``)."""
        if self.eval_loader is None:
            return {}
        from .schedule_free import FlatAdamWScheduleFree

        use_shadow = self.cfg.eval_snapshot == "shadow" and self.optimizer.shadow is not None
        sf_flip = isinstance(self.optimizer, FlatAdamWScheduleFree) and self.optimizer.train_mode
        if sf_flip:
            self.optimizer.eval()  # schedule-free: evaluate the averaged iterate x, as the reference does
        if use_shadow:
            self.optimizer.ema_swap()
        self.model.eval()
        meters = DistributedAverageMeters(self.dist)
        try:
            eval_cfg = dataclasses.replace(self.cfg, diffusion_batch_size=1, diffusion_chunk_size=0)
            for i, batch in enumerate(self.eval_loader):
                try:
                    with self._autocast():
                        _, ld, counts, _ = training_step(
                            self.model, self.stage_batch(batch), cfg=eval_cfg, model_cfg=self.model_cfg,
                            global_step=i, device=self.device, num_recycles=self.cfg.max_recycles,
                        )  # fmt: skip
                    meters.update({f"eval/{k}": v for k, v in ld.items()}, {f"eval/{k}": c for k, c in counts.items()})
                except Exception:  # noqa: BLE001 - a bad eval sample must not desynchronise the ranks
                    logger.exception("eval sample %d failed on rank %d", i, self.dist.rank)
        finally:
            self.model.train()
            if use_shadow:
                self.optimizer.ema_swap()
            if sf_flip:
                self.optimizer.train()
        return meters.sync()

    # ------------------------------------------------------------------ main loop
    def run(self, resume: str | None = None) -> TrainState:
        cfg, st = self.cfg, self.state
        self._dump_run_files()
        if resume:
            self.load_checkpoint(resume)
        elif cfg.auto_resume and (latest := self.ckpt.find_latest()):
            logger.info("auto-resume from %s", latest)
            self.load_checkpoint(latest, own_run=True)
        if self.train_loader is None:
            raise ValueError("Trainer.run needs a train_loader")
        gc.freeze()  # long-lived objects out of the collector's way before workers fork
        shutdown = ShutdownCoordinator(self.dist)
        ckpt_request = CheckpointRequestHandler()
        acc = cfg.accumulate_grad_batches
        if cfg.eval_before and self.eval_loader is not None:
            self._log(self.evaluate())
        self._last_ckpt_wall = time.time()
        data_wait = 0.0
        it = iter(self.train_loader)
        stopped = False
        self.callbacks.fire("on_train_start", self)
        while st.effective_step < cfg.max_steps and not stopped:
            t0 = time.perf_counter()
            try:
                batch = next(it)
            except StopIteration:
                st.epoch += 1
                it = iter(self.train_loader)
                batch = next(it)
            data_wait += time.perf_counter() - t0
            record_ids = batch.pop("_record_id", None) if isinstance(batch, dict) else None
            self.callbacks.fire("on_step_start", self, batch)
            self.timer.start()
            t_step = time.perf_counter()
            _, loss_dict, counts = self.micro_step(batch, record_ids)
            self.meters.update({f"train/{k}": v for k, v in loss_dict.items()},
                               {f"train/{k}": c for k, c in counts.items()})  # fmt: skip
            if st.global_step % acc == 0:
                result = self.engine.step_or_skip(st)
                boundary = any(iv > 0 and st.effective_step % iv == 0 for iv in (cfg.checkpoint_interval, cfg.eval_interval))
                if boundary or st.global_step % (cfg.log_interval * acc) == 0 or st.effective_step >= cfg.max_steps:
                    # a decision that depends on the step number follows: settle the fused step's verdict first
                    result = self.engine.resolve(st) or result
                self.callbacks.fire("on_step_end" if result.advanced else "on_skip_step", self, result)
                if result.advanced:
                    if result.grad_norm is not None:
                        self.meters.update({"train/grad_norm": result.grad_norm})
                    self._after_optimizer_step(ckpt_request)
            self.timer.stop()
            if cfg.slow_step_log_threshold_s > 0:
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                dt = time.perf_counter() - t_step
                if dt > cfg.slow_step_log_threshold_s:
                    logger.warning("SLOW_STEP rank=%d step=%d dt=%.1fs records=%s", self.dist.rank, st.global_step, dt,
                                   record_ids)  # fmt: skip
            if st.global_step % (cfg.log_interval * acc) == 0:
                mean_ms, max_ms, _ = self.timer.flush()
                wait = torch.tensor(data_wait, device=self.device)
                if self.dist.is_distributed:
                    torch.distributed.all_reduce(wait, op=torch.distributed.ReduceOp.MAX)
                vals = self.meters.sync()
                vals.update({"train/step_ms": mean_ms, "train/step_ms_max": max_ms, "train/data_wait_s": float(wait),
                             "train/lr": self.scheduler.get_last_lr()[0], "train/step": st.effective_step})  # fmt: skip
                self._log(vals)
                data_wait = 0.0
            stopped = shutdown.tick()
        self.engine.resolve(st)
        self.callbacks.fire("on_train_end", self)
        if stopped and st.global_step % acc != 0:
            # shutdown inside an accumulation window: drop the partial gradients and go back to the last boundary, so the
            # resumed run starts on a full window (reference: training/trainer.py:1322-1345)
            self.optimizer.zero_grad()
            st.global_step -= st.global_step % acc
        if stopped and self.dist.is_main:
            logger.info("stop requested: writing checkpoint at step %d and leaving", st.effective_step)
        self.save_checkpoint("checkpoint_final.pt" if not stopped else None, background=False)
        self.ckpt.wait_for_io()
        self.ckpt.close()
        destroy_process_group_safely(self.dist)
        return st

    def _after_optimizer_step(self, ckpt_request) -> None:
        cfg, st = self.cfg, self.state
        want = st.effective_step % cfg.checkpoint_interval == 0
        if self.dist.is_main:  # wall clock and signals are rank 0's alone; the others follow its broadcast
            want = want or ckpt_request.consume()
            if cfg.checkpoint_every_hours > 0 and time.time() - self._last_ckpt_wall > cfg.checkpoint_every_hours * 3600:
                want = True
        if self.dist.is_distributed:  # rank 0 decides, every rank takes part in the RNG gather
            flag = torch.tensor([int(want)], device=self.device)
            torch.distributed.broadcast(flag, src=0)
            want = bool(flag.item())
        if want:
            self.save_checkpoint()
            self._last_ckpt_wall = time.time()  # whatever triggered it, the hourly timer starts over
        if self.eval_loader is not None and st.effective_step % cfg.eval_interval == 0:
            self.callbacks.fire("on_eval_start", self)
            vals = self.evaluate()
            self.callbacks.fire("on_eval_end", self, vals)
            self._log(vals)
            total = vals.get("eval/total")
            if total is not None and total < st.best_eval_loss:
                st.best_eval_loss = total
                self.save_checkpoint("checkpoint_best.pt")

    def _log(self, values: dict) -> None:
        if not values or not self.dist.is_main:
            return
        for t in self.trackers:
            t.log(values, self.state.effective_step)
        if not self.trackers:
            logger.info("step %d: %s", self.state.effective_step,
                        " ".join(f"{k}={v:.4g}" for k, v in sorted(values.items()) if isinstance(v, (int, float))))  # fmt: skip


def _plain(cfg) -> dict:
    """Dataclass tree → plain dict that ``yaml.safe_dump`` accepts (tuples become lists)."""

    def conv(v):
        if dataclasses.is_dataclass(v):
            return {f.name: conv(getattr(v, f.name)) for f in dataclasses.fields(v)}
        if isinstance(v, (list, tuple)):
            return [conv(x) for x in v]
        if isinstance(v, dict):
            return {k: conv(x) for k, x in v.items()}
        return v

    return conv(cfg)
