"""One training micro-step and the optimizer step with cross-rank skip consensus.

``training_step`` mirrors the reference's (training/step.py:99-209): pick the
recycle count (same on every rank), run ``forward_training`` under autocast,
evaluate the loss per batch element in fp32. ``OptimizerEngine.step_or_skip``
mirrors ``WrappedOptimizer.step_or_skip`` (training/optim.py:627-804): every
rank, every sync step, gathers the loss-NaN flags and the gradient norms; all
ranks skip together; too many consecutive skips abort. The gradient path
underneath is the flat-buffer optimizer and ``GradSync`` rather than DDP.
"""

from __future__ import annotations

import logging
import random
from dataclasses import dataclass
from typing import Literal

import torch

from ..models.precision import fp32_guard
from ..parallel.dist import DistInfo, all_gather_scalar, collective_guard
from ..parallel.grad_sync import GradSync
from .collectives import slice_batch_dict
from .flat_optimizer import FlatAdamW
from .objective import training_loss
from .state import TrainState

logger = logging.getLogger(__name__)


def is_chunked_diffusion_active(cfg) -> bool:
    return cfg.diffusion_chunk_size > 0 and cfg.diffusion_batch_size % cfg.diffusion_chunk_size == 0


def pick_num_recycles(cfg, global_step: int) -> int:
    """Uniform in ``[0, max_recycles]``; with ``uniform_recycle`` seeded by the step so all ranks agree."""
    if cfg.uniform_recycle:
        return random.Random(cfg.seed + global_step).randint(0, cfg.max_recycles)
    return random.randint(0, cfg.max_recycles)


def prepare_features(features: dict, device) -> dict:
    return {k: (v.to(device, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in features.items()}


def aggregate_sample_losses(per_sample: list[dict]):
    """Mean of each reported term over the samples that emitted it, plus those counts."""
    sums, counts = {}, {}
    for ld in per_sample:
        for k, v in ld.items():
            sums[k] = sums[k] + v if k in sums else v
            counts[k] = counts.get(k, 0) + 1
    return {k: v / counts[k] for k, v in sums.items()}, counts


def training_step(model, features, *, cfg, model_cfg, global_step: int, device, num_recycles: int | None = None):
    """Forward + loss of one micro-batch. Returns ``(total_loss, loss_dict, loss_counts, num_recycles)``.

    With chunked diffusion the per-chunk losses are back-propagated inside the
    forward (each divided by ``accumulate_grad_batches``); the returned total
    still has to be back-propagated by the caller for the remaining terms.
    """
    features = prepare_features(features, device)
    if num_recycles is None:
        num_recycles = pick_num_recycles(cfg, global_step)
    chunked = is_chunked_diffusion_active(cfg)
    acc = cfg.accumulate_grad_batches

    def backward_fn(loss):
        (loss / acc).backward()

    pred = model.forward_training(
        features, num_recycles=num_recycles, diffusion_batch_size=cfg.diffusion_batch_size,
        mini_rollout_steps=cfg.mini_rollout_steps, mini_rollout_samples=cfg.mini_rollout_samples, seed=global_step,
        fused_ce=cfg.use_fused_ce_loss, diffusion_chunk_size=cfg.diffusion_chunk_size if chunked else 0,
        backward_fn=backward_fn if chunked else None, loss_cfg=cfg if chunked else None,
        compute_confidence=cfg.alpha_confidence > 0, msa_precropped=cfg.msa_precrop,
        chain_perm_gate_k=(cfg.chain_perm_gate_k if cfg.chain_perm_stability_gate else 1),
        permute_gt_before_noise=cfg.permute_gt_before_noise, compute_diffusion=not cfg.train_confidence_only,
    )  # fmt: skip
    loss_fn = fp32_guard(model_cfg.precision.fp32_loss)(training_loss)
    B = cfg.batch_size_per_rank
    totals, dicts = [], []
    for b in range(B):
        loss_b, ld_b = loss_fn(slice_batch_dict(pred, b, B), slice_batch_dict(features, b, B), cfg)
        totals.append(loss_b)
        dicts.append(ld_b)
    total = torch.stack(totals).mean()
    loss_dict, counts = aggregate_sample_losses(dicts)
    for group in ("cond_drop", "null_pair"):
        for k, v in pred.get(f"__{group}__", {}).items():
            loss_dict[f"{group}/{k}"] = v
            counts[f"{group}/{k}"] = 1
    return total, loss_dict, counts, num_recycles


@dataclass
class StepResult:
    advanced: bool
    was_nan: bool
    reason: Literal["loss", "grad"] | None
    grad_norm: torch.Tensor | None
    nan_ranks: list[int]


class OptimizerEngine:
    """Owns optimizer, schedule and gradient reduction; enforces the skip-together contract."""

    def __init__(self, optimizer: FlatAdamW, scheduler, dist_info: DistInfo, cfg, grad_sync: GradSync | None = None):
        self.optimizer, self.scheduler, self.dist, self.cfg = optimizer, scheduler, dist_info, cfg
        self.grad_sync = grad_sync or GradSync(dist_info)
        self._nan_accum: torch.Tensor | None = None
        self._window_record_ids: list[str] = []

    def add_microstep_loss(self, loss: torch.Tensor, record_ids=None) -> None:
        """OR this micro-step's non-finite flag into the device-side accumulator (no sync, no collective)."""
        if self._nan_accum is None:
            self._nan_accum = torch.zeros(1, device=loss.device)
        self._nan_accum.add_((~torch.isfinite(loss.detach())).float().view(1))
        for rid in record_ids or ():
            if rid is not None:
                self._window_record_ids.append(rid)

    # ------------------------------------------------------------------ one-kernel step (CUDA)
    def resolve(self, state: TrainState) -> StepResult | None:
        """Settle the outcome of the last fused step on the host (its result block was copied back asynchronously).

        The fused step is launched without waiting for its verdict and booked as advanced. If the device-side consensus
        skipped it (non-finite loss or gradient on any rank, an outlier norm, a wait for a peer that ran out), the
        bookkeeping is taken back here: step counters, bias-correction count, EMA count and schedule position. Called
        at the start of the next optimizer step - a whole forward/backward later, when the copy has long landed - and by
        the trainer before it takes a decision that depends on the step number.
        """
        pending, self._pending = getattr(self, "_pending", None), None
        if pending is None:
            return None
        res = pending["peer"].read_result()
        state.last_grad_norm = torch.tensor(res["norm"])
        if self.cfg.per_rank_grad_clip and self.dist.is_distributed:
            finite = [n for n in res["local_norms"] if n == n and abs(n) != float("inf")]
            if finite:
                state.last_grad_norm_rank_mean = torch.tensor(sum(finite) / len(finite))
                state.last_grad_norm_rank_max = torch.tensor(max(finite))
        if res["advanced"]:
            return StepResult(True, False, None, state.last_grad_norm, [])
        opt, attempted = self.optimizer, pending["attempted"]
        opt.step_count -= 1
        if pending["ema"]:
            opt.ema_updates -= 1
        self.scheduler.last_epoch -= 1
        self.scheduler._apply()
        state.effective_step -= 1
        state.consecutive_nan_skips = pending["skips_before"]
        self._window_record_ids = pending["records"]
        if res["reason"] == "timeout":
            pending["peer"].status.zero_()
            raise RuntimeError(f"Step {attempted}: a bounded wait for another rank ran out inside the fused optimizer step "
                               "(a rank left or fell far behind); parameters were not updated")
        if res["reason"] == "loss":
            ranks = [r for r, f in enumerate(res["loss_flags"]) if f != 0.0]
            if self.dist.is_main:
                logger.warning("Step %d: NaN/Inf loss in accumulation window (ranks=%s), skipped", attempted, ranks)
            self._report_records(attempted, ranks, "NaN/Inf loss window")
            self._account_skip(state, attempted, "loss")
            return StepResult(False, True, "loss", None, ranks)
        norms = res["local_norms"] if (self.cfg.per_rank_grad_clip and self.dist.is_distributed) else [res["norm"]] * self.dist.world_size
        thr = self.cfg.grad_norm_skip_threshold
        ranks = [r for r, n in enumerate(norms) if not (n == n and abs(n) != float("inf")) or (thr > 0 and n > thr)]
        if self.dist.is_main:
            logger.warning("Step %d: non-finite or outlier gradient norm (ranks=%s, norm of the average %.3e), skipped",
                           attempted, ranks, res["norm"])  # fmt: skip
        self._report_records(attempted, ranks, "bad gradient")
        self._account_skip(state, attempted, "grad")
        return StepResult(False, True, "grad", state.last_grad_norm, ranks)

    def _step_fused(self, state: TrainState, peer) -> StepResult:
        cfg, opt = self.cfg, self.optimizer
        self.resolve(state)  # the previous step's verdict first: it fixes this step's counters
        per_rank = bool(cfg.per_rank_grad_clip and self.dist.is_distributed)
        dev = opt.flat_grad.device
        clip = cfg.grad_clip_norm if cfg.grad_clip_norm and cfg.grad_clip_norm > 0 else 0.0
        if per_rank:
            local = opt.grad_norm(True)
            c = torch.clamp(clip / (local + 1e-6), max=1.0) if clip > 0 else torch.ones((), device=dev)
            coef = torch.where(torch.isfinite(local), c, torch.ones_like(c))
        else:
            local, coef = torch.zeros((), device=dev), torch.ones((), device=dev)
        g0 = opt.param_groups[0]
        step = opt.step_count + 1
        b1, b2 = g0["betas"]
        ema = opt.shadow
        peer.fused_step(opt, coef=coef, loss_flag=self._nan_accum, local_norm=local, lr=g0["lr"], betas=(b1, b2), eps=g0["eps"],
                        bc1=1.0 - b1**step, bc2=1.0 - b2**step, ema=ema, ema_w=1.0 - opt.ema_decay, clip_norm=clip,
                        skip_threshold=cfg.grad_norm_skip_threshold, per_rank_clip=per_rank)  # fmt: skip
        self._nan_accum.zero_()
        from ..ops import autograd_ops

        autograd_ops.invalidate_weight_cache()  # stacked bf16 copies were built from the old parameter values
        self._pending = {"peer": peer, "attempted": state.effective_step + 1, "ema": ema is not None,
                         "skips_before": state.consecutive_nan_skips, "records": list(self._window_record_ids)}  # fmt: skip
        opt.step_count = step
        if ema is not None:
            opt.ema_updates += 1
        self.scheduler.step()
        self._window_record_ids.clear()
        state.effective_step += 1
        state.consecutive_nan_skips = 0
        state.last_grad_norm = peer.result[2]  # device scalar, no host read here
        return StepResult(True, False, None, peer.result[2], [])

    def step_or_skip(self, state: TrainState) -> StepResult:
        """MUST be called by every rank on every sync step."""
        assert self._nan_accum is not None, "add_microstep_loss must run at least once before step_or_skip"
        cfg, opt = self.cfg, self.optimizer
        peer = self.grad_sync.fused_step_engine(opt)
        if peer is not None:
            return self._step_fused(state, peer)
        with collective_guard("step_or_skip", self.dist):
            flags = all_gather_scalar(self._nan_accum, self.dist)
            bad = bool(flags.any().item())
            self._nan_accum.zero_()
            attempted = state.effective_step + 1
            if bad:
                opt.zero_grad()
                ranks = (flags > 0).nonzero().flatten().tolist()
                if self.dist.is_main:
                    logger.warning("Step %d: NaN/Inf loss in accumulation window (ranks=%s), skipping", attempted, ranks)
                self._report_records(attempted, ranks, "NaN/Inf loss window")
                self._account_skip(state, attempted, "loss")
                return StepResult(False, True, "loss", None, ranks)

            local, global_norm, scale = self.grad_sync.clip_and_average(
                opt, cfg.grad_clip_norm, cfg.per_rank_grad_clip, fp64_norm=True
            )
            state.last_grad_norm = local.detach()
            if global_norm is not None:
                state.last_grad_norm_global = global_norm.detach()
            check = local.float()
            if global_norm is not None:  # per-rank mode: a reduction that failed returns a NaN norm of the average
                check = torch.where(torch.isfinite(global_norm.float()), check, global_norm.float())
            if opt.flat_grad.is_cuda:  # a kernel whose bounded wait ran out left garbage behind: skip on every rank
                from ..ops import native

                if native.available():
                    bad_kernel = torch.ops.df3.gemm_status() != 0
                    peer_eng = getattr(self.grad_sync, "_peer", None)
                    if peer_eng is not None:
                        bad_kernel = bad_kernel or int(peer_eng.status.item()) != 0
                        peer_eng.status.zero_()
                    if bad_kernel:
                        logger.error("Step %d: a kernel reported a wait that ran out on rank %d; the step is skipped", attempted, self.dist.rank)
                        check = torch.full_like(check, float("nan"))
            norms = all_gather_scalar(check, self.dist)
            finite = torch.isfinite(norms)
            if bool(finite.any().item()):
                state.last_grad_norm_rank_mean = norms[finite].mean()
                state.last_grad_norm_rank_max = norms[finite].max()
            if not bool(finite.all().item()):
                return self._skip_bad_grad(state, attempted, local, norms, (~finite).nonzero().flatten().tolist(),
                                           "NaN/Inf in grads")  # fmt: skip
            thr = cfg.grad_norm_skip_threshold
            if thr > 0 and bool((norms > thr).any().item()):
                return self._skip_bad_grad(state, attempted, local, norms, (norms > thr).nonzero().flatten().tolist(),
                                           f"grad outlier exceeded skip_threshold={thr:.3e}")  # fmt: skip
            if cfg.grad_norm_log_threshold > 0 and self._window_record_ids and local.item() > cfg.grad_norm_log_threshold:
                logger.warning("Step %d: rank %d grad_norm=%.3e exceeded log_threshold=%.3e window record_ids=%s",
                               attempted, self.dist.rank, local.item(), cfg.grad_norm_log_threshold,
                               self._window_record_ids)  # fmt: skip
            opt.step(grad_scale=scale)
            opt.zero_grad()
            self.scheduler.step()
            self._window_record_ids.clear()
            state.effective_step += 1
            state.consecutive_nan_skips = 0
            return StepResult(True, False, None, local, [])

    def _report_records(self, attempted, ranks, what):
        if self.dist.rank in ranks and self._window_record_ids:
            logger.warning("Step %d: rank %d %s record_ids=%s", attempted, self.dist.rank, what, self._window_record_ids)
        self._window_record_ids.clear()

    def _skip_bad_grad(self, state, attempted, norm, norms, ranks, why):
        self.optimizer.zero_grad()
        if self.dist.is_main:
            detail = ", ".join(f"rank{r}={norms[r].item():.3e}" for r in ranks)
            logger.warning("Step %d: %s (ranks=%s, %s), skipping", attempted, why, ranks, detail)
        self._report_records(attempted, ranks, why)
        self._account_skip(state, attempted, "grad")
        return StepResult(False, True, "grad", norm, ranks)

    def _account_skip(self, state, attempted, reason):
        state.consecutive_nan_skips += 1
        limit = self.cfg.max_consecutive_nan_skips
        if limit > 0 and state.consecutive_nan_skips >= limit:
            msg = (f"Aborting: {state.consecutive_nan_skips} consecutive non-finite {reason} skips at step "
                   f"{attempted} (limit={limit}).")  # fmt: skip
            logger.critical(msg)
            raise RuntimeError(msg)
