"""Training loop of the complex language model (reference: complexlm/trainer.py:41-375).

One process per GPU; gradients are averaged with one all-reduce over a flat view of all gradients (the packed batches
have different token counts per rank, so the loss is normalised by the local number of scored positions, as in the
reference's DDP set-up). AdamW takes the model's parameter groups, whose ``lr_scale`` carries the muP step rule; the
schedule is linear warm-up then cosine to ``min_lr_frac``. Evaluation scores fixed masked positions twice: with the whole
complex visible and with every chain alone; ``delta`` is what the partner chains were worth.
"""

from __future__ import annotations

import json
import math
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .config import ExperimentConfig, to_dict
from .data import PackedComplexStream, build_views, drop_overlapping_clusters, evaluation_batches
from .model import IGNORE_INDEX, ComplexLM, PackedBatch

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def lr_at(step: int, cfg) -> float:
    if step < cfg.warmup_steps:
        return cfg.lr * (step + 1) / max(cfg.warmup_steps, 1)
    t = min(1.0, (step - cfg.warmup_steps) / max(cfg.max_steps - cfg.warmup_steps, 1))
    return cfg.lr * (cfg.min_lr_frac + (1 - cfg.min_lr_frac) * 0.5 * (1 + math.cos(math.pi * t)))


def masked_lm_metrics(logits: torch.Tensor, batch: PackedBatch) -> dict[str, torch.Tensor]:
    """Sums (not means) per group, so they can be added over batches and ranks: loss, correct, count."""
    scored = batch.labels != IGNORE_INDEX
    loss = F.cross_entropy(logits.float(), batch.labels, ignore_index=IGNORE_INDEX, reduction="none")
    hit = (logits.argmax(-1) == batch.labels) & scored
    n_ent = torch.zeros(batch.n_complexes, device=logits.device)
    ent_key = batch.complex_index.long() * (int(batch.entity_index.max()) + 1) + batch.entity_index.long()
    uniq = torch.unique(ent_key)
    n_ent.index_add_(0, (uniq // (int(batch.entity_index.max()) + 1)), torch.ones_like(uniq, dtype=torch.float))
    n_ch = (batch.complex_cu[1:] - batch.complex_cu[:-1]).float()  # tokens; chains per complex below
    chains_per_cx = torch.zeros(batch.n_complexes, device=logits.device)
    first = torch.ones_like(batch.chain_index, dtype=torch.bool)
    first[1:] = batch.chain_index[1:] != batch.chain_index[:-1]
    chains_per_cx.index_add_(0, batch.complex_index.long()[first], torch.ones(int(first.sum()), device=logits.device))
    homo = ((n_ent == 1) & (chains_per_cx > 1))[batch.complex_index.long()]
    hetero = (n_ent > 1)[batch.complex_index.long()]
    groups = {"all": scored, "homomer": scored & homo, "heteromer": scored & hetero,
              "interface": scored & batch.iface & batch.iface_known, "non_interface": scored & ~batch.iface & batch.iface_known,
              "unlabelled": scored & ~batch.iface_known, "heteromer_interface": scored & hetero & batch.iface & batch.iface_known}  # fmt: skip
    del n_ch
    out = {}
    for name, sel in groups.items():
        out[f"{name}/loss"] = (loss * sel).sum()
        out[f"{name}/correct"] = (hit & sel).sum().float()
        out[f"{name}/count"] = sel.sum().float()
    return out


class ComplexLMTrainer:
    def __init__(self, cfg: ExperimentConfig, output_dir: str, resume: str | None = None, device: str | None = None):
        self.cfg, self.out = cfg, output_dir
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        if self.world > 1 and not dist.is_initialized():
            dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
        if device is None:
            device = f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        torch.manual_seed(cfg.train.seed)
        self.model = ComplexLM(cfg.model).to(self.device)
        groups = self.model.param_groups(cfg.train.weight_decay)
        self.opt = torch.optim.AdamW(groups, lr=cfg.train.lr, betas=(cfg.train.beta1, cfg.train.beta2), eps=cfg.train.eps,
                                     fused=self.device.type == "cuda")  # fmt: skip
        self.step = 0
        self.train_views = build_views(cfg.data)
        self.eval_views = build_views(cfg.data, cfg.eval_sources) if cfg.eval_sources else []
        if cfg.train.eval_cluster_disjoint and self.eval_views:
            drop_overlapping_clusters(self.eval_views, self.train_views)
        # no sources configured: the caller feeds train_step() with its own batches (benchmarks, tests)
        self.stream = PackedComplexStream(self.train_views, cfg.data, cfg.data.seed, self.rank) if self.train_views else None
        self.amp = DTYPES[cfg.train.dtype] if self.device.type == "cuda" else torch.float32
        if self.world > 1:  # every rank starts from rank 0's weights
            for p in self.model.parameters():
                dist.broadcast(p.data, 0)
        if self.rank == 0:
            os.makedirs(output_dir, exist_ok=True)
            with open(os.path.join(output_dir, "config.json"), "w") as f:
                json.dump(to_dict(cfg), f, indent=1)
        if cfg.train.esmc_weights and not resume:  # warm start; a resumed run already carries trained weights
            from .esmc import load_esmc

            report = load_esmc(self.model, cfg.train.esmc_weights)
            if self.rank == 0:
                with open(os.path.join(output_dir, "esmc_warm_start.json"), "w") as f:
                    json.dump(report, f, indent=1)
        if resume:
            self.load_checkpoint(resume)

    # --- one optimizer step ------------------------------------------------------------------------------------
    def _forward_loss(self, batch: PackedBatch):
        with torch.autocast(self.device.type, dtype=self.amp, enabled=self.amp != torch.float32):
            logits = self.model(batch).logits
        m = masked_lm_metrics(logits, batch)
        return m["all/loss"] / m["all/count"].clamp(min=1), m

    def _sync_grads(self) -> None:
        if self.world == 1:
            return
        grads = [p.grad for p in self.model.parameters() if p.grad is not None]
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat)
        flat.div_(self.world)
        at = 0
        for g in grads:
            g.copy_(flat[at : at + g.numel()].view_as(g))
            at += g.numel()

    def train_step(self, batches: list[PackedBatch]) -> dict[str, float]:
        self.model.train()
        lr = lr_at(self.step, self.cfg.train)
        for g in self.opt.param_groups:
            g["lr"] = lr * g.get("lr_scale", 1.0)
        total, metrics = 0.0, None
        for b in batches:
            loss, metrics = self._forward_loss(b.to(self.device, non_blocking=True))
            (loss / len(batches)).backward()
            total += float(loss.detach()) / len(batches)
        self._sync_grads()
        norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.cfg.train.grad_clip or float("inf"))
        if torch.isfinite(norm):
            self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        self.step += 1
        acc = float(metrics["all/correct"] / metrics["all/count"].clamp(min=1))
        return {"loss": total, "accuracy": acc, "grad_norm": float(norm), "lr": lr}

    def train(self, max_steps: int | None = None) -> dict[str, float]:
        cfg = self.cfg.train
        it = iter(self.stream)
        last, t0 = {}, time.time()
        while self.step < (max_steps or cfg.max_steps):
            last = self.train_step([next(it) for _ in range(cfg.accum_steps)])
            if self.rank == 0 and cfg.log_every and self.step % cfg.log_every == 0:
                self.log({**last, "steps_per_s": cfg.log_every / max(time.time() - t0, 1e-9)}, "train")
                t0 = time.time()
            if cfg.eval_every and self.eval_views and self.step % cfg.eval_every == 0:
                ev = self.evaluate()
                if self.rank == 0:
                    self.log(ev, "eval")
            if cfg.save_every and self.step % cfg.save_every == 0 and self.rank == 0:
                self.save_checkpoint()
        if self.rank == 0:
            self.save_checkpoint(final=True)
        return last

    # --- evaluation --------------------------------------------------------------------------------------------
    @torch.no_grad()
    def evaluate(self) -> dict[str, float]:
        self.model.eval()
        sums: dict[str, torch.Tensor] = {}
        for b in evaluation_batches(self.eval_views, self.cfg.data, self.cfg.train.eval_batches)[self.rank :: self.world]:
            b = b.to(self.device)
            for tag, view in (("", b), ("_single", b.chains_only())):
                with torch.autocast(self.device.type, dtype=self.amp, enabled=self.amp != torch.float32):
                    logits = self.model(view).logits
                for k, v in masked_lm_metrics(logits, b).items():
                    group, what = k.split("/")
                    key = f"{group}/{what}{tag}"
                    sums[key] = sums.get(key, 0) + v
        if self.world > 1 and sums:
            keys = sorted(sums)
            flat = torch.stack([sums[k] for k in keys])
            dist.all_reduce(flat)
            sums = dict(zip(keys, flat))
        out = {}
        for key in [k for k in sums if k.endswith("/count")]:
            g = key[: -len("/count")]
            n = float(sums[key])
            if n == 0:
                continue
            out[f"{g}/loss"] = float(sums[f"{g}/loss"]) / n
            out[f"{g}/accuracy"] = float(sums[f"{g}/correct"]) / n
            out[f"{g}/loss_single"] = float(sums[f"{g}/loss_single"]) / n
            out[f"{g}/delta"] = out[f"{g}/loss_single"] - out[f"{g}/loss"]
        return out

    # --- bookkeeping -------------------------------------------------------------------------------------------
    def log(self, metrics: dict[str, float], prefix: str) -> None:
        row = {"step": self.step, **{f"{prefix}/{k}": v for k, v in metrics.items()}}
        with open(os.path.join(self.out, "metrics.jsonl"), "a") as f:
            f.write(json.dumps(row) + "\n")
        print(" ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in row.items()), flush=True)

    def save_checkpoint(self, final: bool = False) -> str:
        path = os.path.join(self.out, "final.pt" if final else f"step_{self.step:07d}.pt")
        torch.save({"model": self.model.state_dict(), "optimizer": self.opt.state_dict(), "step": self.step,
                    "config": to_dict(self.cfg)}, path + ".tmp")  # fmt: skip
        os.replace(path + ".tmp", path)
        keep = self.cfg.train.keep_last
        old = sorted(f for f in os.listdir(self.out) if f.startswith("step_") and f.endswith(".pt"))
        for f in old[:-keep] if keep else []:
            os.remove(os.path.join(self.out, f))
        return path

    def load_checkpoint(self, path: str) -> None:
        ck = torch.load(path, map_location=self.device, weights_only=False)
        self.model.load_state_dict(ck["model"])
        self.opt.load_state_dict(ck["optimizer"])
        self.step = int(ck["step"])
