"""Experiment description of the complex language model (reference: complexlm/config.py:13-351).

Field names and defaults follow the reference's YAML files, so its ``plm-*.yaml`` configs load here; ``base:`` names a
parent file in the same directory, ``overrides`` are dotted ``section.key=value`` pairs applied last.
"""

from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass, field
from typing import Any

import yaml

LAYER_KINDS = ("c", "g", "r", "x")  # chain+RoPE, complex no-position, complex+RoPE, other-chains-only


@dataclass
class ComplexLMConfig:
    d_model: int = 768
    n_heads: int = 12
    n_layers: int = 24
    layer_pattern: str = "cg"
    expansion_ratio: float = 8 / 3
    norm: str = "rmsnorm"
    norm_eps: float = 1e-5
    qk_layernorm: bool = True
    bias: bool = False
    scale_residue: bool = True
    rope_theta: float = 10000.0
    max_position: int = 4096
    vocab_size: int = 33
    attn_impl: str = "varlen"
    embed_dropout: float = 0.0
    chain_signal: str = "none"
    esmc_compat: bool = False
    mup: bool = False
    mup_base_width: int = 256
    init_std: float = 0.02

    def __post_init__(self):
        if self.d_model % self.n_heads:
            raise ValueError("d_model must be divisible by n_heads")
        if not self.layer_pattern or any(k not in LAYER_KINDS for k in self.layer_pattern):
            raise ValueError(f"layer_pattern uses kinds {LAYER_KINDS}")
        if self.norm not in ("rmsnorm", "layernorm") or self.attn_impl not in ("varlen", "sdpa"):
            raise ValueError("norm is rmsnorm|layernorm, attn_impl is varlen|sdpa")
        if "x" in self.layer_pattern and self.attn_impl != "sdpa":
            raise ValueError("kind 'x' has no packed-segment form: set attn_impl='sdpa'")

    @property
    def kinds(self) -> list[str]:
        return [self.layer_pattern[i % len(self.layer_pattern)] for i in range(self.n_layers)]

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    @property
    def width_mult(self) -> float:
        return self.d_model / self.mup_base_width if self.mup else 1.0

    @property
    def base_head_dim(self) -> int:
        return self.mup_base_width // self.n_heads if self.mup else self.head_dim


@dataclass
class SourceConfig:
    name: str = ""
    weight: float = 1.0
    homo_weight: float | None = None
    hetero_weight: float | None = None
    cluster_balanced: bool = True
    interface_masking: bool = True
    max_complexes: int | None = None
    date_max: int | None = None
    date_min: int | None = None
    allow_undated: bool = False
    exclude_ids: str | None = None
    holdout_every: int = 0
    holdout_side: str = "train"


@dataclass
class MaskingConfig:
    rate: float = 0.15
    interface_rate: float = 0.30
    mask_token_frac: float = 0.8
    random_token_frac: float = 0.1
    homomer_paired: bool = True


@dataclass
class DataConfig:
    data_root: str = "/data/plm/store"
    sources: list[SourceConfig] = field(default_factory=list)
    token_budget: int = 16384
    max_chain_len: int = 2048
    max_complex_len: int = 4096
    max_chains: int = 16
    min_chains: int = 1
    permute_chains: bool = True
    masking: MaskingConfig = field(default_factory=MaskingConfig)
    num_workers: int = 6
    prefetch_factor: int = 4
    seed: int = 0


@dataclass
class TrainConfig:
    max_steps: int = 100_000
    lr: float = 4e-4
    min_lr_frac: float = 0.1
    warmup_steps: int = 2000
    weight_decay: float = 0.01
    beta1: float = 0.9
    beta2: float = 0.98
    eps: float = 1e-8
    grad_clip: float = 1.0
    accum_steps: int = 1
    dtype: str = "bf16"
    esmc_weights: str | None = None
    compile: bool = False
    log_every: int = 20
    eval_every: int = 2000
    eval_batches: int = 20
    save_every: int = 5000
    eval_cluster_disjoint: bool = True
    keep_last: int = 3
    wandb_project: str | None = None
    wandb_entity: str | None = None
    wandb_run_name: str | None = None
    diagnostics_every: int = 0
    seed: int = 0


@dataclass
class ExperimentConfig:
    model: ComplexLMConfig = field(default_factory=ComplexLMConfig)
    data: DataConfig = field(default_factory=DataConfig)
    train: TrainConfig = field(default_factory=TrainConfig)
    eval_sources: list[SourceConfig] = field(default_factory=list)


def _build(cls, raw: dict):
    kwargs: dict[str, Any] = {}
    hints = {f.name: f for f in dataclasses.fields(cls)}
    for k, v in (raw or {}).items():
        if k not in hints:
            raise KeyError(f"{cls.__name__} has no field {k!r}")
        default = hints[k].default_factory() if hints[k].default_factory is not dataclasses.MISSING else hints[k].default
        if dataclasses.is_dataclass(default) and isinstance(v, dict):
            v = _build(type(default), v)
        elif k in ("sources", "eval_sources") and isinstance(v, list):
            v = [_build(SourceConfig, s) if isinstance(s, dict) else s for s in v]
        kwargs[k] = v
    return cls(**kwargs)


def _merge(base: dict, top: dict) -> dict:
    out = dict(base)
    for k, v in top.items():
        out[k] = _merge(out[k], v) if isinstance(v, dict) and isinstance(out.get(k), dict) else v
    return out


def _read(path: str) -> dict:
    with open(path) as f:
        raw = yaml.safe_load(f) or {}
    parent = raw.pop("base", None)
    if parent:
        raw = _merge(_read(os.path.join(os.path.dirname(path), parent)), raw)
    return raw


def load_experiment(path: str | None = None, overrides: dict[str, Any] | None = None) -> ExperimentConfig:
    raw = _read(path) if path else {}
    for dotted, value in (overrides or {}).items():
        node = raw
        *parents, leaf = dotted.split(".")
        for p in parents:
            node = node.setdefault(p, {})
        node[leaf] = yaml.safe_load(value) if isinstance(value, str) else value
    return _build(ExperimentConfig, raw)


def to_dict(cfg) -> dict:
    return dataclasses.asdict(cfg)
