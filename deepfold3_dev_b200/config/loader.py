"""YAML / JSON config files with ``base:`` inheritance and ``--override k=v``.

Behaviour follows the reference loader (config_loader.py:18-193 and
scripts/train.py:108-130): a file may name a ``base:`` file (relative to
itself); nested mappings merge key by key while lists and scalars replace;
top-level ``datasets:`` / ``eval_datasets:`` move under ``training``; dotted
overrides coerce ``true/false/null``, ints and floats.
"""

from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Any

import yaml

from .schema import DatasetConfig, ModelConfig, TrainingConfig

_STRATEGIES = ("uniform", "weighted")
_FORMATS = ("df3", "of3", "of3pdb")
_CROP_KEYS = ("contiguous", "spatial", "interface")


def deep_merge(base: dict, override: dict) -> dict:
    out = dict(base)
    for key, val in override.items():
        if isinstance(val, dict) and isinstance(out.get(key), dict):
            out[key] = deep_merge(out[key], val)
        else:
            out[key] = val
    return out


def _read(path: Path) -> dict:
    ext = path.suffix.lower()
    text = path.read_text()
    if ext == ".json":
        return json.loads(text)
    if ext in (".yaml", ".yml"):
        return yaml.safe_load(text) or {}
    raise ValueError(f"Unsupported config file extension: {ext} (expected .json, .yaml, or .yml)")


def resolve_config(config_path: str | Path, _chain: tuple[Path, ...] = ()) -> dict:
    """Load ``config_path`` and fold in its chain of ``base:`` files."""
    path = Path(config_path).resolve()
    if path in _chain:
        raise ValueError("Circular config base reference: " + " -> ".join(map(str, (*_chain, path))))
    if not path.exists():
        raise FileNotFoundError(f"Config file not found: {path}")
    data = _read(path)
    parent = data.pop("base", None)
    if parent is None:
        return data
    parent_path = Path(parent)
    if not parent_path.is_absolute():
        parent_path = path.parent / parent_path
    return deep_merge(resolve_config(parent_path, (*_chain, path)), data)


def normalize_datasets(raw: list[dict]) -> list[dict]:
    """Validate dataset entries and fill every ``DatasetConfig`` field."""
    out = []
    for i, entry in enumerate(raw):
        where = f"datasets[{i}]"
        if not isinstance(entry, dict):
            raise ValueError(f"{where}: expected a mapping, got {type(entry).__name__}")
        for need in ("name", "data_dir"):
            if need not in entry:
                raise ValueError(f"{where}: missing required field '{need}'")
        strategy, fmt = entry.get("strategy", "uniform"), entry.get("format", "df3")
        if strategy not in _STRATEGIES:
            raise ValueError(f"{where}: invalid strategy '{strategy}', must be one of {set(_STRATEGIES)}")
        if fmt not in _FORMATS:
            raise ValueError(f"{where}: invalid format '{fmt}', must be one of {set(_FORMATS)}")
        excl = entry.get("exclude_loss_mol_types") or []
        if not isinstance(excl, list):
            raise ValueError(f"{where}: exclude_loss_mol_types must be a list of integers")
        try:
            excl = [int(x) for x in excl]
        except (TypeError, ValueError) as exc:
            raise ValueError(f"{where}: exclude_loss_mol_types must contain integers ({exc})") from exc
        cw = entry.get("crop_weights")
        if cw is not None:
            if not isinstance(cw, dict):
                raise ValueError(f"{where}: crop_weights must be a mapping, got {type(cw).__name__}")
            extra = sorted(set(cw) - set(_CROP_KEYS))
            if extra:
                raise ValueError(f"{where}: unknown crop_weights keys {extra} (use {set(_CROP_KEYS)})")
            try:
                cw = {k: float(v) for k, v in cw.items()}
            except (TypeError, ValueError) as exc:
                raise ValueError(f"{where}: crop_weights values must be numbers ({exc})") from exc
        out.append(
            dict(
                name=entry["name"],
                data_dir=entry["data_dir"],
                weight=float(entry.get("weight", 1.0)),
                strategy=strategy,
                is_distillation=bool(entry.get("is_distillation", False)),
                format=fmt,
                cutoff_date=str(entry.get("cutoff_date", "")),
                exclude_loss_mol_types=excl,
                crop_weights=cw,
                template_struct_space=bool(
                    entry.get("template_struct_space", entry.get("monomer_template_struct_space", False))
                ),
                max_template_date=str(entry.get("max_template_date", "")),
                of3_cache_dir=str(entry.get("of3_cache_dir", "")),
                template_cache_dir=str(entry.get("template_cache_dir", "")),
                curator_weights=str(entry.get("curator_weights", "")),
            )
        )
    return out


def load_config(config_path: str | Path) -> dict:
    """Resolved config dict with dataset lists normalised under ``training``."""
    data = resolve_config(config_path)
    for top, dest in (("datasets", "extra_datasets"), ("eval_datasets", "eval_datasets")):
        raw = data.pop(top, None)
        if raw is not None:
            data.setdefault("training", {})[dest] = normalize_datasets(raw)
    return data


def coerce_scalar(text: str) -> Any:
    """``--override`` value text → bool / None / int / float / JSON list / str."""
    low = text.strip().lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("null", "none"):
        return None
    for cast in (int, float):
        try:
            return cast(text)
        except ValueError:
            pass
    if text[:1] in "[{":
        try:
            return json.loads(text)
        except json.JSONDecodeError:
            pass
    return text


def apply_dict(cfg, data: dict, path: str = "") -> None:
    """Set fields of dataclass ``cfg`` from a nested dict; unknown keys raise."""
    names = {f.name: f for f in dataclasses.fields(cfg)}
    for key, val in data.items():
        if key not in names:
            raise KeyError(f"unknown config key '{path}{key}' for {type(cfg).__name__}")
        cur = getattr(cfg, key)
        if dataclasses.is_dataclass(cur) and isinstance(val, dict):
            apply_dict(cur, val, f"{path}{key}.")
        elif key in ("extra_datasets", "eval_datasets") and isinstance(val, list):
            setattr(cfg, key, [DatasetConfig(**v) if isinstance(v, dict) else v for v in val])
        else:
            if isinstance(cur, tuple) and isinstance(val, list):
                val = tuple(val)
            setattr(cfg, key, val)


def apply_override(cfg, dotted: str, value: Any) -> None:
    """``a.b.c=value`` on a dataclass tree."""
    *parents, leaf = dotted.split(".")
    node = cfg
    for p in parents:
        if not hasattr(node, p):
            raise KeyError(f"override '{dotted}': no field '{p}' on {type(node).__name__}")
        node = getattr(node, p)
    if not hasattr(node, leaf):
        raise KeyError(f"override '{dotted}': no field '{leaf}' on {type(node).__name__}")
    cur = getattr(node, leaf)
    if isinstance(cur, tuple) and isinstance(value, list):
        value = tuple(value)
    setattr(node, leaf, value)


def build_configs(
    config_files: list[str] | tuple[str, ...] = (), overrides: list[str] | tuple[str, ...] = ()
) -> tuple[TrainingConfig, ModelConfig]:
    """``--config`` files (later wins) then ``--override`` items → ``(TrainingConfig, ModelConfig)``.

    An override key is looked up under ``training`` first, then ``model``;
    the prefixes ``training.`` / ``model.`` pick one explicitly.
    """
    merged: dict = {}
    for f in config_files:
        merged = deep_merge(merged, load_config(f))
    train_cfg, model_cfg = TrainingConfig(), ModelConfig()
    apply_dict(train_cfg, merged.get("training", {}), "training.")
    apply_dict(model_cfg, merged.get("model", {}), "model.")
    for item in overrides:
        if "=" not in item:
            raise ValueError(f"--override expects key=value, got {item!r}")
        key, text = item.split("=", 1)
        value = coerce_scalar(text)
        if key.startswith("training."):
            apply_override(train_cfg, key[len("training.") :], value)
        elif key.startswith("model."):
            apply_override(model_cfg, key[len("model.") :], value)
        else:
            try:
                apply_override(train_cfg, key, value)
            except KeyError:
                apply_override(model_cfg, key, value)
    train_cfg.__post_init__()
    model_cfg.__post_init__()
    return train_cfg, model_cfg
