"""Loading files written by the reference package.

``.pt`` checkpoints of the reference pickle its config dataclasses under ``deepfold3.model.config``. When that
package is not importable, ``install_pickle_aliases`` registers alias modules whose classes are this package's
field-compatible dataclasses, so ``torch.load`` of such a checkpoint resolves.
"""

from __future__ import annotations

import importlib.util
import sys
import types


def install_pickle_aliases(force: bool = False) -> bool:
    """Alias ``deepfold3.model.config`` to ``deepfold3_dev_b200.config.schema``; returns True if aliases were installed."""
    if not force and "deepfold3" not in sys.modules:
        try:
            if importlib.util.find_spec("deepfold3") is not None:
                return False  # the real package is importable: nothing to do
        except (ImportError, ValueError):
            pass
    if not force and "deepfold3.model.config" in sys.modules:
        return False
    from .config import schema

    root = sys.modules.get("deepfold3") or types.ModuleType("deepfold3")
    model = sys.modules.get("deepfold3.model") or types.ModuleType("deepfold3.model")
    root.__path__ = getattr(root, "__path__", [])
    model.__path__ = getattr(model, "__path__", [])
    root.model, model.config = model, schema
    sys.modules.update({"deepfold3": root, "deepfold3.model": model, "deepfold3.model.config": schema})
    return True


def torch_load_compat(path: str, **kwargs):
    """``torch.load`` that retries with the aliases when the pickled config classes cannot be found."""
    import torch

    try:
        return torch.load(path, **kwargs)
    except ModuleNotFoundError as exc:
        if "deepfold3" not in str(exc):
            raise
        install_pickle_aliases(force=True)
        return torch.load(path, **kwargs)
