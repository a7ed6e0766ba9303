"""Per-token training masks carried next to an example (reference: data/masking.py:24-170).

A ``TokenMask`` holds named boolean / float arrays over the tokens of a structure (for instance ``fixed``: tokens
whose coordinates are given and must not contribute to the loss, or ``design``: tokens to be redesigned). It follows
the example through cropping with ``select`` and turns into per-token loss weights.
"""

from __future__ import annotations

import dataclasses

import numpy as np


@dataclasses.dataclass
class TokenMask:
    arrays: dict

    def select(self, indices: np.ndarray) -> "TokenMask":
        return TokenMask({k: v[indices] for k, v in self.arrays.items()})

    def get(self, name: str):
        return self.arrays.get(name)

    @classmethod
    def load(cls, path_or_npz) -> "TokenMask":
        z = np.load(path_or_npz) if isinstance(path_or_npz, (str, bytes)) else path_or_npz
        return cls({k: np.asarray(z[k]) for k in z.files})

    def save(self, path: str) -> None:
        np.savez_compressed(path, **self.arrays)

    @classmethod
    def fixed_from_chains(cls, asym_id: np.ndarray, fixed_chains) -> "TokenMask":
        return cls({"fixed": np.isin(asym_id, np.asarray(list(fixed_chains)))})

    def loss_weight(self, num_tokens: int, exclude=("fixed",)) -> np.ndarray:
        w = np.ones(num_tokens, dtype=np.float32)
        for name in exclude:
            m = self.arrays.get(name)
            if m is not None:
                w = w * (1.0 - m.astype(np.float32))
        return w

    @staticmethod
    def loss_weight_excluding_mol_types(mol_type: np.ndarray, excluded) -> np.ndarray:
        return (~np.isin(mol_type, np.asarray(list(excluded)))).astype(np.float32)
