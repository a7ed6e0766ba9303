"""Infinite, resumable index streams (reference: data/sample/weighted.py:198-446, data/sample/multi.py:19-200).

``WeightedClusterSampler`` draws examples with probability proportional to
``sum over chains beta_chain * alpha_type / |cluster|`` plus the interface terms; every rank draws the same
global stream from the shared seed and keeps ``stream[rank::world]``. ``MultiDatasetSampler`` mixes several
datasets by weight and yields offsets into their concatenation. Both expose ``state_dict`` /
``load_state_dict`` so a resumed run continues the stream.
"""

from __future__ import annotations

import torch

ALPHA = {"protein": 3.0, "nucleic": 3.0, "ligand": 1.0}
BETA_CHAIN, BETA_INTERFACE = 0.5, 1.0


def example_weight(chains: list[dict], interfaces: list[dict] | None = None) -> float:
    """``chains``: ``[{"type": "protein"|"nucleic"|"ligand", "cluster_size": int}]``; interfaces likewise."""
    w = sum(BETA_CHAIN * ALPHA.get(c.get("type", "protein"), 1.0) / max(1, int(c.get("cluster_size", 1))) for c in chains)
    for i in interfaces or ():
        w += BETA_INTERFACE * ALPHA.get(i.get("type", "protein"), 1.0) / max(1, int(i.get("cluster_size", 1)))
    return max(w, 1e-8)


class WeightedClusterSampler:
    def __init__(self, weights, seed: int = 0, rank: int = 0, world_size: int = 1, block: int = 4096):
        self.weights = torch.as_tensor(weights, dtype=torch.double)
        self.seed, self.rank, self.world, self.block = seed, rank, world_size, block
        self.drawn = 0  # global draws consumed (a multiple of ``block`` plus the cursor)
        self._buf, self._cursor, self._epoch = None, 0, 0

    def _refill(self):
        g = torch.Generator().manual_seed(self.seed + 1_000_003 * self._epoch)
        self._buf = torch.multinomial(self.weights, self.block * self.world, replacement=True, generator=g)[self.rank :: self.world]
        self._epoch += 1
        self._cursor = 0

    def __iter__(self):
        return self

    def __next__(self) -> int:
        if self._buf is None or self._cursor >= len(self._buf):
            self._refill()
        i = int(self._buf[self._cursor])
        self._cursor += 1
        return i

    def state_dict(self) -> dict:
        return {"epoch": self._epoch, "cursor": self._cursor, "seed": self.seed}

    def load_state_dict(self, sd: dict) -> None:
        self.seed = sd.get("seed", self.seed)
        self._epoch = max(0, int(sd["epoch"]) - 1)
        self._refill()
        self._cursor = int(sd["cursor"])


class MultiDatasetSampler:
    """Mixture of per-dataset samplers; yields ``offset_of_dataset + index``."""

    def __init__(self, samplers: list, sizes: list[int], mix_weights: list[float], seed: int = 0):
        self.samplers, self.sizes = samplers, sizes
        self.offsets = [0]
        for s in sizes[:-1]:
            self.offsets.append(self.offsets[-1] + s)
        self.mix = torch.as_tensor(mix_weights, dtype=torch.double)
        self.gen = torch.Generator().manual_seed(seed)

    def __iter__(self):
        return self

    def __next__(self) -> int:
        d = int(torch.multinomial(self.mix, 1, generator=self.gen))
        return self.offsets[d] + next(self.samplers[d])

    def state_dict(self) -> dict:
        return {"gen": self.gen.get_state(), "samplers": [s.state_dict() for s in self.samplers]}

    def load_state_dict(self, sd: dict) -> None:
        self.gen.set_state(sd["gen"])
        for s, st in zip(self.samplers, sd["samplers"]):
            s.load_state_dict(st)
