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


def _alpha(mol_type: int) -> float:
    from . import const

    if mol_type == const.MOL_PROTEIN:
        return ALPHA["protein"]
    if mol_type in (const.MOL_RNA, const.MOL_DNA):
        return ALPHA["nucleic"]
    if mol_type == const.MOL_NONPOLYMER:
        return ALPHA["ligand"]
    return 1.0


def anchor_tables(records) -> list[tuple[list[tuple[str, int, int]], list[float]]]:
    """Per manifest record, the crop anchors it offers and their weights ``w_a`` (AF3 SI 2.5.1-2.5.3; reference:
    data/sample/weighted.py:100-196). An anchor is ``("chain", chain_id, -1)`` with ``w = beta_chain * alpha(type) /
    |chain cluster|`` or ``("interface", chain_1, chain_2)`` with ``w = beta_interface * (alpha_1 + alpha_2) /
    |interface cluster|``; an interface cluster is the unordered pair of the two chains' clusters, and cluster sizes
    count valid members over the whole record list. Drawing a record by the sum of its ``w_a`` (``record_weights``)
    and then one of its anchors in proportion to ``w_a`` equals drawing from the flat table of all anchors.
    """
    chain_count: dict = {}
    face_count: dict = {}
    for r in records:
        by_id = {c.chain_id: c for c in r.chains}
        for c in r.chains:
            if c.valid:
                chain_count[c.cluster_id] = chain_count.get(c.cluster_id, 0) + 1
        for f in r.interfaces:
            a, b = by_id.get(f.chain_1), by_id.get(f.chain_2)
            if f.valid and a is not None and b is not None and a.valid and b.valid:
                key = frozenset((a.cluster_id, b.cluster_id))
                face_count[key] = face_count.get(key, 0) + 1
    out = []
    for r in records:
        by_id = {c.chain_id: c for c in r.chains}
        anchors, weights = [], []
        for c in r.chains:
            if c.valid:
                anchors.append(("chain", int(c.chain_id), -1))
                weights.append(BETA_CHAIN * _alpha(c.mol_type) / max(1, chain_count.get(c.cluster_id, 1)))
        for f in r.interfaces:
            a, b = by_id.get(f.chain_1), by_id.get(f.chain_2)
            if f.valid and a is not None and b is not None and a.valid and b.valid:
                size = max(1, face_count.get(frozenset((a.cluster_id, b.cluster_id)), 1))
                anchors.append(("interface", int(a.chain_id), int(b.chain_id)))
                weights.append(BETA_INTERFACE * (_alpha(a.mol_type) + _alpha(b.mol_type)) / size)
        out.append((anchors, weights))
    return out


def record_weights(tables) -> list[float]:
    """The record marginal of ``anchor_tables``: the sum of a record's anchor weights (a record without a valid anchor
    keeps a vanishing weight so that the sampler's distribution stays defined)."""
    return [max(float(sum(w)), 1e-12) for _, w in tables]


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
