"""Training-set filters of AF3 supplement 2.5.4 on a parsed ``Structure`` / ``Record`` pair.

Reference: data/prepare/filters.py:29-699. Structure-level rules reject an entry (resolution, method, release window,
chain and residue budgets, tight heavy-atom clashes); chain-level rules clear ``valid`` on single chains (resolved
length window, all-unknown chains, unknown fraction, broken CA trace, chains that sit inside another chain) and on
every interface that touches such a chain. ``select_interface_chains`` is the per-sample spatial pre-crop of large
assemblies around the sampled chain or interface.
"""

from __future__ import annotations

import random
from dataclasses import dataclass

import numpy as np
from scipy.spatial import cKDTree

from .. import const
from ..types import ChainInfo, Record, Structure, StructureInfo


@dataclass
class StructureFilterConfig:
    # entry level
    max_resolution: float | None = None
    min_resolution: float | None = None
    allowed_methods: frozenset[str] | None = None
    max_release_date: str | None = None
    min_release_date: str | None = None
    max_chains: int = 300
    max_total_residues: int = 16384
    min_polymer_chains: int = 1
    # chain level
    min_residues: int = 4
    max_residues: int = 5000
    max_ca_dist: float = 10.0
    clash_freq: float = 0.3
    clash_dist: float = 1.7
    max_unk_fraction: float | None = None
    # whole-entry geometry check
    max_tight_clashes: int | None = None
    tight_clash_dist: float = 0.8
    # X-ray entries: leave out ligand chains made of buffer / precipitant molecules only (AF3 supplement table 9)
    drop_crystallization_aids: bool = True


def _chain_residues(st: Structure, ci: ChainInfo) -> np.ndarray:
    c = st.chains[ci.chain_id]
    return st.residues[int(c["res_idx"]) : int(c["res_idx"]) + int(c["res_num"])]


def _resolved_xyz(st: Structure, asym: int) -> np.ndarray:
    a = st.atoms[st.chain_atoms(st.chains[asym])]
    a = a[a["is_present"]]
    return np.stack([a["x"], a["y"], a["z"]], -1).astype(np.float64) if len(a) else np.zeros((0, 3))


def resolved_count(st: Structure, ci: ChainInfo) -> int:
    return int(_chain_residues(st, ci)["is_present"].sum())


def unknown_fraction(st: Structure, ci: ChainInfo) -> float:
    res = _chain_residues(st, ci)
    res = res[res["is_present"]]
    if not len(res):
        return 1.0
    unk = (res["res_type"] == const.RES_TYPE_ORDER["UNK"]) | (res["res_type"] == const.RES_TYPE_ORDER["N"])
    return float(unk.mean())


def ca_trace_ok(st: Structure, ci: ChainInfo, max_dist: float) -> bool:
    """Protein chains only: neighbouring residues (by residue number) keep their CA atoms within ``max_dist``."""
    if ci.mol_type != const.MOL_PROTEIN:
        return True
    pts, ids = [], []
    for r in _chain_residues(st, ci):
        atoms = st.atoms[int(r["atom_idx"]) : int(r["atom_idx"]) + int(r["atom_num"])]
        hit = np.nonzero((atoms["name"] == b"CA") & atoms["is_present"])[0]
        if len(hit):
            a = atoms[hit[0]]
            pts.append((a["x"], a["y"], a["z"]))
            ids.append(int(r["res_id"]))
    if len(pts) < 2:
        return True
    pts, ids = np.asarray(pts, np.float64), np.asarray(ids)
    step = np.linalg.norm(pts[1:] - pts[:-1], axis=1)
    return not bool(np.any((ids[1:] - ids[:-1] == 1) & (step > max_dist)))


def count_tight_clashes(st: Structure, dist: float = 0.8) -> int:
    """Heavy-atom pairs of different residues closer than ``dist`` that are not bonded."""
    present = np.nonzero(st.atoms["is_present"])[0]
    if len(present) < 2:
        return 0
    xyz = st.coords()[present].astype(np.float64)
    pairs = cKDTree(xyz).query_pairs(dist, output_type="ndarray")
    if not len(pairs):
        return 0
    res_of = np.repeat(np.arange(len(st.residues)), st.residues["atom_num"])
    i, j = present[pairs[:, 0]], present[pairs[:, 1]]
    bonded = {(int(a), int(b)) for a, b in zip(st.bonds["atom_1"], st.bonds["atom_2"])}
    keep = res_of[i] != res_of[j]
    return sum(1 for a, b in zip(i[keep], j[keep]) if (int(a), int(b)) not in bonded and (int(b), int(a)) not in bonded)


def clashing_chains(st: Structure, rec: Record, freq: float = 0.3, dist: float = 1.7) -> set[int]:
    """Chains with more than ``freq`` of their atoms within ``dist`` of another chain, removed worst-first.

    After each removal the fractions are recomputed (removing one chain can clear its neighbours). Ties go to the
    chain with fewer atoms, then to the larger chain id.
    """
    xyz = {ci.chain_id: _resolved_xyz(st, ci.chain_id) for ci in rec.chains}
    xyz = {k: v for k, v in xyz.items() if len(v)}
    trees = {k: cKDTree(v) for k, v in xyz.items()}
    alive, removed = set(xyz), set()
    while len(alive) > 1:
        worst = None
        for a in alive:
            hit = np.zeros(len(xyz[a]), bool)
            for b in alive:
                if b != a:
                    d, _ = trees[b].query(xyz[a], distance_upper_bound=dist)
                    hit |= np.isfinite(d)
            frac = float(hit.mean())
            key = (frac, -len(xyz[a]), a)
            if frac > freq and (worst is None or key > worst[0]):
                worst = (key, a)
        if worst is None:
            break
        alive.discard(worst[1])
        removed.add(worst[1])
    return removed


def filter_structure_metadata(info: StructureInfo | None, cfg: StructureFilterConfig, num_chains: int | None = None,
                              num_residues: int | None = None, num_polymer_chains: int | None = None) -> str | None:  # fmt: skip
    """Reason the entry is rejected, or ``None``. Unknown resolution / dates fail a filter that asks about them."""
    info = info or StructureInfo()
    if cfg.max_resolution is not None and (info.resolution is None or info.resolution > cfg.max_resolution):
        return f"resolution {info.resolution} > {cfg.max_resolution}"
    if cfg.min_resolution is not None and info.resolution is not None and info.resolution < cfg.min_resolution:
        return f"resolution {info.resolution} < {cfg.min_resolution}"
    if cfg.allowed_methods is not None and (info.method or "").upper() not in {m.upper() for m in cfg.allowed_methods}:
        return f"method {info.method!r} not allowed"
    if cfg.max_release_date is not None and (info.released is None or info.released > cfg.max_release_date):
        return f"released {info.released} after {cfg.max_release_date}"
    if cfg.min_release_date is not None and info.released is not None and info.released < cfg.min_release_date:
        return f"released {info.released} before {cfg.min_release_date}"
    if num_chains is not None and num_chains > cfg.max_chains:
        return f"{num_chains} chains > {cfg.max_chains}"
    if num_residues is not None and num_residues > cfg.max_total_residues:
        return f"{num_residues} residues > {cfg.max_total_residues}"
    if num_polymer_chains is not None and num_polymer_chains < cfg.min_polymer_chains:
        return f"{num_polymer_chains} polymer chains < {cfg.min_polymer_chains}"
    return None


def filter_structure(st: Structure, rec: Record, cfg: StructureFilterConfig | None = None) -> tuple[Record, dict[str, str]]:
    """Clear ``valid`` on failing chains and their interfaces (in place); returns the reasons by chain name."""
    cfg = cfg or StructureFilterConfig()
    why: dict[str, str] = {}
    for ci in rec.chains:
        polymer = ci.mol_type != const.MOL_NONPOLYMER
        n = resolved_count(st, ci)
        if polymer and not (cfg.min_residues <= n <= cfg.max_residues):
            why[ci.chain_name] = f"length {n} not in [{cfg.min_residues}, {cfg.max_residues}]"
        elif not polymer and n == 0:
            why[ci.chain_name] = "no resolved atoms"
        elif polymer and unknown_fraction(st, ci) >= 1.0:
            why[ci.chain_name] = "all residues unknown"
        elif polymer and cfg.max_unk_fraction is not None and unknown_fraction(st, ci) > cfg.max_unk_fraction:
            why[ci.chain_name] = f"UNK fraction {unknown_fraction(st, ci):.2f} > {cfg.max_unk_fraction:.2f}"
        elif not ca_trace_ok(st, ci, cfg.max_ca_dist):
            why[ci.chain_name] = f"consecutive CA > {cfg.max_ca_dist:.0f} A"
        if ci.chain_name in why:
            ci.valid = False
    for asym in clashing_chains(st, rec, cfg.clash_freq, cfg.clash_dist):
        ci = rec.chains[asym]
        ci.valid = False
        why[ci.chain_name] = "chain clashing"
    if cfg.max_tight_clashes is not None:
        n = count_tight_clashes(st, cfg.tight_clash_dist)
        if n > cfg.max_tight_clashes:
            for ci in rec.chains:
                ci.valid = False
                why.setdefault(ci.chain_name, f"{n} atom pairs below {cfg.tight_clash_dist} A")
    ok = {ci.chain_id for ci in rec.chains if ci.valid}
    for face in rec.interfaces:
        face.valid = face.valid and face.chain_1 in ok and face.chain_2 in ok
    return rec, why


def select_interface_chains(st: Structure, anchor: tuple[str, int, int] | None = None, max_chains: int = 20,
                            interface_distance: float = 15.0, ligand_inclusion_distance: float = 5.0,
                            rng: random.Random | None = None) -> set[int]:  # fmt: skip
    """Chains to keep when an assembly has more than ``max_chains`` polymer chains.

    A reference atom is drawn from the anchor (``("chain", a, _)`` or ``("interface", a, b)``; for an interface, from
    the atoms of ``a`` within ``interface_distance`` of ``b`` and the other way round); the ``max_chains`` polymer
    chains nearest to it stay, anchor chains always, and ligands within ``ligand_inclusion_distance`` of a kept chain
    come back in.
    """
    rng = rng or random.Random(0)
    every = [int(c["asym_id"]) for c in st.chains]
    polymer = [a for a in every if int(st.chains[a]["mol_type"]) != const.MOL_NONPOLYMER]
    if len(polymer) <= max_chains:
        return set(every)
    xyz = {a: _resolved_xyz(st, a) for a in every}
    forced = [] if anchor is None else ([anchor[1]] if anchor[0] == "chain" else [anchor[1], anchor[2]])
    forced = [a for a in forced if a in xyz]
    pool = np.zeros((0, 3))
    if len(forced) == 2 and len(xyz[forced[0]]) and len(xyz[forced[1]]):
        ta, tb = cKDTree(xyz[forced[0]]), cKDTree(xyz[forced[1]])
        da, _ = tb.query(xyz[forced[0]], distance_upper_bound=interface_distance)
        db, _ = ta.query(xyz[forced[1]], distance_upper_bound=interface_distance)
        pool = np.concatenate([xyz[forced[0]][np.isfinite(da)], xyz[forced[1]][np.isfinite(db)]])
    if not len(pool):
        src = [xyz[a] for a in forced if len(xyz[a])] or [xyz[a] for a in polymer if len(xyz[a])]
        pool = np.concatenate(src) if src else np.zeros((1, 3))
    ref = pool[rng.randrange(len(pool))]
    ranked = sorted((float(np.linalg.norm(xyz[a] - ref, axis=1).min()), a) for a in polymer if len(xyz[a]))
    keep = set(forced)
    for _, a in ranked:
        if len(keep & set(polymer)) >= max_chains:
            break
        keep.add(a)
    kept_xyz = [xyz[a] for a in keep if len(xyz[a])]
    if kept_xyz:
        tree = cKDTree(np.concatenate(kept_xyz))
        for a in every:
            if a not in keep and a not in polymer and len(xyz[a]):
                d, _ = tree.query(xyz[a], distance_upper_bound=ligand_inclusion_distance)
                if np.isfinite(d).any():
                    keep.add(a)
    return keep
