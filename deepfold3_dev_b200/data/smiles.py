"""Ligands given as SMILES, without a cheminformatics toolkit.

The reference hands SMILES to RDKit for the heavy-atom graph and an ETKDG conformer (data/ccd.py:160-362). Here the
string is parsed directly (organic-subset and bracket atoms, charges, bond orders, branches, ring closures, dots;
stereo marks are read and ignored) and a conformer is embedded from distance targets: bonded pairs at the sum of the
covalent radii (shortened for multiple bonds), 1-3 pairs from the hybridisation angle of the middle atom, all pairs
inside a small ring from the regular polygon, everything else kept at least a van-der-Waals contact apart. The result
is registered as a reference-conformer table entry (atoms named by element and running number, bonds with orders), so
a SMILES ligand flows through tokenisation, the bond matrix and the atom-permutation tables like a dictionary ligand.
The geometry is a plausible embedding, not a force-field minimum.
"""

from __future__ import annotations

import hashlib
import math
import re

import numpy as np

ORGANIC = ("Cl", "Br", "B", "C", "N", "O", "P", "S", "F", "I")
AROMATIC = {"b": "B", "c": "C", "n": "N", "o": "O", "p": "P", "s": "S", "se": "SE", "as": "AS"}
NUMBER = {"H": 1, "B": 5, "C": 6, "N": 7, "O": 8, "F": 9, "NA": 11, "MG": 12, "AL": 13, "SI": 14, "P": 15, "S": 16, "CL": 17,
          "K": 19, "CA": 20, "MN": 25, "FE": 26, "CO": 27, "NI": 28, "CU": 29, "ZN": 30, "AS": 33, "SE": 34, "BR": 35, "I": 53,
          "PT": 78, "AU": 79, "HG": 80}  # fmt: skip
SYMBOL = {v: k for k, v in NUMBER.items()}
RADIUS = {1: 0.31, 5: 0.84, 6: 0.76, 7: 0.71, 8: 0.66, 9: 0.57, 14: 1.11, 15: 1.07, 16: 1.05, 17: 1.02, 33: 1.19, 34: 1.20,
          35: 1.20, 53: 1.39}  # fmt: skip
BOND_ORDER = {"-": 1, "=": 2, "#": 3, ":": 4, "/": 1, "\\": 1}
_BRACKET = re.compile(r"\[(\d+)?([A-Za-z][a-z]?)(@{1,2}[A-Z0-9]*)?(H\d*)?([+-]+\d*|[+-]\d+)?(:\d+)?\]")


def parse_smiles(smiles: str):
    """``(elements, charges, bonds, aromatic)`` of the heavy atoms: atomic numbers, formal charges, ``(i, j, order)`` with
    order 4 for aromatic bonds, and per-atom aromatic flags. Explicit hydrogens ``[H]`` are dropped."""
    elements, charges, aromatic, bonds = [], [], [], []
    keep: list[bool] = []
    stack: list[int] = []
    rings: dict[str, tuple[int, int | None]] = {}
    prev, pending = None, None
    i, n = 0, len(smiles)

    def add_atom(symbol: str, charge: int, arom: bool):
        nonlocal prev, pending
        z = NUMBER.get(symbol.upper())
        if z is None:
            raise ValueError(f"SMILES: unknown element {symbol!r} in {smiles!r}")
        elements.append(z), charges.append(charge), aromatic.append(arom), keep.append(z != 1)
        idx = len(elements) - 1
        if prev is not None:
            order = pending if pending is not None else (4 if arom and aromatic[prev] else 1)
            bonds.append((prev, idx, order))
        prev, pending = idx, None

    while i < n:
        ch = smiles[i]
        if ch == "[":
            m = _BRACKET.match(smiles, i)
            if not m:
                raise ValueError(f"SMILES: bad bracket atom at {i} in {smiles!r}")
            sym, sign = m.group(2), m.group(5) or ""
            charge = 0
            if sign:
                digits = re.sub(r"[+-]", "", sign)
                charge = (int(digits) if digits else sign.count("+") + sign.count("-")) * (1 if "+" in sign else -1)
            arom = sym in AROMATIC
            add_atom(AROMATIC.get(sym, sym), charge, arom)
            i = m.end()
        elif smiles.startswith(("Cl", "Br"), i):
            add_atom(smiles[i : i + 2], 0, False)
            i += 2
        elif ch in "BCNOPSFI":
            add_atom(ch, 0, False)
            i += 1
        elif ch in "bcnops":
            add_atom(AROMATIC[ch], 0, True)
            i += 1
        elif ch in BOND_ORDER:
            pending = BOND_ORDER[ch]
            i += 1
        elif ch == "(":
            stack.append(prev)
            i += 1
        elif ch == ")":
            if not stack:
                raise ValueError(f"SMILES: unbalanced ')' in {smiles!r}")
            prev = stack.pop()
            i += 1
        elif ch == ".":
            prev, pending = None, None
            i += 1
        elif ch.isdigit() or ch == "%":
            label = smiles[i + 1 : i + 3] if ch == "%" else ch
            i += 3 if ch == "%" else 1
            if prev is None:
                raise ValueError(f"SMILES: ring closure before any atom in {smiles!r}")
            if label in rings:
                other, order = rings.pop(label)
                order = pending if pending is not None else order
                if order is None:
                    order = 4 if aromatic[prev] and aromatic[other] else 1
                bonds.append((other, prev, order))
            else:
                rings[label] = (prev, pending)
            pending = None
        else:
            raise ValueError(f"SMILES: unexpected character {ch!r} at {i} in {smiles!r}")
    if rings or stack:
        raise ValueError(f"SMILES: unclosed ring or branch in {smiles!r}")
    new = np.cumsum(keep) - 1
    bonds = [(int(new[a]), int(new[b]), o) for a, b, o in bonds if keep[a] and keep[b]]
    pick = [k for k, ok in enumerate(keep) if ok]
    return [elements[k] for k in pick], [charges[k] for k in pick], bonds, [aromatic[k] for k in pick]


def _small_rings(n: int, bonds) -> list[list[int]]:
    """One shortest cycle through every bond that closes a ring (cycles of at most 8 atoms)."""
    adj = [set() for _ in range(n)]
    for a, b, _ in bonds:
        adj[a].add(b), adj[b].add(a)
    rings, seen = [], set()
    for a, b, _ in bonds:
        # shortest path a -> b that does not use the bond itself
        prev = {a: -1}
        frontier = [a]
        while frontier and b not in prev:
            nxt = []
            for u in frontier:
                for v in adj[u]:
                    if v not in prev and not (u == a and v == b):
                        prev[v] = u
                        nxt.append(v)
            frontier = nxt
        if b in prev:
            path = [b]
            while path[-1] != a:
                path.append(prev[path[-1]])
            key = frozenset(path)
            if len(path) <= 8 and key not in seen:
                seen.add(key)
                rings.append(path)
    return rings


def embed_3d(elements, bonds, aromatic=None, seed: int = 0, iterations: int = 400) -> np.ndarray:
    """Coordinates ``[n, 3]`` (Angstrom, centred) that meet the distance targets described in the module text."""
    n = len(elements)
    if n == 1:
        return np.zeros((1, 3), dtype=np.float32)
    aromatic = aromatic or [False] * n
    rad = np.array([RADIUS.get(int(z), 1.2) for z in elements])
    target = np.zeros((n, n))
    weight = np.zeros((n, n))
    adj: list[dict[int, int]] = [dict() for _ in range(n)]
    for a, b, o in bonds:
        adj[a][b] = adj[b][a] = o
        d = rad[a] + rad[b] - {1: 0.0, 2: 0.13, 3: 0.2, 4: 0.07}.get(o, 0.0)
        target[a, b] = target[b, a] = d
        weight[a, b] = weight[b, a] = 1.0
    for c in range(n):  # 1-3 distances from the angle at c
        nb = list(adj[c])
        orders = list(adj[c].values())
        if 3 in orders or orders.count(2) >= 2:
            angle = math.pi
        elif aromatic[c] or 2 in orders or 4 in orders:
            angle = 2 * math.pi / 3
        else:
            angle = math.radians(109.5)
        for x in range(len(nb)):
            for y in range(x + 1, len(nb)):
                a, b = nb[x], nb[y]
                if weight[a, b] == 0.0:
                    d = math.sqrt(target[a, c] ** 2 + target[b, c] ** 2 - 2 * target[a, c] * target[b, c] * math.cos(angle))
                    target[a, b] = target[b, a] = d
                    weight[a, b] = weight[b, a] = 0.6
    for ring in _small_rings(n, bonds):  # regular polygon: fixes all distances inside the ring, which also makes it flat
        k = len(ring)
        side = np.mean([target[ring[t], ring[(t + 1) % k]] for t in range(k)])
        r = side / (2 * math.sin(math.pi / k))
        for x in range(k):
            for y in range(x + 1, k):
                d = 2 * r * math.sin(math.pi * min(y - x, k - (y - x)) / k)
                a, b = ring[x], ring[y]
                if adj[a].get(b) is None:
                    target[a, b] = target[b, a] = d
                    weight[a, b] = weight[b, a] = 0.6
    # connected aromatic systems (fused rings count as one) with the atoms bonded to them: kept flat during the descent
    planar_sets, seen = [], set()
    for start in range(n):
        if not aromatic[start] or start in seen:
            continue
        comp, todo = {start}, [start]
        while todo:
            u = todo.pop()
            for v in adj[u]:
                if aromatic[v] and v not in comp:
                    comp.add(v)
                    todo.append(v)
        seen |= comp
        planar_sets.append(sorted(comp | {v for u in comp for v in adj[u]}))
    rng = np.random.default_rng(seed)
    x = rng.normal(size=(n, 3)) * (1.5 * n ** (1 / 3))
    free = (weight == 0.0) & ~np.eye(n, dtype=bool)
    contact = 3.0
    step = 0.2
    for it in range(iterations):
        diff = x[:, None, :] - x[None, :, :]
        dist = np.linalg.norm(diff, axis=-1) + 1e-9
        pull = weight * (dist - target)                       # constrained pairs: spring to the target
        push = np.where(free & (dist < contact), 0.5 * (dist - contact), 0.0)   # others: only pushed apart
        grad = ((pull + push) / dist)[:, :, None] * diff
        x = x - step * grad.sum(axis=1)
        for members in planar_sets:  # pull every aromatic system half-way onto its best-fit plane
            pts = x[members]
            centre = pts.mean(axis=0)
            normal = np.linalg.svd(pts - centre)[2][2]
            x[members] = pts - 0.5 * ((pts - centre) @ normal)[:, None] * normal
        if it == iterations // 2:
            step = 0.1
    return (x - x.mean(axis=0)).astype(np.float32)


def component_from_smiles(smiles: str) -> tuple[str, dict]:
    """``(code, table entry)`` for a SMILES ligand: ``atoms`` (element symbol + running number per element),
    ``elements``, ``charges``, ``coords``, ``bonds`` ``[i, j, order]``. The code is ``L`` + 7 hex digits of the string's
    hash, so the same string always maps to the same component."""
    elements, charges, bonds, aromatic = parse_smiles(smiles)
    if not elements:
        raise ValueError(f"SMILES {smiles!r} has no heavy atoms")
    digest = hashlib.sha256(smiles.encode()).hexdigest()
    counts: dict[int, int] = {}
    names = []
    for z in elements:
        counts[z] = counts.get(z, 0) + 1
        names.append(f"{SYMBOL.get(z, 'X')}{counts[z]}"[:4])
    coords = embed_3d(elements, bonds, aromatic, seed=int(digest[:8], 16))
    entry = {"atoms": names, "elements": list(elements), "charges": list(charges), "coords": coords.round(3).tolist(),
             "bonds": [[a, b, o] for a, b, o in bonds], "smiles": smiles}  # fmt: skip
    return "L" + digest[:7].upper(), entry
