"""Ground-truth relabelling under molecular symmetry: chains, residue atoms, ligand atoms.

Three symmetries leave a structure unchanged but change atom labels
(AF3 supplement 4.2 / 4.3): identical chains can be exchanged, some side-chain
atoms can be exchanged within a residue (ASP OD1/OD2, PHE ring, ...), and a
ligand's graph automorphisms permute its atoms. Before a loss compares a
prediction with the ground truth, the ground truth is relabelled to the
member of its symmetry orbit closest to the prediction.

Reference behaviour: data/symmetry/chain_perm.py:121-830 and
data/symmetry/atom_perms.py:73-623. The decision rules are the same; the
implementation is tensor-level where the reference loops in Python.
"""

from __future__ import annotations

from collections import defaultdict

import numpy as np
import torch

MOL_NONPOLYMER = 3

# residue name -> pairs of atom names that may be exchanged together (one group per residue)
RESIDUE_SWAPS: dict[str, tuple[tuple[str, str], ...]] = {
    "ASP": (("OD1", "OD2"),),
    "GLU": (("OE1", "OE2"),),
    "PHE": (("CD1", "CD2"), ("CE1", "CE2")),
    "TYR": (("CD1", "CD2"), ("CE1", "CE2")),
    "ARG": (("NH1", "NH2"),),
    "LEU": (("CD1", "CD2"),),
    "VAL": (("CG1", "CG2"),),
    "A": (("OP1", "OP2"),),
    "G": (("OP1", "OP2"),),
    "C": (("OP1", "OP2"),),
    "U": (("OP1", "OP2"),),
    "DA": (("OP1", "OP2"),),
    "DG": (("OP1", "OP2"),),
    "DC": (("OP1", "OP2"),),
    "DT": (("OP1", "OP2"),),
}


def build_residue_symmetry_pairs(res_name: str, atom_names: list[str]) -> list[tuple[int, int]]:
    """Index pairs into ``atom_names`` that ``res_name``'s symmetry exchanges; pairs with a missing atom are dropped."""
    pos = {n: i for i, n in enumerate(atom_names)}
    return [(pos[a], pos[b]) for a, b in RESIDUE_SWAPS.get(res_name, ()) if a in pos and b in pos]


def _as_long(table, device):
    if table is None:
        return None
    t = table if isinstance(table, torch.Tensor) else torch.as_tensor(np.asarray(table))
    return t.to(dtype=torch.long, device=device)


def _grouped_swap(pred, gt, ia, ib, valid, group):
    """Exchange ``gt[..., ia]`` and ``gt[..., ib]`` for every group whose summed squared error drops.

    ``pred`` / ``gt``: ``[..., L, 3]`` flat atom lists; ``ia``, ``ib``, ``group``: ``[P]``;
    ``valid``: ``[P]`` bool. Decisions are independent per leading index and joint per group.
    """
    pa, pb, ga, gb = pred[..., ia, :], pred[..., ib, :], gt[..., ia, :], gt[..., ib, :]
    v = valid.to(gt.dtype)
    keep_cost = ((pa - ga).pow(2).sum(-1) + (pb - gb).pow(2).sum(-1)) * v
    swap_cost = ((pa - gb).pow(2).sum(-1) + (pb - ga).pow(2).sum(-1)) * v
    _, inv = torch.unique(group, return_inverse=True)
    n_groups = int(inv.max()) + 1
    zeros = keep_cost.new_zeros(*keep_cost.shape[:-1], n_groups)
    better = zeros.index_add(-1, inv, swap_cost) < zeros.index_add(-1, inv, keep_cost)
    do = (better.index_select(-1, inv) & valid).unsqueeze(-1)
    out = gt.clone()
    out[..., ia, :] = torch.where(do, gb, ga)
    out[..., ib, :] = torch.where(do, ga, gb)
    return out


def apply_token_atom_permutation(pred_pos, gt_pos, atom_mask, swap_pairs):
    """Residue-internal swaps. ``swap_pairs``: ``[P, 3]`` rows ``(token, atom_a, atom_b)``; one group per token."""
    pairs = _as_long(swap_pairs, gt_pos.device)
    if pairs is None or pairs.numel() == 0:
        return gt_pos.detach()
    pairs = pairs[pairs[:, 1] != pairs[:, 2]]  # collate padding rows are (0, 0, 0)
    if pairs.numel() == 0:
        return gt_pos.detach()
    M = gt_pos.shape[-2]
    tok, a, b = pairs.unbind(1)
    valid = atom_mask[tok, a].bool() & atom_mask[tok, b].bool()
    flat = lambda t: t.detach().reshape(*t.shape[:-3], -1, 3)  # noqa: E731
    out = _grouped_swap(flat(pred_pos), flat(gt_pos), tok * M + a, tok * M + b, valid, tok)
    return out.reshape(gt_pos.shape)


def apply_ligand_token_swap(pred_pos, gt_pos, atom_mask, swap_pairs):
    """Swaps between single-atom tokens (slot 0). ``swap_pairs``: ``[P, 2]`` or ``[P, 3]`` with a group id column."""
    pairs = _as_long(swap_pairs, gt_pos.device)
    if pairs is None or pairs.numel() == 0:
        return gt_pos.detach()
    pairs = pairs[pairs[:, 0] != pairs[:, 1]]
    if pairs.numel() == 0:
        return gt_pos.detach()
    M = gt_pos.shape[-2]
    a, b = pairs[:, 0], pairs[:, 1]
    group = pairs[:, 2] if pairs.shape[1] >= 3 else torch.arange(pairs.shape[0], device=pairs.device)
    valid = atom_mask[a, 0].bool() & atom_mask[b, 0].bool()
    flat = lambda t: t.detach().reshape(*t.shape[:-3], -1, 3)  # noqa: E731
    return _grouped_swap(flat(pred_pos), flat(gt_pos), a * M, b * M, valid, group).reshape(gt_pos.shape)


def apply_ligand_token_permutation(pred_pos, gt_pos, atom_mask, perm_table):
    """Whole-automorphism choice per ligand.

    ``perm_table``: ``[R, 4]`` rows ``(ligand, permutation, dst_token, src_token)`` listing the moved
    atoms of each non-identity automorphism. Per leading index and ligand the permutation with the
    most negative ``sum |pred_dst - gt_src|^2 - |pred_dst - gt_dst|^2`` is applied, provided all of
    its atoms are resolved; none is applied if none beats the identity.
    """
    tab = _as_long(perm_table, gt_pos.device)
    if tab is None or tab.numel() == 0:
        return gt_pos.detach()
    tab = tab[tab[:, 2] != tab[:, 3]]
    if tab.numel() == 0:
        return gt_pos.detach()
    lig, dst, src = tab[:, 0], tab[:, 2], tab[:, 3]
    ok = atom_mask[dst, 0].bool() & atom_mask[src, 0].bool()
    p_dst = pred_pos[..., dst, 0, :].detach()
    g_src, g_dst = gt_pos[..., src, 0, :].detach(), gt_pos[..., dst, 0, :].detach()
    delta = ((p_dst - g_src).pow(2).sum(-1) - (p_dst - g_dst).pow(2).sum(-1)) * ok.to(p_dst.dtype)
    uniq, gid = torch.unique(tab[:, :2], dim=0, return_inverse=True)
    G = uniq.shape[0]
    cost = delta.new_zeros(*delta.shape[:-1], G).index_add(-1, gid, delta)
    unresolved = delta.new_zeros(G).index_add(0, gid, (~ok).to(delta.dtype)) > 0
    cost = cost.masked_fill(unresolved, float("inf"))
    # best group per ligand: minimise over the groups of each ligand
    lig_of_group = uniq[:, 0]
    ligs, lig_inv = torch.unique(lig_of_group, return_inverse=True)
    big = cost.new_full((*cost.shape[:-1], ligs.numel(), G), float("inf"))
    sel = torch.zeros(ligs.numel(), G, dtype=torch.bool, device=cost.device)
    sel[lig_inv, torch.arange(G, device=cost.device)] = True
    per_lig = torch.where(sel, cost.unsqueeze(-2), big)  # [..., L, G]
    best_cost, best_g = per_lig.min(-1)  # [..., L]
    chosen = torch.zeros(*cost.shape[:-1], G, dtype=torch.bool, device=cost.device)
    chosen.scatter_(-1, best_g, best_cost < 0.0)
    # a group index can be written by a ligand that does not own it only if that ligand's best cost is inf -> False
    row_on = chosen.index_select(-1, gid)  # [..., R]
    # a token is listed once per permutation of its ligand, and at most one of those permutations is switched on: add
    # the chosen move as a difference (rows that stay off add zero) instead of writing every row, where the last
    # write of a repeated index would win
    move = torch.where(row_on.unsqueeze(-1), g_src - g_dst, torch.zeros_like(g_dst))
    out = gt_pos.detach().clone()
    first = out[..., :, 0, :].clone()
    first.index_add_(-2, dst, move)
    out[..., :, 0, :] = first
    return out


# --------------------------------------------------------------------------- chains


def _kabsch(p: np.ndarray, q: np.ndarray):
    """``(R, t)`` with ``R p + t ~ q`` for matched ``[K, 3]`` point sets, reflection-free."""
    pm, qm = p.mean(0), q.mean(0)
    u, _, vt = np.linalg.svd((p - pm).T @ (q - qm))
    d = np.eye(3)
    d[2, 2] = np.sign(np.linalg.det(vt.T @ u.T))
    r = vt.T @ d @ u.T
    return r, qm - r @ pm


def _components(order, bonds):
    """Chains joined by covalent inter-chain bonds form one unit; returns the list of member tuples."""
    parent = {a: a for a in order}

    def find(x):
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    for bond in bonds or ():
        a, b = int(bond[0]), int(bond[1])
        if a in parent and b in parent:
            parent[find(a)] = find(b)
    groups = defaultdict(list)
    for a in order:
        groups[find(a)].append(a)
    return [tuple(v) for v in groups.values()]


def _component_signature(members, ent_of, bonds):
    """Isomorphism invariant of a component: entity multiset plus the multiset of bonded entity pairs."""
    mem = set(members)
    edges = sorted(
        tuple(sorted((ent_of[int(b[0])], ent_of[int(b[1])]))) for b in bonds or () if int(b[0]) in mem and int(b[1]) in mem
    )
    return (tuple(sorted(ent_of[a] for a in members)), tuple(edges))


def compute_chain_permutation_tokens(pred_pos, gt_pos, atom_mask, asym_id, entity_id, token_to_rep_atom=None,
                                     mol_type=None, seq_mask=None, sym_token_index=None,
                                     inter_chain_bonds=None) -> dict[int, int]:  # fmt: skip
    """``{predicted chain: ground-truth chain}`` by anchor-frame greedy matching.

    One global frame is fitted by aligning a predicted chain of the anchor
    entity onto the ground-truth anchor chain; in that frame every predicted
    unit (chain plus covalently attached chains) takes the nearest unused
    ground-truth unit of the same symmetry class. Every candidate anchor is
    tried and the assignment with the least summed squared centroid distance
    wins. Identity when no two units are interchangeable.
    """
    asym = asym_id.detach().cpu().numpy()
    ent = entity_id.detach().cpu().numpy()
    mol = mol_type.detach().cpu().numpy() if mol_type is not None else None
    sym = sym_token_index.detach().cpu().numpy() if sym_token_index is not None else None
    valid = seq_mask.detach().cpu().numpy().astype(bool) if seq_mask is not None else np.ones(len(asym), bool)
    order = list(dict.fromkeys(int(a) for a, v in zip(asym, valid) if v))
    ent_of = {a: int(ent[(asym == a) & valid][0]) for a in order}
    comps = _components(order, inter_chain_bonds)
    classes = defaultdict(list)
    for ci, members in enumerate(comps):
        classes[_component_signature(members, ent_of, inter_chain_bonds)].append(ci)
    identity = {a: a for a in order}
    if not any(len(v) > 1 for v in classes.values()):
        return identity  # nothing interchangeable: no device-to-host copy of coordinates needed

    with torch.no_grad():
        if token_to_rep_atom is not None:
            rep = token_to_rep_atom.to(device=pred_pos.device, dtype=torch.long)
            ar = torch.arange(rep.shape[0], device=pred_pos.device)
            P = pred_pos[ar, rep].double().cpu().numpy()
            G = gt_pos[ar, rep].double().cpu().numpy()
            R = atom_mask[ar, rep].bool().cpu().numpy()
            per_token = 1
        else:
            per_token = pred_pos.shape[-2]
            P = pred_pos.reshape(-1, 3).double().cpu().numpy()
            G = gt_pos.reshape(-1, 3).double().cpu().numpy()
            R = atom_mask.reshape(-1).bool().cpu().numpy()
            sym = None

    rows, cen_p, cen_g, lig = {}, {}, {}, {}
    for a in order:
        tok = np.where((asym == a) & valid)[0]
        idx = tok if per_token == 1 else (tok[:, None] * per_token + np.arange(per_token)).reshape(-1)
        rows[a] = idx
        m = R[idx]
        cen_p[a] = P[idx][m].mean(0) if m.any() else None
        cen_g[a] = G[idx][m].mean(0) if m.any() else None
        lig[a] = bool(mol is not None and np.all(mol[tok] == MOL_NONPOLYMER))
    resolved = [a for a in order if cen_p[a] is not None]
    if len(resolved) < 2:
        return identity
    natoms = {a: int(R[rows[a]].sum()) for a in resolved}
    by_ent = defaultdict(list)
    for a in resolved:
        by_ent[ent_of[a]].append(a)
    anchor_ent = min(
        by_ent, key=lambda e: (all(lig[a] for a in by_ent[e]), len(by_ent[e]), -max(natoms[a] for a in by_ent[e]))
    )
    gt_anchor = max(by_ent[anchor_ent], key=lambda a: natoms[a])

    def unit_centroids(cen):
        out = {}
        for ci, members in enumerate(comps):
            ok = [a for a in members if cen.get(a) is not None]
            out[ci] = cen[min(ok, key=lambda a: (lig[a], -natoms[a]))] if ok else None
        return out

    ucp, ucg = unit_centroids(cen_p), unit_centroids(cen_g)

    def matched_points(pa):
        ip, ig = rows[pa], rows[gt_anchor]
        if sym is None:
            if len(ip) != len(ig):
                return None
            both = R[ip] & R[ig]
            return (P[ip][both], G[ig][both]) if both.sum() >= 3 else None
        first = {}
        for r in ip[R[ip]]:
            first.setdefault(int(sym[r]), r)
        rp, rg, seen = [], [], set()
        for r in ig[R[ig]]:
            s = int(sym[r])
            if s in first and s not in seen:
                seen.add(s)
                rp.append(first[s])
                rg.append(r)
        return (P[rp], G[rg]) if len(rp) >= 3 else None

    best, best_score = None, np.inf
    for pa in by_ent[anchor_ent]:
        pts = matched_points(pa)
        if pts is None:
            continue
        rot, trans = _kabsch(*pts)
        trial, score = dict(identity), 0.0
        for members in classes.values():
            used = set()
            for pc in members:
                if ucp[pc] is None:
                    continue
                moved = rot @ ucp[pc] + trans
                cands = [(float(((moved - ucg[gc]) ** 2).sum()), gc) for gc in members if gc not in used and ucg[gc] is not None]
                if not cands:
                    continue
                _, gc = min(cands)
                used.add(gc)
                taken = set()
                for p in comps[pc]:  # chains inside the matched units: nearest of the same entity
                    if cen_p[p] is None:
                        continue
                    mp = rot @ cen_p[p] + trans
                    opts = [(float(((mp - cen_g[g]) ** 2).sum()), g) for g in comps[gc]
                            if g not in taken and cen_g[g] is not None and ent_of[g] == ent_of[p]]  # fmt: skip
                    if opts:
                        d, g = min(opts)
                        taken.add(g)
                        trial[p] = g
                        score += d
        if score < best_score:
            best, best_score = trial, score
    return best if best is not None else identity


def chain_permutation_index(asym_id, chain_assignment, sym_token_index=None, device=None):
    """``(index, keep)``: ``gt_new[i] = gt[index[i]]``; ``keep[i]`` False where token ``i`` has no partner.

    Without ``sym_token_index`` chains map position by position and pairs of unequal length are left
    alone; with it, tokens map by their per-chain ordinal.
    """
    dev = device if device is not None else asym_id.device
    n = int(asym_id.shape[0])
    asym = asym_id.detach().cpu().numpy()
    index, keep = np.arange(n), np.ones(n, bool)
    sym = sym_token_index.detach().cpu().numpy() if sym_token_index is not None else None
    for p, g in (chain_assignment or {}).items():
        if int(p) == int(g):
            continue
        pr, gr = np.where(asym == int(p))[0], np.where(asym == int(g))[0]
        if sym is None:
            if len(pr) == len(gr):
                index[pr] = gr
            continue
        table = {}
        if len(set(sym[gr].tolist())) != len(gr):
            continue  # duplicated ordinals: mapping undefined, leave the chain alone
        for r in gr:
            table[int(sym[r])] = r
        for r in pr:
            hit = table.get(int(sym[r]))
            if hit is None:
                keep[r] = False
            else:
                index[r] = hit
    return torch.from_numpy(index).to(dev), torch.from_numpy(keep).to(dev)


def apply_chain_permutation_tokens(gt_pos, atom_mask, asym_id, chain_assignment, sym_token_index=None):
    if not chain_assignment or all(int(k) == int(v) for k, v in chain_assignment.items()):
        return gt_pos.detach(), atom_mask.detach()
    index, keep = chain_permutation_index(asym_id, chain_assignment, sym_token_index, device=gt_pos.device)
    return gt_pos.index_select(-3, index).detach(), (atom_mask.index_select(0, index) & keep.unsqueeze(-1)).detach()


def graph_automorphisms(elements, edges, limit: int = 1000, orders=None) -> list[list[int]]:
    """Atom permutations of a ligand that keep its chemistry: ``perm[i]`` is the atom that takes the place of atom ``i``,
    elements, bonds (and bond orders when given) preserved. The identity comes first; the search stops at ``limit``
    permutations. This is what the ligand atom-permutation loss consumes as ``ligand_perms`` (reference:
    data/symmetry/ligand_perms.py:110-172, there through RDKit substructure matching; here a direct search: colour
    refinement by element and neighbourhood, then backtracking over atoms of equal colour)."""
    n = len(elements)
    adj: list[dict[int, int]] = [dict() for _ in range(n)]
    for k, (a, b) in enumerate(edges):
        order = 1 if orders is None else int(orders[k])
        adj[a][b] = adj[b][a] = order
    colour = [(int(e), len(adj[i])) for i, e in enumerate(elements)]
    for _ in range(n):  # 1-dimensional Weisfeiler-Leman refinement until stable
        sig = [(colour[i], tuple(sorted((colour[j], o) for j, o in adj[i].items()))) for i in range(n)]
        ids = {s_: k for k, s_ in enumerate(sorted(set(sig)))}
        new = [ids[s_] for s_ in sig]
        if len(set(new)) == len(set(colour)):
            colour = new
            break
        colour = new
    # visit atoms so that each one (after the first of a component) touches an atom already placed
    order_, seen = [], set()
    for start in sorted(range(n), key=lambda i: (sum(1 for c in colour if c == colour[i]), i)):
        if start in seen:
            continue
        queue = [start]
        seen.add(start)
        while queue:
            i = queue.pop(0)
            order_.append(i)
            for j in sorted(adj[i]):
                if j not in seen:
                    seen.add(j)
                    queue.append(j)
    out: list[list[int]] = []
    perm, used = [-1] * n, [False] * n

    def place(depth: int) -> bool:
        if depth == n:
            out.append(list(perm))
            return len(out) >= limit
        i = order_[depth]
        placed = order_[:depth]
        for j in range(n):
            if used[j] or colour[j] != colour[i]:
                continue
            if any(adj[i].get(k) != adj[j].get(perm[k]) for k in placed):
                continue
            perm[i], used[j] = j, True
            if place(depth + 1):
                return True
            perm[i], used[j] = -1, False
        return False

    place(0)
    out.sort(key=lambda p_: p_ != list(range(n)))
    return out


def symmetry_features(feats: dict, max_ligand_atoms: int = 64, max_perms: int = 32) -> dict:
    """The permutation tables of one (cropped) example, built from its own features so that every index refers to the
    tokens that survived the crop (reference: data/feature/featurizer.py training extras, symmetry/atom_perms.py,
    symmetry/ligand_perms.py):

    ``atom_swap_pairs`` ``[P, 3]``   (token, atom slot a, atom slot b) for the exchangeable atoms of standard residues;
    ``ligand_perms``    ``[R, 4]``   (ligand, permutation, destination token, source token) for every non-identity
                                     automorphism of each ligand whose atoms are all present in the crop.
    """
    from . import const

    res_type = feats["res_type"].tolist()
    mol_type = feats["mol_type"].tolist()
    chars = feats["ref_atom_name_chars"]
    mask = feats["ref_mask"]
    names_of = lambda t: ["".join(chr(int(c) + 32) for c in chars[t, a]).strip() for a in range(int(mask[t].sum()))]  # noqa: E731
    swaps = []
    for t, (rt, mt) in enumerate(zip(res_type, mol_type)):
        if mt == const.MOL_NONPOLYMER or int(mask[t].sum()) <= 1:
            continue
        name = const.RES_TYPE_INDEX_TO_NAME.get(int(rt))
        if name in RESIDUE_SWAPS:
            swaps += [(t, a, b) for a, b in build_residue_symmetry_pairs(name, names_of(t))]
    out = {"atom_swap_pairs": torch.tensor(swaps, dtype=torch.long).reshape(-1, 3)}
    # ligands: atom tokens of non-polymer chains grouped by (chain, residue)
    groups: dict[tuple[int, int], list[int]] = {}
    asym, resi = feats["asym_id"].tolist(), feats["residue_index"].tolist()
    for t, mt in enumerate(mol_type):
        if mt == const.MOL_NONPOLYMER and int(mask[t].sum()) == 1:
            groups.setdefault((asym[t], resi[t]), []).append(t)
    bonds = feats.get("bond_matrix")
    rows = []
    for lig, members in enumerate(groups.values()):
        if not 1 < len(members) <= max_ligand_atoms or bonds is None:
            continue
        idx = torch.tensor(members)
        sub = bonds[idx][:, idx].reshape(len(members), len(members)) > 0
        edges = [(int(a), int(b)) for a, b in torch.nonzero(torch.triu(sub, 1)).tolist()]
        if not edges:
            continue
        elements = feats["ref_element"][idx, 0].tolist()
        perms = graph_automorphisms(elements, edges, limit=max_perms + 1)
        for pid, perm in enumerate(perms[1:]):
            rows += [(lig, pid, members[dst], members[src]) for dst, src in enumerate(perm) if dst != src]
    out["ligand_perms"] = torch.tensor(rows, dtype=torch.long).reshape(-1, 4)
    return out
