"""Synthetic complexes with the exact feature schema of the real pipeline.

Used by the benchmarks, the smoke test and the CPU tests: random sequences,
standard heavy-atom layouts per residue, an MSA mutated from the query,
templates as noisy copies of the target and a random-walk ground truth. Only
``torch`` and the chemistry tables are imported, so the same generator can feed
any implementation of the model.
"""

from __future__ import annotations

import math

import torch

from . import const

M = const.MAX_ATOMS_PER_TOKEN
_AA = const.PROTEIN_RES3
_RNA = ("A", "G", "C", "U")
_DNA = ("DA", "DG", "DC", "DT")


def _random_walk(n: int, step: float, g: torch.Generator) -> torch.Tensor:
    d = torch.randn(n, 3, generator=g)
    d = d / d.norm(dim=-1, keepdim=True).clamp(min=1e-6) * step
    return torch.cumsum(d, dim=0)


def synthetic_complex(chains, *, num_msa: int = 16, num_templates: int = 0, seed: int = 0, mutation_rate: float = 0.3,
                      gap_rate: float = 0.1, sigma_data: float = 16.0, with_gt: bool = True, msa_rows_total=None,
                      pad_to: int | None = None) -> dict:  # fmt: skip
    """Feature dict (no batch axis) for a complex.

    Args:
        chains: list of ``(kind, length)`` with ``kind`` in ``protein | rna | dna | ligand``; identical
            ``(kind, length, tag)`` triples with the same optional third element ``tag`` share an entity.
        num_msa: MSA rows (query included).
        num_templates: template slots, filled with noisy copies of the target backbone.
        msa_rows_total: if given, the MSA is tiled to this many rows (pre-cropped recycling stacks).
        pad_to: pad the token axis to this length with masked tokens.
    """
    g = torch.Generator().manual_seed(seed)
    res_type, mol_type, asym, entity, sym_id, res_idx, tok_idx = [], [], [], [], [], [], []
    atom_names: list[tuple[str, ...]] = []
    entity_of: dict = {}
    copies: dict = {}
    for ci, spec in enumerate(chains):
        kind, length = spec[0], spec[1]
        key = (kind, length, spec[2]) if len(spec) > 2 else (kind, length, ci)
        ent = entity_of.setdefault(key, len(entity_of))
        copy = copies.get(ent, 0)
        copies[ent] = copy + 1
        seq_g = torch.Generator().manual_seed(seed * 7919 + ent)  # copies of one entity share a sequence
        for i in range(length):
            if kind == "protein":
                name, mt = _AA[int(torch.randint(0, 20, (1,), generator=seq_g))], const.MOL_PROTEIN
                atoms = const.RESIDUE_ATOMS[name]
            elif kind == "rna":
                name, mt = _RNA[int(torch.randint(0, 4, (1,), generator=seq_g))], const.MOL_RNA
                atoms = const.RESIDUE_ATOMS[name]
            elif kind == "dna":
                name, mt = _DNA[int(torch.randint(0, 4, (1,), generator=seq_g))], const.MOL_DNA
                atoms = const.RESIDUE_ATOMS[name]
            elif kind == "ligand":
                name, mt = "UNK", const.MOL_NONPOLYMER
                atoms = (("C", "N", "O")[int(torch.randint(0, 3, (1,), generator=seq_g))] + str(i + 1),)
            else:
                raise ValueError(f"unknown chain kind {kind!r}")
            res_type.append(const.RES_TYPE_ORDER[name])
            mol_type.append(mt)
            asym.append(ci)
            entity.append(ent)
            sym_id.append(copy)
            res_idx.append(0 if kind == "ligand" else i)  # a ligand is one residue of many single-atom tokens
            tok_idx.append(len(tok_idx))
            atom_names.append(atoms)
    N = len(res_type)
    ref_mask = torch.zeros(N, M, dtype=torch.bool)
    ref_element = torch.zeros(N, M, dtype=torch.long)
    ref_chars = torch.zeros(N, M, 4, dtype=torch.long)
    rep = torch.zeros(N, dtype=torch.long)
    frame_atom = torch.zeros(N, 3, dtype=torch.long)
    frames_mask = torch.zeros(N, dtype=torch.bool)
    for i, atoms in enumerate(atom_names):
        k = len(atoms)
        ref_mask[i, :k] = True
        for a, nm in enumerate(atoms):
            ref_element[i, a] = const.atom_element(nm)
            ref_chars[i, a] = torch.tensor(const.encode_atom_name(nm))
        if mol_type[i] != const.MOL_NONPOLYMER:
            rep[i] = atoms.index(const.representative_atom("", mol_type[i]))
            frame_atom[i] = torch.tensor([atoms.index(x) for x in const.frame_atoms(mol_type[i])])
            frames_mask[i] = True
    asym_t = torch.tensor(asym)
    # reference conformers: atoms jittered around the origin, one conformer id per residue (per ligand for ligands)
    ref_pos = torch.randn(N, M, 3, generator=g) * 1.5 * ref_mask.unsqueeze(-1)
    uid = torch.zeros(N, dtype=torch.long)
    nxt = -1
    last = None
    for i in range(N):
        key = (asym[i], res_idx[i])
        if key != last:
            nxt += 1
            last = key
        uid[i] = nxt
    feats = {
        "res_type": torch.tensor(res_type),
        "mol_type": torch.tensor(mol_type),
        "asym_id": asym_t,
        "entity_id": torch.tensor(entity),
        "sym_id": torch.tensor(sym_id),
        "residue_index": torch.tensor(res_idx),
        "token_index": torch.tensor(tok_idx),
        "seq_mask": torch.ones(N, dtype=torch.bool),
        "pair_mask": torch.ones(N, N, dtype=torch.bool),
        "ref_pos": ref_pos,
        "ref_mask": ref_mask,
        "ref_element": ref_element,
        "ref_charge": torch.zeros(N, M),
        "ref_atom_name_chars": ref_chars,
        "ref_space_uid": uid.unsqueeze(-1).expand(N, M).contiguous(),
        "token_to_rep_atom": rep,
        "token_to_center_atom": rep.clone(),
        "frame_atom_index": frame_atom,
        "frame_token_index": torch.arange(N).unsqueeze(-1).expand(N, 3).contiguous(),
        "frames_mask": frames_mask,
    }
    # MSA: query row + rows mutated at ``mutation_rate`` with ``gap_rate`` gaps (polymer columns only)
    query = feats["res_type"].clone()
    S = max(1, num_msa)
    msa = query.unsqueeze(0).repeat(S, 1)
    if S > 1:
        mut = torch.rand(S - 1, N, generator=g) < mutation_rate
        gap = torch.rand(S - 1, N, generator=g) < gap_rate
        rnd = torch.randint(0, 20, (S - 1, N), generator=g)
        is_prot = (feats["mol_type"] == const.MOL_PROTEIN).unsqueeze(0)
        body = torch.where(mut & is_prot, rnd, msa[1:])
        msa[1:] = torch.where(gap & is_prot, torch.full_like(body, const.MSA_GAP), body)
    if msa_rows_total is not None and msa_rows_total > S:
        msa = msa.repeat(math.ceil(msa_rows_total / S), 1)[:msa_rows_total]
        S = msa_rows_total
    feats["msa"] = msa
    feats["msa_mask"] = torch.ones(S, N, dtype=torch.bool)
    feats["deletion_matrix"] = torch.zeros(S, N, dtype=torch.long)
    onehot = torch.nn.functional.one_hot(msa.clamp(max=30), 31).float()
    feats["profile"] = onehot.mean(0)
    feats["deletion_mean"] = torch.zeros(N)

    gt = None
    if with_gt or num_templates > 0:
        centers = torch.zeros(N, 3)
        for ci in range(len(chains)):
            sel = asym_t == ci
            n = int(sel.sum())
            kind = chains[ci][0]
            walk = _random_walk(n, 1.5 if kind == "ligand" else 3.8, g)
            centers[sel] = walk + torch.randn(3, generator=g) * sigma_data
        gt = (centers.unsqueeze(1) + torch.randn(N, M, 3, generator=g) * 1.5) * ref_mask.unsqueeze(-1)
        # the token-centre atom sits on the walk itself
        gt[torch.arange(N), rep] = centers
    if with_gt:
        feats["atom_gt_positions"] = gt
        feats["atom_gt_mask"] = ref_mask.clone()
        feats["resolution"] = torch.tensor(2.0)
        feats["is_distillation"] = torch.tensor(False)
    if num_templates > 0:
        T = num_templates
        ar = torch.arange(N)
        ca = gt[ar, rep]
        is_prot = feats["mol_type"] == const.MOL_PROTEIN
        cb_slot = torch.tensor([a.index("CB") if "CB" in a else min(1, len(a) - 1) for a in atom_names])
        frames, pbs, cas = [], [], []
        for t in range(T):
            noisy = gt + torch.randn(N, M, 3, generator=g) * 0.5
            n_, ca_, c_ = noisy[ar, frame_atom[:, 0]], noisy[ar, frame_atom[:, 1]], noisy[ar, frame_atom[:, 2]]
            e1 = torch.nn.functional.normalize(c_ - ca_, dim=-1)
            u = n_ - ca_
            e2 = torch.nn.functional.normalize(u - e1 * (u * e1).sum(-1, keepdim=True), dim=-1)
            frames.append(torch.stack([e1, e2, torch.linalg.cross(e1, e2)], dim=-2))
            pbs.append(noisy[ar, cb_slot])
            cas.append(noisy[ar, rep])
        pm = is_prot.float().unsqueeze(0).expand(T, N).contiguous()
        feats.update(
            template_aatype=feats["res_type"].unsqueeze(0).expand(T, N).contiguous(),
            template_pseudo_beta=torch.stack(pbs),
            template_pseudo_beta_mask=pm,
            template_backbone_frame=torch.stack(frames),
            template_backbone_mask=pm.clone(),
            template_ca=torch.stack(cas),
            template_mask=torch.ones(T),
        )
        del ca
    if pad_to is not None and pad_to > N:
        feats = pad_tokens(feats, pad_to)
    return feats


def pad_tokens(feats: dict, n_pad: int) -> dict:
    """Right-pad every token-indexed axis to ``n_pad`` with zeros / False (masked tokens)."""
    N = feats["res_type"].shape[0]
    out = {}
    for k, v in feats.items():
        if not isinstance(v, torch.Tensor) or v.dim() == 0:
            out[k] = v
            continue
        t = v
        for d in range(t.dim()):
            if t.shape[d] == N and k not in ("template_mask",):
                pad = [0, 0] * (t.dim() - d - 1) + [0, n_pad - N]
                t = torch.nn.functional.pad(t, pad)
        out[k] = t
    return out


def batch_features(samples: list[dict]) -> dict:
    """Stack per-example feature dicts on a new leading batch axis (shapes must already agree)."""
    out = {}
    for k in samples[0]:
        vals = [s[k] for s in samples]
        out[k] = torch.stack(vals) if isinstance(vals[0], torch.Tensor) else vals[0]
    return out


def split_lengths(total: int, parts: int) -> list[int]:
    base = total // parts
    return [base + (1 if i < total % parts else 0) for i in range(parts)]
