"""``Structure`` (+ per-chain MSAs, templates) -> the training feature dict.

Reference: data/tokenize/tokenizer.py (one token per standard residue, one per heavy atom for ligands and modified
residues) and data/feature/featurizer.py:37-1760 (feature table plus the training extras: ground-truth positions and
masks in the dense token-atom layout, token bonds, resolution). The output has the keys the model and the losses read
and is what ``FeatureDirDataset`` stores as ``<id>.pt``; cropping happens later, on the features.

Reference conformers of standard residues come from ``ref_conformers``. A ligand or modified residue that the
conformer table does not list uses its own observed coordinates (centred) as the conformer; the per-sample random
rotation applied by the dataset removes the pose. Unresolved atoms of such a component have no conformer entry and are
left out of the token list.
"""

from __future__ import annotations

import numpy as np
import torch

from . import const, ref_conformers
from .inference_input import _token_features
from .types import MSA, Record, Structure

M = const.MAX_ATOMS_PER_TOKEN


def tokenize_structure(st: Structure, keep_asym: set[int] | None = None, atomize: set[int] | None = None):
    """Token table (the dict ``_token_features`` consumes) plus, per token, the rows of ``st.atoms`` it covers.

    ``atomize``: rows of ``st.residues`` (standard polymer residues) to tokenise per heavy atom, the way modified
    residues and ligands always are (the training-time regulariser of the reference, data/tokenize/atomize.py:109-319).
    ``tok["col"]`` is the position of a token's residue inside its chain: the alignment / template column it reads.
    ``tok["chain_len"]`` maps a chain to its number of residues.
    """
    tok: dict[str, list] = {k: [] for k in ("res_type", "mol_type", "asym", "entity", "sym", "res_idx", "atoms", "col")}
    tok["chain_len"] = {}
    atom_rows: list[np.ndarray] = []
    chain_cols: dict[int, tuple[int, int]] = {}
    atomize = atomize or set()
    for c in st.chains:
        asym = int(c["asym_id"])
        if keep_asym is not None and asym not in keep_asym:
            continue
        start = len(tok["res_type"])
        mt = int(c["mol_type"])
        first = int(c["res_idx"])
        tok["chain_len"][asym] = int(c["res_num"])
        for ordinal, r in enumerate(st.residues[first : first + int(c["res_num"])]):
            a0, n = int(r["atom_idx"]), int(r["atom_num"])
            rows = np.arange(a0, a0 + n)
            name = r["name"].decode().strip()
            common = (int(r["res_type"]), mt, asym, int(c["entity_id"]), int(c["sym_id"]), int(r["res_id"]), ordinal)
            standard = bool(r["is_standard"]) and mt != const.MOL_NONPOLYMER and name in const.RESIDUE_ATOMS
            if standard and (first + ordinal) not in atomize:
                names, elements, charges, coords = ref_conformers.get_ref_atoms(name)
                _push(tok, common, (name, names, elements, charges, coords))
                atom_rows.append(rows[:M])
                continue
            if standard:  # atomised on request: its tokens look like those of a modified residue
                unk = const.RES_TYPE_ORDER["UNK"] if mt == const.MOL_PROTEIN else const.RES_TYPE_ORDER["N"]
                common = (unk, *common[1:])
            # per-atom tokens
            ref = ref_conformers.get_ref_atoms(name)
            atoms = st.atoms[rows]
            if ref is not None:
                by_name = {an: k for k, an in enumerate(ref[0])}
            present = atoms["is_present"]
            centre = np.zeros(3) if not present.any() else np.stack([atoms["x"], atoms["y"], atoms["z"]], -1)[present].mean(0)
            for k, a in enumerate(atoms):
                an = a["name"].decode().strip()
                if ref is not None and an in by_name:
                    j = by_name[an]
                    entry = (name, [an], [ref[1][j]], [ref[2][j]], ref[3][j : j + 1])
                elif a["is_present"]:
                    xyz = np.array([[a["x"], a["y"], a["z"]]], dtype=np.float32) - centre.astype(np.float32)
                    entry = (name, [an], [int(a["element"])], [float(a["charge"])], xyz)
                else:
                    continue
                _push(tok, common, entry)
                atom_rows.append(rows[k : k + 1])
        if len(tok["res_type"]) > start:
            chain_cols[asym] = (start, len(tok["res_type"]))
    return tok, atom_rows, chain_cols


def _push(tok, common, atoms):
    for key, v in zip(("res_type", "mol_type", "asym", "entity", "sym", "res_idx", "col"), common):
        tok[key].append(v)
    tok["atoms"].append(atoms)


def token_bonds(st: Structure, atom_rows: list[np.ndarray], feats: dict, atomize: set[int] | None = None) -> torch.Tensor:
    """[N, N] bool: bonds between tokens where at least one side is an atom token (ligand / modified residue).

    The structure's bond table holds the bonds a file states explicitly (ligands, links, modified residues). The bonds
    inside a standard residue are implied by its name, so for the residues in ``atomize`` (standard residues tokenised
    per atom) they come from ``const.RESIDUE_BONDS``, and the links to the neighbouring residues of the chain from
    ``const.POLYMER_LINK``."""
    N = len(atom_rows)
    owner = np.full(len(st.atoms), -1, dtype=np.int64)
    for t, rows in enumerate(atom_rows):
        owner[rows] = t
    out = torch.zeros(N, N, dtype=torch.bool)
    if atomize:
        def atoms_of(res_row):
            r = st.residues[res_row]
            a0, n = int(r["atom_idx"]), int(r["atom_num"])
            return {st.atoms["name"][k].decode().strip(): k for k in range(a0, a0 + n)}

        def join(a, b):
            ta, tb = (owner[a], owner[b]) if a is not None and b is not None else (-1, -1)
            if ta >= 0 and tb >= 0 and ta != tb:
                out[ta, tb] = out[tb, ta] = True

        for c in st.chains:
            first, count, mt = int(c["res_idx"]), int(c["res_num"]), int(c["mol_type"])
            link = const.POLYMER_LINK.get(mt)
            for ri in range(first, first + count):
                if ri not in atomize:
                    continue
                mine = atoms_of(ri)
                for x, y in const.RESIDUE_BONDS.get(st.residues[ri]["name"].decode().strip(), ()):
                    join(mine.get(x), mine.get(y))
                if link is not None:
                    if ri > first:
                        join(atoms_of(ri - 1).get(link[0]), mine.get(link[1]))
                    if ri + 1 < first + count:
                        join(mine.get(link[0]), atoms_of(ri + 1).get(link[1]))
    single = np.array([len(r) == 1 for r in atom_rows])
    a, b = owner[st.bonds["atom_1"]], owner[st.bonds["atom_2"]]
    ok = (a >= 0) & (b >= 0) & (a != b)
    a, b = a[ok], b[ok]
    ok = single[a] | single[b]
    out[a[ok], b[ok]] = True
    out[b[ok], a[ok]] = True
    return out


def msa_block(feats: dict, chain_cols: dict[int, tuple[int, int]], paired: dict[int, MSA] | None,
              unpaired: dict[int, MSA] | None, max_rows: int = const.MAX_MSA_ROWS, token_col=None, chain_len=None) -> dict:  # fmt: skip
    """Query row, then paired rows (row i of every chain), then each chain's own rows in its own columns.

    ``token_col`` ``[N]``: the alignment column every token reads (its residue's position in the chain; several atom
    tokens of one residue share a column) and ``chain_len``: residues per chain, i.e. the width an alignment must
    have. Without them a chain's tokens and its alignment columns correspond one to one."""
    N = feats["res_type"].shape[0]
    rows = [feats["res_type"].numpy().astype(np.int64)]
    dels = [np.zeros(N, dtype=np.int64)]

    def width(asym):
        s, e = chain_cols[asym]
        return chain_len[asym] if chain_len is not None else e - s

    def cols(asym):
        s, e = chain_cols[asym]
        return np.asarray(token_col[s:e]) if token_col is not None else np.arange(e - s)

    def fits(asym, msa):
        return msa is not None and not msa.is_empty and msa.sequences.shape[1] == width(asym)

    pm = {a: m for a, m in (paired or {}).items() if a in chain_cols and fits(a, m)}
    if len(pm) > 1:
        for r in range(1, min(m.sequences.shape[0] for m in pm.values())):
            row, d = np.full(N, const.MSA_GAP, dtype=np.int64), np.zeros(N, dtype=np.int64)
            for a, m in pm.items():
                s, e = chain_cols[a]
                row[s:e], d[s:e] = m.sequences[r][cols(a)], m.deletion_matrix[r][cols(a)]
            rows.append(row), dels.append(d)
    for a, m in (unpaired or {}).items():
        if a not in chain_cols or not fits(a, m):
            continue
        s, e = chain_cols[a]
        for r in range(1, m.sequences.shape[0]):
            if len(rows) >= max_rows:
                break
            row, d = np.full(N, const.MSA_GAP, dtype=np.int64), np.zeros(N, dtype=np.int64)
            row[s:e], d[s:e] = m.sequences[r][cols(a)], m.deletion_matrix[r][cols(a)]
            rows.append(row), dels.append(d)
    msa = torch.as_tensor(np.stack(rows[:max_rows]))
    deletion = torch.as_tensor(np.stack(dels[:max_rows]))
    onehot = torch.nn.functional.one_hot(msa.clamp(max=const.MSA_VOCAB_SIZE - 1), const.MSA_VOCAB_SIZE).float()
    return {"msa": msa, "msa_mask": torch.ones_like(msa, dtype=torch.bool), "deletion_matrix": deletion,
            "profile": onehot.mean(0)[:, : const.RES_TYPE_COUNT], "deletion_mean": deletion.float().mean(0)}  # fmt: skip


def featurize_structure(st: Structure, record: Record | None = None, paired_msa: dict[int, MSA] | None = None,
                        unpaired_msa: dict[int, MSA] | None = None, only_valid: bool = True,
                        max_msa_rows: int = const.MAX_MSA_ROWS, with_msa: bool = True, atomize: set[int] | None = None) -> dict:  # fmt: skip
    """The unbatched, uncropped feature dict of one entry (tensors on CPU). ``with_msa=False`` leaves the alignment
    block out and returns the token range of every chain under ``"_chain_cols"`` instead, for callers that crop first
    and read alignments only for what survives (``attach_cropped_msa``)."""
    keep = None
    if record is not None and only_valid:
        keep = {c.chain_id for c in record.chains if c.valid}
    tok, atom_rows, chain_cols = tokenize_structure(st, keep, atomize)
    if not tok["res_type"]:
        raise ValueError(f"{st.name}: no tokens after filtering")
    token_col, chain_len = np.asarray(tok.pop("col"), dtype=np.int64), tok.pop("chain_len")
    feats = _token_features(tok)
    N = len(atom_rows)
    gt = torch.zeros(N, M, 3)
    gt_mask = torch.zeros(N, M, dtype=torch.bool)
    xyz = st.coords()
    for t, rows in enumerate(atom_rows):
        k = len(rows)
        gt[t, :k] = torch.as_tensor(xyz[rows])
        gt_mask[t, :k] = torch.as_tensor(st.atoms["is_present"][rows])
    gt_mask &= feats["ref_mask"]
    feats["atom_gt_positions"] = gt * gt_mask.unsqueeze(-1)
    feats["atom_gt_mask"] = gt_mask
    feats["bond_matrix"] = token_bonds(st, atom_rows, feats, atomize).float().unsqueeze(-1)  # [N, N, 1], read by the trunk
    if with_msa:
        feats.update(msa_block(feats, chain_cols, paired_msa, unpaired_msa, max_msa_rows, token_col, chain_len))
    else:
        feats["_chain_cols"] = dict(chain_cols)
        feats["_token_col"], feats["_chain_len"] = token_col, dict(chain_len)
    info = record.structure_info if record is not None else None
    feats["resolution"] = torch.tensor(float(info.resolution) if info and info.resolution else const.RESOLUTION_UNKNOWN)
    feats["is_distillation"] = torch.tensor(False)
    return feats


def attach_cropped_msa(feats: dict, keep, chain_cols: dict[int, tuple[int, int]], load_msa, load_paired=None,
                       max_msa_rows: int = const.MAX_MSA_ROWS, token_col=None, chain_len=None) -> tuple[dict, int, int]:
    """Alignment block of an example that was cropped first (reference: data/module/dataset.py:425-602).

    ``feats`` are the cropped features, ``keep`` the sorted indices of the surviving tokens in the uncropped example
    (``None``: nothing was cut) and ``chain_cols`` the uncropped token range of every chain. ``load_msa(asym_id)`` /
    ``load_paired(asym_id)`` are called only for chains that still have tokens; their alignments are cut to the
    surviving columns before rows are assembled, so a 384-token crop of a large assembly never reads the alignments
    of the chains it dropped. Returns the features and how many alignments were read and skipped."""
    n_all = max((e for _, e in chain_cols.values()), default=0)
    keep_np = np.arange(n_all) if keep is None else np.asarray(keep)
    new_cols, unpaired, paired, read, skipped = {}, {}, {}, 0, 0
    for asym, (s, e) in chain_cols.items():
        pos = np.flatnonzero((keep_np >= s) & (keep_np < e))
        if len(pos) == 0:
            skipped += 1
            continue
        new_cols[asym] = (int(pos[0]), int(pos[-1]) + 1)
        # alignment column of every surviving token: its residue's position in the chain (``token_col``) when the
        # chain holds atom tokens, else simply its offset inside the chain
        cols = np.asarray(token_col)[keep_np[pos]] if token_col is not None else keep_np[pos] - s
        want = chain_len[asym] if chain_len is not None else e - s
        for loader, store in ((load_msa, unpaired), (load_paired, paired)):
            m = loader(asym) if loader is not None else None
            if m is None or m.is_empty or m.sequences.shape[1] != want:
                continue
            read += 1
            store[asym] = MSA(m.sequences[:, cols], m.mask[:, cols], m.deletion_matrix[:, cols])
    out = dict(feats)
    out.update(msa_block(out, new_cols, paired or None, unpaired or None, max_msa_rows))
    return out, read, skipped


def attach_cropped_templates(feats: dict, keep, chain_cols: dict[int, tuple[int, int]], token_col, chain_len, load_templates,
                             max_templates: int = 4) -> tuple[dict, int]:
    """Template features of an example that was cropped first. ``load_templates(asym_id)`` returns the ``TemplateChain``
    list of a chain (its query indices count residues of the chain) and is called only for chains that still have
    tokens. Slot ``t`` of every chain shares row ``t`` of the template axis; the model only lets a template inform
    pairs inside one chain. Returns the features (always ``max_templates`` rows) and the number of templates used."""
    from . import templates as tpl

    N = int(feats["res_type"].shape[0])
    out = tpl.template_features(0, [], max_templates, num_tokens=N)
    n_all = max((e for _, e in chain_cols.values()), default=0)
    keep_np = np.arange(n_all) if keep is None else np.asarray(keep)
    used = 0
    for asym, (s, e) in chain_cols.items():
        pos = np.flatnonzero((keep_np >= s) & (keep_np < e))
        if len(pos) == 0:
            continue
        chains = load_templates(asym) or []
        if not chains:
            continue
        per_res = tpl.template_features(int(chain_len[asym]), chains, max_templates)
        cols = torch.as_tensor(np.asarray(token_col)[keep_np[pos]])
        where = torch.as_tensor(pos)
        for k, v in per_res.items():
            if k == "template_mask":
                out[k] = torch.maximum(out[k], v)
            else:
                out[k][:, where] = v.index_select(1, cols)
        used += min(len(chains), max_templates)
    return out, used
