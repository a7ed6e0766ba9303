"""Features of one prediction job (reference: data/module/dataset.py:1039-1258, ``InferenceInput.from_*``).

Tokenisation: one token per standard residue or nucleotide; ligands, ions and modified residues are one
token per heavy atom. Every chain contributes its own MSA block (its columns, gaps elsewhere), the first
row is the query of the whole complex. The result is the unbatched feature dict the model's ``forward``
consumes.
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch

from . import const, ref_conformers
from .parse import a3m as a3m_mod
from .parse.json_input import JobInput, LigandChainInput, NucleotideChainInput, ProteinChainInput, parse_json_input

M = const.MAX_ATOMS_PER_TOKEN


@dataclasses.dataclass
class InferenceInput:
    features: dict
    chain_names: list[str]
    name: str = "job"
    seeds: list[int] = dataclasses.field(default_factory=lambda: [0])

    @property
    def num_tokens(self) -> int:
        return int(self.features["res_type"].shape[0])

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_sequence(cls, sequence: str, mol_type: str = "protein", name: str = "job", msa_crop_size: int = 16384):
        mt = const.MOL_TYPE_IDS[mol_type.upper()]
        chain = ProteinChainInput(["A"], sequence.upper()) if mt == const.MOL_PROTEIN else NucleotideChainInput(["A"], sequence.upper(), mt)
        return cls.from_job(JobInput(name, [chain]), msa_crop_size=msa_crop_size)

    @classmethod
    def from_a3m(cls, path: str, mol_type: str = "protein", name: str | None = None, msa_crop_size: int = 16384):
        with open(path) as f:
            text = f.read()
        query = a3m_mod.parse_a3m(text, max_rows=1).sequences[0].replace("-", "")
        mt = const.MOL_TYPE_IDS[mol_type.upper()]
        chain = (ProteinChainInput(["A"], query, unpaired_msa=text) if mt == const.MOL_PROTEIN
                 else NucleotideChainInput(["A"], query, mt, unpaired_msa=text))  # fmt: skip
        return cls.from_job(JobInput(name or "job", [chain]), msa_crop_size=msa_crop_size)

    @classmethod
    def from_json(cls, path: str, msa_crop_size: int = 16384) -> list[InferenceInput]:
        return [cls.from_job(job, msa_crop_size=msa_crop_size) for job in parse_json_input(path)]

    @classmethod
    def from_job(cls, job: JobInput, msa_crop_size: int = 16384, msa_pairing: str = "auto",
                 pdb_mmcif_dir: str | None = None) -> InferenceInput:  # fmt: skip
        if job.user_ccd:
            if "data_" in job.user_ccd and "\n" in job.user_ccd:
                ref_conformers.load_component_text(job.user_ccd)
            else:
                ref_conformers.load_table(job.user_ccd)
        needed = set()
        for chain in job.chains:
            needed.update(getattr(chain, "ccd_codes", ()) or ())
            needed.update(code for code, _ in (getattr(chain, "modifications", ()) or ()))
        ref_conformers.ensure_components(needed)
        tok: dict[str, list] = {k: [] for k in ("res_type", "mol_type", "asym", "entity", "sym", "res_idx", "atoms")}
        chain_names, chain_cols, chain_msas = [], [], []
        entity_of: dict = {}
        copies: dict = {}
        asym = 0
        for chain in job.chains:
            key = (type(chain).__name__, getattr(chain, "sequence", None), tuple(getattr(chain, "ccd_codes", ())),
                   getattr(chain, "smiles", None), tuple(getattr(chain, "modifications", ())))  # fmt: skip
            ent = entity_of.setdefault(key, len(entity_of))
            for cid in chain.ids:
                start = len(tok["res_type"])
                _tokenize_chain(chain, tok, asym, ent, copies.get(ent, 0))
                copies[ent] = copies.get(ent, 0) + 1
                chain_cols.append((start, len(tok["res_type"])))
                chain_msas.append(chain)
                chain_names.append(cid)
                asym += 1
        feats = _token_features(tok)
        feats.update(_msa_features(feats, chain_cols, chain_msas, msa_crop_size, msa_pairing))
        feats.update(_template_features(feats, chain_cols, chain_msas, mmcif_dir=pdb_mmcif_dir, max_date=job.max_template_date))
        feats["bond_matrix"] = _bond_matrix(tok, chain_names, job.bonded_atom_pairs)
        return cls(feats, chain_names, job.name, list(job.seeds))


def _bond_matrix(tok, chain_names, bonded_atom_pairs) -> torch.Tensor:
    """[N, N, 1] float: bonds between atom tokens of one component (from its dictionary entry) and the job's explicit
    ``bondedAtomPairs`` (chain id, 1-based residue, atom name), where at least one end is an atom token."""
    N = len(tok["res_type"])
    out = torch.zeros(N, N, 1)
    where: dict[tuple[int, int, str], int] = {}
    groups: dict[tuple[int, int], list[int]] = {}
    for i in range(N):
        names = tok["atoms"][i][1]
        key = (tok["asym"][i], tok["res_idx"][i])
        if len(names) == 1:  # an atom token (ligand, ion or atomised residue)
            where[(key[0], key[1], names[0])] = i
            groups.setdefault(key, []).append(i)
        else:
            for a in names:
                where.setdefault((key[0], key[1], a), i)
    for key, members in groups.items():
        code = tok["atoms"][members[0]][0]
        entry = ref_conformers._TABLE.get(str(code).upper())
        if not entry or not entry.get("bonds"):
            continue
        atom_names = entry["atoms"]
        for a, b, _order in entry["bonds"]:
            i, j = where.get((key[0], key[1], atom_names[a])), where.get((key[0], key[1], atom_names[b]))
            if i is not None and j is not None and i != j:
                out[i, j, 0] = out[j, i, 0] = 1.0
    asym_of = {name: k for k, name in enumerate(chain_names)}
    for pair in bonded_atom_pairs or ():
        ends = []
        for chain, res, atom in (pair.a, pair.b):
            ends.append(where.get((asym_of.get(chain, -1), int(res) - 1, atom)))
        if None not in ends and ends[0] != ends[1]:
            out[ends[0], ends[1], 0] = out[ends[1], ends[0], 0] = 1.0
    return out


def _template_features(feats, chain_cols, chains, max_templates: int = 4, mmcif_dir: str | None = None,
                       max_date: str | None = None) -> dict:  # fmt: skip
    """Template features of the protein chains that list hits; each chain fills its own token columns."""
    from . import templates as tpl

    N = int(feats["res_type"].shape[0])
    merged = None
    for (s, e), c in zip(chain_cols, chains):
        hits = getattr(c, "templates", None)
        L = len(getattr(c, "sequence", ""))
        if not hits or L == 0:
            continue
        loaded = tpl.load_json_templates(hits, hits[0].get("_base_dir", "."), max_templates, mmcif_dir, max_date)
        if not loaded:
            continue
        # features per residue of the chain, then one copy per token of that residue (a modified residue is several
        # atom tokens that all point at the residue's template column)
        per_res = tpl.template_features(L, loaded, max_templates)
        col = feats["residue_index"][s:e].clamp(0, L - 1)
        if merged is None:
            merged = tpl.template_features(0, [], max_templates, num_tokens=N)
        for k, v in per_res.items():
            if k == "template_mask":
                merged[k] = torch.maximum(merged[k], v)
            else:
                merged[k][:, s:e] = v.index_select(1, col)
    return merged or {}


def _component(name: str):
    rec = ref_conformers.get_ref_atoms(name)
    if rec is None:
        raise ValueError(
            f"no reference conformer for component {name!r}: pass a conformer table (userCCD / --ccd) that lists it"
        )
    return rec


def _tokenize_chain(chain, tok, asym, ent, sym):
    def add(res_type, mol_type, res_idx, atoms):
        tok["res_type"].append(res_type)
        tok["mol_type"].append(mol_type)
        tok["asym"].append(asym)
        tok["entity"].append(ent)
        tok["sym"].append(sym)
        tok["res_idx"].append(res_idx)
        tok["atoms"].append(atoms)

    if isinstance(chain, LigandChainInput):
        codes = list(chain.ccd_codes)
        if chain.smiles and not codes:
            # no dictionary entry: heavy-atom graph and an embedded conformer straight from the string
            from .smiles import component_from_smiles

            code, entry = component_from_smiles(chain.smiles)
            ref_conformers._TABLE.setdefault(code, entry)
            codes = [code]
        for r, code in enumerate(codes):
            names, elements, charges, coords = _component(code)
            for a in range(len(names)):  # one token per atom, all sharing the residue index
                add(const.RES_TYPE_ORDER["UNK"], const.MOL_NONPOLYMER, r, (code, [names[a]], [elements[a]], [charges[a]], coords[a : a + 1]))
        return
    mt = chain.mol_type
    table = {const.MOL_PROTEIN: const.PROTEIN_1TO3, const.MOL_RNA: const.RNA_1TO3, const.MOL_DNA: const.DNA_1TO3}[mt]
    unk = "UNK" if mt == const.MOL_PROTEIN else "N"
    mods = {pos - 1: code for code, pos in getattr(chain, "modifications", [])}
    for i, c in enumerate(chain.sequence):
        name = table.get(c, unk)
        if i in mods and ref_conformers.get_ref_atoms(mods[i]) is not None:  # modified residue: atom tokens
            names, elements, charges, coords = _component(mods[i])
            for a in range(len(names)):
                add(const.RES_TYPE_ORDER[name], mt, i, (mods[i], [names[a]], [elements[a]], [charges[a]], coords[a : a + 1]))
            continue
        names, elements, charges, coords = _component(name)
        add(const.RES_TYPE_ORDER[name], mt, i, (name, names, elements, charges, coords))


def _token_features(tok) -> dict:
    N = len(tok["res_type"])
    ref_pos = torch.zeros(N, M, 3)
    ref_mask = torch.zeros(N, M, dtype=torch.bool)
    ref_element = torch.zeros(N, M, dtype=torch.long)
    ref_charge = torch.zeros(N, M)
    ref_chars = torch.zeros(N, M, 4, dtype=torch.long)
    rep = torch.zeros(N, dtype=torch.long)
    frame_atom = torch.zeros(N, 3, dtype=torch.long)
    frames_mask = torch.zeros(N, dtype=torch.bool)
    uid = torch.zeros(N, dtype=torch.long)
    last, nxt = None, -1
    for i in range(N):
        _, names, elements, charges, coords = tok["atoms"][i]
        k = min(len(names), M)
        ref_mask[i, :k] = True
        ref_pos[i, :k] = torch.as_tensor(np.asarray(coords[:k], dtype=np.float32))
        ref_element[i, :k] = torch.tensor(elements[:k])
        ref_charge[i, :k] = torch.tensor([float(c) for c in charges[:k]])
        for a in range(k):
            ref_chars[i, a] = torch.tensor(const.encode_atom_name(names[a]))
        mt = tok["mol_type"][i]
        if mt != const.MOL_NONPOLYMER and len(names) > 1:
            want = const.representative_atom("", mt)
            rep[i] = names.index(want) if want in names else 0
            fa = const.frame_atoms(mt)
            if all(x in names for x in fa):
                frame_atom[i] = torch.tensor([names.index(x) for x in fa])
                frames_mask[i] = True
        key = (tok["asym"][i], tok["res_idx"][i])
        if key != last:
            nxt, last = nxt + 1, key
        uid[i] = nxt
    # conformers are expressed around the centroid of their residue (atom tokens of one ligand share one frame)
    total = torch.zeros(nxt + 1, 3).index_add_(0, uid, ref_pos.sum(1))
    count = torch.zeros(nxt + 1).index_add_(0, uid, ref_mask.sum(1).float())
    center = (total / count.clamp(min=1).unsqueeze(-1))[uid].unsqueeze(1)
    ref_pos = (ref_pos - center) * ref_mask.unsqueeze(-1)
    return {
        "res_type": torch.tensor(tok["res_type"]), "mol_type": torch.tensor(tok["mol_type"]),
        "asym_id": torch.tensor(tok["asym"]), "entity_id": torch.tensor(tok["entity"]), "sym_id": torch.tensor(tok["sym"]),
        "residue_index": torch.tensor(tok["res_idx"]), "token_index": torch.arange(N),
        "seq_mask": torch.ones(N, dtype=torch.bool), "pair_mask": torch.ones(N, N, dtype=torch.bool),
        "ref_pos": ref_pos, "ref_mask": ref_mask, "ref_element": ref_element, "ref_charge": ref_charge,
        "ref_atom_name_chars": ref_chars, "ref_space_uid": uid.unsqueeze(-1).expand(N, M).contiguous(),
        "token_to_rep_atom": rep, "token_to_center_atom": rep.clone(), "frame_atom_index": frame_atom,
        "frame_token_index": torch.arange(N).unsqueeze(-1).expand(N, 3).contiguous(), "frames_mask": frames_mask,
    }  # fmt: skip


def _msa_features(feats, chain_cols, chains, max_rows: int, msa_pairing: str = "auto") -> dict:
    N = feats["res_type"].shape[0]
    query = feats["res_type"].clone()
    rows, dels = [query.numpy()], [np.zeros(N, dtype=np.int64)]
    # paired rows first (row i of every chain that has a paired alignment), then per-chain blocks
    # a chain's alignment has one column per residue; its tokens (one per residue, or several atom tokens for a modified
    # residue) read the column of their residue
    def col(s, e):
        return feats["residue_index"][s:e].numpy()

    def usable(c, cols):
        return bool(getattr(c, "sequence", "")) and int(feats["mol_type"][cols[0]]) != const.MOL_NONPOLYMER

    def width_ok(m, c):
        return len(m.sequences) > 0 and len(m.sequences[0]) == len(c.sequence)

    paired = [(cols, a3m_mod.parse_a3m(c.paired_msa), c) for cols, c in zip(chain_cols, chains)
              if getattr(c, "paired_msa", None) and usable(c, cols)]  # fmt: skip
    paired = [(cols, m) for cols, m, c in paired if width_ok(m, c)]
    if len(paired) <= 1 and msa_pairing in ("auto", "species"):
        # no explicit paired alignments: pair the unpaired ones by species when several distinct chains carry headers
        cand = [(cols, a3m_mod.parse_a3m(c.unpaired_msa, dedup=False), c) for cols, c in zip(chain_cols, chains)
                if getattr(c, "unpaired_msa", None) and usable(c, cols)]  # fmt: skip
        cand = [(cols, m) for cols, m, c in cand if width_ok(m, c)]
        if len({m.sequences[0] for _, m in cand}) > 1:
            from .msa.pairing import pair_by_species

            joined, res = pair_by_species([m for _, m in cand], max_rows=min(max_rows, 8191))
            if len(res.rows) > 1:
                paired = [(cols, m) for (cols, _), m in zip(cand, joined)]
    if len(paired) > 1:
        depth = min(len(m) for _, m in paired)
        for r in range(1, depth):
            row, d = np.full(N, const.MSA_GAP, dtype=np.int64), np.zeros(N, dtype=np.int64)
            for (s, e), m in paired:
                mt = int(feats["mol_type"][s])
                row[s:e] = np.asarray(a3m_mod.encode_sequence(m.sequences[r], mt))[col(s, e)]
                d[s:e] = np.asarray(m.deletions[r])[col(s, e)]
            rows.append(row)
            dels.append(d)
    for (s, e), c in zip(chain_cols, chains):
        text = getattr(c, "unpaired_msa", None)
        if not text or not usable(c, (s, e)):
            continue  # ligands and chains without an alignment contribute only the query row
        m = a3m_mod.parse_a3m(text, max_rows=max_rows)
        if len(m.sequences[0]) != len(c.sequence):
            continue  # an alignment of another sequence: its columns mean nothing here
        mt = int(feats["mol_type"][s])
        for r in range(1, len(m)):
            row, d = np.full(N, const.MSA_GAP, dtype=np.int64), np.zeros(N, dtype=np.int64)
            row[s:e] = np.asarray(a3m_mod.encode_sequence(m.sequences[r], mt))[col(s, e)]
            d[s:e] = np.asarray(m.deletions[r])[col(s, e)]
            rows.append(row)
            dels.append(d)
            if len(rows) >= max_rows:
                break
    msa = torch.as_tensor(np.stack(rows[:max_rows]))
    deletion = torch.as_tensor(np.stack(dels[:max_rows]))
    onehot = torch.nn.functional.one_hot(msa, const.MSA_VOCAB_SIZE).float()
    return {"msa": msa, "msa_mask": torch.ones_like(msa, dtype=torch.bool), "deletion_matrix": deletion,
            "profile": onehot.mean(0), "deletion_mean": deletion.float().mean(0)}  # fmt: skip
