"""Template features from aligned template chains (reference: data/feature/featurizer.py:420-560).

Inputs are template hits whose coordinates are already available as arrays (a chain's residue names and
per-residue atom coordinates in ``const.RESIDUE_ATOMS`` order); reading them out of mmCIF files is the
preparation step that needs gemmi. Features, per template ``t`` and query token ``i``:
``template_aatype``, ``template_pseudo_beta`` (+ mask: CB, or CA for glycine), ``template_backbone_frame`` (+ mask:
rows e1, e2, e3 from N, CA, C), ``template_ca``, ``template_mask``.
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch

from . import const


@dataclasses.dataclass
class TemplateChain:
    res_names: list  # three-letter names, one per template residue
    coords: np.ndarray  # [L, 24, 3] atoms in const.RESIDUE_ATOMS order
    atom_mask: np.ndarray  # [L, 24] bool
    query_to_hit: dict  # 0-based query residue -> 0-based template residue


def _frames(n, ca, c):
    e1 = c - ca
    e1 = e1 / np.linalg.norm(e1, axis=-1, keepdims=True).clip(1e-8)
    u = n - ca
    e2 = u - e1 * (u * e1).sum(-1, keepdims=True)
    e2 = e2 / np.linalg.norm(e2, axis=-1, keepdims=True).clip(1e-8)
    return np.stack([e1, e2, np.cross(e1, e2)], axis=-2)


def template_features(query_len: int, templates: list[TemplateChain], max_templates: int = 4, token_offset: int = 0,
                      num_tokens: int | None = None) -> dict:  # fmt: skip
    """Features of up to ``max_templates`` templates for a chain occupying tokens ``[offset, offset + query_len)``."""
    n = num_tokens or query_len
    T = max_templates
    out = {
        "template_aatype": torch.full((T, n), const.RES_TYPE_ORDER["-"], dtype=torch.long),
        "template_pseudo_beta": torch.zeros(T, n, 3), "template_pseudo_beta_mask": torch.zeros(T, n),
        "template_backbone_frame": torch.eye(3).expand(T, n, 3, 3).clone(), "template_backbone_mask": torch.zeros(T, n),
        "template_ca": torch.zeros(T, n, 3), "template_mask": torch.zeros(T),
    }  # fmt: skip
    for t, tpl in enumerate(templates[:T]):
        out["template_mask"][t] = 1.0
        for q, h in tpl.query_to_hit.items():
            if not (0 <= q < query_len and 0 <= h < len(tpl.res_names)):
                continue
            i = token_offset + q
            name = tpl.res_names[h]
            out["template_aatype"][t, i] = const.RES_TYPE_ORDER.get(name, const.RES_TYPE_ORDER["UNK"])
            atoms = const.RESIDUE_ATOMS.get(name, const.RESIDUE_ATOMS["UNK"])
            xyz, ok = tpl.coords[h], tpl.atom_mask[h]
            idx = {a: k for k, a in enumerate(atoms)}
            if all(a in idx and ok[idx[a]] for a in ("N", "CA", "C")):
                fr = _frames(xyz[idx["N"]], xyz[idx["CA"]], xyz[idx["C"]])
                out["template_backbone_frame"][t, i] = torch.as_tensor(fr, dtype=torch.float32)
                out["template_backbone_mask"][t, i] = 1.0
                out["template_ca"][t, i] = torch.as_tensor(xyz[idx["CA"]], dtype=torch.float32)
            pb = "CB" if ("CB" in idx and ok[idx["CB"]]) else "CA"
            if pb in idx and ok[idx[pb]]:
                out["template_pseudo_beta"][t, i] = torch.as_tensor(xyz[idx[pb]], dtype=torch.float32)
                out["template_pseudo_beta_mask"][t, i] = 1.0
    return out


# ---------------------------------------------------------------------------------------------------------------
# template hits from files (reference: data/parse/templates.py:85-125 CIGAR pairs, :730-760 mmCIF hits,
# :911-990 the JSON hit lists that accompany prediction jobs)
# ---------------------------------------------------------------------------------------------------------------
def cigar_to_index_pairs(cigar: str, query_start: int, target_start: int) -> tuple[list[int], list[int]]:
    """CIGAR of an m8 hit (1-based starts) -> parallel 0-based ``(query indices, template indices)`` of matches."""
    import re

    q, t = query_start - 1, target_start - 1
    qi, ti = [], []
    for count, op in re.findall(r"(\d+)([MIDX=])", cigar):
        n = int(count)
        if op in "MX=":
            qi.extend(range(q, q + n)), ti.extend(range(t, t + n))
            q, t = q + n, t + n
        elif op == "I":  # present in the query only
            q += n
        else:  # "D": present in the target only
            t += n
    return qi, ti


def parse_m8(text: str) -> list[dict]:
    """Rows of an mmseqs ``.m8`` file with a trailing CIGAR column -> ``[{name, chainId, queryIndices, templateIndices,
    identity, evalue}]`` in file order."""
    hits = []
    for line in text.splitlines():
        f = line.split("\t")
        if len(f) < 13:
            continue
        qi, ti = cigar_to_index_pairs(f[12], int(f[6]), int(f[8]))
        pdb, _, chain = f[1].partition("_")
        hits.append({"name": f[1], "pdb_id": pdb.lower(), "chainId": chain, "queryIndices": qi, "templateIndices": ti,
                     "identity": float(f[2]), "evalue": float(f[10])})  # fmt: skip
    return hits


def reconcile_hit_with_chain(mapping: dict[int, int], hit_sequence: str, hit_start: int, chain_sequence: str,
                             min_identity: float = 0.5) -> dict[int, int] | None:  # fmt: skip
    """Move a query -> target mapping from the sequence the search database holds to the sequence of the structure file.

    Search tools align against a sequence database built from deposited SEQRES records; the structure file read later
    may be a newer revision of the entry (residues added or removed at the ends, a corrected stretch), so a target
    position of the hit need not be the same position of the chain. ``hit_sequence`` is the ungapped target residues of
    the hit, the first of them at position ``hit_start`` (0-based) of the database sequence; ``mapping`` values count
    positions of that database sequence. The hit residues are aligned to ``chain_sequence`` by longest common blocks:
    positions inside a common block and inside an equally long substituted stretch are carried over, positions the
    chain does not have are dropped. When the hit already sits at ``hit_start`` in the chain the mapping comes back
    unchanged. ``None`` when fewer than ``min_identity`` of the hit's residues find their residue in the chain (the
    wrong chain or entry). Same purpose as the reference's gap-insertion realignment
    (data/parse/template_realign.py:21-163), which assumes the structure only loses residues relative to SEQRES.
    """
    import difflib

    if chain_sequence[hit_start : hit_start + len(hit_sequence)] == hit_sequence:
        return dict(mapping)
    moved, same = {}, 0
    for op, a0, a1, b0, b1 in difflib.SequenceMatcher(None, hit_sequence, chain_sequence, autojunk=False).get_opcodes():
        if op == "equal" or (op == "replace" and a1 - a0 == b1 - b0):
            same += (a1 - a0) if op == "equal" else 0
            for k in range(a1 - a0):
                moved[hit_start + a0 + k] = b0 + k
    if not hit_sequence or same < min_identity * len(hit_sequence):
        return None
    return {q: moved[t] for q, t in mapping.items() if t in moved}


def template_chain_from_mmcif(path: str, chain_id: str | None, query_indices, template_indices,
                              hit_sequence: str | None = None, hit_start: int | None = None) -> TemplateChain | None:  # fmt: skip
    """One hit: ``template_indices`` count positions of the chain's full (SEQRES) sequence, 0-based.

    ``chain_id`` is matched against author chain names first, then label names; ``None`` takes the first protein chain.
    Only protein chains give templates. Returns ``None`` when the chain is absent. With ``hit_sequence`` (the hit's
    ungapped target residues, starting at ``hit_start``, default the smallest template index) the indices are first
    reconciled with the chain's own sequence (``reconcile_hit_with_chain``); a hit that does not fit the chain is dropped.
    """
    from .parse.mmcif import parse_mmcif

    st, rec = parse_mmcif(path, use_assembly=False)
    pick = None
    for ci in rec.chains:
        if ci.mol_type != const.MOL_PROTEIN:
            continue
        if chain_id is None or ci.auth_chain_name == chain_id or ci.chain_name == chain_id:
            pick = ci
            break
    if pick is None:
        return None
    c = st.chains[pick.chain_id]
    res = st.residues[int(c["res_idx"]) : int(c["res_idx"]) + int(c["res_num"])]
    L, A = len(res), const.MAX_ATOMS_PER_TOKEN
    coords, mask, names = np.zeros((L, A, 3), np.float32), np.zeros((L, A), bool), []
    xyz = st.coords()
    for k, r in enumerate(res):
        name = const.RES_TYPE_INDEX_TO_NAME.get(int(r["res_type"]), "UNK")
        names.append(name)
        a0, n = int(r["atom_idx"]), int(r["atom_num"])
        atoms = st.atoms[a0 : a0 + n]
        if bool(r["is_standard"]):
            m = min(n, A)
            coords[k, :m], mask[k, :m] = xyz[a0 : a0 + m], atoms["is_present"][:m]
            continue
        order = {a: j for j, a in enumerate(const.RESIDUE_ATOMS.get(name, const.RESIDUE_ATOMS["UNK"]))}
        for j, a in enumerate(atoms):  # modified residue: copy the atoms its parent also has
            slot = order.get(a["name"].decode().strip())
            if slot is not None and a["is_present"]:
                coords[k, slot], mask[k, slot] = xyz[a0 + j], True
    mapping = {int(q): int(t) for q, t in zip(query_indices, template_indices)}
    if hit_sequence and mapping:
        letters = "".join(const.PROTEIN_3TO1.get(nm, "X") for nm in names)
        start = min(mapping.values()) if hit_start is None else int(hit_start)
        mapping = reconcile_hit_with_chain(mapping, hit_sequence.replace("-", "").upper(), start, letters)
        if not mapping:
            return None
    return TemplateChain(names, coords, mask, mapping)


def load_json_templates(entries: list[dict], base_dir: str = ".", max_templates: int = 4, mmcif_dir: str | None = None,
                        max_date: str | None = None) -> list[TemplateChain]:
    """Hit list of a prediction job: ``[{"name" | "mmcifPath": file, "chainId", "queryIndices", "templateIndices"}]``;
    with ``"templateSequence"`` (the target residues the search tool aligned, optionally ``"templateSequenceStart"``)
    the indices are reconciled with the sequence of the structure file. An entry may instead carry the file's text under ``"mmcif"``, or only a ``"pdbId"`` that is looked up in the local
    mmCIF mirror ``mmcif_dir``. With ``max_date`` (YYYY-MM-DD) a hit released later is dropped: the entry's
    ``"releaseDate"`` decides when present, else the release date in the structure file; a hit whose date cannot be
    determined is kept. Unreadable hits are skipped."""
    import os
    import tempfile

    out = []
    for e in entries:
        if len(out) >= max_templates:
            break
        path = e.get("mmcifPath") or e.get("name")
        tmp = None
        if "mmcif" in e and e["mmcif"]:
            tmp = tempfile.NamedTemporaryFile("w", suffix=".cif", delete=False)
            tmp.write(e["mmcif"]), tmp.close()
            path = tmp.name
        elif path and not os.path.isabs(path):
            path = os.path.join(base_dir, path)
        elif not path and e.get("pdbId") and mmcif_dir:
            path = find_pdb_mmcif(str(e["pdbId"]), mmcif_dir)
        try:
            if path and os.path.exists(path):
                if max_date and not e.get("releaseDate"):
                    from .parse.mmcif import parse_mmcif

                    released = getattr(parse_mmcif(path, use_assembly=False)[1].structure_info, "released", None)
                    if released and str(released)[:10] > max_date:
                        continue
                hit = template_chain_from_mmcif(path, e.get("chainId"), e["queryIndices"], e["templateIndices"],
                                                e.get("templateSequence"), e.get("templateSequenceStart"))
                if hit is not None:
                    out.append(hit)
        except (ValueError, KeyError, IndexError):
            pass
        finally:
            if tmp is not None:
                os.unlink(tmp.name)
    return out


# ---------------------------------------------------------------------------------------------------------------
# template preparation for prediction jobs and a per-chain coordinate cache
# (reference: scripts/prepare_templates.py, scripts/build_pdb_cache.py, data/parse/pdb_chain_cache.py)
# ---------------------------------------------------------------------------------------------------------------
def find_pdb_mmcif(pdb_id: str, root: str) -> str | None:
    """``root/<id>.cif[.gz]`` or the wwPDB divided layout ``root/<middle two characters>/<id>.cif[.gz]``."""
    import os

    pid = pdb_id.lower()
    for base in (root, os.path.join(root, pid[1:3])):
        for ext in (".cif", ".cif.gz"):
            path = os.path.join(base, pid + ext)
            if os.path.exists(path):
                return path
    return None


def save_template_chain(chain: TemplateChain, path: str) -> None:
    np.savez_compressed(path, res_names=np.array(chain.res_names), coords=chain.coords.astype(np.float32), atom_mask=chain.atom_mask)


def load_template_chain(path: str, query_indices, template_indices) -> TemplateChain:
    z = np.load(path)
    return TemplateChain([str(x) for x in z["res_names"]], z["coords"], z["atom_mask"],
                         {int(q): int(t) for q, t in zip(query_indices, template_indices)})  # fmt: skip


def build_chain_cache(mmcif_dir: str, out_dir: str, limit: int = 0) -> int:
    """One ``<pdb>_<chain>.npz`` (residue names, dense atom coordinates, mask) per protein chain of every entry."""
    import os

    from .parse.mmcif import parse_mmcif
    from .prepare.pipeline import find_mmcif_files

    os.makedirs(out_dir, exist_ok=True)
    n = 0
    for path in find_mmcif_files(mmcif_dir)[: limit or None]:
        try:
            _st, rec = parse_mmcif(path, use_assembly=False)
        except Exception:  # noqa: BLE001 - unreadable entries are skipped
            continue
        for ci in rec.chains:
            if ci.mol_type != const.MOL_PROTEIN:
                continue
            chain = template_chain_from_mmcif(path, ci.auth_chain_name or ci.chain_name, [], [])
            if chain is not None:
                save_template_chain(chain, os.path.join(out_dir, f"{rec.id}_{ci.auth_chain_name or ci.chain_name}.npz"))
                n += 1
    return n


def prepare_job_templates(m8_text: str, mmcif_dir: str, out_dir: str, index: int = 0, max_templates: int = 4,
                          max_release_date: str | None = None, min_aligned: int = 10, query_length: int | None = None) -> list[dict]:  # fmt: skip
    """Hits of one query -> ``out_dir/templates_<index>.json`` plus a copy of each hit's mmCIF next to it.

    Hits are taken in file order (best first). A hit is skipped when its entry is missing, released after
    ``max_release_date`` (entries without a date are skipped when a cut-off is set), aligned over fewer than
    ``min_aligned`` positions, or repeats an entry and chain already taken.
    """
    import json
    import os
    import shutil

    from .parse.mmcif import read_structure_info

    os.makedirs(out_dir, exist_ok=True)
    taken, seen = [], set()
    for hit in parse_m8(m8_text):
        if len(taken) >= max_templates:
            break
        key = (hit["pdb_id"], hit["chainId"])
        if key in seen or len(hit["queryIndices"]) < min_aligned:
            continue
        if query_length is not None and max(hit["queryIndices"], default=0) >= query_length:
            continue
        src = find_pdb_mmcif(hit["pdb_id"], mmcif_dir)
        if src is None:
            continue
        if max_release_date is not None:
            info = read_structure_info(src)
            if info is None or info.released is None or info.released > max_release_date:
                continue
        if template_chain_from_mmcif(src, hit["chainId"], hit["queryIndices"], hit["templateIndices"]) is None:
            continue
        seen.add(key)
        name = f"{hit['pdb_id']}_{hit['chainId']}.cif" + (".gz" if src.endswith(".gz") else "")
        shutil.copyfile(src, os.path.join(out_dir, name))
        taken.append({"name": name, "chainId": hit["chainId"], "queryIndices": hit["queryIndices"], "templateIndices": hit["templateIndices"]})
    with open(os.path.join(out_dir, f"templates_{index}.json"), "w") as f:
        json.dump(taken, f)
    return taken


# ---------------------------------------------------------------------------------------------------------------
# templates of training examples (reference: data/module/dataset.py:748-900, data/prepare/template_search.py:110-216,
# :504-509): per-sequence hit lists prepared once, filtered and sampled per example at load time
# ---------------------------------------------------------------------------------------------------------------
def monomer_template_index(root: str, msa_id: str) -> str | None:
    """The hit list of a sequence: ``<root>/monomer_templates/<first two characters>/<msa_id>.json`` (the reference's
    sharded layout) or ``<root>/templates/<msa_id>.json``; ``None`` when neither exists."""
    from . import io_cache

    import os

    key = str(msa_id)
    shard = key[:2].lower() if len(key) >= 2 else "__"
    for path in (os.path.join(root, "monomer_templates", shard, f"{key}.json"), os.path.join(root, "templates", f"{key}.json")):
        if io_cache.exists(path):
            return path
    return None


def passes_hit_filters(hit: dict, query_length: int, max_subsequence_ratio: float = 0.95, min_hit_length: int = 10,
                       min_align_ratio: float = 0.1) -> bool:  # fmt: skip
    """AF3 SI 2.4 per-hit filters on an m8-style hit (1-based ``qstart qend tstart tend``, ``identity`` 0..1): the
    template span has at least ``min_hit_length`` residues, the alignment covers at least ``min_align_ratio`` of the
    query, and a near-identical hit (>= 0.99) spanning more than ``max_subsequence_ratio`` of the query is a copy of
    the query and is dropped."""
    span = int(hit["tend"]) - int(hit["tstart"]) + 1
    aligned = int(hit["qend"]) - int(hit["qstart"]) + 1
    q = max(int(query_length), 1)
    if span < min_hit_length or aligned / q < min_align_ratio:
        return False
    return not (span / q > max_subsequence_ratio and float(hit.get("identity", 0.0)) >= 0.99)


def template_cutoff(released: str | None, cutoff_days: int = 60, max_template_date: str | None = None,
                    default_cutoff: str | None = None) -> str | None:  # fmt: skip
    """Latest template release date an example may see: ``min(max_template_date, released - cutoff_days)``; an example
    without a release date falls back to ``default_cutoff``. ``None`` means that no bound can be established, and the
    caller must then use no template at all (a template newer than the example would leak its answer)."""
    import datetime

    per_record = default_cutoff
    if released:
        try:
            per_record = (datetime.date.fromisoformat(str(released)[:10]) - datetime.timedelta(days=cutoff_days)).isoformat()
        except ValueError:
            pass
    if per_record is None:
        return max_template_date
    return per_record if max_template_date is None else min(max_template_date, per_record)


def sample_training_templates(hits: list[dict], record_id: str, cutoff: str | None, rng, max_templates: int = 4) -> list[dict]:
    """Hits a training example may use: not the example's own entry, released (with a known date) on or before
    ``cutoff``; then ``k = min(Uniform{0..n}, max_templates)`` of them drawn without replacement (AF3 SI 2.4). Accepts
    the reference's hit records (``template_pdb_id``, ``template_chain_id``, ``release_date``) and this package's
    (``pdbId``, ``chainId``, ``releaseDate``)."""
    if cutoff is None:
        return []
    own = str(record_id).upper()
    ok = []
    for h in hits:
        pdb = str(h.get("template_pdb_id") or h.get("pdbId") or "").upper()
        date = h.get("release_date") or h.get("releaseDate")
        if pdb and pdb != own and date and str(date)[:10] <= cutoff:
            ok.append(h)
    k = min(rng.randint(0, len(ok)), max_templates) if ok else 0
    return rng.sample(ok, k) if k else []


def hit_index_pairs(hit: dict) -> tuple[list[int], list[int]]:
    """0-based (query, template) index lists of a hit: explicit lists, or a CIGAR string with 1-based starts."""
    if "queryIndices" in hit:
        return list(hit["queryIndices"]), list(hit["templateIndices"])
    return cigar_to_index_pairs(hit["cigar"], int(hit["qstart"]), int(hit["tstart"]))


def chain_cache_path(cache_dir: str, pdb_id: str, chain_id: str) -> str | None:
    """``<cache>/<pdb>_<chain>.npz``, flat or under a two-character shard directory, in either letter case of the id."""
    import os

    for pdb in (pdb_id.lower(), pdb_id.upper()):
        name = f"{pdb}_{chain_id}.npz"
        for path in (os.path.join(cache_dir, name), os.path.join(cache_dir, pdb[1:3].lower(), name), os.path.join(cache_dir, pdb[:2].lower(), name)):
            if os.path.exists(path):
                return path
    return None


def build_monomer_template_index(data_dir: str, m8_dir: str, release_dates: dict[str, str], lengths: dict[str, int] | None = None,
                                 max_hits: int = 20, log=None) -> tuple[int, int]:
    """``<m8_dir>/<msa_id>.m8`` (template search results per distinct sequence, 13 columns with CIGAR) ->
    ``<data_dir>/monomer_templates/<shard>/<msa_id>.json``: the hits that pass the AF3 per-hit filters, best first, at
    most ``max_hits`` per sequence, each with the release date of its entry (``release_dates``: entry id -> date; hits
    of unknown date are written with ``null`` and never used in training). The date cut-off itself is applied per
    example when it is loaded, because one sequence occurs in examples of different dates. Returns ``(sequences
    written, hits written)`` (reference: data/prepare/template_search.py:181-216, :440-503)."""
    import json
    import os

    written = total = 0
    dates = {k.lower(): v for k, v in release_dates.items()}
    for name in sorted(os.listdir(m8_dir)):
        if not name.endswith(".m8"):
            continue
        msa_id = name[:-3]
        with open(os.path.join(m8_dir, name)) as f:
            rows = [line.rstrip("\n").split("\t") for line in f if line.strip()]
        hits = []
        for r in rows:
            if len(r) < 13:
                continue
            pdb, _, chain = r[1].partition("_")
            hit = {"template_pdb_id": pdb.lower(), "template_chain_id": chain or "A", "identity": float(r[2]), "evalue": float(r[10]),
                   "qstart": int(r[6]), "qend": int(r[7]), "tstart": int(r[8]), "tend": int(r[9]), "cigar": r[12],
                   "release_date": dates.get(pdb.lower()), "index_space": "seqres"}  # fmt: skip
            qlen = (lengths or {}).get(msa_id, hit["qend"])
            if passes_hit_filters(hit, qlen):
                hits.append(hit)
            if len(hits) >= max_hits:
                break
        if not hits:
            continue
        shard = msa_id[:2].lower() if len(msa_id) >= 2 else "__"
        out = os.path.join(data_dir, "monomer_templates", shard)
        os.makedirs(out, exist_ok=True)
        with open(os.path.join(out, f"{msa_id}.json"), "w") as f:
            json.dump(hits, f)
        written, total = written + 1, total + len(hits)
    if log:
        log(f"{written} sequences, {total} template hits -> {os.path.join(data_dir, 'monomer_templates')}")
    return written, total
