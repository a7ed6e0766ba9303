"""Dataset maintenance commands around a prepared training directory.

Reference: scripts/prepare.py:554-1615 (``fetch-ccd``, ``build-ccd-cache``, ``export-complexes``, ``import-of3``,
``import-msa``, ``import-paired-msa``, ``enrich-manifest``, ``drop-obsolete``, ``build-of3-cache``,
``stamp-template-index-space``), scripts/pack.py, scripts/build_masks.py, scripts/refilter.py and
scripts/warmup_triton.py. The commands keep the reference's names and options; what they do is stated on this
package's own data layer (``data/types.py`` records, ``data/paths.py`` layout).
"""

from __future__ import annotations

import glob
import gzip
import json
import os
import shutil

import click
import numpy as np

from ..data import paths


def _load(data_dir):
    from ..data.types import load_manifest

    path = paths.manifest(data_dir)
    if not os.path.exists(path):
        raise click.ClickException(f"{path} not found: run `prepare structures` first")
    return path, load_manifest(path)


def _chain_sequences(data_dir, records):
    """``{msa_id: (one-letter sequence, mol_type)}`` of every polymer chain, read from the stored structures."""
    from ..data import const
    from ..data.types import Structure

    out = {}
    for rec in records:
        want = {c.chain_id: c for c in rec.chains if c.mol_type != const.MOL_NONPOLYMER and c.msa_id not in out}
        if not want:
            continue
        st = Structure.load(paths.structure(data_dir, rec.id))
        seqs = st.chain_canonical_seqs or {}
        for chain_id, c in want.items():
            if chain_id in seqs:
                out[c.msa_id] = (seqs[chain_id], c.mol_type)
    return out


# --------------------------------------------------------------------------------------------------------- chemical components
@click.command("fetch-ccd")
@click.option("--output", required=True, type=click.Path(), help="Directory to save components.cif.gz in.")
@click.option("--from-file", type=click.Path(exists=True), default=None, help="Copy a local components.cif[.gz] instead of downloading.")
@click.option("--url", default="https://files.wwpdb.org/pub/pdb/data/monomers/components.cif.gz", show_default=True)
def fetch_ccd(output, from_file, url):
    """Get the wwPDB chemical component dictionary (about 100 MB) for `build-ccd-cache`."""
    os.makedirs(output, exist_ok=True)
    if from_file:
        dst = os.path.join(output, os.path.basename(from_file))
        shutil.copyfile(from_file, dst)
    else:
        import urllib.request

        dst = os.path.join(output, "components.cif.gz")
        try:
            with urllib.request.urlopen(url, timeout=60) as r, open(dst + ".part", "wb") as f:
                shutil.copyfileobj(r, f)
        except OSError as exc:
            raise click.ClickException(f"download failed ({exc}); fetch the file elsewhere and pass --from-file") from exc
        os.replace(dst + ".part", dst)
    click.echo(f"CCD components saved to: {dst}")


@click.command("build-ccd-cache")
@click.option("--components-cif", required=True, type=click.Path(exists=True))
@click.option("--output", required=True, type=click.Path(), help="JSON cache to write.")
@click.option("--ref-pos", is_flag=True, help="ETKDG reference conformers (needs RDKit).")
@click.option("--automorphisms", is_flag=True, help="Heavy-atom graph automorphisms of every ligand.")
@click.option("--workers", default=1, type=int)
def build_ccd_cache(components_cif, output, ref_pos, automorphisms, workers):
    """One JSON with every component's atoms, ideal coordinates, charges, leaving atoms and bonds; with
    --automorphisms also the atom permutations the ligand-permutation loss uses (graph search, no RDKit)."""
    from ..data.ccd import export_table

    if ref_pos:
        try:
            import rdkit  # noqa: F401
        except ImportError as exc:
            raise click.ClickException("--ref-pos generates conformers with RDKit, which is not installed; the cache "
                                       "keeps the dictionary's ideal coordinates without it") from exc
    n = export_table(components_cif, output, None)
    if automorphisms:
        from ..data.symmetry import graph_automorphisms

        with open(output) as f:
            table = json.load(f)
        for comp in table.values():
            heavy = [i for i, e in enumerate(comp["elements"]) if e != 1]
            if not 1 < len(heavy) <= 64:
                continue
            index = {a: k for k, a in enumerate(heavy)}
            bonds = [(index[a], index[b], o) for a, b, o in comp["bonds"] if a in index and b in index]
            perms = graph_automorphisms([comp["elements"][i] for i in heavy], [(a, b) for a, b, _ in bonds], limit=1000,
                                        orders=[o for _, _, o in bonds])  # fmt: skip
            if len(perms) > 1:
                comp["heavy_atoms"] = [comp["atoms"][i] for i in heavy]
                comp["automorphisms"] = perms
        with open(output, "w") as f:
            json.dump(table, f)
    click.echo(f"{n} components -> {output}")


# --------------------------------------------------------------------------------------------------------- manifest tools
@click.command("export-complexes")
@click.option("--data-dir", required=True, type=click.Path(exists=True))
@click.option("--output", required=True, type=click.Path())
@click.option("--all-mol-types", is_flag=True, help="Include nucleic-acid chains, not just proteins.")
def export_complexes(data_dir, output, all_mol_types):
    """``{record id: [sequence, ...]}`` of every record with more than one qualifying chain (input of paired-MSA searches)."""
    from ..data import const

    _, records = _load(data_dir)
    seqs = _chain_sequences(data_dir, records)
    out = {}
    for rec in records:
        keep = [seqs[c.msa_id][0] for c in rec.chains
                if c.msa_id in seqs and (all_mol_types or c.mol_type == const.MOL_PROTEIN)]  # fmt: skip
        if len(keep) > 1:
            out[rec.id] = keep
    with open(output, "w") as f:
        json.dump(out, f)
    click.echo(f"{len(out)} complexes -> {output}")


def _query_of(a3m_path):
    opener = gzip.open if a3m_path.endswith(".gz") else open
    with opener(a3m_path, "rt") as f:
        seq = []
        for line in f:
            if line.startswith(">"):
                if seq:
                    break
                continue
            if line.startswith("#"):
                continue
            seq.append(line.strip())
    return "".join(ch for ch in "".join(seq) if ch.isupper() or ch == "-").replace("-", "")


def _store_alignment(src, dst_base, mol_type, keep_a3m):
    from ..data.parse.a3m import msa_from_a3m_file

    if os.path.exists(dst_base + ".npz"):
        return False
    os.makedirs(os.path.dirname(dst_base), exist_ok=True)
    msa_from_a3m_file(src, mol_type).save(dst_base + ".npz")
    if keep_a3m:
        shutil.copyfile(src, dst_base + ".a3m")
    return True


@click.command("import-msa")
@click.option("--data-dir", required=True, type=click.Path(exists=True))
@click.option("--msa-dir", required=True, type=click.Path(exists=True), help="A3M files, any naming, scanned recursively.")
@click.option("--workers", default=1, type=int, show_default=True)
@click.option("--keep-a3m", is_flag=True)
def import_msa(data_dir, msa_dir, workers, keep_a3m):
    """Attach existing A3M files to the chains whose sequence equals the file's query; writes msa/<msa_id>.npz."""
    _, records = _load(data_dir)
    by_seq = {}
    for msa_id, (seq, mol_type) in _chain_sequences(data_dir, records).items():
        by_seq.setdefault(seq, []).append((msa_id, mol_type))
    files = [p for p in glob.glob(os.path.join(msa_dir, "**", "*.a3m*"), recursive=True) if os.path.isfile(p)]
    jobs = []
    for path in files:
        for msa_id, mol_type in by_seq.get(_query_of(path), ()):
            jobs.append((path, os.path.join(data_dir, "msa", str(msa_id)), mol_type, keep_a3m))
    if workers > 1 and len(jobs) > 1:
        from concurrent.futures import ProcessPoolExecutor

        with ProcessPoolExecutor(workers) as pool:
            written = sum(pool.map(_store_alignment, *zip(*jobs)))
    else:
        written = sum(_store_alignment(*j) for j in jobs)
    click.echo(f"{len(files)} alignments scanned, {len(jobs)} matched a chain, {written} written")


@click.command("import-paired-msa")
@click.option("--data-dir", required=True, type=click.Path(exists=True))
@click.option("--paired-dir", required=True, type=click.Path(exists=True), help="<record id>/<msa_id>.paired.a3m")
@click.option("--workers", default=1, type=int, show_default=True)
@click.option("--keep-a3m", is_flag=True)
def import_paired_msa(data_dir, paired_dir, workers, keep_a3m):
    """Attach paired alignments made outside: rows of msa_paired/<record id>/<msa_id>.npz pair up across the chains of a record."""
    path, records = _load(data_dir)
    written = touched = 0
    for rec in records:
        src_dir = os.path.join(paired_dir, rec.id)
        if not os.path.isdir(src_dir):
            continue
        for c in rec.chains:
            src = os.path.join(src_dir, f"{c.msa_id}.paired.a3m")
            if not os.path.exists(src):
                continue
            key = f"{rec.id}/{c.msa_id}"
            written += _store_alignment(src, os.path.join(data_dir, "msa_paired", key), c.mol_type, keep_a3m)
            if c.paired_msa_id != key:
                c.paired_msa_id, touched = key, touched + 1
    if touched:
        from ..data.types import save_manifest

        save_manifest(records, path)
    click.echo(f"{written} paired alignments written, {touched} chains pointed at them")


def _read_entries_idx(path):
    """wwPDB entries.idx: IDCODE, HEADER, ACCESSION DATE (mm/dd/yy), COMPOUND, SOURCE, AUTHORS, RESOLUTION, EXPERIMENT TYPE."""
    out = {}
    with open(path, errors="replace") as f:
        for line in f:
            cols = line.rstrip("\n").split("\t")
            if len(cols) < 8 or len(cols[0]) != 4:
                continue
            date = None
            parts = cols[2].split("/")
            if len(parts) == 3 and all(p.isdigit() for p in parts):
                mm, dd, yy = (int(p) for p in parts)
                date = f"{(1900 if yy >= 70 else 2000) + yy:04d}-{mm:02d}-{dd:02d}"
            try:
                res = float(cols[6].split(",")[0])
            except ValueError:
                res = None
            out[cols[0].lower()] = {"resolution": res, "method": cols[7].strip() or None, "deposited": date}
    return out


@click.command("enrich-manifest")
@click.option("--data-dir", required=True, type=click.Path(exists=True))
@click.option("--idx", type=click.Path(exists=True), default=None, help="wwPDB derived_data/index/entries.idx")
@click.option("--mmcif-cache", type=click.Path(exists=True), default=None, help="JSON written by `scan-mmcif`.")
def enrich_manifest(data_dir, idx, mmcif_cache):
    """Fill blank resolution / method / deposited / released fields of the manifest; fields already set are kept."""
    from ..data.types import StructureInfo, save_manifest

    if not idx and not mmcif_cache:
        raise click.ClickException("give --idx and/or --mmcif-cache")
    sources = []
    if idx:
        sources.append(_read_entries_idx(idx))
    if mmcif_cache:
        with open(mmcif_cache) as f:
            rows = json.load(f)
        rows = rows.values() if isinstance(rows, dict) else rows
        sources.append({str(r["id"]).lower(): r for r in rows if "id" in r})
    path, records = _load(data_dir)
    filled = 0
    for rec in records:
        info = rec.structure_info or StructureInfo()
        for table in sources:
            row = table.get(rec.id.lower()[:4]) or table.get(rec.id.lower())
            if not row:
                continue
            for field in ("resolution", "method", "deposited", "released"):
                if getattr(info, field) in (None, "") and row.get(field) not in (None, ""):
                    setattr(info, field, row[field])
                    filled += 1
        rec.structure_info = info
    save_manifest(records, path)
    click.echo(f"{filled} fields filled in {len(records)} records")


@click.command("drop-obsolete")
@click.option("--data-dir", required=True, type=click.Path(exists=True))
@click.option("--ids-file", type=click.Path(exists=True), default=None, help="obsolete.dat or a JSON list of ids (default: download).")
@click.option("--delete-files", is_flag=True, help="Also delete the dropped records' structure / mask files.")
def drop_obsolete(data_dir, ids_file, delete_files):
    """Remove records whose PDB entry has been made obsolete."""
    from ..data.types import save_manifest

    if ids_file:
        with open(ids_file) as f:
            text = f.read()
    else:
        import urllib.request

        try:
            with urllib.request.urlopen("https://files.wwpdb.org/pub/pdb/data/status/obsolete.dat", timeout=60) as r:
                text = r.read().decode()
        except OSError as exc:
            raise click.ClickException(f"download failed ({exc}); pass --ids-file") from exc
    if text.lstrip().startswith("["):
        gone = {str(i).lower() for i in json.loads(text)}
    else:  # "OBSLTE    31-JUL-94 116L     216L"
        gone = {cols[2].lower() for cols in (line.split() for line in text.splitlines()) if len(cols) >= 3 and cols[0] == "OBSLTE"}
    path, records = _load(data_dir)
    keep = [r for r in records if r.id.lower()[:4] not in gone]
    dropped = [r for r in records if r.id.lower()[:4] in gone]
    save_manifest(keep, path)
    if delete_files:
        for r in dropped:
            for p in (paths.structure(data_dir, r.id), paths.mask(data_dir, r.id), paths.features(data_dir, r.id)):
                if os.path.exists(p):
                    os.remove(p)
    click.echo(f"{len(dropped)} obsolete records dropped, {len(keep)} kept")


# --------------------------------------------------------------------------------------------------------- OpenFold 3 data
@click.command("import-of3")
@click.option("--of3-dir", required=True, type=click.Path(exists=True), help="<id>/<id>.npz or flat *.npz atom arrays.")
@click.option("--output", required=True, type=click.Path())
@click.option("--cache", type=click.Path(exists=True), default=None, help="OpenFold 3 dataset_cache.json (resolution, dates).")
@click.option("--limit", type=int, default=None)
def import_of3(of3_dir, output, cache, limit):
    """Convert OpenFold 3 preprocessed structures (atom-array .npz) into this package's structures + manifest."""
    from ..data.of3 import convert_directory

    n, skipped = convert_directory(of3_dir, output, cache, limit)
    click.echo(f"{n} structures imported into {output} ({skipped} skipped)")


@click.command("build-of3-cache")
@click.option("--cache-file", required=True, type=click.Path(exists=True))
@click.option("--output", required=True, type=click.Path(), help="Directory for the columnar cache.")
@click.option("--no-templates", is_flag=True)
def build_of3_cache(cache_file, output, no_templates):
    """Turn an OpenFold 3 dataset cache JSON into memory-mappable ``.npy`` columns (one open per worker instead of one
    multi-gigabyte JSON parse per worker)."""
    from ..data.of3 import build_columnar_cache

    entries, chains = build_columnar_cache(cache_file, output, not no_templates)
    click.echo(f"{entries} entries, {chains} chains -> {output}")


@click.command("stamp-template-index-space")
@click.option("--data-dir", required=True, type=click.Path(exists=True))
@click.option("--space", type=click.Choice(["struct", "seqres"]), default="struct", show_default=True)
@click.option("--workers", default=16, type=int, show_default=True)
@click.option("--dry-run", is_flag=True)
def stamp_template_index_space(data_dir, space, workers, dry_run):
    """Record in every template index file which residue numbering its template-side positions use (positions among
    the resolved residues, or positions in the full sequence), so that the loader need not be told per dataset."""
    files = []
    for sub in ("templates", "monomer_templates"):
        files += glob.glob(os.path.join(data_dir, sub, "**", "*.json"), recursive=True)
    changed = 0
    for path in files:
        with open(path) as f:
            doc = json.load(f)
        holder = doc if isinstance(doc, dict) else None
        if holder is None:
            doc = holder = {"hits": doc}
        if holder.get("index_space") == space:
            continue
        if "index_space" in holder and holder["index_space"] != space:
            raise click.ClickException(f"{path} is already stamped {holder['index_space']!r}")
        changed += 1
        if dry_run:
            continue
        holder["index_space"] = space
        tmp = path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(doc, f)
        os.replace(tmp, path)
    click.echo(f"{len(files)} index files, {changed} {'would be ' if dry_run else ''}stamped {space!r}")


@click.command("backfill-template-dates")
@click.option("--data-dir", required=True, type=click.Path(exists=True))
@click.option("--release-dates", required=True, type=click.Path(exists=True),
              help="JSON {entry id: YYYY-MM-DD}, or the table `scan-mmcif` writes (rows with id and released).")
@click.option("--dry-run", is_flag=True)
def backfill_template_dates(data_dir, release_dates, dry_run):
    """Fill missing ``release_date`` fields of the template hit lists under DATA_DIR from a table of release dates.
    Hit lists written without dates make the fail-closed date filter drop every template in training; this edits
    the JSON in place instead of parsing the search results again."""
    with open(release_dates) as f:
        table = json.load(f)
    if isinstance(table, list):
        table = {str(r.get("id", "")): r.get("released") or r.get("release_date") for r in table if isinstance(r, dict)}
    dates = {str(k).lower(): str(v)[:10] for k, v in table.items() if v}
    files = []
    for sub in ("templates", "monomer_templates"):
        files += glob.glob(os.path.join(data_dir, sub, "**", "*.json"), recursive=True)
    filled = unknown = touched = 0
    for path in files:
        with open(path) as f:
            doc = json.load(f)
        hits = doc.get("hits", []) if isinstance(doc, dict) else doc
        changed = False
        for h in hits:
            if not isinstance(h, dict) or h.get("release_date"):
                continue
            entry = str(h.get("template_pdb_id") or h.get("pdb_id") or h.get("pdbId") or "").lower()
            if entry in dates:
                h["release_date"], changed, filled = dates[entry], True, filled + 1
            else:
                unknown += 1
        if changed:
            touched += 1
            if not dry_run:
                tmp = path + ".tmp"
                with open(tmp, "w") as f:
                    json.dump(doc, f)
                os.replace(tmp, path)
    click.echo(f"{len(files)} hit lists: {filled} dates {'would be ' if dry_run else ''}filled in {touched} files, {unknown} hits without a known date")


@click.command("msa-worklist")
@click.option("--data-dir", "data_dirs", required=True, multiple=True, type=click.Path(exists=True), help="Prepared dataset root (repeatable).")
@click.option("--output", required=True, type=click.Path(), help="Directory for combined.fasta, complexes.json, stats.json.")
def msa_worklist(data_dirs, output):
    """What is still to be searched: protein sequences of the datasets that have no alignment yet (``combined.fasta``,
    one entry per distinct sequence, named by its alignment id), and the heteromeric records whose chains lack a paired
    alignment (``complexes.json``: ``{record id: [sequence, ...]}``), with counts in ``stats.json``. The two files are
    the inputs of ``msa-batch``."""
    from ..data import const

    os.makedirs(output, exist_ok=True)
    missing, complexes = {}, {}
    stats = {"records": 0, "protein_sequences": 0, "with_alignment": 0, "heteromers": 0, "heteromers_paired": 0}
    for data_dir in data_dirs:
        _, records = _load(data_dir)
        seqs = _chain_sequences(data_dir, records)
        have = {m for m, (_, mol) in seqs.items() if mol == const.MOL_PROTEIN and paths.msa(data_dir, m) is not None}
        protein = {m for m, (_, mol) in seqs.items() if mol == const.MOL_PROTEIN}
        stats["records"] += len(records)
        stats["protein_sequences"] += len(protein)
        stats["with_alignment"] += len(have)
        for m in sorted(protein - have):
            missing.setdefault(m, seqs[m][0])
        for rec in records:
            chains = [c for c in rec.chains if c.mol_type == const.MOL_PROTEIN and c.msa_id in seqs]
            if len({c.msa_id for c in chains}) < 2:
                continue
            stats["heteromers"] += 1
            if all(getattr(c, "paired_msa_id", None) for c in chains):
                stats["heteromers_paired"] += 1
                continue
            complexes[rec.id] = [seqs[c.msa_id][0] for c in chains]
            for c in chains:  # a paired search needs the unpaired queries too
                if c.msa_id not in have:
                    missing.setdefault(c.msa_id, seqs[c.msa_id][0])
    with open(os.path.join(output, "combined.fasta"), "w") as f:
        for m, seq in missing.items():
            f.write(f">{m}\n{seq}\n")
    with open(os.path.join(output, "complexes.json"), "w") as f:
        json.dump(complexes, f)
    stats.update(sequences_to_search=len(missing), complexes_to_pair=len(complexes))
    with open(os.path.join(output, "stats.json"), "w") as f:
        json.dump(stats, f, indent=1)
    click.echo(json.dumps(stats))


# --------------------------------------------------------------------------------------------------------- packs, kernels
@click.command("pack")
@click.argument("src_dir", type=click.Path(exists=True))
@click.argument("out_dir", type=click.Path(), required=False)
@click.option("--shard-size", type=int, default=1 << 30, show_default=True, help="Bytes per tar shard.")
@click.option("--include", multiple=True, help="Pack only paths under this prefix, e.g. structures/ (repeatable).")
def pack(src_dir, out_dir, shard_size, include):
    """Bundle the files under SRC_DIR (recursively) into tar shards with a sorted index. OUT_DIR defaults to
    SRC_DIR/_pack, where the datasets find it by themselves; rerun after an interruption to continue."""
    from ..data.pack import PACK_DIRNAME, build_pack

    out_dir = out_dir or os.path.join(src_dir, PACK_DIRNAME)
    click.echo(f"{build_pack(src_dir, out_dir, shard_size, include)} files -> {out_dir}")


@click.command("pack-verify")
@click.argument("src_dir", type=click.Path(exists=True))
@click.argument("pack_dir", type=click.Path(exists=True), required=False)
@click.option("--sample", type=int, default=0, help="Check only this many files (0 = all).")
@click.option("--checksums", is_flag=True, help="Also re-hash every shard against SHA256SUMS.")
def pack_verify(src_dir, pack_dir, sample, checksums):
    """Compare the files under SRC_DIR byte for byte with what the pack returns for their paths."""
    from ..data.pack import PACK_DIRNAME, Pack, _sha256, _walk

    pack_dir = pack_dir or os.path.join(src_dir, PACK_DIRNAME)
    pk = Pack(pack_dir)
    names = _walk(src_dir, pk.include)
    total = len(names)
    if sample:
        names = names[:: max(1, len(names) // sample)][:sample]
    bad = []
    for name in names:
        with open(os.path.join(src_dir, name), "rb") as f:
            if not pk.exists(name) or pk.read_bytes(name) != f.read():
                bad.append(name)
    pk.close()
    if bad:
        raise click.ClickException(f"{len(bad)} of {len(names)} files differ or are missing, first: {bad[:5]}")
    if not pk.legacy and not sample and len(pk) != total:
        raise click.ClickException(f"the pack holds {len(pk)} files, the source {total}")
    if checksums and os.path.exists(os.path.join(pack_dir, "SHA256SUMS")):
        with open(os.path.join(pack_dir, "SHA256SUMS")) as f:
            for line in f:
                digest, rel = line.split()
                if _sha256(os.path.join(pack_dir, rel)) != digest:
                    raise click.ClickException(f"{rel}: checksum mismatch")
    click.echo(f"{len(names)} files verified")


@click.command("warmup-kernels")
@click.option("--tokens", type=int, multiple=True, default=(384,), help="Token counts to run the pair-shaped kernels at.")
@click.option("--build/--no-build", default=True, help="Compile the extension first if it is stale.")
def warmup_kernels(tokens, build):
    """Build (if needed) and load the sm_100a extension and run each kernel family once per token count, so that the
    first training step or prediction pays no one-time cost (the reference's `warmup-triton` autotunes its Triton
    kernels at this point; these kernels have nothing to tune)."""
    import torch

    from ..ops import build as ops_build
    from ..ops import native

    if build:
        click.echo(ops_build.build())
    nat = native.require()
    if not torch.cuda.is_available():
        raise click.ClickException("no CUDA device")
    from .. import ops

    for n in tokens:
        z = torch.randn(1, n, n, 128, device="cuda").bfloat16()
        mask = torch.ones(1, n, n, device="cuda")
        w = torch.randn(256, 128, device="cuda") * 0.05
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            z0 = ops.layer_norm(z, None, None)
            ops.triangle_contract_norm(z0, w, w, mask, True, None, None)
            ops.sigmoid_gate_mul(z0, w[:128], z0)
            bias = ops.head_bias_planes(z0, w[:4])
            qkv = ops.stacked_linear(z0, w[:128], w[:128], w[:128]).view(1, n, n, 3, 4, 32)
            ops.grid_attention(qkv, bias, mask, 32**-0.5, False)
            ops.transition(z, None, None, torch.randn(1024, 128, device="cuda") * 0.05, torch.randn(128, 512, device="cuda") * 0.05)
        torch.cuda.synchronize()
        click.echo(f"{n} tokens: ok")
    nat.check_status()
    click.echo(json.dumps(ops.census(), indent=1))


COMMANDS = (fetch_ccd, build_ccd_cache, export_complexes, import_msa, import_paired_msa, enrich_manifest, drop_obsolete,
            import_of3, build_of3_cache, stamp_template_index_space, backfill_template_dates, msa_worklist, pack, pack_verify,
            warmup_kernels)
