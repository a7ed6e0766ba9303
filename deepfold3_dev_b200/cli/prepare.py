"""``prepare`` command group and the dataset-inspection commands.

Reference: scripts/prepare.py:316-1546 (sub-commands ``structures``, ``filter``, ``cluster``, ``msa`` ...),
scripts/scan_mmcif.py, scripts/refilter.py, scripts/inspect_example.py, scripts/build_masks.py, scripts/pack.py.
"""

from __future__ import annotations

import json
import os

import click


@click.group()
def prepare():
    """Turn mmCIF archives into training examples: structures -> filter -> cluster -> features -> pack."""


def _filter_cfg(max_resolution, max_release_date, min_release_date, max_chains, max_unk_fraction, max_tight_clashes):
    from ..data.prepare import StructureFilterConfig

    return StructureFilterConfig(max_resolution=max_resolution, max_release_date=max_release_date,
                                 min_release_date=min_release_date, max_chains=max_chains,
                                 max_unk_fraction=max_unk_fraction, max_tight_clashes=max_tight_clashes)  # fmt: skip


_FILTER_OPTIONS = [
    click.option("--max-resolution", type=float, default=9.0),
    click.option("--max-release-date", default=None, help="YYYY-MM-DD; entries without a date fail this filter."),
    click.option("--min-release-date", default=None),
    click.option("--max-chains", type=int, default=300),
    click.option("--max-unk-fraction", type=float, default=None),
    click.option("--max-tight-clashes", type=int, default=None),
]


def _with(options):
    def deco(f):
        for o in reversed(options):
            f = o(f)
        return f

    return deco


@prepare.command("structures")
@click.argument("mmcif_dir", type=click.Path(exists=True))
@click.argument("out_dir", type=click.Path())
@click.option("--workers", type=int, default=max(1, (os.cpu_count() or 2) // 2))
@click.option("--no-assembly", is_flag=True, help="Keep the asymmetric unit instead of biological assembly 1.")
@click.option("--limit", type=int, default=0)
@_with(_FILTER_OPTIONS)
def structures(mmcif_dir, out_dir, workers, no_assembly, limit, **filt):
    """Parse and filter every mmCIF under MMCIF_DIR; writes structures/*.npz, manifest.json, sequences.fasta."""
    from ..data.prepare import prepare_directory

    counts = prepare_directory(mmcif_dir, out_dir, _filter_cfg(**filt), workers, not no_assembly, limit)
    click.echo(json.dumps(counts))


@prepare.command("ccd-table")
@click.argument("components_cif", type=click.Path(exists=True))
@click.argument("out_json", type=click.Path())
@click.option("--code", "codes", multiple=True, help="Only these component codes (default: all).")
def ccd_table(components_cif, out_json, codes):
    """Export reference conformers (ideal coordinates, charges, leaving atoms, bonds) from components.cif[.gz] to JSON."""
    from ..data.ccd import export_table

    click.echo(f"{export_table(components_cif, out_json, set(codes) or None)} components -> {out_json}")


@prepare.command("filter")
@click.argument("data_dir", type=click.Path(exists=True))
@click.option("--output", type=click.Path(), default=None, help="Manifest to write (default: in place).")
@_with(_FILTER_OPTIONS)
def refilter(data_dir, output, **filt):
    """Re-apply the filters to an existing manifest from the stored structures (no mmCIF parsing)."""
    from ..data.prepare import filter_structure, filter_structure_metadata
    from ..data.types import Structure, load_manifest, save_manifest

    cfg = _filter_cfg(**filt)
    path = os.path.join(data_dir, "manifest.json")
    kept, dropped = [], 0
    for rec in load_manifest(path):
        for c in rec.chains:
            c.valid = True
        for i in rec.interfaces:
            i.valid = True
        st = Structure.load(os.path.join(data_dir, "structures", f"{rec.id}.npz"))
        if filter_structure_metadata(rec.structure_info, cfg, len(rec.chains), len(st.residues)) is not None:
            dropped += 1
            continue
        rec, _ = filter_structure(st, rec, cfg)
        if any(c.valid for c in rec.chains):
            kept.append(rec)
        else:
            dropped += 1
    save_manifest(kept, output or path)
    click.echo(f"{len(kept)} kept, {dropped} dropped")


@prepare.command("cluster")
@click.argument("data_dir", type=click.Path(exists=True))
@click.option("--pdb-clusters", type=click.Path(exists=True), default=None, help="wwPDB clusters-by-entity-40.txt.")
@click.option("--identity", type=float, default=0.4)
def cluster(data_dir, pdb_clusters, identity):
    """Assign cluster ids (sampling weights use them) to every chain of the manifest."""
    from ..data.prepare import cluster_records
    from ..data.prepare.clustering import load_pdb_clusters
    from ..data.prepare.pipeline import load_fasta
    from ..data.types import load_manifest, save_manifest

    path = os.path.join(data_dir, "manifest.json")
    recs = load_manifest(path)
    fasta = os.path.join(data_dir, "sequences.fasta")
    seqs = load_fasta(fasta) if os.path.exists(fasta) else {}
    cluster_records(recs, seqs, load_pdb_clusters(pdb_clusters) if pdb_clusters else None, identity)
    save_manifest(recs, path)
    click.echo(f"{len({str(c.cluster_id) for r in recs for c in r.chains})} clusters over {len(recs)} entries")


@prepare.command("features")
@click.argument("data_dir", type=click.Path(exists=True))
@click.option("--msa-dir", type=click.Path(), default=None, help="Directory of <msa_id>.a3m (or .npz) alignments.")
@click.option("--max-msa-rows", type=int, default=16384)
@click.option("--ccd", type=click.Path(exists=True), default=None,
              help="components.cif[.gz] or a JSON conformer table: reference conformers of ligands and modified residues.")
def features(data_dir, msa_dir, max_msa_rows, ccd):
    """Featurise every manifest entry into features/<id>.pt plus the flat manifest the training datasets read."""
    import torch

    from ..data import ref_conformers

    ref_conformers.set_ccd_source(ccd)

    from ..data.featurize import featurize_structure
    from ..data.parse.a3m import msa_from_a3m_file
    from ..data.types import MSA, Structure, load_manifest

    out = os.path.join(data_dir, "features")
    os.makedirs(out, exist_ok=True)
    flat = []
    for rec in load_manifest(os.path.join(data_dir, "manifest.json")):
        st = Structure.load(os.path.join(data_dir, "structures", f"{rec.id}.npz"))
        if ccd:  # one pass over the dictionary for the components this entry needs and does not know yet
            ref_conformers.ensure_components({r["name"].decode().strip() for r in st.residues if not r["is_standard"]})
        msas = {}
        for c in rec.chains:
            if not msa_dir:
                continue
            base = os.path.join(msa_dir, str(c.msa_id))
            if os.path.exists(base + ".npz"):
                msas[c.chain_id] = MSA.load(base + ".npz")
            elif os.path.exists(base + ".a3m"):
                msas[c.chain_id] = msa_from_a3m_file(base + ".a3m", c.mol_type, max_msa_rows)
        try:
            feats = featurize_structure(st, rec, unpaired_msa=msas, max_msa_rows=max_msa_rows)
        except ValueError as exc:
            click.echo(f"skip {rec.id}: {exc}")
            continue
        torch.save(feats, os.path.join(out, f"{rec.id}.pt"))
        d = rec.to_dict()
        flat.append({"id": rec.id, "chains": d["chains"], "interfaces": d["interfaces"],
                     "resolution": (d.get("structure_info") or {}).get("resolution") or 0.0})  # fmt: skip
    with open(os.path.join(out, "manifest.json"), "w") as f:
        json.dump(flat, f)
    click.echo(f"{len(flat)} examples -> {out}")


@prepare.command("pack")
@click.argument("src_dir", type=click.Path(exists=True))
@click.argument("out_dir", type=click.Path())
@click.option("--shard-size", default="1G")
def pack(src_dir, out_dir, shard_size):
    """Bundle a directory of small files into tar shards with an index (read back transparently by the datasets)."""
    from ..data.pack import build_pack

    units = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    size = int(float(shard_size[:-1]) * units[shard_size[-1].upper()]) if shard_size[-1].upper() in units else int(shard_size)
    click.echo(f"{build_pack(src_dir, out_dir, size)} files -> {out_dir}")


@prepare.command("monomer-templates")
@click.argument("data_dir", type=click.Path(exists=True))
@click.option("--m8-dir", type=click.Path(exists=True), required=True, help="<msa_id>.m8 template search results (13 columns, CIGAR last).")
@click.option("--release-dates", type=click.Path(exists=True), default=None, help="JSON {entry id: YYYY-MM-DD}.")
@click.option("--pdb-mmcif-dir", type=click.Path(exists=True), default=None, help="Read release dates from a local mmCIF mirror instead.")
@click.option("--max-hits", type=int, default=20, show_default=True)
def monomer_templates(data_dir, m8_dir, release_dates, pdb_mmcif_dir, max_hits):
    """Template hit lists per distinct sequence of a prepared dataset, for training (`monomer_templates/`)."""
    from ..data import templates as tpl
    from ..data.types import load_manifest

    if release_dates:
        with open(release_dates) as f:
            dates = json.load(f)
    elif pdb_mmcif_dir:
        from ..data.parse.mmcif import read_structure_info

        ids = set()
        for name in os.listdir(m8_dir):
            if name.endswith(".m8"):
                with open(os.path.join(m8_dir, name)) as f:
                    ids.update(line.split("\t")[1].partition("_")[0].lower() for line in f if "\t" in line)
        dates = {}
        for pdb in sorted(ids):
            path = tpl.find_pdb_mmcif(pdb, pdb_mmcif_dir)
            info = read_structure_info(path) if path else None
            if info is not None and info.released:
                dates[pdb] = info.released
    else:
        raise click.ClickException("give --release-dates or --pdb-mmcif-dir")
    lengths = {}
    manifest = os.path.join(data_dir, "manifest.json")
    if os.path.exists(manifest):
        for rec in load_manifest(manifest):
            for c in rec.chains:
                lengths[str(c.msa_id)] = int(c.num_residues)
    tpl.build_monomer_template_index(data_dir, m8_dir, dates, lengths, max_hits, click.echo)


@prepare.command("masks")
@click.argument("data_dir", type=click.Path(exists=True))
@click.option("--exclude-mol-type", "exclude", multiple=True, type=click.Choice(["protein", "dna", "rna", "ligand"]))
def masks(data_dir, exclude):
    """Write masks/<id>.npz token masks (loss weight 0 for the excluded molecule classes)."""
    import numpy as np

    from ..data import const
    from ..data.featurize import tokenize_structure
    from ..data.types import Structure, load_manifest

    ids = {"protein": const.MOL_PROTEIN, "dna": const.MOL_DNA, "rna": const.MOL_RNA, "ligand": const.MOL_NONPOLYMER}
    drop = {ids[e] for e in exclude}
    out = os.path.join(data_dir, "masks")
    os.makedirs(out, exist_ok=True)
    n = 0
    for rec in load_manifest(os.path.join(data_dir, "manifest.json")):
        st = Structure.load(os.path.join(data_dir, "structures", f"{rec.id}.npz"))
        tok, _, _ = tokenize_structure(st, {c.chain_id for c in rec.chains if c.valid})
        mt = np.asarray(tok["mol_type"])
        np.savez_compressed(os.path.join(out, f"{rec.id}.npz"), loss_weight=(~np.isin(mt, list(drop))).astype(np.float32))
        n += 1
    click.echo(f"{n} masks -> {out}")


@click.command("scan-mmcif")
@click.argument("mmcif_dir", type=click.Path(exists=True))
@click.option("--output", type=click.Path(), default=None, help="TSV to write (default: stdout).")
def scan_mmcif(mmcif_dir, output):
    """Table of id, resolution, method, deposition and release date for every mmCIF under a directory."""
    from ..data.parse.mmcif import read_structure_info
    from ..data.prepare.pipeline import find_mmcif_files

    lines = ["id\tresolution\tmethod\tdeposited\treleased"]
    for path in find_mmcif_files(mmcif_dir):
        info = read_structure_info(path)
        name = os.path.basename(path).split(".")[0]
        lines.append(f"{name}\tunreadable\t\t\t" if info is None else
                     f"{name}\t{info.resolution}\t{info.method}\t{info.deposited}\t{info.released}")  # fmt: skip
    text = "\n".join(lines) + "\n"
    if output:
        with open(output, "w") as f:
            f.write(text)
    else:
        click.echo(text, nl=False)


@click.command("inspect-example")
@click.argument("path", type=click.Path(exists=True))
def inspect_example(path):
    """Summarise one stored example: a ``.npz`` structure, a ``.pt`` feature dict or an mmCIF file."""
    from ..data import const

    if path.endswith(".pt"):
        import torch

        feats = torch.load(path, map_location="cpu", weights_only=False)
        for k, v in feats.items():
            click.echo(f"{k:28s} {tuple(v.shape) if hasattr(v, 'shape') else v!r} {getattr(v, 'dtype', '')}")
        return
    if path.endswith(".npz"):
        from ..data.types import Structure

        st = Structure.load(path)
    else:
        from ..data.parse.mmcif import parse_mmcif

        st, rec = parse_mmcif(path)
        click.echo(f"info: {rec.structure_info}")
    click.echo(f"{st.name}: {len(st.chains)} chains, {len(st.residues)} residues, {len(st.atoms)} atoms "
               f"({int(st.atoms['is_present'].sum())} resolved), {len(st.bonds)} bonds")  # fmt: skip
    for c in st.chains:
        click.echo(f"  chain {c['name'].decode():4s} asym {int(c['asym_id']):3d} entity {int(c['entity_id']):3d} copy {int(c['sym_id']):2d} "
                   f"{const.MOL_TYPE_NAMES[int(c['mol_type'])]:10s} {int(c['res_num']):5d} residues {int(c['atom_num']):6d} atoms")  # fmt: skip




# ---------------------------------------------------------------------------------------------------------------
# side language model (reference: scripts/plm_prepare.py, scripts/plm_train.py)
# ---------------------------------------------------------------------------------------------------------------
@click.group("plm-prepare")
def plm_prepare():
    """Build, cluster and inspect the stores the complex language model trains on."""


@plm_prepare.command("structure")
@click.option("--data-dir", type=click.Path(exists=True), required=True, help="Output of `prepare structures`.")
@click.option("--output", type=click.Path(), required=True)
@click.option("--source", required=True)
def plm_structure(data_dir, output, source):
    from ..complexlm.prepare import build_from_structures

    click.echo(json.dumps(build_from_structures(data_dir, output, source)))


@plm_prepare.command("pairs")
@click.option("--fasta", type=click.Path(exists=True), required=True)
@click.option("--pairs", type=click.Path(exists=True), required=True, help="Two sequence ids per line.")
@click.option("--output", type=click.Path(), required=True)
@click.option("--source", required=True)
def plm_pairs(fasta, pairs, output, source):
    from ..complexlm.prepare import build_from_pairs

    click.echo(json.dumps(build_from_pairs(fasta, pairs, output, source)))


@plm_prepare.command("cluster")
@click.option("--store", "stores", multiple=True, required=True, type=click.Path(exists=True))
@click.option("--identity", type=float, default=0.4)
def plm_cluster(stores, identity):
    from ..complexlm.prepare import cluster_stores

    click.echo(json.dumps(cluster_stores(list(stores), identity)))


@plm_prepare.command("stats")
@click.option("--store", type=click.Path(exists=True), required=True)
def plm_stats(store):
    from ..complexlm.prepare import store_stats

    click.echo(json.dumps(store_stats(store)))


@click.command("plm-train")
@click.option("--config", type=click.Path(exists=True), default=None)
@click.option("--output", type=click.Path(), required=True)
@click.option("--resume", type=click.Path(exists=True), default=None)
@click.option("--override", "overrides", multiple=True, help="section.key=value (repeatable).")
@click.option("--dry-run", is_flag=True, help="Build everything, run one step, write nothing but the config.")
def plm_train(config, output, resume, overrides, dry_run):
    """Train the complex language model (launch under torch.distributed.run for several GPUs)."""
    from ..complexlm.config import load_experiment
    from ..complexlm.trainer import ComplexLMTrainer

    cfg = load_experiment(config, dict(o.split("=", 1) for o in overrides))
    trainer = ComplexLMTrainer(cfg, output, resume)
    if dry_run:
        click.echo(json.dumps(trainer.train_step([next(iter(trainer.stream))])))
        return
    click.echo(json.dumps(trainer.train()))


@click.command("evaluate")
@click.argument("predicted", type=click.Path(exists=True))
@click.argument("experimental", type=click.Path(exists=True))
@click.option("--assembly", is_flag=True, help="Expand biological assembly 1 of the experimental entry.")
def evaluate(predicted, experimental, assembly):
    """lDDT, TM-score, GDT-TS, RMSD and DockQ of a predicted mmCIF against an experimental one."""
    from ..evaluation.compare import compare_files

    click.echo(json.dumps(compare_files(predicted, experimental, assembly), indent=1))


@click.group("eval-sweep")
def eval_sweep():
    """Fold a benchmark set with checkpoints of a run, score it against experimental structures, follow the trajectory."""


def _sweep_targets(inputs, truth, category, max_tokens):
    from ..evaluation.sweep import discover_targets

    targets = discover_targets(inputs, truth, set(category) or None, max_tokens)
    if not targets:
        raise click.ClickException(f"no job under {inputs}/<category>/*.json")
    return targets


@eval_sweep.command("run")
@click.option("--inputs", type=click.Path(exists=True), required=True, help="inputs/<category>/<name>.json")
@click.option("--run-dir", type=click.Path(), required=True)
@click.option("--ckpt-dir", type=click.Path(exists=True), default=None, help="step_<N>.safetensors / checkpoint_<N>.pt")
@click.option("--steps", default="0", help="Comma list of checkpoint steps, newest first is usual; 0 with no --ckpt-dir: random weights.")
@click.option("--category", multiple=True)
@click.option("--max-tokens", type=int, default=1024, show_default=True)
@click.option("--gpus", default=None, help="Comma list of device indices (default: all visible).")
@click.option("--seed", "seeds", default="42,43,44,45", show_default=True)
@click.option("--num-samples", type=int, default=5, show_default=True)
@click.option("--dry-run", is_flag=True, help="Print the per-GPU commands only.")
@click.argument("extra", nargs=-1)
def eval_sweep_run(inputs, run_dir, ckpt_dir, steps, category, max_tokens, gpus, seeds, num_samples, dry_run, extra):
    """One prediction process per GPU over a length-balanced share of the targets; a re-run fills the gaps. Arguments
    after `--` go to `inference-batch` unchanged."""
    from ..evaluation.sweep import resolve_checkpoint, run_sweep

    targets = _sweep_targets(inputs, None, category, max_tokens)
    if gpus is None:
        import torch

        gpus = ",".join(str(i) for i in range(max(1, torch.cuda.device_count())))
    failed = 0
    for step in (int(s) for s in steps.split(",")):
        params = resolve_checkpoint(ckpt_dir, step) if ckpt_dir else None
        if ckpt_dir and params is None:
            click.echo(f"step {step}: no checkpoint in {ckpt_dir}, skipped")
            continue
        click.echo(f"step {step}: {len(targets)} target(s), weights {params or 'random'}")
        failed += run_sweep(targets, os.path.join(run_dir, "pred", f"step_{step}"), params, [int(g) for g in gpus.split(",")],
                            [int(s) for s in seeds.split(",")], num_samples, list(extra), dry_run, click.echo)  # fmt: skip
    if failed:
        raise click.ClickException(f"{failed} prediction process(es) failed; see _gpu*.log under the pred directories")


@eval_sweep.command("score")
@click.option("--inputs", type=click.Path(exists=True), required=True)
@click.option("--truth", type=click.Path(exists=True), required=True, help="Directory of experimental mmCIF files named like the jobs.")
@click.option("--run-dir", type=click.Path(exists=True), required=True)
@click.option("--steps", default=None, help="Comma list (default: every pred/step_* present).")
@click.option("--category", multiple=True)
@click.option("--max-tokens", type=int, default=1024, show_default=True)
@click.option("--assembly", is_flag=True)
def eval_sweep_score(inputs, truth, run_dir, steps, category, max_tokens, assembly):
    """Score every predicted structure, then write per-step summaries and the trajectory over steps."""
    import glob as _glob

    from ..evaluation.sweep import score_step, summarize, trajectory

    targets = _sweep_targets(inputs, truth, category, max_tokens)
    found = sorted(int(os.path.basename(d)[5:]) for d in _glob.glob(os.path.join(run_dir, "pred", "step_*")))
    for step in ([int(s) for s in steps.split(",")] if steps else found):
        out = os.path.join(run_dir, "eval", f"step_{step}")
        rows = score_step(os.path.join(run_dir, "pred", f"step_{step}"), targets, os.path.join(out, "scores.csv"), assembly, click.echo)
        for row in summarize(rows, os.path.join(out, "summary.csv")):
            if row["fold_class"] == "all":
                click.echo(f"step {step} {row['category']}: {row['targets']} targets, lDDT mean {row['lddt_mean']:.3f} "
                           f"oracle {row['lddt_oracle']:.3f}, TM mean {row['tm_score_mean']:.3f} oracle {row['tm_score_oracle']:.3f}")  # fmt: skip
    traj = trajectory(run_dir, os.path.join(run_dir, "trajectory.csv"))
    click.echo(f"{len(traj)} trajectory row(s) -> {os.path.join(run_dir, 'trajectory.csv')}")


@click.command("prepare-templates")
@click.option("--m8", "m8_path", type=click.Path(exists=True), required=True, help="Template search hits (mmseqs .m8 with CIGAR).")
@click.option("--pdb-mmcif-dir", type=click.Path(exists=True), required=True)
@click.option("--output-dir", type=click.Path(), required=True)
@click.option("--index", type=int, default=0, help="Chain index in the job (names the JSON file).")
@click.option("--max-templates", type=int, default=4)
@click.option("--max-template-date", default=None, help="YYYY-MM-DD release cut-off.")
def prepare_templates(m8_path, pdb_mmcif_dir, output_dir, index, max_templates, max_template_date):
    """Turn template search hits into the templates JSON and mmCIF files a prediction job points at."""
    from ..data.templates import prepare_job_templates

    with open(m8_path) as f:
        hits = prepare_job_templates(f.read(), pdb_mmcif_dir, output_dir, index, max_templates, max_template_date)
    click.echo(f"{len(hits)} templates -> {output_dir}/templates_{index}.json")


@click.command("build-pdb-cache")
@click.argument("mmcif_dir", type=click.Path(exists=True))
@click.argument("out_dir", type=click.Path())
@click.option("--limit", type=int, default=0)
def build_pdb_cache(mmcif_dir, out_dir, limit):
    """Cache dense per-chain coordinates of every protein chain under MMCIF_DIR for template featurisation."""
    from ..data.templates import build_chain_cache

    click.echo(f"{build_chain_cache(mmcif_dir, out_dir, limit)} chains -> {out_dir}")


@click.command("inspect-checkpoint")
@click.argument("path", type=click.Path(exists=True))
@click.option("--depth", type=int, default=2, help="Module-name depth of the grouping.")
def inspect_checkpoint(path, depth):
    """Parameter counts, norms, non-finite values and EMA distance of a .pt / .safetensors checkpoint, by module."""
    from ..utils.run_tools import checkpoint_report

    click.echo(json.dumps(checkpoint_report(path, depth), indent=1, default=str))


@click.command("run-status")
@click.argument("run_dir", type=click.Path(exists=True))
def run_status_cmd(run_dir):
    """Progress, throughput, loss trend and skipped steps of a training run directory."""
    from ..utils.run_tools import run_status

    click.echo(json.dumps(run_status(run_dir), indent=1))


@click.group("triage")
def triage():
    """Diagnostics for a run that misbehaves: non-finite values, diverging paths, gradient agreement, series, mirror images."""


def _triage_model(config, overrides, params, tokens, seed):
    """The model of a recipe (random weights unless ``params``) and one synthetic example of ``tokens`` tokens."""
    import torch

    from ..config.loader import build_configs
    from ..data.synthetic import split_lengths, synthetic_complex
    from ..models.model import DeepFold3

    tc, mc = build_configs(list(config), list(overrides))
    torch.manual_seed(seed)
    model = DeepFold3(mc)
    if params:
        from ..training.checkpointing import load_pretrained_weights

        load_pretrained_weights(model, params)
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    model.to(dev)
    feats = synthetic_complex([("protein", n) for n in split_lengths(tokens, 2)], num_msa=min(mc.msa_crop_size, 64), seed=seed)
    feats = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in feats.items()}
    return model, tc, mc, feats, dev


@triage.command("activations")
@click.option("--config", multiple=True, type=click.Path(exists=True))
@click.option("--override", multiple=True)
@click.option("--params", type=click.Path(exists=True), default=None)
@click.option("--tokens", type=int, default=64, show_default=True)
@click.option("--seed", type=int, default=0)
@click.option("--compare-disabled", default=None, help="Run a second trace with DF3_DISABLE_OPS set to this list and report where the two part.")
@click.option("--top", type=int, default=10, show_default=True)
def triage_activations(config, override, params, tokens, seed, compare_disabled, top):
    """Trace every submodule of one prediction-mode forward: first non-finite output, largest magnitudes, and with
    --compare-disabled the first module where the kernel path and the PyTorch statement differ."""
    import dataclasses

    import torch

    from ..utils import triage as T

    model, _, mc, feats, dev = _triage_model(config, override, params, tokens, seed)
    model.eval()

    def run():
        with torch.no_grad(), torch.autocast(dev.type, dtype=torch.bfloat16, enabled=dev.type == "cuda"):
            model(dict(feats), seed=seed, num_recycles=1, num_samples=1)

    rows = T.activation_trace(model, run)
    bad = T.first_nonfinite(rows)
    out = {"modules_called": len(rows), "first_nonfinite": dataclasses.asdict(bad) if bad else None,
           "largest": [dataclasses.asdict(r) for r in T.largest_activations(rows, top)]}  # fmt: skip
    if compare_disabled:
        keep = os.environ.get("DF3_DISABLE_OPS")
        os.environ["DF3_DISABLE_OPS"] = compare_disabled
        try:
            other = T.activation_trace(model, run)
        finally:
            if keep is None:
                os.environ.pop("DF3_DISABLE_OPS", None)
            else:
                os.environ["DF3_DISABLE_OPS"] = keep
        out["differences"] = T.diff_traces(rows, other)[:top]
    click.echo(json.dumps(out, indent=1))


@triage.command("grad-spread")
@click.option("--config", multiple=True, type=click.Path(exists=True))
@click.option("--override", multiple=True)
@click.option("--params", type=click.Path(exists=True), default=None)
@click.option("--tokens", type=int, default=64, show_default=True)
@click.option("--examples", type=int, default=8, show_default=True)
@click.option("--seed", type=int, default=0)
def triage_grad_spread(config, override, params, tokens, examples, seed):
    """Norms and directional agreement of per-example gradients over synthetic examples (one forward + backward each)."""
    import torch

    from ..data.synthetic import split_lengths, synthetic_complex
    from ..training.engine import training_step
    from ..utils import triage as T

    model, tc, mc, _, dev = _triage_model(config, override, params, tokens, seed)
    model.train()
    spread = T.GradientSpread()
    for i in range(examples):
        feats = synthetic_complex([("protein", n) for n in split_lengths(tokens, 2)], num_msa=min(mc.msa_crop_size, 64), seed=seed + 1 + i)
        batch = {k: (v.unsqueeze(0).to(dev) if torch.is_tensor(v) else [v]) for k, v in feats.items()}
        model.zero_grad(set_to_none=True)
        with torch.autocast(dev.type, dtype=torch.bfloat16, enabled=dev.type == "cuda"):
            loss, *_ = training_step(model, batch, cfg=tc, model_cfg=mc, global_step=i, device=dev, num_recycles=1)
        loss.backward()
        spread.add(T.flat_gradient(model))
    click.echo(json.dumps(spread.result(), indent=1))


@triage.command("distogram")
@click.option("--config", multiple=True, type=click.Path(exists=True))
@click.option("--override", multiple=True)
@click.option("--params", type=click.Path(exists=True), default=None)
@click.option("--example", type=click.Path(exists=True), default=None, help="A stored feature file (.pt) with ground truth; default: a synthetic complex.")
@click.option("--tokens", type=int, default=64, show_default=True)
@click.option("--recycles", type=int, default=1, show_default=True)
@click.option("--seed", type=int, default=0)
@click.option("--save", type=click.Path(), default=None, help="Write the true and expected distance maps as .npz.")
def triage_distogram(config, override, params, example, tokens, recycles, seed, save):
    """Distogram head against the true distances of one example: bin accuracy, cross-entropy, error of the expected distance."""
    import torch

    from ..utils.triage import distogram_agreement

    model, _, _, feats, dev = _triage_model(config, override, params, tokens, seed)
    if example:
        feats = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in torch.load(example, map_location="cpu", weights_only=False).items()}
    with torch.autocast(dev.type, dtype=torch.bfloat16, enabled=dev.type == "cuda"):
        out = distogram_agreement(model, feats, recycles, seed)
    maps = {k: out.pop(k) for k in ("true_distance", "expected_distance") if k in out}
    if save and maps:
        import numpy as np

        np.savez_compressed(save, **{k: v.numpy() for k, v in maps.items()})
    click.echo(json.dumps(out, indent=1))


@triage.command("series")
@click.argument("run_dir", type=click.Path(exists=True))
@click.option("--prefix", default="act_rms", show_default=True)
@click.option("--window", type=int, default=50, show_default=True)
@click.option("--ceiling", type=float, default=None)
def triage_series(run_dir, prefix, window, ceiling):
    """Latest value, median and log-slope of every logged series with the prefix, fastest-growing first."""
    from ..utils.triage import series_summary

    click.echo(json.dumps(series_summary(run_dir, prefix, window, ceiling), indent=1))


@triage.command("handedness")
@click.argument("pred", type=click.Path(exists=True))
@click.argument("ref", type=click.Path(exists=True))
def triage_handedness(pred, ref):
    """Is the predicted structure a mirror image of the reference? Per matched chain."""
    from ..utils.triage import handedness_of_files

    click.echo(json.dumps(handedness_of_files(pred, ref), indent=1))


def register(cli) -> None:
    for cmd in (prepare, scan_mmcif, inspect_example, plm_prepare, plm_train, evaluate, eval_sweep, prepare_templates, build_pdb_cache, inspect_checkpoint, run_status_cmd,
                triage):  # fmt: skip
        cli.add_command(cmd)

