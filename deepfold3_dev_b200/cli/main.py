"""``deepfold3`` command line (reference: scripts/cli.py and scripts/{train,inference,inference_batch,export_weights,
convert_weights}.py).

    python -m deepfold3_dev_b200.cli train --config configs/initial.yaml --output runs/a --dataset pdb:/data/pdb
    python -m deepfold3_dev_b200.cli inference --json job.json --params weights.safetensors --output out/
    python -m deepfold3_dev_b200.cli inference-batch --inputs-file jobs.txt --params ... --output-template 'out/{name}'
    python -m deepfold3_dev_b200.cli export runs/a/checkpoint_1000.pt weights.safetensors --snapshot shadow
"""

from __future__ import annotations

import logging
import os
import re

import click

DTYPES = {"bf16": "bfloat16", "fp32": "float32", "fp16": "float16"}


def _setup_logging():
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s: %(message)s")


def apply_det_recipe() -> None:
    """Bit-reproducible run: deterministic algorithms, no TF32, cuBLAS workspace pinned."""
    import torch

    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    torch.use_deterministic_algorithms(True, warn_only=True)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cudnn.benchmark = False


@click.group()
def cli():
    """DeepFold3 on B200."""


# ------------------------------------------------------------------------------------------------ train
def _read_id_list(path):
    """Record ids, one per line (blank lines and ``#`` comments skipped), lower-cased; ``None`` without a file."""
    if not path:
        return None
    with open(path) as f:
        return {line.split()[0].lower() for line in f if line.strip() and not line.startswith("#")}


def _filter_ids(dataset, include, exclude) -> int:
    """Keep the records of ``dataset`` named in ``include`` (when given) and not named in ``exclude``; returns how many
    were dropped. Datasets without a record list (synthetic data) are left alone."""
    records = getattr(dataset, "records", None)
    if records is None or (include is None and exclude is None):
        return 0
    rid = lambda r: str(r["id"] if isinstance(r, dict) else r.id).lower()  # noqa: E731
    kept = [r for r in records if (include is None or rid(r) in include) and (exclude is None or rid(r) not in exclude)]
    dropped = len(records) - len(kept)
    dataset.records = kept
    if hasattr(dataset, "_anchors"):
        dataset._anchors = None  # sampling weights follow the surviving records
    return dropped


class EvalLoader:
    """A fixed, rank-strided set of evaluation examples, re-iterable: every call of the trainer's evaluation sees the
    same examples (the datasets draw crops from a per-index seed), one example per batch."""

    def __init__(self, parts, limit: int, rank: int, world: int):
        from ..data import datasets as ds

        self.collate = ds.collate
        self.items = []
        for p in parts:
            self.items += [(p, i) for i in range(len(p))]
        self.items = self.items[: max(0, limit)][rank::world]

    def __len__(self):
        return len(self.items)

    def __iter__(self):
        for part, i in self.items:
            yield self.collate([part[i]])


def build_training_stream(tc, mc, info, datasets, data_dir=None, synthetic=False, num_workers=None, include=None, exclude=None,
                          eval_cutoff_date=None, return_eval: bool = False):
    """``(stream, sampler)`` for the training loop: the datasets named on the command line (or in the config's mixture),
    weighted cluster sampling per dataset, a weighted mixture over datasets, token-budget batching and a prefetch thread.
    Shared by ``train`` and by the input-pipeline check of the cluster recipes.

    A dataset is ``name:path[:weight[:strategy[:distill[:format[:tpl_struct_space]]]]]``. ``include`` / ``exclude`` are
    sets of record ids. ``eval_cutoff_date`` splits structure datasets by release date: entries released on or before
    it train, later ones form the evaluation set; with ``return_eval`` the result is ``(stream, sampler, eval_loader)``
    (the evaluation loader also takes the recipe's ``eval_datasets``; ``None`` when there is nothing to evaluate on)."""
    from ..data import datasets as ds
    from ..data.samplers import MultiDatasetSampler, WeightedClusterSampler

    specs = list(datasets) or ([f"data:{data_dir}"] if data_dir else [])
    extra = {}  # per-dataset settings that only the config file carries (date cut-off, crop weights)
    if not specs and not synthetic:
        for d in getattr(tc, "extra_datasets", []) or []:
            if d.data_dir:
                specs.append(f"{d.name or 'data'}:{d.data_dir}:{d.weight}:{d.strategy}:{int(d.is_distillation)}")
                extra[d.data_dir] = {"cutoff_date": d.cutoff_date, "crop_weights": d.crop_weights, "format": d.format,
                                     "of3_cache_dir": d.of3_cache_dir}
    eval_parts = []
    if synthetic or not specs:
        if not synthetic:
            raise click.ClickException("give --dataset / --data-dir, or --synthetic")
        data = ds.SyntheticDataset(tc.max_tokens, 2, min(mc.msa_crop_size, 1024), 4, seed=tc.seed + info.rank)
        sampler = iter(range(1 << 62))
        stream = ds.BatchStream(data, sampler, tc.batch_size_per_rank, tc.max_tokens)
    else:
        parts, weights = [], []
        for spec in specs:
            f = spec.split(":")
            name, path = f[0], f[1]
            weights.append(float(f[2]) if len(f) > 2 and f[2] else 1.0)
            distill = len(f) > 4 and f[4].lower() in ("1", "true", "distill")
            kw = {k: v for k, v in extra.get(path, {}).items() if v}
            if len(f) > 5 and f[5]:
                kw["format"] = f[5]
            if eval_cutoff_date:
                kw["cutoff_date"] = eval_cutoff_date
            structured = kw.get("format", "df3") != "df3" or os.path.isdir(os.path.join(path, "structures"))
            if "cutoff_date" in kw and not structured:
                kw.pop("cutoff_date")  # feature directories carry no dates; the cut-off is applied when they are prepared
            d = mc.data
            common = dict(max_tokens=tc.max_tokens, max_atoms=tc.max_atoms, is_distillation=distill, seed=tc.seed,
                          pdb_chain_cache_dir=getattr(tc, "pdb_chain_cache_dir", None) or None, max_templates=d.max_templates,
                          template_cutoff_days=d.template_cutoff_days, max_template_date=d.max_template_date,
                          default_template_cutoff_date=d.default_template_cutoff_date,
                          slow_sample_log_threshold_s=tc.slow_sample_log_threshold_s)  # fmt: skip
            parts.append(ds.open_dataset(path, atomize_prob=d.atomize_prob, atomize_source=d.atomize_source,
                                         atomize_max_residues=d.atomize_max_residues, **common, **kw))  # fmt: skip
            dropped = _filter_ids(parts[-1], include, exclude)
            logging.getLogger(__name__).info("dataset %s: %d examples from %s%s", name, len(parts[-1]), path,
                                             f" ({dropped} dropped by the id lists)" if dropped else "")  # fmt: skip
            if eval_cutoff_date and structured and kw.get("format", "df3") == "df3":
                later = ds.open_dataset(path, **common, **{**kw, "keep_after": True})  # no atomisation in evaluation
                _filter_ids(later, include, exclude)
                if len(later):
                    eval_parts.append(later)
        samplers = [WeightedClusterSampler(p.weights(), tc.seed + 17 * i, info.rank, info.world_size) for i, p in enumerate(parts)]
        sampler = MultiDatasetSampler(samplers, [len(p) for p in parts], weights, tc.seed)

        class _Concat:
            def __getitem__(self, i):
                for p, off in zip(parts, sampler.offsets):
                    if i < off + len(p):
                        return p[i - off]
                raise IndexError(i)

        stream = ds.BatchStream(_Concat(), sampler, tc.batch_size_per_rank, tc.max_tokens)
    workers = tc.num_workers if num_workers is None else num_workers
    if workers > 0 and not synthetic:
        base = stream
        stream = ds.PrefetchStream(lambda w: base, depth=max(2, getattr(tc, "prefetch_factor", 2) * workers), workers=1)
    if not return_eval:
        return stream, sampler
    for d in getattr(tc, "eval_datasets", []) or []:  # evaluation sets named by the recipe
        if d.data_dir and os.path.exists(d.data_dir):
            kw = {k: v for k, v in {"cutoff_date": d.cutoff_date, "format": d.format, "of3_cache_dir": d.of3_cache_dir}.items() if v}
            if kw.get("format", "df3") == "df3":
                kw["keep_after"] = bool(d.cutoff_date)
            eval_parts.append(ds.open_dataset(d.data_dir, max_tokens=tc.max_tokens, max_atoms=tc.max_atoms, seed=tc.seed, **kw))
    loader = EvalLoader(eval_parts, int(getattr(tc, "eval_samples", 1024)), info.rank, info.world_size) if eval_parts else None
    return stream, sampler, (loader if loader is not None and len(loader) else None)


@cli.command()
@click.option("--data-dir", type=click.Path(), default=None, help="Directory of featurised examples (one dataset).")
@click.option("--output", type=click.Path(), required=True)
@click.option("--params", type=click.Path(), default=None, help="Initial weights (.safetensors / .pt).")
@click.option("--resume", default=None, help="Checkpoint path, or 'auto' for the latest in --output.")
@click.option("--config", "configs", multiple=True, type=click.Path(exists=True))
@click.option("--lr", type=float, default=None)
@click.option("--max-steps", type=int, default=None)
@click.option("--max-tokens", type=int, default=None)
@click.option("--grad-accum", type=int, default=None)
@click.option("--seed", type=int, default=None)
@click.option("--deterministic", is_flag=True)
@click.option("--dtype", type=click.Choice(list(DTYPES)), default=None)
@click.option("--wandb", "wandb_project", default=None)
@click.option("--wandb-entity", default=None)
@click.option("--override", "overrides", multiple=True, help="key=value on the training or model config.")
@click.option("--dataset", "datasets", multiple=True, help="name:path[:weight[:strategy[:distill]]] (repeatable).")
@click.option("--synthetic", is_flag=True, help="Train on generated examples of the configured crop size.")
@click.option("--num-workers", type=int, default=None, help="Background data threads (default: training.num_workers).")
@click.option("--ccd", type=click.Path(exists=True), default=None, help="components.cif[.gz] or a JSON conformer table.")
@click.option("--ccd-cache", type=click.Path(exists=True), default=None, help="JSON conformer table from build-ccd-cache.")
@click.option("--include-list", type=click.Path(exists=True), default=None, help="Record ids to train on, one per line.")
@click.option("--exclude-list", type=click.Path(exists=True), default=None, help="Record ids to leave out, one per line.")
@click.option("--eval-cutoff-date", default=None, help="YYYY-MM-DD: structure entries released later form the evaluation set.")
@click.option("--mmcif-dir", type=click.Path(exists=True), default=None,
              help="Local mmCIF mirror: template chains missing from the per-chain cache are read from it.")
def train(data_dir, output, params, resume, configs, lr, max_steps, max_tokens, grad_accum, seed, deterministic, dtype,
          wandb_project, wandb_entity, overrides, datasets, synthetic, num_workers, ccd, ccd_cache, include_list,
          exclude_list, eval_cutoff_date, mmcif_dir):  # fmt: skip
    """Train the model (one process per GPU; launch with torch.distributed.run for several)."""
    _setup_logging()
    import faulthandler
    import signal

    faulthandler.enable()  # a fatal signal prints every thread's Python stack
    if hasattr(signal, "SIGUSR1"):
        faulthandler.register(signal.SIGUSR1, all_threads=True)  # `kill -USR1 <pid>`: where is this rank right now?
    from ..config.loader import build_configs
    from ..parallel.dist import init_process_group
    from ..training.tracking import build_trackers
    from ..training.trainer import Trainer, _plain

    tc, mc = build_configs(list(configs), list(overrides))
    tc.output_dir = output
    for key, val in (("lr", lr), ("max_steps", max_steps), ("max_tokens", max_tokens), ("accumulate_grad_batches", grad_accum),
                     ("seed", seed), ("dtype", dtype), ("params_path", params)):  # fmt: skip
        if val is not None:
            setattr(tc, key, val)
    if deterministic:
        tc.deterministic = True
        apply_det_recipe()
    info = init_process_group(tc.collective_timeout_s)
    for table in (ccd, ccd_cache):
        if table:
            from ..data import ref_conformers

            ref_conformers.set_ccd_source(table)  # a JSON table is read now, a components.cif is looked up per component
    if mmcif_dir:
        os.environ["DF3_TEMPLATE_MMCIF_DIR"] = mmcif_dir  # read by the datasets' template loader as the fallback source
    stream, sampler, eval_loader = build_training_stream(
        tc, mc, info, list(datasets), data_dir, synthetic, num_workers, include=_read_id_list(include_list),
        exclude=_read_id_list(exclude_list), eval_cutoff_date=eval_cutoff_date, return_eval=True,
    )  # fmt: skip
    trackers = build_trackers(output, info.is_main, wandb_project, wandb_entity, {"training": _plain(tc), "model": _plain(mc)})
    trainer = Trainer(tc, mc, train_loader=stream, eval_loader=eval_loader, sampler=sampler if hasattr(sampler, "state_dict") else None,
                      dist_info=info, trackers=trackers)  # fmt: skip
    if resume == "auto":
        resume = trainer.ckpt.find_latest()
    state = trainer.run(resume)
    for t in trackers:
        t.close()
    click.echo(f"finished at step {state.effective_step}")


# ------------------------------------------------------------------------------------------------ inference
def _inference_options(f):
    opts = [
        click.option("--params", type=click.Path(), default=None, help=".safetensors / .pt; random weights if omitted."),
        click.option("--num-recycles", type=int, default=10),
        click.option("--num-samples", type=int, default=5),
        click.option("--msa-crop-size", type=int, default=16384),
        click.option("--snapshot", type=click.Choice(["auto", "shadow", "average", "fast"]), default="auto"),
        click.option("--seed", "seeds", type=int, multiple=True),
        click.option("--device", default=None),
        click.option("--optim", type=click.Choice(["none", "inference", "inference-cueq", "train-matched"]), default="inference"),
        click.option("--precision", type=click.Choice(list(DTYPES)), default="bf16"),
        click.option("--hoist-sampler/--no-hoist-sampler", default=True,
                     help="Compute everything that does not depend on the noise level once per prediction and replay the "
                          "denoiser from a CUDA graph (default). --no-hoist-sampler runs the per-block statement eagerly."),
        click.option("--msa-search", type=click.Choice(["none", "server", "local"]), default="none", show_default=True,
                     help="Search alignments (and template hits) for protein chains of a JSON job that carry none: the ColabFold "
                          "MMseqs2 API, or the staged local pipeline over --msa-db-dir."),
        click.option("--msa-db-dir", type=click.Path(), default=None, help="ColabFold databases for --msa-search local."),
        click.option("--msa-cache-dir", type=click.Path(), default="~/.cache/deepfold3/msa", show_default=True),
        click.option("--logits-scheme", type=click.Choice(["float32", "float16", "int8", "int8_softmax", "int4_softmax", "f16", "u8", "f32"]),
                     default="int8_softmax", show_default=True, help="How logits.npz stores the head logits (f16 / u8 / f32: earlier names)."),
        click.option("--bucket/--no-bucket", default=True),
        click.option("--sample-chunk", type=int, default=0),
        click.option("--guidance", "guidance", multiple=True,
                     help="W[@TARGET[@LO..HI]] with TARGET full | all (every interface) | A:B[,C:D] (repeatable); scale[:drop[:lo-hi]] also accepted."),
        click.option("--allow-guidance-overlap", is_flag=True),
        click.option("--restraint", "restraints", multiple=True, help="SEL:SEL[@DIST[@LO..HI]] pulls two residue groups together (repeatable)."),
        click.option("--restraint-pair", "restraint_pairs", multiple=True, help="Like --restraint, residue i of one side with residue i of the other."),
        click.option("--repel", "repels", multiple=True, help="SEL:SEL[@DIST[@LO..HI]] keeps two groups at least DIST apart."),
        click.option("--restraint-rigid/--restraint-residues", default=True, help="Move whole chains rigidly, or the named residues alone."),
        click.option("--restraint-after-step/--restraint-before-step", default=False),
        click.option("--restraint-after-sigma", type=float, default=16.0),
        click.option("--restraint-max-step", type=float, default=2.0),
        click.option("--restraint-weight", type=float, default=0.0),
        click.option("--msa-pairing", type=click.Choice(["auto", "species", "none"]), default="auto"),
        click.option("--matmul-precision", type=click.Choice(["highest", "high", "medium"]), default=None),
        click.option("--plot-confidences", is_flag=True, help="Write a pLDDT / PAE figure next to every confidences JSON."),
        click.option("--allow-missing-keys", is_flag=True),
        click.option("--ccd", type=click.Path(), default=None, help="components.cif[.gz] or a JSON conformer table, for ligands and modified residues."),
        click.option("--det", is_flag=True, help="Deterministic recipe."),
    ]
    for o in reversed(opts):
        f = o(f)
    return f


def _prepare_model(params, device, optim, snapshot, allow_missing_keys, det, ccd):
    import torch

    from ..data import ref_conformers
    from ..inference.weights import build_model

    if det:
        apply_det_recipe()
    if ccd:
        ref_conformers.set_ccd_source(ccd)
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    model, cfg = build_model(params, device, optim, snapshot, allow_missing=allow_missing_keys)
    return model, cfg, device


def _job_steering(inp, guidance, allow_overlap, restraints, restraint_pairs, repels, weight, rigid, after_step, after_sigma, max_step):
    """Guidance terms and restraint arguments of one job (selectors are resolved against the job's chains)."""
    from ..models.guidance import build_guidance_terms, parse_guidance_spec
    from ..models.restraints import build_restraints, parse_restraint_spec

    feats = inp.features
    chain_index = {name: i for i, name in enumerate(inp.chain_names)}
    n = int(feats["res_type"].shape[0])
    terms = None
    if guidance:
        if all("@" in g or g.replace(".", "", 1).replace("-", "", 1).isdigit() for g in guidance) and not any(":" in g.split("@")[0] for g in guidance):
            specs = [parse_guidance_spec(g) for g in guidance]
            terms = build_guidance_terms(specs, feats["asym_id"], chain_index, n, feats["residue_index"], allow_overlap)
        else:
            terms = _guidance_terms(guidance)
    specs = [parse_restraint_spec(t) for t in restraints] + [parse_restraint_spec(t, paired=True) for t in restraint_pairs]
    specs += [parse_restraint_spec(t, repel=True) for t in repels]
    kwargs = None
    if specs:
        built = build_restraints(specs, feats["asym_id"], chain_index, n, feats["residue_index"])
        kwargs = dict(restraints=built, restraint_weight=weight or 1.0, restraint_rigid=rigid, restraint_max_step=max_step,
                      restraint_after_step=after_step, restraint_after_sigma=after_sigma)  # fmt: skip
    return terms, kwargs


def _attach_templates(inp, hits_path: str, mmcif_dir: str | None, cache_dir: str) -> None:
    """Template features of a single-chain job from a hit file (.m8 / .hhr / templates JSON)."""
    import json

    from ..data import templates as tpl

    n = inp.num_tokens
    if hits_path.endswith(".json"):
        with open(hits_path) as f:
            chains = tpl.load_json_templates(json.load(f), os.path.dirname(os.path.abspath(hits_path)))
    else:
        if not mmcif_dir:
            raise click.ClickException("--templates with .m8 / .hhr hits needs --pdb-mmcif-dir")
        with open(hits_path) as f:
            text = f.read()
        if hits_path.endswith(".hhr"):
            from ..data.parse.hhr import parse_hhr

            rows = []
            for h in parse_hhr(text):
                pairs = sorted(h.query_to_hit_mapping.items())
                rows.append({"pdb_id": h.pdb_id.lower(), "chainId": h.chain_id, "queryIndices": [q for q, _ in pairs],
                             "templateIndices": [t for _, t in pairs], "seq": h.hit_sequence.replace("-", "")})  # fmt: skip
            chains = []
            for r in rows:
                src = tpl.find_pdb_mmcif(r["pdb_id"], mmcif_dir)
                hit = tpl.template_chain_from_mmcif(src, r["chainId"], r["queryIndices"], r["templateIndices"], r["seq"]) if src else None
                if hit is not None:
                    chains.append(hit)
        else:
            hits = tpl.prepare_job_templates(text, mmcif_dir, cache_dir, query_length=n)
            chains = tpl.load_json_templates(hits, cache_dir)
    if chains:
        inp.features.update(tpl.template_features(n, chains))


def _apply_hoist(hoist: bool) -> None:
    if not hoist:
        os.environ["DF3_GRAPH_SAMPLER"] = "0"
        os.environ["DF3_DIFFUSION_FAST"] = "0"


def parse_inputs_file(path: str) -> list[tuple[str, str | None, dict]]:
    """Lines of an ``--inputs-file``: ``json_path [output_dir] [key=value ...]``, tab-separated when the line holds a tab,
    else split on blanks; ``#`` starts a comment. Known keys: ``seeds=42,66`` (this job's seeds), and for a guidance
    sweep ``group=NAME`` and ``pairs=H:A,L:A``. Returns ``[(json_path, output_dir or None, {key: value})]``."""
    out = []
    with open(path) as f:
        for raw in f:
            line = raw.split("#", 1)[0].strip()
            if not line:
                continue
            fields = [x.strip() for x in line.split("\t")] if "\t" in line else line.split()
            fields = [x for x in fields if x]
            keyed = [x for x in fields[1:] if re.match(r"[a-z_]+=", x)]
            plain = [x for x in fields[1:] if x not in keyed]
            extras = dict(x.split("=", 1) for x in keyed)
            out.append((fields[0], plain[0] if plain else None, extras))
    return out


def load_guidance_sweep(path: str) -> dict[str, list[tuple[str, tuple[str, ...]]]]:
    """``{"groups": {GROUP: [{"name": N, "guidance": ["W@TARGET", ...]}, ...]}}`` -> ``{GROUP: [(name, specs)]}``. Every
    entry is one guidance setting; its results go to the line's output directory with ``{cfg}`` replaced by the name."""
    import json

    with open(path) as f:
        data = json.load(f)
    groups = {}
    for group, items in data["groups"].items():
        entries = [(str(it["name"]), tuple(str(g) for g in it.get("guidance", ()))) for it in items]
        names = [n for n, _ in entries]
        if len(set(names)) != len(names):
            raise click.UsageError(f"--guidance-sweep: duplicate entry names in group {group!r}")
        groups[group] = entries
    return groups


def sweep_entries(groups, out_dir: str, extras: dict) -> list[tuple[str, str, tuple[str, ...]]]:
    """``[(entry name, output directory, guidance specs)]`` for one inputs-file line under a guidance sweep."""
    group = extras.get("group")
    if group not in groups:
        raise click.UsageError(f"--guidance-sweep: {out_dir} names group {group!r}; known groups: {sorted(groups)}")
    if "{cfg}" not in out_dir:
        raise click.UsageError(f"--guidance-sweep: the output directory {out_dir} has no {{cfg}} placeholder")
    out = []
    for name, specs in groups[group]:
        if any("{pairs}" in t for t in specs) and not extras.get("pairs"):
            raise click.UsageError(f"--guidance-sweep: entry {name!r} needs pairs=... on the line of {out_dir}")
        out.append((name, out_dir.replace("{cfg}", name), tuple(t.replace("{pairs}", extras.get("pairs", "")) for t in specs)))
    return out


def _msa_search_fn(mode: str, db_dir: str | None, cache_dir: str | None):
    """The ``msa_search`` argument of ``parse_json_input`` for the ``--msa-search`` choice."""
    from ..data.parse import json_input

    if mode == "server":
        return json_input.msa_search_from_server(cache_dir)
    if mode == "local":
        if not db_dir:
            raise click.ClickException("--msa-search local needs --msa-db-dir")
        from ..data.msa.mmseqs_pipeline import MmseqsSettings

        return json_input.msa_search_local(MmseqsSettings(db_dir, use_templates=True), cache_dir)
    return None


def _plot_outputs(out_dir: str) -> None:
    from ..io.plot import plot_confidences

    for base, _dirs, files in os.walk(out_dir):
        for f in files:
            if (f == "confidences.json" or f.endswith("_confidences.json")) and "summary" not in f:
                try:
                    plot_confidences(os.path.join(base, f))
                except Exception as exc:  # noqa: BLE001 - a figure must not fail the prediction
                    logging.getLogger(__name__).warning("plot of %s failed: %r", f, exc)


def _guidance_terms(specs):
    from ..models.diffusion_modules import GuidanceTerm

    terms = []
    for s in specs:
        f = s.split(":")
        rng = None
        if len(f) > 2 and f[2]:
            lo, hi = f[2].split("-")
            rng = (float(lo), float(hi))
        terms.append(GuidanceTerm(scale=float(f[0]), sigma_range=rng))
    return terms or None


@cli.command()
@click.option("--msa", type=click.Path(exists=True), default=None, help="A3M alignment of a single chain.")
@click.option("--json", "json_path", type=click.Path(exists=True), default=None, help="Job description (any dialect).")
@click.option("--sequence", default=None, help="A single sequence, no alignment.")
@click.option("--mol-type", type=click.Choice(["protein", "dna", "rna"]), default="protein")
@click.option("--output", type=click.Path(), required=True)
@click.option("--templates", "templates_path", type=click.Path(exists=True), default=None,
              help="Template hits for a single-chain job: mmseqs .m8 with CIGAR, HHsearch .hhr, or a templates JSON.")
@click.option("--pdb-mmcif-dir", type=click.Path(exists=True), default=None, help="Where the hits' mmCIF files are.")
@click.option("--template-cache", type=click.Path(), default=None, help="Directory for the prepared template files.")
@_inference_options
def inference(msa, json_path, sequence, mol_type, output, templates_path, pdb_mmcif_dir, template_cache, params, num_recycles, num_samples, msa_crop_size, snapshot,
              seeds, device, optim, precision, hoist_sampler, msa_search, msa_db_dir, msa_cache_dir, logits_scheme, bucket, sample_chunk, guidance, allow_guidance_overlap,
              restraints, restraint_pairs, repels, restraint_rigid, restraint_after_step, restraint_after_sigma,
              restraint_max_step, restraint_weight, msa_pairing, matmul_precision, plot_confidences,
              allow_missing_keys, ccd, det):  # fmt: skip
    """Predict the structure of one job."""
    _setup_logging()
    _apply_hoist(hoist_sampler)
    import torch

    from ..data.inference_input import InferenceInput
    from ..inference.runner import run_job

    dist_info = None
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # launched with one process per GPU: every prediction is spread over the GPUs (row-sharded trunk, samples dealt out)
        from ..parallel.dist import init_process_group

        dist_info = init_process_group(timeout_s=1800.0)
        device = str(dist_info.device)
    model, cfg, device = _prepare_model(params, device, optim, snapshot, allow_missing_keys, det, ccd)
    if dist_info is not None:
        import torch.distributed as dist

        for tensor in list(model.parameters()) + list(model.buffers()):
            dist.broadcast(tensor.data, 0)
    if matmul_precision:
        torch.set_float32_matmul_precision(matmul_precision)
    if json_path:
        from ..data.parse.json_input import parse_json_input

        inputs = [InferenceInput.from_job(job, msa_crop_size, msa_pairing, pdb_mmcif_dir)
                  for job in parse_json_input(json_path, msa_search=_msa_search_fn(msa_search, msa_db_dir, msa_cache_dir))]
    elif msa:
        inputs = [InferenceInput.from_a3m(msa, mol_type, msa_crop_size=msa_crop_size)]
    elif sequence:
        inputs = [InferenceInput.from_sequence(sequence, mol_type, msa_crop_size=msa_crop_size)]
    else:
        raise click.ClickException("one of --json, --msa, --sequence is required")
    if templates_path and not json_path:
        _attach_templates(inputs[0], templates_path, pdb_mmcif_dir, template_cache or os.path.join(output, "templates"))
    model.cfg.msa_crop_size = msa_crop_size
    for inp in inputs:
        out_dir = output if len(inputs) == 1 else os.path.join(output, inp.name)
        terms, rkw = _job_steering(inp, guidance, allow_guidance_overlap, restraints, restraint_pairs, repels, restraint_weight,
                                   restraint_rigid, restraint_after_step, restraint_after_sigma, restraint_max_step)  # fmt: skip
        summaries = run_job(model, inp, out_dir, device, list(seeds) or None, num_recycles, num_samples,
                            getattr(torch, DTYPES[precision]), bucket, sample_chunk, logits_scheme=logits_scheme,
                            guidance_terms=terms, restraint_kwargs=rkw, manifest_fields={"params": params, "optim": optim},
                            dist_info=dist_info)  # fmt: skip
        if dist_info is not None and dist_info.rank != 0:
            continue
        if plot_confidences:
            _plot_outputs(out_dir)
        best = max(summaries, key=lambda s: s["ranking_score"])
        click.echo(f"{inp.name}: {len(summaries)} samples, best ranking score {best['ranking_score']:.3f} "
                   f"(seed {best['seed']}, sample {best['sample']}) -> {out_dir}")  # fmt: skip


@cli.command("inference-batch")
@click.option("--inputs-file", type=click.Path(exists=True), required=True, help="One JSON path per line.")
@click.option("--output-template", default="out/{name}", help="Output directory per job; {name} is the job name.")
@click.option("--skip-existing/--no-skip-existing", default=True)
@click.option("--save-distogram/--no-save-distogram", default=True)
@click.option("--shard", default=None, help="I/N: take every N-th job starting at I (one process per GPU; default from RANK / WORLD_SIZE).")
@click.option("--pdb-mmcif-dir", type=click.Path(exists=True), default=None, help="Local mmCIF mirror for template hits named by PDB id.")
@click.option("--guidance-sweep", type=click.Path(exists=True), default=None,
              help="JSON of guidance settings per group; every inputs-file line names its group (group=...), its output "
                   "directory carries {cfg}, and {pairs} in a guidance value takes the line's pairs=... Not with --guidance.")
@_inference_options
def inference_batch(inputs_file, output_template, skip_existing, save_distogram, shard, pdb_mmcif_dir, guidance_sweep, params, num_recycles, num_samples,
                    msa_crop_size, snapshot, seeds, device, optim, precision, hoist_sampler, msa_search, msa_db_dir, msa_cache_dir, logits_scheme, bucket, sample_chunk,
                    guidance, allow_guidance_overlap, restraints, restraint_pairs, repels, restraint_rigid,
                    restraint_after_step, restraint_after_sigma, restraint_max_step, restraint_weight, msa_pairing,
                    matmul_precision, plot_confidences, allow_missing_keys, ccd, det):  # fmt: skip
    """Predict many jobs with one model load; finished seeds are skipped on a re-run."""
    _setup_logging()
    import torch

    from ..data.inference_input import InferenceInput
    from ..inference.runner import run_job

    part = None
    if shard is None and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        shard = f"{os.environ.get('RANK', '0')}/{os.environ['WORLD_SIZE']}"
    if shard:
        part = tuple(int(x) for x in shard.split("/"))
        if len(part) != 2 or not 0 <= part[0] < part[1]:
            raise click.ClickException(f"--shard {shard}: need I/N with 0 <= I < N")
        if device is None and torch.cuda.is_available():
            device = f"cuda:{int(os.environ.get('LOCAL_RANK', part[0] % max(torch.cuda.device_count(), 1)))}"
    model, cfg, device = _prepare_model(params, device, optim, snapshot, allow_missing_keys, det, ccd)
    model.cfg.msa_crop_size = msa_crop_size
    if matmul_precision:
        torch.set_float32_matmul_precision(matmul_precision)
    from ..data.parse.json_input import parse_json_input

    _apply_hoist(hoist_sampler)
    if guidance_sweep and guidance:
        raise click.UsageError("--guidance-sweep and --guidance exclude each other")
    groups = load_guidance_sweep(guidance_sweep) if guidance_sweep else None
    lines = parse_inputs_file(inputs_file)
    if part is not None:
        lines = lines[part[0] :: part[1]]
    done = failed = 0
    search_fn = _msa_search_fn(msa_search, msa_db_dir, msa_cache_dir)
    for p, line_out, extras in lines:
        try:
            job_seeds = [int(x) for x in extras["seeds"].split(",")] if extras.get("seeds") else (list(seeds) or None)
            for job in parse_json_input(p, msa_search=search_fn):
                inp = InferenceInput.from_job(job, msa_crop_size, msa_pairing, pdb_mmcif_dir)
                base_dir = (line_out or output_template).replace("{name}", inp.name)
                # one run per guidance setting of the line's sweep group, all on one trunk per seed; or one run
                shared = {} if groups is not None else None
                runs = sweep_entries(groups, base_dir, extras) if groups is not None else [(None, base_dir, tuple(guidance))]
                for cfg_name, out_dir, specs in runs:
                    terms, rkw = _job_steering(inp, specs, allow_guidance_overlap, restraints, restraint_pairs, repels,
                                               restraint_weight, restraint_rigid, restraint_after_step, restraint_after_sigma,
                                               restraint_max_step)  # fmt: skip
                    fields = {"params": params, "input": p} | ({"guidance_setting": cfg_name} if cfg_name else {})
                    run_job(model, inp, out_dir, device, job_seeds, num_recycles, num_samples,
                            getattr(torch, DTYPES[precision]), bucket, sample_chunk, skip_existing, logits_scheme,
                            save_distogram, terms, rkw, manifest_fields=fields, trunk_cache=shared)  # fmt: skip
                    if plot_confidences:
                        _plot_outputs(out_dir)
                done += 1
        except click.UsageError:
            raise
        except Exception as exc:  # noqa: BLE001 - one bad job must not stop the batch
            failed += 1
            logging.getLogger(__name__).exception("job %s failed: %s", p, exc)
    click.echo(f"{done} jobs done, {failed} failed")
    if failed:
        raise SystemExit(1)


# ------------------------------------------------------------------------------------------------ weights
@cli.command()
@click.argument("checkpoint", type=click.Path(exists=True))
@click.argument("output", type=click.Path())
@click.option("--snapshot", type=click.Choice(["auto", "shadow", "average", "fast"]), default="auto")
def export(checkpoint, output, snapshot):
    """Write one weight snapshot of a ``.pt`` checkpoint as ``.safetensors`` with the model config embedded."""
    from ..inference.weights import load_state
    from ..training.checkpointing import save_safetensors

    state, cfg = load_state(checkpoint, snapshot)
    save_safetensors(output, state, cfg)
    click.echo(f"{len(state)} tensors -> {output}")


@cli.command()
@click.argument("af3_params", type=click.Path(exists=True))
@click.argument("output", type=click.Path())
def convert(af3_params, output):
    """Convert an AlphaFold 3 parameter file (``.bin`` / ``.bin.zst``) to ``.safetensors``."""
    from ..config.schema import ModelConfig
    from ..convert.af3 import convert_file
    from ..training.checkpointing import save_safetensors

    state = convert_file(af3_params)
    save_safetensors(output, state, ModelConfig())
    click.echo(f"{len(state)} tensors -> {output}")


def _mmseqs_options(fn):
    """Options of the staged local pipeline, shared by ``msa`` and ``msa-batch``."""
    for opt in reversed([
        click.option("--db-dir", type=click.Path(), default=None,
                     help="Directory with the ColabFold databases (uniref30_2302_db, colabfold_envdb_202108_db, pdb100_230517): "
                          "runs the staged search / expand / re-align / filter pipeline."),
        click.option("--use-env/--no-use-env", default=True, help="Also search the environmental database."),
        click.option("--use-templates", is_flag=True, help="Also search the PDB sequences; writes an m8 table with CIGAR strings."),
        click.option("--gpu", is_flag=True, help="GPU prefilter (databases made with makepaddedseqdb)."),
        click.option("--gpu-server", is_flag=True, help="Use a running `mmseqs gpuserver` (deploy/msa/gpuserver.sh)."),
        click.option("--threads", type=int, default=32, show_default=True),
        click.option("--mmseqs", "mmseqs_binary", default="mmseqs", show_default=True),
    ]):  # fmt: skip
        fn = opt(fn)
    return fn


def _mmseqs_settings(db_dir, use_env, use_templates, gpu, gpu_server, threads, mmseqs_binary):
    from ..data.msa.mmseqs_pipeline import MmseqsSettings

    return MmseqsSettings(db_dir, use_env=use_env, use_templates=use_templates, gpu=gpu, gpu_server=gpu_server, threads=threads,
                          binary=mmseqs_binary)  # fmt: skip


@cli.command()
@click.argument("fasta_or_sequence")
@click.option("--output", type=click.Path(), required=True, help="A3M file to write.")
@click.option("--db", default=None, help="One local MMseqs2 target database (plain search); see also --db-dir.")
@click.option("--cache-dir", type=click.Path(), default="~/.cache/deepfold3/msa")
@click.option("--host", default=None, help="MSA server URL.")
@_mmseqs_options
def msa(fasta_or_sequence, output, db, cache_dir, host, db_dir, use_env, use_templates, gpu, gpu_server, threads, mmseqs_binary):
    """Search an alignment for one sequence: the staged local pipeline (--db-dir), a plain local search (--db), or the
    ColabFold MMseqs2 API."""
    from ..data.msa import mmseqs_pipeline, search
    from ..data.parse.a3m import read_fasta_like

    seq = fasta_or_sequence
    if os.path.exists(seq):
        with open(seq) as f:
            seq = read_fasta_like(f.read())[1][0]
    cache = search.MsaCache(os.path.expanduser(cache_dir))
    if db_dir:
        settings = _mmseqs_settings(db_dir, use_env, use_templates, gpu, gpu_server, threads, mmseqs_binary)
        res = mmseqs_pipeline.search_monomer_batch([seq], settings, cache)[0]
        a3m = res["a3m"]
        if use_templates:
            with open(os.path.splitext(output)[0] + ".m8", "w") as f:
                f.write(res["m8"])
    else:
        a3m = search.search_local(seq, db, cache) if db else search.search_server([seq], cache, host or search.DEFAULT_HOST)[0]
    with open(output, "w") as f:
        f.write(a3m)
    click.echo(f"{a3m.count('>')} rows -> {output}")


@cli.command("msa-batch")
@click.option("--inputs-file", type=click.Path(exists=True), required=True, help="One job JSON per line.")
@click.option("--output-dir", type=click.Path(), required=True)
@click.option("--db", default=None)
@click.option("--cache-dir", type=click.Path(), default="~/.cache/deepfold3/msa")
@click.option("--paired/--no-paired", default=False, help="With --db-dir: also write paired alignments per complex.")
@_mmseqs_options
def msa_batch(inputs_file, output_dir, db, cache_dir, paired, db_dir, use_env, use_templates, gpu, gpu_server, threads, mmseqs_binary):
    """Search alignments for every distinct protein sequence of many jobs; writes ``{sha1}.a3m`` per sequence (and
    ``{sha1}.m8`` with --use-templates, ``paired/{job}/{sha1}.a3m`` with --paired). With --db-dir all sequences go
    through the databases in one pass."""
    import hashlib

    from ..data.msa import mmseqs_pipeline, search
    from ..data.parse.json_input import ProteinChainInput, parse_json_input

    os.makedirs(output_dir, exist_ok=True)
    cache = search.MsaCache(os.path.expanduser(cache_dir))
    seqs: dict[str, None] = {}
    complexes: dict[str, list[str]] = {}
    with open(inputs_file) as f:
        for line in f:
            if line.strip() and not line.startswith("#"):
                for job in parse_json_input(line.strip()):
                    prot = [c for c in job.chains if isinstance(c, ProteinChainInput)]
                    seqs.update(dict.fromkeys(c.sequence for c in prot if not c.unpaired_msa))
                    complexes[job.name] = [c.sequence for c in prot]
    sha = lambda s: hashlib.sha1(s.encode()).hexdigest()  # noqa: E731
    if db_dir:
        settings = _mmseqs_settings(db_dir, use_env, use_templates, gpu, gpu_server, threads, mmseqs_binary)
        todo = list(seqs)
        for s, res in zip(todo, mmseqs_pipeline.search_monomer_batch(todo, settings, cache)):
            with open(os.path.join(output_dir, sha(s) + ".a3m"), "w") as f:
                f.write(res["a3m"])
            if use_templates:
                with open(os.path.join(output_dir, sha(s) + ".m8"), "w") as f:
                    f.write(res["m8"])
        n_paired = 0
        if paired:
            names = [n for n, chains in complexes.items() if len(set(chains)) > 1]
            for name, blocks in zip(names, mmseqs_pipeline.search_pair_batch([complexes[n] for n in names], settings, cache)):
                os.makedirs(os.path.join(output_dir, "paired", name), exist_ok=True)
                for s, block in zip(dict.fromkeys(complexes[name]), blocks):
                    with open(os.path.join(output_dir, "paired", name, sha(s) + ".a3m"), "w") as f:
                        f.write(block)
                n_paired += 1
        click.echo(f"{len(seqs)} sequences searched, {n_paired} complexes paired")
        return
    for s in sorted(seqs):
        a3m = search.search_local(s, db, cache) if db else search.search_server([s], cache)[0]
        with open(os.path.join(output_dir, sha(s) + ".a3m"), "w") as f:
            f.write(a3m)
    click.echo(f"{len(seqs)} sequences searched")


@cli.command()
@click.argument("confidences_json", type=click.Path(exists=True))
@click.option("--output", type=click.Path(), default=None, help="PNG path (default: next to the JSON).")
def plot(confidences_json, output):
    """Plot pLDDT per token and the PAE matrix of one sample."""
    from ..io.plot import plot_confidences

    path = plot_confidences(confidences_json, output)
    click.echo(path)


@cli.command("bench-kernels")
@click.option("--op", default="all")
def bench_kernels(op):
    """Per-kernel timings on the current GPU."""
    import sys

    from ..ops import microbench

    sys.argv = ["microbench", "--op", op]
    microbench.main()


from . import prepare as _prepare  # noqa: E402

_prepare.register(cli)

from . import dataset_tools as _dataset_tools  # noqa: E402

for _command in _dataset_tools.COMMANDS:
    cli.add_command(_command)
# names the reference uses for commands that live in the `prepare` group here, and for its kernel warm-up
cli.add_command(_prepare.masks, "build-masks")
cli.add_command(_prepare.refilter, "refilter")
cli.add_command(_dataset_tools.warmup_kernels, "warmup-triton")


def main():
    cli()


if __name__ == "__main__":
    main()
