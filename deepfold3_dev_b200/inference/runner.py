"""Prediction jobs: features -> model -> files (reference: scripts/inference.py, scripts/inference_batch.py:145-633).

Output tree of one job::

    {out}/seed-{s}_sample-{i}/model.cif, confidences.json, logits.npz
    {out}/seed-{s}_distogram.npz
    {out}/ranking_scores.csv, {job}_summary_confidences.json, run_manifest.json

The trunk runs once per seed; samples can be drawn in chunks (``sample_chunk``) that reuse it, each
chunk re-seeded from (seed, chunk index). File writing happens on a background thread.
"""

from __future__ import annotations

import dataclasses
import logging
import os
import time

import torch

from ..io import confidences as conf
from ..io import logit_codec
from ..io.background_writer import BackgroundWriter, logits_to_host
from ..io.mmcif import save_mmcif
from ..io.run_manifest import new_manifest, write_manifest
from ..models import bucket
from ..ops import census

logger = logging.getLogger(__name__)


def sample_chunks(num_samples: int, chunk: int) -> list[int]:
    if chunk <= 0 or chunk >= num_samples:
        return [num_samples]
    return [chunk] * (num_samples // chunk) + ([num_samples % chunk] if num_samples % chunk else [])


def sample_chunk_seed(seed: int, chunk_index: int) -> int:
    return seed if chunk_index == 0 else (seed * 1_000_003 + chunk_index) % (2**31 - 1)


def _concat_outputs(parts):
    first = parts[0]
    if len(parts) == 1:
        return first
    fields = {}
    for f in dataclasses.fields(first):
        vals = [getattr(p, f.name) for p in parts]
        fields[f.name] = vals[0] if (f.name == "distogram" or vals[0] is None) else torch.cat(vals, 0)
    return dataclasses.replace(first, **fields)


def sample_dir(out_dir: str, seed: int, sample: int) -> str:
    return os.path.join(out_dir, f"seed-{seed}_sample-{sample}")


def seed_done(out_dir: str, seed: int, num_samples: int) -> bool:
    return all(os.path.exists(os.path.join(sample_dir(out_dir, seed, i), "confidences.json")) for i in range(num_samples))


@torch.inference_mode()
def predict(model, features: dict, seed: int, num_recycles: int, num_samples: int, device, dtype=torch.bfloat16,
            use_bucket: bool = True, sample_chunk: int = 0, guidance_terms=None, restraint_kwargs=None,
            trunk_cache: dict | None = None):  # fmt: skip
    """One seed: returns the unpadded ``DeepFold3Output`` with ``num_samples`` samples. ``trunk_cache`` (a dict the
    caller owns) keeps the padded features, the trunk output and the distogram of every (seed, recycles) it has seen, so
    that several guidance or restraint settings of one job run the trunk once per seed (reference:
    scripts/inference_batch.py:360-460, one trunk shared by the entries of a guidance sweep)."""
    amp = torch.autocast(device_type=torch.device(device).type, dtype=dtype, enabled=dtype != torch.float32)
    kw = dict(restraint_kwargs or {})
    key = (seed, num_recycles)
    with amp:
        if trunk_cache is not None and key in trunk_cache:
            feats, n, trunk, disto = trunk_cache[key]
        else:
            feats = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in features.items()}
            n = int(feats["res_type"].shape[0])
            if use_bucket:
                feats, n = bucket.pad_features(feats)
            trunk = model.run_evoformer(feats, num_recycles, seed=seed)
            disto = model.distogram_head(trunk[0]["pair"])
            if trunk_cache is not None:
                trunk_cache[key] = (feats, n, trunk, disto)
        parts = []
        for ci, k in enumerate(sample_chunks(num_samples, sample_chunk)):
            parts.append(model.sample_from_trunk(feats, trunk, seed=sample_chunk_seed(seed, ci), num_samples=k,
                                                 guidance_terms=guidance_terms, distogram=disto, **kw))  # fmt: skip
    return bucket.unpad_output(_concat_outputs(parts), n)


def rank_samples(num_samples: int, rank: int, world: int) -> list[int]:
    """Sample indices drawn by ``rank`` when one prediction is spread over ``world`` GPUs (round-robin)."""
    return list(range(rank, num_samples, world))


@torch.inference_mode()
def predict_distributed(model, features: dict, seed: int, num_recycles: int, num_samples: int, dist_info, dtype=torch.bfloat16,
                        use_bucket: bool = True, axial: bool = True, guidance_terms=None, restraint_kwargs=None):  # fmt: skip
    """One prediction on all GPUs of a node. The trunk runs once, its Pairformer stack row-sharded over the ranks
    (``parallel/axial.py``; every rank ends with the full pair tensor), then each rank draws its share of the samples as
    one batch, seeded from (seed, rank) like chunk ``rank`` of a chunked single-GPU run, and scores them with the
    confidence head. Returns ``(sample indices, output)`` for this
    rank; ``output`` is ``None`` on ranks without a sample (the reference spreads whole jobs over processes instead:
    bench/scripts/run_sweep.py:96-168)."""
    device = dist_info.device
    feats = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in features.items()}
    n = int(feats["res_type"].shape[0])
    if use_bucket:
        feats, n = bucket.pad_features(feats)
    if axial and dist_info.world_size > 1:
        from ..parallel.axial import AxialComm

        if getattr(model.evoformer, "_axial_comm", None) is None:
            model.evoformer._axial_comm = AxialComm(dist_info)
    amp = torch.autocast(device_type=torch.device(device).type, dtype=dtype, enabled=dtype != torch.float32)
    kw = dict(restraint_kwargs or {})
    mine = rank_samples(num_samples, dist_info.rank, dist_info.world_size)
    with amp:
        trunk = model.run_evoformer(feats, num_recycles, seed=seed)
        comm = getattr(model.evoformer, "_axial_comm", None)
        if comm is not None:
            comm.check()
        if not mine:
            return mine, None
        disto = model.distogram_head(trunk[0]["pair"])
        out = model.sample_from_trunk(feats, trunk, seed=sample_chunk_seed(seed, dist_info.rank), num_samples=len(mine),
                                      guidance_terms=guidance_terms, distogram=disto, **kw)  # fmt: skip
    return mine, bucket.unpad_output(out, n)


def write_seed(out_dir: str, job_name: str, seed: int, output, features: dict, chain_names, writer: BackgroundWriter,
               logits_scheme: str = "int8_softmax", save_distogram: bool = True, indices=None) -> list[dict]:  # fmt: skip
    """Files of the samples in ``output``; ``indices`` are their numbers within the seed when ``output`` holds only a
    subset (one prediction spread over several GPUs)."""
    host = logits_to_host(output)
    feats = {k: v.cpu() if isinstance(v, torch.Tensor) else v for k, v in features.items()}
    summaries = []
    S = host.atom_positions.shape[0]
    numbers = list(range(S)) if indices is None else list(indices)
    for i, number in enumerate(numbers):
        d = sample_dir(out_dir, seed, number)
        os.makedirs(d, exist_ok=True)
        s = conf.sample_summary(number, seed, host.plddt[i].float(), host.pae[i].float(), host.pde[i].float(),
                                host.atom_positions[i].float(), feats)  # fmt: skip
        summaries.append(s)
        one = dataclasses.replace(host, atom_positions=host.atom_positions[i : i + 1], atom_mask=host.atom_mask[i : i + 1],
                                  plddt=host.plddt[i : i + 1])  # fmt: skip
        writer.submit(save_mmcif, os.path.join(d, "model.cif"), one, feats, title=f"{job_name} seed {seed} sample {number}",
                      chain_names=chain_names)  # fmt: skip
        writer.submit(conf.save_confidences_json, os.path.join(d, "confidences.json"), s)
        heads = {"plddt": host.plddt[i], "pae": host.pae[i], "pde": host.pde[i]}
        if host.exp_resolved is not None:
            heads["exp_resolved"] = host.exp_resolved[i]
        writer.submit(logit_codec.save_logits, os.path.join(d, "logits.npz"), heads, logits_scheme)
    if save_distogram and host.distogram is not None:
        writer.submit(logit_codec.save_logits, os.path.join(out_dir, f"seed-{seed}_distogram.npz"),
                      {"distogram": host.distogram}, logits_scheme)  # fmt: skip
    return summaries


def run_job(model, inp, out_dir: str, device, seeds=None, num_recycles: int = 10, num_samples: int = 5,
            dtype=torch.bfloat16, use_bucket: bool = True, sample_chunk: int = 0, skip_existing: bool = False,
            logits_scheme: str = "int8_softmax", save_distogram: bool = True, guidance_terms=None, restraint_kwargs=None,
            manifest_fields: dict | None = None, dist_info=None, trunk_cache: dict | None = None) -> list[dict]:  # fmt: skip
    """All seeds of one job; returns the per-sample summaries (also written as CSV / JSON). With a ``dist_info`` of more
    than one rank every prediction is spread over the ranks (``predict_distributed``): each rank writes the sample
    folders of its own samples, rank 0 the files that summarise the job."""
    spread = dist_info is not None and dist_info.world_size > 1
    main = not spread or dist_info.rank == 0
    os.makedirs(out_dir, exist_ok=True)
    manifest = new_manifest(job=inp.name, num_tokens=inp.num_tokens, num_samples=num_samples, num_recycles=num_recycles,
                            **(manifest_fields or {}))  # fmt: skip
    mpath = os.path.join(out_dir, "run_manifest.json")
    if main:
        write_manifest(mpath, manifest)
    summaries, timings = [], {}
    census(reset=True)
    with BackgroundWriter() as writer:
        for seed in seeds if seeds is not None else inp.seeds:
            if skip_existing and seed_done(out_dir, seed, num_samples):
                logger.info("seed %d already complete, skipping", seed)
                continue
            t0 = time.time()
            indices = None
            if spread:
                indices, out = predict_distributed(model, inp.features, seed, num_recycles, num_samples, dist_info, dtype,
                                                   use_bucket, True, guidance_terms, restraint_kwargs)  # fmt: skip
            else:
                out = predict(model, inp.features, seed, num_recycles, num_samples, device, dtype, use_bucket, sample_chunk,
                              guidance_terms, restraint_kwargs, trunk_cache)  # fmt: skip
            if torch.cuda.is_available() and torch.device(device).type == "cuda":
                torch.cuda.synchronize()
            timings[f"seed-{seed}"] = time.time() - t0
            mine = []
            if out is not None:
                mine = write_seed(out_dir, inp.name, seed, out, inp.features, inp.chain_names, writer, logits_scheme,
                                  save_distogram and main, indices)  # fmt: skip
            if spread:
                import torch.distributed as dist

                gathered = [None] * dist_info.world_size
                dist.all_gather_object(gathered, mine)
                mine = sorted((s for part in gathered for s in part), key=lambda s: s.get("sample", 0))
            summaries += mine
    if torch.cuda.is_available() and torch.device(device).type == "cuda":
        from ..ops import autograd_ops

        autograd_ops.check_status()  # a kernel wait that ran out anywhere in the job makes its files suspect: fail loudly
    if not main:
        return summaries
    if summaries:
        conf.save_ranking_scores_csv(os.path.join(out_dir, "ranking_scores.csv"), summaries)
        conf.save_summary_confidences_json(os.path.join(out_dir, f"{inp.name}_summary_confidences.json"), summaries, inp.name)
    manifest.update(status="done", seconds_per_seed=timings, kernel_census=census())
    write_manifest(mpath, manifest)
    return summaries
