"""Training examples -> batches (reference: data/module/dataset.py:238-602, data/module/collate.py:31-130,
training/data.py:40-561).

``FeatureDirDataset`` reads examples that were featurised ahead of time (one ``.pt`` feature dict per
example, optionally inside pack shards, see ``data/pack.py``) and applies the training-time steps:
crop to the token / atom budget, random rotation of each reference conformer, bookkeeping keys. Building
those files from mmCIF needs gemmi / RDKit, which are not installable offline; ``SyntheticDataset``
generates examples of the same schema for benchmarks and tests.
"""

from __future__ import annotations

import json
import logging
import os

import torch

from . import cropper, io_cache, pack as packs
from .synthetic import split_lengths, synthetic_complex

PAD_VALUES = {"msa": 21}

logger = logging.getLogger(__name__)


def rotate_reference_conformers(feats: dict, gen: torch.Generator) -> dict:
    """Independent random rotation + small translation of every ``ref_space_uid`` group (AF3 §2.8)."""
    from ..models.diffusion_modules import random_rigid_transforms

    uid = feats["ref_space_uid"]
    groups = int(uid.max()) + 1
    rot, trans = random_rigid_transforms((groups,), uid.device, gen)
    R, t = rot[uid], trans[uid] * 0.0
    pos = torch.einsum("nmij,nmj->nmi", R, feats["ref_pos"]) + t
    return {**feats, "ref_pos": pos * feats["ref_mask"].unsqueeze(-1)}


class SyntheticDataset:
    def __init__(self, num_tokens=384, num_chains=2, num_msa=1024, num_templates=4, length=1 << 30, seed=0):
        self.cfg = (num_tokens, num_chains, num_msa, num_templates)
        self.length, self.seed = length, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i: int) -> dict:
        n, c, s, t = self.cfg
        chains = [("protein", L) for L in split_lengths(n, c)]
        f = synthetic_complex(chains, num_msa=s, num_templates=t, seed=self.seed + i)
        f["_record_id"] = f"synthetic-{self.seed + i}"
        return f


class FeatureDirDataset:
    """Directory of ``<id>.pt`` feature dicts plus optional ``manifest.json`` (``[{id, chains, interfaces, ...}]``)."""

    def __init__(self, root: str, max_tokens: int = 384, max_atoms: int = 0, crop_weights: dict | None = None,
                 is_distillation: bool = False, seed: int = 0, pack=None, atomize_prob: float = 0.0,
                 atomize_source: str = "random", atomize_max_residues: int = 0):  # fmt: skip
        self.root, self.max_tokens, self.max_atoms = root, max_tokens, max_atoms
        self.atomize_prob, self.atomize_max_residues = atomize_prob, atomize_max_residues  # the source is always "random" here
        self.crop_weights, self.is_distillation, self.seed = crop_weights, is_distillation, seed
        self.pack = pack if pack is not None else packs.register(root)
        man = os.path.join(root, "manifest.json")
        if os.path.exists(man):
            with open(man) as f:
                self.records = json.load(f)
        else:
            names = set(n for n in os.listdir(root) if n.endswith(".pt"))
            if self.pack is not None:
                names |= {k for k in self.pack.keys() if k.endswith(".pt") and "/" not in k}
            self.records = [{"id": n[:-3]} for n in sorted(names)]
        self.bad = 0

    def __len__(self):
        return len(self.records)

    def weights(self) -> list[float]:
        from .samplers import example_weight

        return [example_weight(r.get("chains", [{}]), r.get("interfaces")) for r in self.records]

    def _load(self, rec) -> dict:
        name = rec["id"] + ".pt"
        if self.pack is not None and self.pack.exists(name):
            import io

            return torch.load(io.BytesIO(self.pack.read_bytes(name)), map_location="cpu", weights_only=False)
        return torch.load(os.path.join(self.root, name), map_location="cpu", weights_only=False)

    def __getitem__(self, i: int) -> dict:
        rec = self.records[i % len(self.records)]
        gen = torch.Generator().manual_seed(self.seed * 7_654_321 + i)
        feats = self._load(rec)
        if self.atomize_prob > 0:
            from .atomize import atomize_stored_features

            feats = atomize_stored_features(feats, gen, self.atomize_prob, self.atomize_max_residues)
        feats, strategy = cropper.crop(feats, self.max_tokens, self.max_atoms, gen, self.crop_weights)
        feats = rotate_reference_conformers(feats, gen)
        feats.setdefault("resolution", torch.tensor(float(rec.get("resolution", 0.0))))
        feats["is_distillation"] = torch.tensor(bool(self.is_distillation))
        feats["_record_id"] = rec["id"]
        feats["_crop"] = strategy
        return feats


def collate(samples: list[dict], pad_tokens_to: int | None = None, pad_msa_to: int | None = None) -> dict:
    """Right-pad every tensor key to the batch maximum (or to fixed sizes) and stack; keys missing anywhere are dropped."""
    keys = set(samples[0])
    for s in samples[1:]:
        keys &= set(s)
    out = {}
    for k in sorted(keys):
        vals = [s[k] for s in samples]
        if not isinstance(vals[0], torch.Tensor):
            out[k] = vals
            continue
        if vals[0].dim() == 0:
            out[k] = torch.stack(vals)
            continue
        shape = [max(v.shape[d] for v in vals) for d in range(vals[0].dim())]
        if pad_tokens_to or pad_msa_to:
            n = max(int(s["res_type"].shape[0]) for s in samples)
            m = max(int(s["msa"].shape[0]) for s in samples) if "msa" in samples[0] else 0
            for d in range(len(shape)):
                if pad_tokens_to and shape[d] == n and k not in ("template_mask",):
                    shape[d] = max(shape[d], pad_tokens_to)
                elif pad_msa_to and d == 0 and shape[d] == m and k in ("msa", "msa_mask", "deletion_matrix"):
                    shape[d] = max(shape[d], pad_msa_to)
        padded = []
        for v in vals:
            pad = []
            for d in reversed(range(v.dim())):
                pad += [0, shape[d] - v.shape[d]]
            padded.append(torch.nn.functional.pad(v, pad, value=PAD_VALUES.get(k, 0)) if any(pad) else v)
        out[k] = torch.stack(padded)
    return out


class BatchStream:
    """Iterator of collated batches: ``sampler`` -> ``dataset[i]`` -> ``collate``; bad examples are skipped and counted."""

    def __init__(self, dataset, sampler, batch_size: int = 1, pad_tokens_to: int | None = None, max_retries: int = 20):
        self.dataset, self.sampler, self.batch_size = dataset, sampler, batch_size
        self.pad_tokens_to, self.max_retries, self.dropped = pad_tokens_to, max_retries, 0
        self.served = self.retries = 0
        self.errors: dict[str, int] = {}   # exception type -> how many examples it cost (reference: dataset.py:99-191)

    def counters(self) -> dict:
        """Log entries: examples served and dropped, retries, and the drop count per exception type."""
        out = {"data/served": self.served, "data/dropped": self.dropped, "data/retries": self.retries}
        out.update({f"data/dropped/{name}": n for name, n in sorted(self.errors.items())})
        for key in ("msa_read", "msa_skipped"):
            if hasattr(self.dataset, key):
                out[f"data/{key}"] = getattr(self.dataset, key)
        return out

    def __iter__(self):
        return self

    def __next__(self) -> dict:
        items = []
        while len(items) < self.batch_size:
            for attempt in range(self.max_retries):
                try:
                    items.append(self.dataset[next(self.sampler)])
                    self.served += 1
                    self.retries += attempt
                    break
                except StopIteration:
                    raise
                except Exception as exc:  # noqa: BLE001 - a broken example must not stop the run
                    self.dropped += 1
                    name = type(exc).__name__
                    self.errors[name] = self.errors.get(name, 0) + 1
                    if self.errors[name] <= 3:
                        import logging

                        logging.getLogger(__name__).warning("dropping an example (%s: %s)", name, exc)
            else:
                raise RuntimeError(f"{self.max_retries} consecutive examples failed to load")
        return collate(items, self.pad_tokens_to)


class PrefetchStream:
    """Runs an iterator of batches on background threads, ``depth`` batches ahead (reference: training/data.py DataLoader
    wiring with ``num_workers`` / ``prefetch_factor``).

    Loading, cropping and collating are file reads and torch ops, both of which release the interpreter lock, so
    threads overlap them with the training step without the copy through worker processes. Order is preserved with
    one worker; with several workers batches arrive in completion order.
    """

    def __init__(self, make_stream, depth: int = 4, workers: int = 1):
        import queue
        import threading

        self._q: queue.Queue = queue.Queue(maxsize=max(1, depth))
        self._stop = threading.Event()
        self._err: BaseException | None = None
        self._threads = []
        for w in range(max(1, workers)):
            t = threading.Thread(target=self._run, args=(make_stream(w),), name=f"df3-data-{w}", daemon=True)
            t.start()
            self._threads.append(t)

    def _run(self, stream):
        try:
            for batch in stream:
                while not self._stop.is_set():
                    try:
                        self._q.put(batch, timeout=0.2)
                        break
                    except Exception:  # noqa: BLE001 - queue.Full: keep waiting unless stopped
                        continue
                if self._stop.is_set():
                    return
        except BaseException as exc:  # noqa: BLE001 - surfaced by the consumer
            self._err = exc
            self._q.put(None)

    def __iter__(self):
        return self

    def __next__(self):
        item = self._q.get()
        if item is None:
            raise RuntimeError(f"data worker failed: {self._err!r}") from self._err
        return item

    def close(self) -> None:
        self._stop.set()


def apply_date_cutoff(records: list, cutoff: str, keep_after: bool = False) -> list:
    """Release-date split (reference: training/data.py:64-92). ``keep_after=False`` keeps entries released on or before
    ``cutoff`` (training side), ``True`` those released after it (evaluation side). An entry without a release date is
    dropped on both sides: it cannot be shown to be on the right side. An empty ``cutoff`` keeps everything."""
    if not cutoff:
        return list(records)
    out = []
    for r in records:
        released = r.structure_info.released if r.structure_info is not None else None
        if not released:
            continue
        if (released > cutoff) == keep_after:
            out.append(r)
    return out


class StructureDataset:
    """Prepared structures featurised on the fly (reference: data/module/dataset.py:238-602, ``TrainingDataset``).

    ``root`` is the output of ``prepare structures``: ``manifest.json``, ``structures/<id>.npz`` and optionally
    ``msa/<msa_id>.npz`` / ``.a3m``. Per sample: pick the anchor chain or interface, pre-crop large assemblies to the
    chains around it, featurise, crop to the token budget, then rotate the reference conformers. MSAs are read only for
    chains that survive the chain pre-crop.
    """

    def __init__(self, root: str, max_tokens: int = 384, max_atoms: int = 0, crop_weights: dict | None = None,
                 is_distillation: bool = False, seed: int = 0, max_chains: int = 20, max_msa_rows: int = 16384,
                 msa_dir: str | None = None, cutoff_date: str = "", keep_after: bool = False, atomize_prob: float = 0.0,
                 atomize_source: str = "random", atomize_max_residues: int = 0, pdb_chain_cache_dir: str | None = None,
                 max_templates: int = 4, template_cutoff_days: int = 60, max_template_date: str | None = None,
                 default_template_cutoff_date: str | None = None, slow_sample_log_threshold_s: float = 0.0):  # fmt: skip
        from .types import load_manifest

        self.slow_threshold_s = slow_sample_log_threshold_s

        self.root, self.max_tokens, self.max_atoms = root, max_tokens, max_atoms
        self.crop_weights, self.is_distillation, self.seed = crop_weights, is_distillation, seed
        self.max_chains, self.max_msa_rows = max_chains, max_msa_rows
        self.atomize = {"atomize_prob": atomize_prob, "atomize_source": atomize_source, "atomize_max_residues": atomize_max_residues}
        # templates: per-sequence hit lists under the dataset root, coordinates from a per-chain cache (`build-pdb-cache`)
        self.pdb_chain_cache_dir, self.max_templates = pdb_chain_cache_dir, max_templates
        self.template_cutoff_days, self.max_template_date = template_cutoff_days, max_template_date
        self.default_template_cutoff_date = default_template_cutoff_date
        self.templates_used = self.templates_dropped = 0
        self.msa_dir = msa_dir or os.path.join(root, "msa")
        packs.register(root)  # structures/ and msa/ may live in {root}/_pack
        if msa_dir:
            packs.register(os.path.dirname(os.path.abspath(msa_dir)))
        self.records = [r for r in load_manifest(os.path.join(root, "manifest.json")) if any(c.valid for c in r.chains)]
        self.records = apply_date_cutoff(self.records, cutoff_date, keep_after)
        self.msa_read = self.msa_skipped = 0  # alignments opened / never opened because their chain was cropped away
        self._anchors = None

    def __len__(self):
        return len(self.records)

    def anchor_tables(self):
        if self._anchors is None:
            from .samplers import anchor_tables

            self._anchors = anchor_tables(self.records)
        return self._anchors

    def weights(self) -> list[float]:
        """Record marginal of the AF3 weighting: the sum of the record's chain and interface anchor weights."""
        from .samplers import record_weights

        return record_weights(self.anchor_tables())

    def _templates(self, rec, chain, rng):
        """Templates of one protein chain for this draw of the example (reference: data/module/dataset.py:772-870)."""
        import json

        from . import const
        from . import templates as tpl

        if chain.mol_type != const.MOL_PROTEIN:
            return []
        index = tpl.monomer_template_index(self.root, chain.msa_id)
        if index is None:
            return []
        try:
            hits = json.loads(io_cache.read_text(index))
        except (OSError, ValueError):
            self.templates_dropped += 1
            return []
        released = rec.structure_info.released if rec.structure_info else None
        cutoff = tpl.template_cutoff(released, self.template_cutoff_days, self.max_template_date, self.default_template_cutoff_date)
        out = []
        for hit in tpl.sample_training_templates(hits, rec.id, cutoff, rng, self.max_templates):
            pdb = str(hit.get("template_pdb_id") or hit.get("pdbId"))
            chain_id = str(hit.get("template_chain_id") or hit.get("chainId") or "A")
            path = tpl.chain_cache_path(self.pdb_chain_cache_dir, pdb, chain_id)
            try:
                q, t = tpl.hit_index_pairs(hit)
                if path is not None:
                    out.append(tpl.load_template_chain(path, q, t))
                    continue
                # not in the per-chain cache: read the entry from the local mmCIF mirror, if one was named
                mirror = os.environ.get("DF3_TEMPLATE_MMCIF_DIR")
                src = tpl.find_pdb_mmcif(pdb, mirror) if mirror else None
                chain_obj = tpl.template_chain_from_mmcif(src, chain_id, q, t) if src else None
                if chain_obj is None:
                    self.templates_dropped += 1
                else:
                    out.append(chain_obj)
            except (KeyError, ValueError, OSError):
                self.templates_dropped += 1
        self.templates_used += len(out)
        return out

    def _msa(self, chain):
        from .parse.a3m import msa_from_a3m_file
        from .types import MSA

        base = os.path.join(self.msa_dir, str(chain.msa_id))
        if io_cache.exists(base + ".npz"):
            return MSA.load(base + ".npz")
        if io_cache.exists(base + ".a3m"):
            return msa_from_a3m_file(base + ".a3m", chain.mol_type, self.max_msa_rows)
        return None

    def __getitem__(self, i: int) -> dict:
        from .types import Structure

        rec = self.records[i % len(self.records)]
        st = Structure.load(os.path.join(self.root, "structures", f"{rec.id}.npz"))
        feats, read, skipped = featurize_record(
            st, rec, lambda chain: self._msa(chain), max_tokens=self.max_tokens, max_atoms=self.max_atoms,
            crop_weights=self.crop_weights, max_chains=self.max_chains, max_msa_rows=self.max_msa_rows,
            seed=self.seed * 7_654_321 + i, is_distillation=self.is_distillation,
            anchors=self.anchor_tables()[i % len(self.records)], **self.atomize,
            load_templates=(lambda chain, rng: self._templates(rec, chain, rng)) if self.pdb_chain_cache_dir else None,
            max_templates=self.max_templates, slow_threshold_s=self.slow_threshold_s,
        )  # fmt: skip
        self.msa_read, self.msa_skipped = self.msa_read + read, self.msa_skipped + skipped
        return feats


def featurize_record(st, rec, load_msa, *, max_tokens: int = 384, max_atoms: int = 0, crop_weights: dict | None = None,
                     max_chains: int = 20, max_msa_rows: int = 16384, seed: int = 0, is_distillation: bool = False,
                     anchors=None, atomize_prob: float = 0.0, atomize_source: str = "random", atomize_max_residues: int = 0,
                     load_templates=None, max_templates: int = 4, slow_threshold_s: float = 0.0):
    """One training example from a stored structure and its manifest record: pick the anchor chain or interface
    (in proportion to the anchor weights of ``anchors = (anchor list, weights)`` when given, else uniformly),
    pre-crop large assemblies to the chains around it, featurise, crop to the token budget, read the alignments of
    what survived (``load_msa(chain_info)`` -> ``MSA`` or ``None``), rotate the reference conformers. Returns the
    features and the numbers of alignments read and skipped. With ``slow_threshold_s > 0`` an example that took longer
    is reported in one ``SLOW_SAMPLE`` log line with the wall time of every phase (reference:
    data/module/dataset.py:565-578)."""
    import random
    import time

    clock = [("start", time.perf_counter())]
    mark = lambda name: clock.append((name, time.perf_counter()))  # noqa: E731

    from .featurize import attach_cropped_msa, attach_cropped_templates, featurize_structure
    from .prepare.filters import select_interface_chains

    gen = torch.Generator().manual_seed(seed)
    rng = random.Random(seed)
    valid = [c for c in rec.chains if c.valid]
    faces = [f for f in rec.interfaces if f.valid]
    if anchors is not None and anchors[0]:
        anchor = rng.choices(anchors[0], weights=anchors[1], k=1)[0]
    elif faces and rng.random() < 0.5:
        f = rng.choice(faces)
        anchor = ("interface", f.chain_1, f.chain_2)
    else:
        anchor = ("chain", rng.choice(valid).chain_id, -1)
    keep = select_interface_chains(st, anchor, max_chains, rng=rng) & {c.chain_id for c in valid}
    old_ids = sorted(keep)
    sub = st.select_chains(old_ids)
    mark("select_chains")
    # crop first, then read alignments only for the chains (and columns) that survived
    atomize = _residues_to_atomize(sub, rng, atomize_prob, atomize_source, atomize_max_residues)
    feats = featurize_structure(sub, None, max_msa_rows=max_msa_rows, with_msa=False, atomize=atomize)
    chain_cols, token_col, chain_len = feats.pop("_chain_cols"), feats.pop("_token_col"), feats.pop("_chain_len")
    mark("featurize")
    # the anchor in the numbering of the featurised sub-structure (chains renumbered in the order of old_ids)
    new_of_old = {c: k for k, c in enumerate(old_ids)}
    crop_anchor = (anchor[0], new_of_old.get(anchor[1], -1), new_of_old.get(anchor[2], -1)) if anchor[1] in new_of_old else None
    feats, strategy, kept = cropper.crop(feats, max_tokens, max_atoms, gen, crop_weights, return_keep=True, anchor=crop_anchor)
    mark("crop")
    feats, read, skipped = attach_cropped_msa(feats, kept, chain_cols, lambda a: load_msa(rec.chains[old_ids[a]]),
                                              max_msa_rows=max_msa_rows, token_col=token_col, chain_len=chain_len)  # fmt: skip
    mark("msa")
    if load_templates is not None:  # ``load_templates(chain_info, rng)`` -> TemplateChain list of a protein chain
        tfeats, _ = attach_cropped_templates(feats, kept, chain_cols, token_col, chain_len,
                                             lambda a: load_templates(rec.chains[old_ids[a]], rng), max_templates)  # fmt: skip
        feats.update(tfeats)
        mark("templates")
    feats = rotate_reference_conformers(feats, gen)
    from .symmetry import symmetry_features

    feats.update(symmetry_features(feats))  # exchangeable atoms and ligand automorphisms, indexed in the cropped example
    mark("symmetry")
    total = clock[-1][1] - clock[0][1]
    if 0 < slow_threshold_s < total:
        phases = " ".join(f"{name}={t1 - t0:.2f}s" for (_, t0), (name, t1) in zip(clock, clock[1:]))
        logger.warning("SLOW_SAMPLE %s total=%.2fs tokens=%d chains=%d %s", rec.id, total, int(feats["res_type"].shape[0]),
                       len(old_ids), phases)  # fmt: skip
    info = rec.structure_info
    feats["resolution"] = torch.tensor(float(info.resolution) if info and info.resolution else 0.0)
    feats["is_distillation"] = torch.tensor(bool(is_distillation))
    feats["_record_id"] = rec.id
    feats["_crop"] = strategy
    return feats, read, skipped


def _residues_to_atomize(st, rng, prob: float, source: str = "random", max_residues: int = 0, interface_distance: float = 15.0) -> set[int]:
    """Rows of ``st.residues`` to tokenise per atom in this example: every standard polymer residue with more than one
    atom is picked with probability ``prob`` (``source="interface"``: only residues whose centre lies within
    ``interface_distance`` of a residue of another chain), at most ``max_residues`` of them (0: no cap). Training only;
    the crop that follows counts the extra tokens (reference: data/tokenize/atomize.py:109-131)."""
    if prob <= 0.0:
        return set()
    import numpy as np

    from . import const

    if source not in ("random", "interface"):
        raise ValueError(f"unknown atomize_source {source!r} (random | interface)")
    eligible, centres, owners = [], [], []
    xyz = st.coords()
    for c in st.chains:
        if int(c["mol_type"]) == const.MOL_NONPOLYMER:
            continue
        first = int(c["res_idx"])
        for k, r in enumerate(st.residues[first : first + int(c["res_num"])]):
            a0, n = int(r["atom_idx"]), int(r["atom_num"])
            present = st.atoms["is_present"][a0 : a0 + n]
            if bool(r["is_standard"]) and n > 1 and present.any():
                eligible.append(first + k)
                centres.append(xyz[a0 : a0 + n][present].mean(0))
                owners.append(int(c["asym_id"]))
    if not eligible:
        return set()
    if source == "interface":
        pts, own = np.asarray(centres), np.asarray(owners)
        d = np.linalg.norm(pts[:, None] - pts[None], axis=-1)
        touch = ((d < interface_distance) & (own[:, None] != own[None])).any(-1)
        eligible = [e for e, t in zip(eligible, touch) if t]
    picked = [e for e in eligible if rng.random() < prob]
    if max_residues > 0 and len(picked) > max_residues:
        picked = rng.sample(picked, max_residues)
    return set(picked)


def open_dataset(path: str, format: str = "df3", of3_cache_dir: str = "", **kw):
    """The dataset behind one entry of a recipe's ``datasets`` list (reference: training/data.py:40-561). ``df3``: a
    directory of ``.pt`` features or the output of ``prepare structures`` (featurised on the fly); ``of3`` / ``of3pdb``:
    an OpenFold 3 structure directory read in place, the latter with its columnar metadata cache (release-date cut-off,
    cluster-balanced weights)."""
    from . import paths

    template_keys = ("pdb_chain_cache_dir", "max_templates", "template_cutoff_days", "max_template_date", "default_template_cutoff_date",
                     "slow_sample_log_threshold_s")  # fmt: skip
    template_kw = {k: kw.pop(k) for k in template_keys if k in kw}  # per-sequence hit lists exist for prepared roots only
    if format in ("of3", "of3pdb"):
        from .of3 import OF3StructureDataset

        cutoff = kw.pop("cutoff_date", "") or None
        kw.pop("keep_after", None)
        return OF3StructureDataset(path, cache_dir=of3_cache_dir or None, max_release_date=cutoff, **kw)
    if format != "df3":
        raise ValueError(f"dataset format must be df3|of3|of3pdb, got {format!r}")
    if paths.is_prepared_root(path):
        return StructureDataset(path, **kw, **template_kw)
    return FeatureDirDataset(path, **kw)
