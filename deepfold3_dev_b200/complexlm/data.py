"""Store, sampling, cropping, masking and packing for the complex language model.

Reference: complexlm/store.py (flat memory-mapped ``.npy`` store, sequences deduplicated globally so two slots are the
same entity exactly when they share a chain row), sampler.py (source -> homo/hetero -> cluster -> member), crop.py
(proportional per-chain budget, window anchored on an interface residue, copies of an entity share the window),
masking.py (15 % / 30 % at interfaces, 80/10/10 corruption, copies of an entity share one draw), dataset.py (pack
examples into one token axis up to the token budget).

Store files under ``{root}``: ``seq.npy`` uint8 [R], ``chain_off.npy`` int64 [C+1], ``chain_cluster.npy`` int32 [C],
``slot_chain.npy`` int32 [S], ``slot_iface.npy`` uint8 (per slot residue, optional), ``cx_off.npy`` int64 [N+1],
``cx_cluster.npy`` int32 [N], ``cx_date.npy`` int32 [N] (YYYYMMDD, 0 unknown), ``ids.txt``, ``meta.json``.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass

import numpy as np
import torch

from .config import DataConfig, MaskingConfig, SourceConfig
from .model import IGNORE_INDEX, MASK_ID, PackedBatch, encode, standard_token_ids


# ---------------------------------------------------------------------------------------------------------------
# store
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class StoredComplex:
    id: str
    chains: list[np.ndarray]  # token ids per slot
    entity: np.ndarray  # chain row per slot (equal rows = same sequence)
    iface: list[np.ndarray] | None
    cluster: int
    date: int

    @property
    def is_homomer(self) -> bool:
        return len(self.chains) > 1 and len(set(self.entity.tolist())) == 1


class ComplexStoreWriter:
    def __init__(self, root: str, source: str, with_iface: bool):
        os.makedirs(root, exist_ok=True)
        self.root, self.source, self.with_iface = root, source, with_iface
        self.row_of: dict[bytes, int] = {}
        self.seqs: list[np.ndarray] = []
        self.slot_chain: list[int] = []
        self.slot_iface: list[np.ndarray] = []
        self.cx_off, self.cx_date, self.ids = [0], [], []

    def add(self, cid: str, sequences: list[str], iface: list[np.ndarray] | None = None, date: int = 0) -> None:
        for k, s in enumerate(sequences):
            ids = encode(s)
            row = self.row_of.setdefault(ids.tobytes(), len(self.seqs))
            if row == len(self.seqs):
                self.seqs.append(ids)
            self.slot_chain.append(row)
            if self.with_iface:
                flags = np.zeros(len(ids), np.uint8) if iface is None else np.asarray(iface[k], np.uint8)
                self.slot_iface.append(flags)
        self.cx_off.append(len(self.slot_chain))
        self.cx_date.append(int(date))
        self.ids.append(cid)

    def close(self, **meta) -> dict:
        save = lambda n, v, dt: np.save(os.path.join(self.root, n), np.asarray(v, dtype=dt))  # noqa: E731
        save("seq.npy", np.concatenate(self.seqs) if self.seqs else np.zeros(0), np.uint8)
        save("chain_off.npy", np.concatenate([[0], np.cumsum([len(s) for s in self.seqs])]), np.int64)
        save("chain_cluster.npy", np.full(len(self.seqs), -1), np.int32)
        save("slot_chain.npy", self.slot_chain, np.int32)
        if self.with_iface:
            save("slot_iface.npy", np.concatenate(self.slot_iface) if self.slot_iface else np.zeros(0), np.uint8)
        save("cx_off.npy", self.cx_off, np.int64)
        save("cx_cluster.npy", np.full(len(self.ids), -1), np.int32)
        save("cx_date.npy", self.cx_date, np.int32)
        with open(os.path.join(self.root, "ids.txt"), "w") as f:
            f.write("\n".join(self.ids) + ("\n" if self.ids else ""))
        info = {"source": self.source, "complexes": len(self.ids), "chains": len(self.seqs), "slots": len(self.slot_chain),
                "with_iface": self.with_iface, **meta}  # fmt: skip
        with open(os.path.join(self.root, "meta.json"), "w") as f:
            json.dump(info, f, indent=1)
        return info


class ComplexStore:
    def __init__(self, root: str):
        self.root = root
        ld = lambda n: np.load(os.path.join(root, n), mmap_mode="r")  # noqa: E731
        self.seq, self.chain_off, self.chain_cluster = ld("seq.npy"), ld("chain_off.npy"), ld("chain_cluster.npy")
        self.slot_chain, self.cx_off = ld("slot_chain.npy"), ld("cx_off.npy")
        self.cx_cluster, self.cx_date = ld("cx_cluster.npy"), ld("cx_date.npy")
        self.has_iface = os.path.exists(os.path.join(root, "slot_iface.npy"))
        if self.has_iface:
            self.slot_iface = ld("slot_iface.npy")
            lens = (self.chain_off[1:] - self.chain_off[:-1])[np.asarray(self.slot_chain)]
            self.slot_iface_off = np.concatenate([[0], np.cumsum(lens)])
        with open(os.path.join(root, "ids.txt")) as f:
            self.ids = [line.strip() for line in f if line.strip()]
        with open(os.path.join(root, "meta.json")) as f:
            self.meta = json.load(f)

    @property
    def name(self) -> str:
        return self.meta.get("source", os.path.basename(self.root.rstrip("/")))

    def __len__(self) -> int:
        return len(self.cx_off) - 1

    def n_entities(self) -> np.ndarray:
        return np.array([len(set(self.slot_chain[self.cx_off[i] : self.cx_off[i + 1]].tolist())) for i in range(len(self))])

    def n_chains(self) -> np.ndarray:
        return np.diff(np.asarray(self.cx_off))

    def example(self, i: int) -> StoredComplex:
        s0, s1 = int(self.cx_off[i]), int(self.cx_off[i + 1])
        rows = np.asarray(self.slot_chain[s0:s1])
        chains = [np.asarray(self.seq[self.chain_off[r] : self.chain_off[r + 1]]) for r in rows]
        iface = None
        if self.has_iface:
            iface = [np.asarray(self.slot_iface[self.slot_iface_off[s] : self.slot_iface_off[s + 1]]).astype(bool) for s in range(s0, s1)]
        return StoredComplex(self.ids[i], chains, rows, iface, int(self.cx_cluster[i]), int(self.cx_date[i]))


# ---------------------------------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------------------------------
def eligible_indices(store: ComplexStore, src: SourceConfig, min_chains: int = 1, max_chains: int = 1 << 30) -> np.ndarray:
    """Complexes a source view may draw: date window (fail-closed on unknown dates), chain count, holdout split, caps."""
    idx = np.arange(len(store))
    date = np.asarray(store.cx_date)
    ok = np.ones(len(store), bool)
    if src.date_max is not None or src.date_min is not None:
        known = date > 0
        ok &= known | src.allow_undated
        if src.date_max is not None:
            ok &= ~known | (date <= src.date_max)
        if src.date_min is not None:
            ok &= ~known | (date > src.date_min)
    n = store.n_chains()
    ok &= (n >= min_chains) & (n <= max_chains)
    if src.holdout_every:
        held = idx % src.holdout_every == 0
        ok &= held if src.holdout_side == "eval" else ~held
    if src.exclude_ids and os.path.exists(src.exclude_ids):
        with open(src.exclude_ids) as f:
            bad = {line.strip() for line in f}
        ok &= np.array([i not in bad for i in store.ids])
    idx = idx[ok]
    return idx[: src.max_complexes] if src.max_complexes else idx


class SourceView:
    """One source of the mixture: homo / hetero buckets, each drawn cluster-first when cluster ids exist."""

    def __init__(self, store: ComplexStore, src: SourceConfig, data: DataConfig):
        self.store, self.cfg = store, src
        idx = eligible_indices(store, src, data.min_chains, data.max_chains)
        ent = store.n_entities()[idx] if len(idx) else np.zeros(0, int)
        nch = store.n_chains()[idx] if len(idx) else np.zeros(0, int)
        homo = (ent == 1) & (nch >= 1)
        self.buckets, self.bucket_w = [], []
        for members, w in ((idx[homo], src.homo_weight), (idx[~homo], src.hetero_weight)):
            if not len(members):
                continue
            clusters = np.asarray(store.cx_cluster)[members]
            groups = None
            if src.cluster_balanced and (clusters >= 0).all():
                order = np.argsort(clusters, kind="stable")
                bounds = np.flatnonzero(np.diff(clusters[order])) + 1
                groups = np.split(members[order], bounds)
            self.buckets.append((members, groups))
            self.bucket_w.append(float(len(members)) if w is None else float(w))
        self.bucket_w = np.asarray(self.bucket_w) / max(sum(self.bucket_w), 1e-12)
        self.indices = idx

    def __len__(self) -> int:
        return len(self.indices)

    def draw(self, rng: np.random.Generator) -> int:
        members, groups = self.buckets[rng.choice(len(self.buckets), p=self.bucket_w)]
        if groups is not None:
            g = groups[rng.integers(len(groups))]
            return int(g[rng.integers(len(g))])
        return int(members[rng.integers(len(members))])

    def clusters_in_use(self) -> set[int]:
        c = np.asarray(self.store.cx_cluster)[self.indices]
        return set(c[c >= 0].tolist())


class MixtureSampler:
    def __init__(self, views: list[SourceView]):
        self.views = [v for v in views if len(v)]
        if not self.views:
            raise ValueError("no source has an eligible complex")
        w = np.array([v.cfg.weight for v in self.views], dtype=np.float64)
        self.p = w / w.sum()

    def draw(self, rng: np.random.Generator) -> tuple[int, int]:
        v = int(rng.choice(len(self.views), p=self.p))
        return v, self.views[v].draw(rng)


def build_views(data: DataConfig, sources: list[SourceConfig] | None = None) -> list[SourceView]:
    return [SourceView(ComplexStore(os.path.join(data.data_root, s.name)), s, data) for s in (sources or data.sources)]


def drop_overlapping_clusters(eval_views: list[SourceView], train_views: list[SourceView]) -> int:
    """Remove evaluation complexes whose complex cluster occurs in training (same clustering run only)."""
    dropped = 0
    for ev in eval_views:
        run = ev.store.meta.get("cluster_run")
        seen = set().union(*[tv.clusters_in_use() for tv in train_views if tv.store.meta.get("cluster_run") == run] or [set()])
        if run is None or not seen:
            continue
        c = np.asarray(ev.store.cx_cluster)[ev.indices]
        keep = ~np.isin(c, list(seen))
        dropped += int((~keep).sum())
        ev.indices = ev.indices[keep]
        ev.buckets = [(m[np.isin(m, ev.indices)], None) for m, _ in ev.buckets]
    return dropped


# ---------------------------------------------------------------------------------------------------------------
# crop + mask
# ---------------------------------------------------------------------------------------------------------------
def crop_complex(rng: np.random.Generator, lengths: list[int], entity: np.ndarray, iface: list[np.ndarray] | None,
                 max_chain_len: int, max_complex_len: int) -> list[tuple[int, int]]:  # fmt: skip
    """``(start, stop)`` per chain. Budgets are proportional shares of ``max_complex_len`` capped at ``max_chain_len``;
    a window is anchored on a random interface residue when there is one; copies of an entity get the same window."""
    total = sum(lengths)
    scale = min(1.0, max_complex_len / max(total, 1))
    windows: dict[int, tuple[int, int]] = {}
    out = []
    for k, n in enumerate(lengths):
        e = int(entity[k])
        if e in windows:
            out.append(windows[e])
            continue
        budget = max(1, min(max_chain_len, int(n * scale)))
        if budget >= n:
            w = (0, n)
        else:
            hot = np.flatnonzero(iface[k]) if iface is not None and iface[k].any() else None
            anchor = int(hot[rng.integers(len(hot))]) if hot is not None else int(rng.integers(n))
            lo = int(np.clip(anchor - int(rng.integers(budget)), 0, n - budget))
            w = (lo, lo + budget)
        windows[e] = w
        out.append(w)
    return out


def apply_masking(rng: np.random.Generator, chains: list[np.ndarray], entity: np.ndarray, iface: list[np.ndarray] | None,
                  cfg: MaskingConfig, interface_masking: bool) -> tuple[list[np.ndarray], list[np.ndarray]]:  # fmt: skip
    """Returns ``(corrupted tokens, labels)`` per chain; labels are ``IGNORE_INDEX`` off the selected positions.

    With ``homomer_paired`` the copies of an entity share one selection and one corruption draw, so the marginal
    masking rate does not grow with the copy number and a copy never reveals what another hides.
    """
    std = standard_token_ids()
    draws: dict[int, tuple[np.ndarray, np.ndarray, np.ndarray]] = {}
    toks, labels = [], []
    for k, ids in enumerate(chains):
        e = int(entity[k]) if cfg.homomer_paired else -1 - k
        if e not in draws or len(draws[e][0]) != len(ids):
            draws[e] = (rng.random(len(ids)), rng.random(len(ids)), std[rng.integers(len(std), size=len(ids))])
        u_sel, u_kind, rand_tok = draws[e]
        rate = np.full(len(ids), cfg.rate)
        if interface_masking and iface is not None:
            flags = iface[k]
            if cfg.homomer_paired:  # one selection for all copies: a residue is "interface" if it is in any copy
                for j in range(len(chains)):
                    if int(entity[j]) == int(entity[k]) and len(iface[j]) == len(flags):
                        flags = flags | iface[j]
            rate = np.where(flags, cfg.interface_rate, cfg.rate)
        sel = u_sel < rate
        out = ids.copy()
        out[sel & (u_kind < cfg.mask_token_frac)] = MASK_ID
        swap = sel & (u_kind >= cfg.mask_token_frac) & (u_kind < cfg.mask_token_frac + cfg.random_token_frac)
        out[swap] = rand_tok[swap]
        lab = np.full(len(ids), IGNORE_INDEX, dtype=np.int64)
        lab[sel] = ids[sel]
        toks.append(out)
        labels.append(lab)
    return toks, labels


# ---------------------------------------------------------------------------------------------------------------
# examples and packing
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class Example:
    tokens: list[np.ndarray]
    labels: list[np.ndarray]
    starts: list[int]
    entity: np.ndarray
    iface: list[np.ndarray]
    iface_known: bool
    source: int

    @property
    def n_res(self) -> int:
        return sum(len(t) for t in self.tokens)


def build_example(rng: np.random.Generator, cx: StoredComplex, data: DataConfig, src: SourceConfig, source_id: int) -> Example:
    order = rng.permutation(len(cx.chains)) if data.permute_chains else np.arange(len(cx.chains))
    order = order[: data.max_chains]
    chains = [cx.chains[i] for i in order]
    entity = cx.entity[order]
    iface = [cx.iface[i] for i in order] if cx.iface is not None else None
    wins = crop_complex(rng, [len(c) for c in chains], entity, iface, data.max_chain_len, data.max_complex_len)
    chains = [c[a:b] for c, (a, b) in zip(chains, wins)]
    iface_c = [f[a:b] for f, (a, b) in zip(iface, wins)] if iface is not None else None
    toks, labels = apply_masking(rng, chains, entity, iface_c, data.masking, src.interface_masking)
    return Example(toks, labels, [a for a, _ in wins], entity, iface_c or [np.zeros(len(c), bool) for c in chains],
                   iface is not None, source_id)  # fmt: skip


def pack(examples: list[Example]) -> PackedBatch:
    tok, lab, pos, gpos, ch, cx, ent, ifc, known = [], [], [], [], [], [], [], [], []
    chain_len, cx_len, sources = [], [], []
    n_chain = n_ent = 0
    for c, ex in enumerate(examples):
        at = 0
        remap: dict[int, int] = {}
        for t, lb, start, e, f in zip(ex.tokens, ex.labels, ex.starts, ex.entity, ex.iface):
            n = len(t)
            tok.append(t), lab.append(lb), ifc.append(f)
            pos.append(np.arange(start, start + n)), gpos.append(np.arange(at, at + n))
            ch.append(np.full(n, n_chain)), cx.append(np.full(n, c))
            ent.append(np.full(n, remap.setdefault(int(e), n_ent + len(remap))))
            known.append(np.full(n, ex.iface_known))
            chain_len.append(n)
            n_chain += 1
            at += n
        n_ent += len(remap)
        cx_len.append(at)
        sources.append(ex.source)
    cat = lambda parts, dt: torch.as_tensor(np.concatenate(parts).astype(dt))  # noqa: E731
    cu = lambda lens: torch.as_tensor(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32))  # noqa: E731
    return PackedBatch(cat(tok, np.int64), cat(lab, np.int64), cat(pos, np.int64), cat(gpos, np.int64), cu(chain_len), cu(cx_len),
                       cat(ch, np.int32), cat(cx, np.int32), cat(ent, np.int32), cat(ifc, bool), cat(known, bool),
                       torch.as_tensor(sources, dtype=torch.int32), max(chain_len), max(cx_len))  # fmt: skip


class PackedComplexStream(torch.utils.data.IterableDataset):
    """Endless stream of packed batches. Draws are i.i.d., so ranks and workers only need different seeds."""

    def __init__(self, views: list[SourceView], data: DataConfig, seed: int = 0, rank: int = 0):
        self.views, self.data, self.seed, self.rank = views, data, seed, rank
        self.sampler = MixtureSampler(views)

    def __iter__(self):
        info = torch.utils.data.get_worker_info()
        rng = np.random.default_rng([self.seed, self.rank, info.id if info else 0])
        pending: list[Example] = []
        size = 0
        while True:
            v, i = self.sampler.draw(rng)
            view = self.sampler.views[v]
            ex = build_example(rng, view.store.example(i), self.data, view.cfg, v)
            if ex.n_res > self.data.token_budget:
                continue
            if size + ex.n_res > self.data.token_budget and pending:
                yield pack(pending)
                pending, size = [], 0
            pending.append(ex)
            size += ex.n_res


def evaluation_batches(views: list[SourceView], data: DataConfig, n_batches: int, seed: int = 0) -> list[PackedBatch]:
    """Fixed evaluation set: masks are seeded from the complex index, so two checkpoints score identical positions."""
    out, pending, size = [], [], 0
    for v, view in enumerate(views):
        for i in view.indices[: max(1, n_batches * 8)]:
            rng = np.random.default_rng([seed, v, int(i)])
            frozen = DataConfig(**{**data.__dict__, "permute_chains": False})
            ex = build_example(rng, view.store.example(int(i)), frozen, view.cfg, v)
            if ex.n_res > data.token_budget:
                continue
            if size + ex.n_res > data.token_budget and pending:
                out.append(pack(pending))
                pending, size = [], 0
                if len(out) >= n_batches:
                    return out
            pending.append(ex)
            size += ex.n_res
    if pending:
        out.append(pack(pending))
    return out[:n_batches]
