"""Where the files of a prepared dataset live (reference: data/paths.py, data/msa/paths.py).

    <root>/manifest.json                 records (chains, interfaces, metadata)
    <root>/structures/<id>.npz           ``Structure`` record arrays
    <root>/msa/<msa_id>.npz | .a3m       per-sequence alignments, keyed by the sha256 of the canonical sequence
    <root>/msa_paired/<msa_id>.npz       rows paired across chains, when a pairing step ran
    <root>/templates/<msa_id>.json       template hit lists (next to the hits' mmCIF files)
    <root>/masks/<id>.npz                optional per-token loss weights
    <root>/features/<id>.pt              optional pre-featurised examples with their own flat manifest
    <root>/sequences.fasta               unique polymer sequences keyed by msa_id (input of the MSA search)
"""

from __future__ import annotations

import os


def manifest(root: str) -> str:
    return os.path.join(root, "manifest.json")


def structure(root: str, record_id: str) -> str:
    return os.path.join(root, "structures", f"{record_id}.npz")


def msa(root: str, msa_id: str, paired: bool = False) -> str | None:
    """The alignment file of a sequence (``.npz`` preferred over ``.a3m``), or ``None`` when there is none."""
    base = os.path.join(root, "msa_paired" if paired else "msa", str(msa_id))
    for ext in (".npz", ".a3m"):
        if os.path.exists(base + ext):
            return base + ext
    return None


def templates(root: str, msa_id: str) -> str:
    return os.path.join(root, "templates", f"{msa_id}.json")


def mask(root: str, record_id: str) -> str:
    return os.path.join(root, "masks", f"{record_id}.npz")


def features(root: str, record_id: str) -> str:
    return os.path.join(root, "features", f"{record_id}.pt")


def is_prepared_root(path: str) -> bool:
    return os.path.isdir(os.path.join(path, "structures")) and os.path.exists(manifest(path))
