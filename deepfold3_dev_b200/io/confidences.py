"""Confidence read-outs from the head's logits, and their files.

Formulas follow AlphaFold 3 as the reference implements them (io/confidences.py:56-501):
bin centres of the 64 error bins, expected pLDDT / PAE / PDE, TM-adjusted PAE with
``d0 = 1.24 (max(n, 19) - 15)^(1/3) - 1.8``, pTM as the best row, ipTM with ``d0`` sized per chain
pair, the clash test and ``ranking = 0.8 ipTM + 0.2 pTM + 0.5 disorder - 100 clash``.
All functions take torch tensors on any device and return tensors or Python floats.
"""

from __future__ import annotations

import csv
import json
import math
import os

import numpy as np
import torch

MAX_ERROR_BIN, NUM_ERROR_BINS, NUM_PLDDT_BINS = 31.0, 64, 50
CLASH_CUTOFF, MIN_CLASHES, MIN_CLASH_FRACTION = 1.1, 100, 0.5
DISORDER_PLDDT = 50.0


def error_bin_centers(max_error_bin: float = MAX_ERROR_BIN, num_bins: int = NUM_ERROR_BINS) -> torch.Tensor:
    breaks = torch.linspace(0.0, max_error_bin, num_bins - 1)
    step = breaks[1] - breaks[0]
    centers = breaks + step / 2
    return torch.cat([centers, centers[-1:] + step])


def compute_plddt(plddt_logits, atom_mask, num_bins: int = NUM_PLDDT_BINS):
    """``[S, N, M * bins]`` logits -> per-atom ``[S, N, M]`` and per-token ``[S, N]`` pLDDT in [0, 100]."""
    S, N = plddt_logits.shape[:2]
    M = atom_mask.shape[-1]
    probs = plddt_logits.reshape(S, N, M, num_bins).float().softmax(-1)
    centers = (torch.arange(num_bins, device=probs.device).float() + 0.5) / num_bins
    per_atom = (probs * centers).sum(-1) * 100.0
    mask = atom_mask.unsqueeze(0).float()
    return per_atom, (per_atom * mask).sum(-1) / mask.sum(-1).clamp(min=1)


def compute_pae(pae_logits, pair_mask, max_error_bin=MAX_ERROR_BIN, num_bins=NUM_ERROR_BINS):
    centers = error_bin_centers(max_error_bin, num_bins).to(pae_logits.device)
    return (pae_logits.float().softmax(-1) * centers).sum(-1) * pair_mask.unsqueeze(0).float()


def compute_pde(pde_logits, pair_mask, max_error_bin=MAX_ERROR_BIN, num_bins=NUM_ERROR_BINS):
    """Expected distance error ``[S, N, N]`` and its masked mean per sample ``[S]``."""
    centers = error_bin_centers(max_error_bin, num_bins).to(pde_logits.device)
    m = pair_mask.unsqueeze(0).float()
    pde = (pde_logits.float().softmax(-1) * centers).sum(-1) * m
    return pde, pde.sum((-1, -2)) / m.sum((-1, -2)).clamp(min=1)


def compute_exp_resolved(logits, atom_mask):
    """``[S, N, M * 2]`` logits -> probability that each atom is experimentally resolved ``[S, N, M]``."""
    S, N = logits.shape[:2]
    M = atom_mask.shape[-1]
    return logits.reshape(S, N, M, 2).float().softmax(-1)[..., 1] * atom_mask.unsqueeze(0).float()


def tm_adjusted_pae(pae_logits, num_tokens, max_error_bin=MAX_ERROR_BIN, num_bins=NUM_ERROR_BINS):
    """``sum_bins p(bin) / (1 + (centre / d0)^2)`` for ``[N, N, bins]`` logits; ``num_tokens`` scalar or ``[N, N]``."""
    centers = error_bin_centers(max_error_bin, num_bins).to(pae_logits.device)
    n = torch.as_tensor(num_tokens, device=pae_logits.device, dtype=torch.float32).clamp(min=19)
    d0 = 1.24 * (n - 15) ** (1.0 / 3) - 1.8
    per_bin = 1.0 / (1.0 + (centers / d0.unsqueeze(-1)) ** 2)
    return (pae_logits.float().softmax(-1) * per_bin).sum(-1)


def compute_ptm(pae_logits, seq_mask, pair_mask, d0_seq_mask=None, **kw) -> float:
    d0_mask = seq_mask if d0_seq_mask is None else d0_seq_mask
    tm = tm_adjusted_pae(pae_logits, float(d0_mask.sum()), **kw)
    m = pair_mask.float()
    rows = (tm * m / m.sum(-1, keepdim=True).clamp(min=1e-8)).sum(-1) * seq_mask.float()
    return float(rows.max())


def compute_iptm(pae_logits, seq_mask, pair_mask, asym_id, d0_pair_mask=None, **kw) -> float:
    """Interface pTM: pairs on different chains only, ``d0`` from the two chains' token counts; NaN for one chain."""
    inter = (asym_id[:, None] != asym_id[None, :]) & pair_mask.bool()
    if not bool(inter.any()):
        return float("nan")
    counts_mask = (seq_mask if d0_pair_mask is None else d0_pair_mask).float()
    ids = asym_id.long()
    per_chain = torch.zeros(int(ids.max()) + 1, device=ids.device).index_add_(0, ids, counts_mask)
    n_pair = per_chain[ids][:, None] + per_chain[ids][None, :]
    tm = tm_adjusted_pae(pae_logits, n_pair, **kw)
    m = inter.float()
    rows = (tm * m / m.sum(-1, keepdim=True).clamp(min=1e-8)).sum(-1) * seq_mask.float() * (m.sum(-1) > 0).float()
    return float(rows.max())


def compute_chain_pair_iptm(pae_logits, seq_mask, pair_mask, asym_id, **kw) -> list[list[float | None]]:
    """Matrix over chains: off-diagonal the ipTM restricted to that chain pair, on the diagonal the chain's own pTM."""
    chains = sorted(int(c) for c in torch.unique(asym_id[seq_mask.bool()]))
    out: list[list[float | None]] = []
    for a in chains:
        row = []
        for b in chains:
            sel = ((asym_id == a) | (asym_id == b)) & seq_mask.bool()
            pm = pair_mask.float() * sel[:, None].float() * sel[None, :].float()
            if a == b:
                row.append(compute_ptm(pae_logits, sel.float(), pm, **kw))
            else:
                v = compute_iptm(pae_logits, sel.float(), pm, asym_id, **kw)
                row.append(None if math.isnan(v) else v)
        out.append(row)
    return out


def has_clash(atom_positions, atom_mask, residue_index, asym_id, polymer_mask, cutoff=CLASH_CUTOFF,
              min_clashes=MIN_CLASHES, min_clash_fraction=MIN_CLASH_FRACTION) -> bool:  # fmt: skip
    """A polymer chain clashes if more than ``min_clashes`` (or half) of its atoms sit within ``cutoff`` of an atom
    on another chain or more than one residue away."""
    sel = atom_mask.bool() & polymer_mask.bool()[:, None]
    if not bool(sel.any()):
        return False
    tok, _ = torch.nonzero(sel, as_tuple=True)
    xyz = atom_positions[sel].float()
    res, chain = residue_index[tok].long(), asym_id[tok].long()
    clashing = torch.zeros(xyz.shape[0], dtype=torch.bool, device=xyz.device)
    for s in range(0, xyz.shape[0], 4096):
        d = torch.cdist(xyz[s : s + 4096], xyz)
        far = (chain[s : s + 4096, None] != chain[None, :]) | ((res[s : s + 4096, None] - res[None, :]).abs() > 1)
        clashing[s : s + 4096] = ((d < cutoff) & far).any(-1)
    for c in torch.unique(chain):
        on = chain == c
        n = int(clashing[on].sum())
        if n > min_clashes or n / max(1, int(on.sum())) > min_clash_fraction:
            return True
    return False


def fraction_disordered(per_token_plddt, polymer_mask, threshold=DISORDER_PLDDT) -> float:
    poly = polymer_mask.bool()
    n = int(poly.sum())
    return 0.0 if n == 0 else float(((per_token_plddt < threshold) & poly).sum()) / n


def compute_ranking_score(ptm: float, iptm: float, frac_disordered: float = 0.0, clash: bool = False) -> float:
    base = ptm if math.isnan(iptm) else 0.8 * iptm + 0.2 * ptm
    return base + 0.5 * frac_disordered - 100.0 * float(clash)


def distogram_bin_centers(first=2.3125, last=21.6875, num_bins=64) -> torch.Tensor:
    breaks = torch.linspace(first, last, num_bins - 1)
    step = breaks[1] - breaks[0]
    return torch.cat([breaks[:1] - step / 2, breaks + step / 2])


def compute_distogram_expected(logits, **kw):
    return (logits.float().softmax(-1) * distogram_bin_centers(**kw).to(logits.device)).sum(-1)


def compute_contact_probs(logits, cutoff: float = 8.0, **kw):
    centers = distogram_bin_centers(**kw).to(logits.device)
    return (logits.float().softmax(-1) * (centers <= cutoff).float()).sum(-1)


# ------------------------------------------------------------------------------------------------ files
def _clean(obj):
    if isinstance(obj, float):
        return None if (math.isnan(obj) or math.isinf(obj)) else obj
    if isinstance(obj, dict):
        return {k: _clean(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_clean(v) for v in obj]
    if isinstance(obj, (np.floating, np.integer)):
        return _clean(obj.item())
    return obj


def sample_summary(sample: int, seed: int, plddt_logits, pae_logits, pde_logits, atom_positions, feats) -> dict:
    """All per-sample scalars and maps of one prediction (inputs are one sample, token axis unpadded)."""
    atom_mask = feats["ref_mask"].float()
    seq_mask = feats["seq_mask"].float()
    pair_mask = seq_mask[:, None] * seq_mask[None, :]
    asym = feats["asym_id"]
    per_atom, per_token = compute_plddt(plddt_logits[None], atom_mask)
    pae = compute_pae(pae_logits[None], pair_mask)[0]
    pde, mean_pde = compute_pde(pde_logits[None], pair_mask)
    ptm = compute_ptm(pae_logits, seq_mask, pair_mask)
    iptm = compute_iptm(pae_logits, seq_mask, pair_mask, asym)
    polymer = feats["mol_type"] != 3
    disorder = fraction_disordered(per_token[0], polymer & seq_mask.bool())
    clash = has_clash(atom_positions, atom_mask, feats["residue_index"], asym, polymer)
    return {
        "seed": seed, "sample": sample, "ptm": ptm, "iptm": iptm, "fraction_disordered": disorder, "has_clash": clash,
        "ranking_score": compute_ranking_score(ptm, iptm, disorder, clash),
        "mean_plddt": float((per_atom[0] * atom_mask).sum() / atom_mask.sum().clamp(min=1)),
        "mean_pde": float(mean_pde[0]),
        "chain_pair_iptm": compute_chain_pair_iptm(pae_logits, seq_mask, pair_mask, asym),
        "atom_plddts": per_atom[0][atom_mask.bool()].tolist(), "token_plddts": per_token[0].tolist(),
        "pae": pae.tolist(), "pde": pde[0].tolist(),
        "token_chain_ids": asym.tolist(), "token_res_ids": feats["residue_index"].tolist(),
    }  # fmt: skip


def save_confidences_json(path: str, summary: dict) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        json.dump(_clean(summary), f)


SCALARS = ("seed", "sample", "ranking_score", "ptm", "iptm", "fraction_disordered", "has_clash", "mean_plddt", "mean_pde")


def save_ranking_scores_csv(path: str, summaries: list[dict]) -> None:
    rows = sorted(summaries, key=lambda s: -s["ranking_score"])
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(SCALARS)
        for s in rows:
            w.writerow([s[k] for k in SCALARS])


def save_summary_confidences_json(path: str, summaries: list[dict], job_name: str | None = None) -> None:
    best = max(summaries, key=lambda s: s["ranking_score"]) if summaries else None
    blob = {"job_name": job_name, "best": None if best is None else {k: best[k] for k in SCALARS},
            "samples": [{k: s[k] for k in SCALARS} | {"chain_pair_iptm": s["chain_pair_iptm"]} for s in summaries]}  # fmt: skip
    with open(path, "w") as f:
        json.dump(_clean(blob), f, indent=1)


def save_sample_logits(path: str, plddt_logits, pae_logits, pde_logits, exp_resolved_logits=None) -> None:
    arrays = {"plddt": plddt_logits, "pae": pae_logits, "pde": pde_logits}
    if exp_resolved_logits is not None:
        arrays["exp_resolved"] = exp_resolved_logits
    np.savez_compressed(path, **{k: v.detach().float().cpu().numpy().astype(np.float16) for k, v in arrays.items()})


def save_distogram_logits(path: str, logits) -> None:
    np.savez_compressed(path, distogram=logits.detach().float().cpu().numpy().astype(np.float16))
