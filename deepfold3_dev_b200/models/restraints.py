"""Distance restraints steered into the diffusion sampler (``--restraint SEL:SEL[@DIST[@LO..HI]]``).

Behaviour follows the reference (model/restraints.py:46-430): a flat-bottom
quadratic penalty ``U = sum_i max(0, d_i - distance)^2`` on the soft-min
distance ``d_i`` from each restrained residue to the partner group; its
gradient either moves atoms directly or is projected on the rigid-body motions
of the chains involved. Nothing is fed to the network.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from dataclasses import dataclass

import torch

from .guidance import ChainSel, parse_selector_pair, parse_sigma_range, selector_mask

DEFAULT_DISTANCE = 6.0
MIN_DISTANCE, MAX_DISTANCE = 2.0, 30.0


@dataclass(frozen=True)
class RestraintSpec:
    groups: tuple[ChainSel, ChainSel]
    distance: float = DEFAULT_DISTANCE
    sigma_range: tuple[float, float] | None = None
    paired: bool = False
    repel: bool = False


@dataclass(frozen=True)
class Restraint:
    tokens_a: torch.Tensor  # [N] bool, residues that must make the contact
    tokens_b: torch.Tensor  # [N] bool, what they must touch
    distance: float = DEFAULT_DISTANCE
    sigma_range: tuple[float, float] | None = None
    chain_a: torch.Tensor | None = None
    chain_b: torch.Tensor | None = None
    pair_index: tuple[tuple[int, int], ...] = ()
    repel: bool = False


def _count(sel: ChainSel) -> int:
    return sum(hi - lo + 1 for lo, hi in sel.ranges)


def parse_restraint_spec(text: str, paired: bool = False, repel: bool = False) -> RestraintSpec:
    fields = text.split("@")
    if len(fields) > 3:
        raise ValueError(f"expected SEL:SEL[@DIST[@LO..HI]], got {text!r}")
    try:
        a, b = parse_selector_pair(fields[0], what="a restraint")
    except ValueError as exc:
        if "chain pair" in str(exc):
            raise ValueError(f"expected two selectors like A/25-40:B, got {fields[0]!r}") from exc
        raise
    distance = float(fields[1]) if len(fields) > 1 else DEFAULT_DISTANCE
    if not MIN_DISTANCE <= distance <= MAX_DISTANCE:
        raise ValueError(f"restraint distance must be {MIN_DISTANCE:g}..{MAX_DISTANCE:g} A, got {distance:g}")
    sigma = parse_sigma_range(fields[2]) if len(fields) > 2 else None
    if paired:
        na, nb = _count(a), _count(b)
        if not (na and nb):
            raise ValueError(f"a paired restraint needs residues on both sides, got {fields[0]!r}")
        if na != nb:
            raise ValueError(f"paired selectors must name the same number of residues, got {na} and {nb}")
    return RestraintSpec((a, b), distance, sigma, paired, repel)


def describe_restraint(spec: RestraintSpec) -> str:
    a, b = spec.groups
    sigma = f" sigma in [{spec.sigma_range[0]:g}, {spec.sigma_range[1]:g}]" if spec.sigma_range else ""
    kind = f" ({_count(a)} pairs)" if spec.paired else ""
    return f"{a}:{b} {'>=' if spec.repel else '<='} {spec.distance:g} A{kind}{sigma}"


def _pair_tokens(spec, asym_id, chain_index, residue_index, n_tokens):
    if residue_index is None:
        raise ValueError("a paired restraint needs the input's residue_index, got none")
    sides = []
    for sel in spec.groups:
        if sel.chain not in chain_index:
            raise ValueError(f"unknown chain {sel.chain!r}, this input has {sorted(chain_index)}")
        in_chain = asym_id == chain_index[sel.chain]
        if n_tokens is not None:
            in_chain = in_chain.clone()
            in_chain[n_tokens:] = False
        idx = []
        for lo, hi in sel.ranges:
            for num in range(lo, hi + 1):
                hit = torch.nonzero(in_chain & (residue_index == num)).flatten()
                if not hit.numel():
                    raise ValueError(f"{sel.chain}/{num} is not a residue of this input")
                idx.append(int(hit[0]))
        sides.append(idx)
    return tuple(zip(*sides, strict=True))


def build_restraints(specs, asym_id, chain_index: Mapping[str, int], n_tokens=None, residue_index=None):
    out = []
    for spec in specs:
        a, b = (selector_mask(s, asym_id, chain_index, residue_index, n_tokens) for s in spec.groups)
        wa, wb = (selector_mask(ChainSel(s.chain), asym_id, chain_index, None, n_tokens) for s in spec.groups)
        pairs = _pair_tokens(spec, asym_id, chain_index, residue_index, n_tokens) if spec.paired else ()
        out.append(Restraint(a, b, spec.distance, spec.sigma_range, wa, wb, pairs, spec.repel))
    return tuple(out)


def active_restraints(restraints: Sequence[Restraint], sigma_hat: float):
    return tuple(r for r in restraints if r.sigma_range is None or r.sigma_range[0] <= sigma_hat <= r.sigma_range[1])


def _soft_min(d: torch.Tensor, sharpness: float) -> torch.Tensor:
    """Softmax(-sharpness d)-weighted mean along the last axis: between min and mean, size-independent."""
    return (torch.softmax(-sharpness * d, dim=-1) * d).sum(-1)


def restraint_gradient(positions, atom_mask, restraints, sharpness: float):
    """``dU/dx`` with the shape of ``positions`` ``[..., N, M, 3]``; callable under ``no_grad`` / ``inference_mode``."""
    if not restraints:
        return torch.zeros_like(positions)
    with torch.inference_mode(False):
        x = torch.empty_like(positions).copy_(positions).requires_grad_(True)
    with torch.inference_mode(False), torch.enable_grad():
        energy = x.new_zeros(())
        M = x.shape[-2]
        flat = x.reshape(*x.shape[:-3], -1, 3)
        for r in restraints:
            if r.pair_index:
                per = []
                for ta, tb in r.pair_index:
                    ia = torch.nonzero(atom_mask[ta]).flatten() + ta * M
                    ib = torch.nonzero(atom_mask[tb]).flatten() + tb * M
                    if ia.numel() and ib.numel():
                        d = torch.cdist(flat[..., ia, :], flat[..., ib, :])
                        per.append(_soft_min(_soft_min(d, sharpness), sharpness))
                if not per:
                    continue
                dist = torch.stack(per, dim=-1)
            else:
                rows = (r.tokens_a.unsqueeze(-1) & atom_mask).reshape(-1)
                cols = (r.tokens_b.unsqueeze(-1) & atom_mask).reshape(-1)
                if not (bool(rows.any()) and bool(cols.any())):
                    continue
                per_atom = _soft_min(torch.cdist(flat[..., rows, :], flat[..., cols, :]), sharpness)
                tok = torch.nonzero(rows).squeeze(-1) // M
                dist = torch.stack([_soft_min(per_atom[..., tok == t], sharpness) for t in torch.unique(tok)], dim=-1)
            gap = (r.distance - dist) if r.repel else (dist - r.distance)
            energy = energy + gap.clamp(min=0.0).pow(2).sum()
        if not energy.requires_grad:
            return torch.zeros_like(positions)
        (grad,) = torch.autograd.grad(energy, x)
    return grad


def rigid_displacement(positions, atom_mask, restraints, weight: float, sharpness: float, max_step: float):
    """Displacement moving every restrained chain as a rigid body.

    Each atom wants ``u_i = -weight/2 dU/dx_i``; per chain the least-squares
    rigid fit is ``t = mean(u)`` over pulled atoms and ``omega`` from
    ``(sum |r|^2 I - r r^T) omega = sum r x u``. Translation and the largest
    rotational displacement are both clipped to ``max_step`` angstroms; the
    rotation is applied exactly (Rodrigues).
    """
    grad = restraint_gradient(positions, atom_mask, restraints, sharpness)
    out = torch.zeros_like(positions)
    if float(grad.abs().max()) == 0.0:
        return out
    fpos = positions.reshape(*positions.shape[:-3], -1, 3)
    fgrad = grad.reshape(*grad.shape[:-3], -1, 3)
    fout = out.reshape(*out.shape[:-3], -1, 3)
    eye = torch.eye(3, dtype=positions.dtype, device=positions.device)
    done = set()
    for r in restraints:
        for chain in (r.chain_a, r.chain_b):
            if chain is None:
                continue
            sel = (chain.unsqueeze(-1) & atom_mask).reshape(-1)
            idx = torch.nonzero(sel).flatten()
            if not idx.numel():
                continue
            key = (int(idx[0]), int(idx.numel()))
            if key in done:
                continue
            done.add(key)
            p, g = fpos[..., idx, :], fgrad[..., idx, :]
            rel = p - p.mean(-2, keepdim=True)
            pulled = (g.abs().sum(-1) > 0).sum(-1).clamp(min=1).unsqueeze(-1)
            force = (-g).sum(-2) / pulled
            torque = torch.cross(rel, -g, dim=-1).sum(-2)
            gram = (rel.pow(2).sum(-1)[..., None, None] * eye - rel.unsqueeze(-1) * rel.unsqueeze(-2)).sum(-3)
            omega = torch.linalg.solve(gram + 1e-6 * eye, torque.unsqueeze(-1)).squeeze(-1) * (idx.numel() / pulled)
            t = force * (0.5 * weight)
            omega = omega * (0.5 * weight)
            t = t * (max_step / t.norm(dim=-1, keepdim=True).clamp(min=max_step))
            radius = rel.norm(dim=-1).amax(-1, keepdim=True)
            cap = max_step / radius.clamp(min=1e-6)
            angle = omega.norm(dim=-1, keepdim=True)
            omega = omega * (cap / angle.clamp(min=cap))
            angle = omega.norm(dim=-1, keepdim=True)
            axis = (omega / angle.clamp(min=1e-12)).unsqueeze(-2)
            cos, sin = torch.cos(angle).unsqueeze(-2), torch.sin(angle).unsqueeze(-2)
            rot = rel * cos + torch.cross(axis.expand_as(rel), rel, dim=-1) * sin
            rot = rot + axis * (axis * rel).sum(-1, keepdim=True) * (1 - cos)
            fout[..., idx, :] = rot - rel + t.unsqueeze(-2)
    return out


def steer(x, atom_mask, restraints, sigma_hat, sigma_data, weight, rigid, max_step, batched):
    """Apply the active restraints to coordinates ``x`` ``[B, S, N, M, 3]`` for the step at ``sigma_hat``.

    The soft-min sharpens from 0.25 to 2.0 per angstrom as the noise falls
    (reference: diffusion.py:1549-1576). Restraints describe one input, so a
    batched call applies them to every batch element with that element's mask.
    """
    active = active_restraints(restraints, sigma_hat)
    if not active:
        return x
    sharp = 0.25 + 1.75 * (1.0 - min(sigma_hat / sigma_data, 1.0))

    def one(xb, mask):
        if rigid:
            return xb + rigid_displacement(xb, mask, active, weight, sharp, max_step)
        move = -0.5 * weight * restraint_gradient(xb, mask, active, sharp)
        norm = move.norm(dim=-1, keepdim=True)
        return xb + move * (max_step / norm.clamp(min=max_step))

    if not batched:
        return one(x[0], atom_mask).unsqueeze(0)
    return torch.stack([one(x[b], atom_mask[b]) for b in range(x.shape[0])])
