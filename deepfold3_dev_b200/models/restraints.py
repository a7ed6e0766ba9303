"""Distance restraints that steer the diffusion sampler: ``--restraint``, ``--restraint-pair``, ``--repel``.

``--restraint SEL:SEL[@DIST[@LO..HI]]`` asks the residues of the first selector to come within ``DIST`` angstroms
(default 6, allowed 2..30) of the second group, optionally only while the sampler's noise level is inside
``LO..HI``; ``--restraint-pair`` pairs the residues of both selectors one to one, ``--repel`` turns "at most" into
"at least". Nothing is fed to the network: the sampler moves the denoised coordinates down the gradient of

    U = sum_r sum_i max(0, +-(d_ri - DIST_r))^2,

where ``d_ri`` is a soft minimum (softmax-weighted mean with weights ``exp(-s d)``) of the distances from residue
``i`` to the partner atoms, so the energy is smooth and independent of group sizes. The gradient is taken by
autograd, then applied either atom by atom or, by default, projected onto rigid motions of the chains involved.
Semantics follow the reference (model/restraints.py:46-430, model/diffusion.py:1549-1576); the code is organised
around two objects, ``RestraintEnergy`` (energy and gradient) and ``RigidMover`` (least-squares rigid projection).
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from dataclasses import dataclass

import torch

from .guidance import ChainSel, parse_selector_pair, parse_sigma_range

DEFAULT_DISTANCE = 6.0
MIN_DISTANCE, MAX_DISTANCE = 2.0, 30.0


@dataclass(frozen=True)
class RestraintSpec:
    """A parsed option, not yet tied to an input."""

    groups: tuple[ChainSel, ChainSel]
    distance: float = DEFAULT_DISTANCE
    sigma_range: tuple[float, float] | None = None
    paired: bool = False
    repel: bool = False


@dataclass(frozen=True)
class Restraint:
    """A spec resolved against one input's tokens."""

    tokens_a: torch.Tensor  # [N] bool: residues that must make (or avoid) the contact
    tokens_b: torch.Tensor  # [N] bool: what they are measured against
    distance: float = DEFAULT_DISTANCE
    sigma_range: tuple[float, float] | None = None
    chain_a: torch.Tensor | None = None  # [N] bool: the whole chain of each side, for the rigid projection
    chain_b: torch.Tensor | None = None
    pair_index: tuple[tuple[int, int], ...] = ()  # token pairs of a one-to-one restraint
    repel: bool = False

    def active_at(self, sigma: float) -> bool:
        return self.sigma_range is None or self.sigma_range[0] <= sigma <= self.sigma_range[1]


def parse_restraint_spec(text: str, paired: bool = False, repel: bool = False) -> RestraintSpec:
    head, *tail = text.split("@")
    if len(tail) > 2:
        raise ValueError(f"a restraint is SEL:SEL[@DIST[@LO..HI]]; {text!r} has too many '@' fields")
    sides = parse_selector_pair(head, what="a restraint")
    dist = DEFAULT_DISTANCE if not tail else float(tail[0])
    if dist < MIN_DISTANCE or dist > MAX_DISTANCE or dist != dist:
        raise ValueError(f"restraint distance {dist:g} A is outside {MIN_DISTANCE:g}..{MAX_DISTANCE:g} A")
    window = parse_sigma_range(tail[1]) if len(tail) == 2 else None
    if paired:
        counts = [s.residue_count() for s in sides]
        if 0 in counts:
            raise ValueError(f"--restraint-pair needs residue numbers on both sides of {head!r}")
        if counts[0] != counts[1]:
            raise ValueError(f"--restraint-pair needs as many residues left as right; {head!r} has {counts[0]} and {counts[1]}")
    return RestraintSpec(sides, dist, window, paired, repel)


def describe_restraint(spec: RestraintSpec) -> str:
    """One log line per restraint, e.g. ``A/25-40:B <= 6 A`` or ``H/31+52:L/50+91 >= 8 A (2 pairs) sigma in [1, 40]``."""
    left, right = spec.groups
    text = f"{left}:{right} {'>=' if spec.repel else '<='} {spec.distance:g} A"
    if spec.paired:
        text += f" ({left.residue_count()} pairs)"
    if spec.sigma_range is not None:
        text += f" sigma in [{spec.sigma_range[0]:g}, {spec.sigma_range[1]:g}]"
    return text


def _one_to_one(spec: RestraintSpec, asym_id, chain_index, residue_index, n_tokens) -> tuple[tuple[int, int], ...]:
    """Token index pairs of a paired restraint: the k-th residue number of the left selector with the k-th of the right."""
    if residue_index is None:
        raise ValueError("--restraint-pair needs residue numbers, but the input carries no residue_index")
    limit = asym_id.shape[-1] if n_tokens is None else n_tokens
    columns = []
    for sel in spec.groups:
        if sel.chain not in chain_index:
            raise ValueError(f"chain {sel.chain!r} is not in this input (chains: {', '.join(sorted(chain_index))})")
        chain_tokens = torch.nonzero(asym_id[:limit] == chain_index[sel.chain]).flatten()
        number_to_token: dict[int, int] = {}
        for tok in chain_tokens.tolist():
            number_to_token.setdefault(int(residue_index[tok]), tok)  # first token of a residue (atomised residues repeat)
        column = []
        for lo, hi in sel.ranges:
            for number in range(lo, hi + 1):
                if number not in number_to_token:
                    raise ValueError(f"residue {sel.chain}/{number} does not exist in this input")
                column.append(number_to_token[number])
        columns.append(column)
    return tuple(zip(columns[0], columns[1], strict=True))


def build_restraints(specs, asym_id, chain_index: Mapping[str, int], n_tokens=None, residue_index=None):
    resolved = []
    for spec in specs:
        left, right = spec.groups
        resolved.append(Restraint(
            tokens_a=left.mask(asym_id, chain_index, residue_index, n_tokens),
            tokens_b=right.mask(asym_id, chain_index, residue_index, n_tokens),
            distance=spec.distance, sigma_range=spec.sigma_range,
            chain_a=ChainSel(left.chain).mask(asym_id, chain_index, None, n_tokens),
            chain_b=ChainSel(right.chain).mask(asym_id, chain_index, None, n_tokens),
            pair_index=_one_to_one(spec, asym_id, chain_index, residue_index, n_tokens) if spec.paired else (),
            repel=spec.repel,
        ))  # fmt: skip
    return tuple(resolved)


def active_restraints(restraints: Sequence[Restraint], sigma_hat: float):
    return tuple(r for r in restraints if r.active_at(sigma_hat))


def soft_min(d: torch.Tensor, sharpness: float) -> torch.Tensor:
    """Weighted mean of ``d`` along the last axis with weights ``softmax(-sharpness d)``: tends to the minimum as the
    sharpness grows and to the plain mean as it vanishes; unlike log-sum-exp it does not drift with the group size."""
    w = torch.softmax(d * (-sharpness), dim=-1)
    return (w * d).sum(dim=-1)


class RestraintEnergy:
    """``U(x)`` of a set of restraints on coordinates ``x [..., N, M, 3]`` with atom mask ``[N, M]``."""

    def __init__(self, atom_mask: torch.Tensor, restraints: Sequence[Restraint], sharpness: float):
        self.mask, self.restraints, self.s = atom_mask, tuple(restraints), float(sharpness)
        self.atoms_per_token = atom_mask.shape[-1]

    def _atoms_of(self, token: int) -> torch.Tensor:
        return torch.nonzero(self.mask[token]).flatten() + token * self.atoms_per_token

    def _residue_distances(self, flat: torch.Tensor, r: Restraint):
        """Soft-min distance of every restrained residue to its partner set, stacked on a new last axis (or None)."""
        if r.pair_index:
            cols = []
            for ta, tb in r.pair_index:
                ia, ib = self._atoms_of(ta), self._atoms_of(tb)
                if len(ia) and len(ib):
                    d = torch.cdist(flat[..., ia, :], flat[..., ib, :])
                    cols.append(soft_min(soft_min(d, self.s), self.s))
            return torch.stack(cols, -1) if cols else None
        from_atoms = (r.tokens_a[:, None] & self.mask).flatten()
        to_atoms = (r.tokens_b[:, None] & self.mask).flatten()
        if not from_atoms.any().item() or not to_atoms.any().item():
            return None
        nearest = soft_min(torch.cdist(flat[..., from_atoms, :], flat[..., to_atoms, :]), self.s)  # per restrained atom
        owner = torch.nonzero(from_atoms).flatten() // self.atoms_per_token
        return torch.stack([soft_min(nearest[..., owner == t], self.s) for t in owner.unique()], -1)

    def value(self, x: torch.Tensor) -> torch.Tensor:
        flat = x.flatten(-3, -2)
        total = x.new_zeros(())
        for r in self.restraints:
            d = self._residue_distances(flat, r)
            if d is None:
                continue
            violation = (r.distance - d) if r.repel else (d - r.distance)
            total = total + violation.clamp_min(0.0).square().sum()
        return total

    def gradient(self, positions: torch.Tensor) -> torch.Tensor:
        """``dU/dx``; works inside ``no_grad`` and ``inference_mode`` blocks (the sampler runs under one)."""
        if not self.restraints:
            return torch.zeros_like(positions)
        with torch.inference_mode(False), torch.enable_grad():
            x = positions.detach().clone().requires_grad_(True)  # clone: an inference tensor cannot require grad
            u = self.value(x)
            if not u.requires_grad:  # no restraint touched an atom
                return torch.zeros_like(positions)
            (g,) = torch.autograd.grad(u, x)
        return g


def restraint_gradient(positions, atom_mask, restraints, sharpness: float):
    return RestraintEnergy(atom_mask, restraints, sharpness).gradient(positions)


class RigidMover:
    """Least-squares rigid motion of a set of atoms towards per-atom wishes.

    Atom ``i`` at offset ``r_i`` from the centroid wants the displacement ``u_i``. The rigid motion ``t + w x r_i``
    closest to those wishes has ``t = mean(u)`` and ``(sum |r|^2 I - r r^T) w = sum r x u``. Wishes here are
    non-zero only on the pulled atoms, so the means run over those; the translation and the largest rotational
    displacement are limited to ``max_step`` angstroms each, and the rotation is applied exactly (Rodrigues) rather
    than as its first-order displacement, which would stretch the chain.
    """

    def __init__(self, gain: float, max_step: float):
        self.gain, self.max_step = gain, max_step

    def displacement(self, pos: torch.Tensor, wish: torch.Tensor) -> torch.Tensor:
        n = pos.shape[-2]
        eye = torch.eye(3, dtype=pos.dtype, device=pos.device)
        r = pos - pos.mean(dim=-2, keepdim=True)
        n_pulled = (wish.abs().sum(-1) > 0).sum(-1).clamp_min(1)[..., None]
        shift = wish.sum(-2) / n_pulled * self.gain
        torque = torch.linalg.cross(r, wish, dim=-1).sum(-2)
        inertia = (r.square().sum(-1)[..., None, None] * eye - r[..., :, None] * r[..., None, :]).sum(-3)
        spin = torch.linalg.solve(inertia + 1e-6 * eye, torque[..., None])[..., 0] * (n / n_pulled) * self.gain
        # limits: translation length, and the arc travelled by the atom farthest from the centroid
        shift = shift * (self.max_step / shift.norm(dim=-1, keepdim=True).clamp_min(self.max_step))
        max_angle = self.max_step / r.norm(dim=-1).amax(-1, keepdim=True).clamp_min(1e-6)
        spin = spin * (max_angle / spin.norm(dim=-1, keepdim=True).clamp_min(max_angle))
        theta = spin.norm(dim=-1, keepdim=True)
        axis = (spin / theta.clamp_min(1e-12))[..., None, :]
        c, s = torch.cos(theta)[..., None, :], torch.sin(theta)[..., None, :]
        turned = r * c + torch.linalg.cross(axis.expand_as(r), r, dim=-1) * s + axis * (axis * r).sum(-1, keepdim=True) * (1 - c)
        return turned - r + shift[..., None, :]


def rigid_displacement(positions, atom_mask, restraints, weight: float, sharpness: float, max_step: float):
    """Displacement field that moves every chain named by a restraint as one rigid body down the energy gradient
    (each atom's wish is ``-weight / 2 dU/dx``)."""
    grad = restraint_gradient(positions, atom_mask, restraints, sharpness)
    moved = torch.zeros_like(positions)
    if not grad.abs().max().item() > 0.0:
        return moved
    flat_pos, flat_wish, flat_out = positions.flatten(-3, -2), (-grad).flatten(-3, -2), moved.view(*moved.shape[:-3], -1, 3)
    mover = RigidMover(0.5 * weight, max_step)
    handled: set[tuple[int, int]] = set()
    for chain in (c for r in restraints for c in (r.chain_a, r.chain_b) if c is not None):
        atoms = torch.nonzero((chain[:, None] & atom_mask).flatten()).flatten()
        if atoms.numel() == 0:
            continue
        tag = (int(atoms[0]), int(atoms.numel()))
        if tag in handled:  # a chain named by several restraints moves once, with the summed gradient
            continue
        handled.add(tag)
        flat_out[..., atoms, :] = mover.displacement(flat_pos[..., atoms, :], flat_wish[..., atoms, :])
    return moved


def steer(x, atom_mask, restraints, sigma_hat, sigma_data, weight, rigid, max_step, batched):
    """Coordinates ``x [B, S, N, M, 3]`` after one steering move at noise level ``sigma_hat``.

    The soft minimum sharpens linearly from 0.25 / A at ``sigma >= sigma_data`` to 2 / A at ``sigma = 0``: early steps see
    a broad, averaged pull, late steps a contact between specific atoms. Restraints belong to one input; in a batched
    call every element is steered with its own atom mask.
    """
    live = active_restraints(restraints, sigma_hat)
    if not live:
        return x
    sharpness = 2.0 - 1.75 * min(sigma_hat / sigma_data, 1.0)

    def move(coords, mask):
        if rigid:
            return coords + rigid_displacement(coords, mask, live, weight, sharpness, max_step)
        step = restraint_gradient(coords, mask, live, sharpness) * (-0.5 * weight)
        length = step.norm(dim=-1, keepdim=True)
        return coords + step * (max_step / length.clamp_min(max_step))

    if batched:
        return torch.stack([move(x[b], atom_mask[b]) for b in range(x.shape[0])])
    return move(x[0], atom_mask)[None]
