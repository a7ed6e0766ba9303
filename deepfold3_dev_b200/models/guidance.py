"""``--guidance W[@TARGET[@LO..HI]]``: selector grammar and resolution to sampler terms.

Grammar (reference: model/guidance.py:39-312). A selector is ``CHAIN`` or
``CHAIN/RANGES`` with ``RANGES`` = ``+``-joined ``N`` or ``LO-HI``. ``TARGET`` is
``full`` (drop all trunk pair conditioning in the unconditional branch),
``all`` (drop every inter-chain block) or comma-joined ``SEL:SEL`` pairs.
"""

from __future__ import annotations

import math
import re
import warnings
from collections.abc import Mapping, Sequence
from dataclasses import dataclass

import torch

FULL, ALL_INTERFACES = "full", "all"
_RANGE = re.compile(r"^(\d+)(?:-(\d+))?$")


@dataclass(frozen=True)
class ChainSel:
    chain: str
    ranges: tuple[tuple[int, int], ...] = ()

    def __str__(self) -> str:
        if not self.ranges:
            return self.chain
        return self.chain + "/" + "+".join(str(lo) if lo == hi else f"{lo}-{hi}" for lo, hi in self.ranges)


@dataclass(frozen=True)
class GuidanceSpec:
    scale: float
    target: str = FULL
    pairs: tuple[tuple[ChainSel, ChainSel], ...] = ()
    sigma_range: tuple[float, float] | None = None


def parse_selector(text: str) -> ChainSel:
    chain, slash, residues = text.partition("/")
    if not chain:
        raise ValueError(f"expected a chain name, got {text!r}")
    if slash and not residues:
        raise ValueError(f"expected residue numbers after '/', got {text!r}")
    ranges = []
    for item in residues.split("+") if residues else ():
        m = _RANGE.match(item)
        if m is None:
            raise ValueError(f"expected a residue number or LO-HI, got {item!r}")
        lo = int(m.group(1))
        hi = int(m.group(2)) if m.group(2) is not None else lo
        if lo > hi:
            raise ValueError(f"residue range needs LO <= HI, got {item!r}")
        ranges.append((lo, hi))
    return ChainSel(chain, tuple(ranges))


def parse_selector_pair(text: str, what: str = "an interface") -> tuple[ChainSel, ChainSel]:
    sides = text.split(":")
    if len(sides) != 2 or not all(sides):
        raise ValueError(f"expected a chain pair like A:B or A/25-40:B, got {text!r}")
    a, b = parse_selector(sides[0]), parse_selector(sides[1])
    if a.chain == b.chain:
        raise ValueError(f"{what} needs two chains, got {text!r}")
    return a, b


def parse_sigma_range(text: str) -> tuple[float, float]:
    parts = text.split("..")
    if len(parts) != 2:
        raise ValueError(f"expected LO..HI, got {text!r}")
    lo, hi = float(parts[0]), float(parts[1])
    if not lo <= hi:
        raise ValueError(f"sigma range needs LO <= HI, got {text!r}")
    return lo, hi


def parse_guidance_spec(text: str) -> GuidanceSpec:
    fields = text.split("@")
    if len(fields) > 3:
        raise ValueError(f"expected W[@TARGET[@LO..HI]], got {text!r}")
    scale = float(fields[0])
    if not math.isfinite(scale):
        raise ValueError(f"guidance weight must be finite, got {fields[0]!r}")
    target = fields[1] if len(fields) > 1 else FULL
    sigma = parse_sigma_range(fields[2]) if len(fields) > 2 else None
    if target in (FULL, ALL_INTERFACES):
        return GuidanceSpec(scale, target, sigma_range=sigma)
    return GuidanceSpec(scale, "pairs", tuple(parse_selector_pair(p) for p in target.split(",")), sigma)


def has_residue_ranges(specs: Sequence[GuidanceSpec]) -> bool:
    return any(sel.ranges for s in specs if s.scale != 1.0 for pair in s.pairs for sel in pair)


def check_guidance_training(specs: Sequence[GuidanceSpec], diffusion) -> None:
    """Refuse a term whose unconditional branch the checkpoint was never trained on."""
    active = [s for s in specs if s.scale != 1.0]
    if active and diffusion.use_conditioning_prob >= 1.0:
        raise ValueError("this checkpoint was trained without conditioning drop (use_conditioning_prob = 1)")
    if any(s.target != FULL for s in active) and diffusion.cond_drop_interface_frac <= 0.0:
        raise ValueError("this checkpoint was trained without interface drop (cond_drop_interface_frac = 0)")


def selector_mask(sel: ChainSel, asym_id, chain_index: Mapping[str, int], residue_index=None, n_tokens=None):
    """``[N]`` bool of the tokens ``sel`` names; tokens at or past ``n_tokens`` (bucket padding) never match."""
    if sel.chain not in chain_index:
        raise ValueError(f"unknown chain {sel.chain!r}, this input has {sorted(chain_index)}")
    mask = asym_id == chain_index[sel.chain]
    if sel.ranges:
        if residue_index is None:
            raise ValueError(f"residue ranges need the input's residue_index, got none for {sel}")
        hit = torch.zeros_like(mask)
        for lo, hi in sel.ranges:
            hit |= (residue_index >= lo) & (residue_index <= hi)
        mask = mask & hit
    if n_tokens is not None:
        mask = mask.clone()
        mask[n_tokens:] = False
    if not bool(mask.any()):
        raise ValueError(f"{sel} selects no token of this input")
    return mask


def _pairs_keep(masks, labels=(), allow_overlap=False):
    n = masks[0][0].numel()
    keep = torch.ones(n, n, dtype=torch.bool, device=masks[0][0].device)
    for k, (a, b) in enumerate(masks):
        drop = a.unsqueeze(-1) & b.unsqueeze(-2)
        drop = drop | drop.T
        if labels and not allow_overlap and bool((drop & ~keep).any()):
            raise ValueError(
                f"{labels[k]} drops pair blocks already dropped by {', '.join(labels[:k])} in the same term "
                "(--allow-guidance-overlap takes the union anyway)"
            )
        keep &= ~drop
    return keep


def build_guidance_terms(specs, asym_id, chain_index, n_tokens=None, residue_index=None, allow_overlap=False):
    """One sampler ``GuidanceTerm`` per spec."""
    from .diffusion_modules import GuidanceTerm, interface_pair_keep

    terms = []
    for spec in specs:
        keep = None
        if spec.target != FULL:
            if len(chain_index) < 2:
                raise ValueError(f"interface guidance needs two chains, this input has {sorted(chain_index)}")
            if spec.target == ALL_INTERFACES:
                keep = interface_pair_keep(asym_id)
            else:
                keep = _pairs_keep(
                    [tuple(selector_mask(s, asym_id, chain_index, residue_index, n_tokens) for s in p) for p in spec.pairs],
                    labels=[f"{a}:{b}" for a, b in spec.pairs],
                    allow_overlap=allow_overlap,
                )
            if n_tokens is not None:
                keep[n_tokens:, :] = True
                keep[:, n_tokens:] = True
        terms.append(GuidanceTerm(spec.scale, keep, spec.sigma_range))
    if not allow_overlap:
        masked = [t for t in terms if t.scale != 1.0 and t.pair_keep is not None]
        for i, a in enumerate(masked):
            for b in masked[i + 1 :]:
                la, ha = a.sigma_range or (-math.inf, math.inf)
                lb, hb = b.sigma_range or (-math.inf, math.inf)
                if not (ha < lb or hb < la) and bool((~a.pair_keep & ~b.pair_keep).any()):
                    warnings.warn(
                        f"guidance terms w={a.scale:g} and w={b.scale:g} drop some of the same pair blocks over the "
                        "same sigma range; those blocks get the sum of both pushes",
                        stacklevel=2,
                    )
                    return tuple(terms)
    return tuple(terms)


# names the reference exposes with a leading underscore, used by its restraint parser
_parse_sel, _sel_mask, _parse_sigma_range = parse_selector, selector_mask, parse_sigma_range
