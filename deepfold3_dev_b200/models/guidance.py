"""Classifier-free guidance from the command line: ``--guidance W[@TARGET[@LO..HI]]``.

What the option means (behaviour of the reference's model/guidance.py:39-312, restated):

* ``W`` is the guidance weight of one term; ``1`` switches the term off.
* ``TARGET`` names the conditioning that the unconditional branch of the term drops: ``full`` (all trunk pair
  conditioning), ``all`` (every block between two different chains) or a comma-separated list of ``SEL:SEL``
  interfaces. A selector ``SEL`` is a chain name, optionally followed by ``/`` and ``+``-joined residue numbers or
  ``LO-HI`` ranges: ``A``, ``B/25-40``, ``H/31-35+50+95-102``.
* ``LO..HI`` limits the term to sampler steps whose noise level lies in that closed interval.

The grammar is held by three small value classes, each of which parses its own text (``ChainSel.parse``,
``SigmaWindow.parse``, ``GuidanceSpec.parse``) and knows how to turn itself into token masks. The module-level
functions are the names the command line and the restraint parser call.
"""

from __future__ import annotations

import math
import warnings
from collections.abc import Mapping, Sequence
from dataclasses import dataclass

import torch

FULL, ALL_INTERFACES, PAIRS = "full", "all", "pairs"


def _closed_interval(item: str) -> tuple[int, int]:
    """``"7"`` -> (7, 7), ``"3-9"`` -> (3, 9). Residue numbers are non-negative integers."""
    first, dash, second = item.partition("-")
    if not first.isdigit() or (dash and not second.isdigit()):
        raise ValueError(f"{item!r} is neither a residue number nor a LO-HI range")
    lo = int(first)
    hi = int(second) if dash else lo
    if hi < lo:
        raise ValueError(f"range {item!r} runs backwards (LO must not exceed HI)")
    return lo, hi


@dataclass(frozen=True)
class ChainSel:
    """A chain, or some residues of it. ``ranges`` holds closed ``(lo, hi)`` residue-number intervals; empty = whole chain."""

    chain: str
    ranges: tuple[tuple[int, int], ...] = ()

    @classmethod
    def parse(cls, text: str) -> "ChainSel":
        name, _, tail = text.partition("/")
        if name == "":
            raise ValueError(f"selector {text!r} does not start with a chain name")
        if "/" in text and tail == "":
            raise ValueError(f"selector {text!r} ends in '/' without residue numbers")
        return cls(name, tuple(_closed_interval(part) for part in tail.split("+")) if tail else ())

    def residue_count(self) -> int:
        return sum(hi - lo + 1 for lo, hi in self.ranges)

    def __str__(self) -> str:
        if not self.ranges:
            return self.chain
        spans = (f"{lo}" if lo == hi else f"{lo}-{hi}" for lo, hi in self.ranges)
        return f"{self.chain}/{'+'.join(spans)}"

    def mask(self, asym_id: torch.Tensor, chain_index: Mapping[str, int], residue_index=None, n_tokens=None) -> torch.Tensor:
        """Boolean ``[N]`` mask of the tokens this selector names. Padding tokens (index >= ``n_tokens``) never match;
        a selector that names nothing is an error, because a silently empty steering term would be a no-op."""
        if self.chain not in chain_index:
            raise ValueError(f"chain {self.chain!r} is not in this input (chains: {', '.join(sorted(chain_index))})")
        picked = asym_id.eq(chain_index[self.chain])
        if self.ranges:
            if residue_index is None:
                raise ValueError(f"selector {self} has residue ranges but the input carries no residue_index")
            inside = [residue_index.ge(lo) & residue_index.le(hi) for lo, hi in self.ranges]
            picked = picked & torch.stack(inside).any(0)
        if n_tokens is not None and n_tokens < picked.shape[-1]:
            picked = picked.clone()
            picked[n_tokens:] = False
        if not picked.any().item():
            raise ValueError(f"selector {self} matches no token of this input")
        return picked


@dataclass(frozen=True)
class SigmaWindow:
    """Closed noise-level interval ``LO..HI``."""

    lo: float
    hi: float

    @classmethod
    def parse(cls, text: str) -> "SigmaWindow":
        lo_text, sep, hi_text = text.partition("..")
        if not sep or ".." in hi_text:
            raise ValueError(f"noise window {text!r} is not of the form LO..HI")
        lo, hi = float(lo_text), float(hi_text)
        if not lo <= hi:  # also catches NaN
            raise ValueError(f"noise window {text!r} has LO above HI")
        return cls(lo, hi)

    def as_tuple(self) -> tuple[float, float]:
        return (self.lo, self.hi)


def _interface(text: str, purpose: str) -> tuple[ChainSel, ChainSel]:
    left, sep, right = text.partition(":")
    if not sep or not left or not right or ":" in right:
        raise ValueError(f"{text!r} is not a pair of selectors (write A:B or A/25-40:B)")
    first, second = ChainSel.parse(left), ChainSel.parse(right)
    if first.chain == second.chain:
        raise ValueError(f"{purpose} joins two different chains, {text!r} names {first.chain!r} twice")
    return first, second


@dataclass(frozen=True)
class GuidanceSpec:
    scale: float
    target: str = FULL                                        # "full", "all" or "pairs"
    pairs: tuple[tuple[ChainSel, ChainSel], ...] = ()         # for target == "pairs"
    sigma_range: tuple[float, float] | None = None

    @classmethod
    def parse(cls, text: str) -> "GuidanceSpec":
        weight_text, *rest = text.split("@")
        if len(rest) > 2:
            raise ValueError(f"--guidance takes W[@TARGET[@LO..HI]]; {text!r} has too many '@' fields")
        weight = float(weight_text)
        if math.isnan(weight) or math.isinf(weight):
            raise ValueError(f"guidance weight {weight_text!r} is not a finite number")
        window = SigmaWindow.parse(rest[1]).as_tuple() if len(rest) == 2 else None
        what = rest[0] if rest else FULL
        if what == FULL or what == ALL_INTERFACES:
            return cls(weight, what, (), window)
        return cls(weight, PAIRS, tuple(_interface(item, "an interface") for item in what.split(",")), window)

    @property
    def active(self) -> bool:
        return self.scale != 1.0


# ---- names used by the command line and by models/restraints.py
def parse_selector(text: str) -> ChainSel:
    return ChainSel.parse(text)


def parse_selector_pair(text: str, what: str = "an interface") -> tuple[ChainSel, ChainSel]:
    return _interface(text, what)


def parse_sigma_range(text: str) -> tuple[float, float]:
    return SigmaWindow.parse(text).as_tuple()


def parse_guidance_spec(text: str) -> GuidanceSpec:
    return GuidanceSpec.parse(text)


def selector_mask(sel: ChainSel, asym_id, chain_index: Mapping[str, int], residue_index=None, n_tokens=None):
    return sel.mask(asym_id, chain_index, residue_index, n_tokens)


def has_residue_ranges(specs: Sequence[GuidanceSpec]) -> bool:
    """Does any active term select by residue number (the caller then needs ``residue_index``)?"""
    for spec in specs:
        if spec.active and any(side.ranges for pair in spec.pairs for side in pair):
            return True
    return False


def check_guidance_training(specs: Sequence[GuidanceSpec], diffusion) -> None:
    """Guidance extrapolates between two branches the network must have seen in training. A checkpoint trained with
    conditioning always on has no unconditional branch at all; one trained without interface drop has never seen a
    partially dropped pair tensor."""
    wanted = [s for s in specs if s.active]
    if not wanted:
        return
    if diffusion.use_conditioning_prob >= 1.0:
        raise ValueError("guidance needs a checkpoint trained with conditioning drop; this one has use_conditioning_prob = 1")
    if diffusion.cond_drop_interface_frac <= 0.0 and any(s.target != FULL for s in wanted):
        raise ValueError("interface guidance needs a checkpoint trained with interface drop; this one has cond_drop_interface_frac = 0")


class _PairKeep:
    """Accumulates the pair blocks one term drops; ``keep`` is the ``[N, N]`` mask of what stays conditioned."""

    def __init__(self, n: int, device):
        self.keep = torch.ones(n, n, dtype=torch.bool, device=device)
        self.seen: list[str] = []

    def drop(self, rows: torch.Tensor, cols: torch.Tensor, label: str, allow_overlap: bool) -> None:
        block = rows[:, None] & cols[None, :]
        block = block | block.transpose(0, 1)
        twice = block & ~self.keep
        if self.seen and not allow_overlap and twice.any().item():
            raise ValueError(f"interface {label} overlaps {', '.join(self.seen)} inside one guidance term; "
                             "pass --allow-guidance-overlap to take the union")  # fmt: skip
        self.keep &= ~block
        self.seen.append(label)


def _windows_meet(a, b) -> bool:
    lo_a, hi_a = a if a is not None else (-math.inf, math.inf)
    lo_b, hi_b = b if b is not None else (-math.inf, math.inf)
    return max(lo_a, lo_b) <= min(hi_a, hi_b)


def build_guidance_terms(specs, asym_id, chain_index, n_tokens=None, residue_index=None, allow_overlap=False):
    """Resolve parsed specs against one input: one sampler ``GuidanceTerm`` per spec, in order."""
    from .diffusion_modules import GuidanceTerm, interface_pair_keep

    terms = []
    for spec in specs:
        keep = None
        if spec.target != FULL:
            if len(chain_index) < 2:
                raise ValueError(f"interface guidance needs at least two chains; this input has {', '.join(sorted(chain_index))}")
            if spec.target == ALL_INTERFACES:
                keep = interface_pair_keep(asym_id)
            else:
                acc = _PairKeep(asym_id.shape[-1], asym_id.device)
                for left, right in spec.pairs:
                    acc.drop(left.mask(asym_id, chain_index, residue_index, n_tokens),
                             right.mask(asym_id, chain_index, residue_index, n_tokens), f"{left}:{right}", allow_overlap)  # fmt: skip
                keep = acc.keep
            if n_tokens is not None:  # bucket padding stays "conditioned": it is masked out everywhere else anyway
                keep[n_tokens:] = True
                keep[:, n_tokens:] = True
        terms.append(GuidanceTerm(spec.scale, keep, spec.sigma_range))
    if not allow_overlap:
        partial = [t for t in terms if t.scale != 1.0 and t.pair_keep is not None]
        clash = next(((a, b) for i, a in enumerate(partial) for b in partial[i + 1 :]
                      if _windows_meet(a.sigma_range, b.sigma_range) and (~a.pair_keep & ~b.pair_keep).any().item()), None)  # fmt: skip
        if clash is not None:
            warnings.warn(f"two guidance terms (w={clash[0].scale:g}, w={clash[1].scale:g}) drop common pair blocks at the same "
                          "noise levels; their pushes add up there", stacklevel=2)  # fmt: skip
    return tuple(terms)
