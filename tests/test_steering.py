"""Guidance and restraint options: grammar, resolution against an input, and the steering move itself (CPU)."""

import math

import pytest
import torch

from deepfold3_dev_b200.models import guidance as G
from deepfold3_dev_b200.models import restraints as R


def _input():
    # chain A: residues 1..6, chain B: residues 1..4, two padding tokens at the end
    asym = torch.tensor([0] * 6 + [1] * 4 + [0, 0])
    resi = torch.tensor(list(range(1, 7)) + list(range(1, 5)) + [0, 0])
    return asym, resi, {"A": 0, "B": 1}, 10


def test_selector_grammar():
    assert G.parse_selector("A") == G.ChainSel("A")
    s = G.parse_selector("H/31-35+50+95-102")
    assert s.ranges == ((31, 35), (50, 50), (95, 102)) and str(s) == "H/31-35+50+95-102" and s.residue_count() == 14
    for bad in ("", "/3", "A/", "A/x", "A/5-3", "A/3-"):
        with pytest.raises(ValueError):
            G.parse_selector(bad)
    with pytest.raises(ValueError):
        G.parse_selector_pair("A:A")
    with pytest.raises(ValueError):
        G.parse_selector_pair("A")
    assert G.parse_sigma_range("0.5..40") == (0.5, 40.0)
    with pytest.raises(ValueError):
        G.parse_sigma_range("4..1")


def test_guidance_spec_grammar():
    assert G.parse_guidance_spec("2.5") == G.GuidanceSpec(2.5, "full")
    assert G.parse_guidance_spec("2@all@1..10") == G.GuidanceSpec(2.0, "all", (), (1.0, 10.0))
    spec = G.parse_guidance_spec("3@A:B/2-3,B:A/5")
    assert spec.target == "pairs" and len(spec.pairs) == 2 and str(spec.pairs[0][1]) == "B/2-3"
    for bad in ("inf", "2@all@1..2@x", "2@A:A"):
        with pytest.raises(ValueError):
            G.parse_guidance_spec(bad)
    assert G.has_residue_ranges([spec]) and not G.has_residue_ranges([G.parse_guidance_spec("1@A:B/2")])


def test_selector_mask_and_terms():
    asym, resi, chains, n = _input()
    m = G.selector_mask(G.parse_selector("A/2-3+6"), asym, chains, resi, n)
    assert m.tolist() == [False, True, True, False, False, True] + [False] * 6
    assert G.selector_mask(G.parse_selector("A"), asym, chains, None, n).sum() == 6  # padding tokens of "chain 0" excluded
    with pytest.raises(ValueError):
        G.selector_mask(G.parse_selector("C"), asym, chains, resi, n)
    with pytest.raises(ValueError):
        G.selector_mask(G.parse_selector("A/40"), asym, chains, resi, n)
    terms = G.build_guidance_terms([G.parse_guidance_spec("2"), G.parse_guidance_spec("3@A/1-2:B")], asym, chains, n, resi)
    assert terms[0].pair_keep is None and terms[0].scale == 2.0
    keep = terms[1].pair_keep
    assert not keep[0, 6] and not keep[6, 0] and not keep[1, 9] and keep[2, 6] and keep[0, 1] and keep[10:, :].all()
    with pytest.raises(ValueError):  # the same block twice inside one term
        G.build_guidance_terms([G.parse_guidance_spec("3@A/1-2:B,A/2:B/1")], asym, chains, n, resi)
    G.build_guidance_terms([G.parse_guidance_spec("3@A/1-2:B,A/2:B/1")], asym, chains, n, resi, allow_overlap=True)
    with pytest.warns(UserWarning):
        G.build_guidance_terms([G.parse_guidance_spec("3@A/1-2:B"), G.parse_guidance_spec("2@A/2:B/1")], asym, chains, n, resi)


def test_guidance_needs_matching_training():
    class D:
        use_conditioning_prob, cond_drop_interface_frac = 1.0, 0.0

    G.check_guidance_training([G.parse_guidance_spec("1")], D)
    with pytest.raises(ValueError):
        G.check_guidance_training([G.parse_guidance_spec("2")], D)
    D.use_conditioning_prob = 0.8
    G.check_guidance_training([G.parse_guidance_spec("2")], D)
    with pytest.raises(ValueError):
        G.check_guidance_training([G.parse_guidance_spec("2@all")], D)


def test_restraint_grammar():
    s = R.parse_restraint_spec("A/2-3:B")
    assert s.distance == 6.0 and s.sigma_range is None and not s.paired
    s = R.parse_restraint_spec("A/2-3:B/1-2@8@0.5..30", paired=True)
    assert s.distance == 8.0 and s.sigma_range == (0.5, 30.0) and R.describe_restraint(s) == "A/2-3:B/1-2 <= 8 A (2 pairs) sigma in [0.5, 30]"
    assert ">=" in R.describe_restraint(R.parse_restraint_spec("A:B@10", repel=True))
    for bad, kw in (("A/2:B@1", {}), ("A/2:B@31", {}), ("A:B", {"paired": True}), ("A/1-2:B/1", {"paired": True}), ("A:B@6@1..2@3", {})):
        with pytest.raises(ValueError):
            R.parse_restraint_spec(bad, **kw)


def _coords():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 12, 3, 3, generator=g) * 2
    x[0, 6:10] += torch.tensor([20.0, 0.0, 0.0])  # chain B far from chain A
    mask = torch.ones(12, 3, dtype=torch.bool)
    mask[10:] = False
    return x, mask


def test_restraint_pulls_groups_together_and_repel_pushes_apart():
    asym, resi, chains, n = _input()
    x, mask = _coords()
    pull = R.build_restraints([R.parse_restraint_spec("A/2-3:B/1-2@6")], asym, chains, n, resi)
    centre = lambda t, lo, hi: t[0, lo:hi].mean((0, 1))  # noqa: E731
    gap0 = (centre(x, 1, 3) - centre(x, 6, 8)).norm()
    for rigid in (True, False):
        with torch.inference_mode():
            y = R.steer(x[None], mask, pull, sigma_hat=1.0, sigma_data=16.0, weight=1.0, rigid=rigid, max_step=2.0, batched=False)[0]
        assert (centre(y, 1, 3) - centre(y, 6, 8)).norm() < gap0
        assert (y - x).norm(dim=-1).max() <= 4.0 + 1e-4  # translation and rotation are limited to max_step each
        if rigid:  # internal distances of a chain are unchanged by a rigid move
            d0 = torch.cdist(x[0, :6].reshape(-1, 3), x[0, :6].reshape(-1, 3))
            d1 = torch.cdist(y[0, :6].reshape(-1, 3), y[0, :6].reshape(-1, 3))
            torch.testing.assert_close(d0, d1, atol=1e-3, rtol=1e-4)
    close = x.clone()
    close[0, 6:10] -= torch.tensor([19.0, 0.0, 0.0])
    push = R.build_restraints([R.parse_restraint_spec("A:B@12", repel=True)], asym, chains, n, resi)
    y = R.steer(close[None], mask, push, 1.0, 16.0, 1.0, True, 2.0, False)[0]
    assert (centre(y, 0, 6) - centre(y, 6, 10)).norm() > (centre(close, 0, 6) - centre(close, 6, 10)).norm()
    # outside its noise window a restraint does nothing; a satisfied one has zero gradient
    windowed = R.build_restraints([R.parse_restraint_spec("A/2-3:B/1-2@6@20..40")], asym, chains, n, resi)
    assert torch.equal(R.steer(x[None], mask, windowed, 1.0, 16.0, 1.0, True, 2.0, False)[0], x)
    assert float(R.restraint_gradient(close, mask, R.build_restraints([R.parse_restraint_spec("A:B@30")], asym, chains, n, resi), 1.0).abs().max()) == 0.0


def test_paired_restraint_indices_and_soft_min():
    asym, resi, chains, n = _input()
    r = R.build_restraints([R.parse_restraint_spec("A/2+5:B/1+4", paired=True)], asym, chains, n, resi)[0]
    assert r.pair_index == ((1, 6), (4, 9))
    d = torch.tensor([1.0, 2.0, 10.0])
    assert abs(float(R.soft_min(d, 50.0)) - 1.0) < 1e-6 and abs(float(R.soft_min(d, 0.0)) - d.mean()) < 1e-6
    assert math.isfinite(float(R.soft_min(d * 100, 2.0)))
