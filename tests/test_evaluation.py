"""Accuracy metrics on constructed cases with known answers."""

import numpy as np
import pytest

from deepfold3_dev_b200.evaluation import metrics


def _helix(n=60):
    t = np.arange(n) * 100.0 * np.pi / 180.0
    return np.stack([2.3 * np.cos(t), 2.3 * np.sin(t), 1.5 * np.arange(n)], 1)


def _rigid(x, seed=0):
    rng = np.random.default_rng(seed)
    q, _ = np.linalg.qr(rng.normal(size=(3, 3)))
    q *= np.sign(np.linalg.det(q))
    return x @ q.T + rng.normal(size=3) * 10


def test_identical_up_to_rigid_motion():
    x = _helix()
    y = _rigid(x)
    assert metrics.rmsd(y, x) < 1e-6 and metrics.lddt(y, x) == pytest.approx(1.0)
    assert metrics.tm_score(y, x) == pytest.approx(1.0, abs=1e-6) and metrics.gdt_ts(y, x) == pytest.approx(1.0)


def test_partial_agreement_is_found_by_the_search():
    x = _helix(80)
    y = x.copy()
    y[40:] = _rigid(x[40:], 3)  # second half moved as a rigid body
    y = _rigid(y, 5)
    g = metrics.gdt_ts(y, x)
    assert 0.45 <= g <= 0.62  # half of the residues superpose exactly
    assert 0.4 < metrics.tm_score(y, x) < 0.75
    assert metrics.rmsd(y, x) > 3.0
    per_atom = metrics.lddt(y, x, per_atom=True)
    assert per_atom[:30].mean() > 0.9 and per_atom[35:45].mean() < per_atom[:30].mean()


def test_mirror_image_scores_low_and_flips_chirality():
    x = _helix(40) + np.random.default_rng(0).normal(size=(40, 3)) * 0.1
    m = x * np.array([1, 1, -1.0])
    assert metrics.tm_score(m, x) < 0.5 and metrics.lddt(m, x) > 0.99  # distances cannot see the mirror
    centers = np.array([[1, 0, 2, 3], [5, 4, 6, 7]])
    assert metrics.chirality_violations(m, centers, x) == 1.0 and metrics.chirality_violations(x, centers, x) == 0.0


def test_dockq_limits():
    rng = np.random.default_rng(0)
    rec = rng.normal(size=(200, 3)) * 6
    lig = rng.normal(size=(80, 3)) * 4 + np.array([11.0, 0, 0])
    same = metrics.dockq(rec, lig, rec, lig)
    assert same["fnat"] == 1.0 and same["dockq"] == pytest.approx(1.0)
    away = metrics.dockq(rec, lig + np.array([40.0, 0, 0]), rec, lig)
    assert away["fnat"] == 0.0 and away["lrmsd"] == pytest.approx(40.0) and away["dockq"] < 0.1


def test_compare_files_roundtrip(tmp_path):
    from test_prepare import _mini_cif

    from deepfold3_dev_b200.evaluation.compare import compare_files

    a, b = tmp_path / "a.cif", tmp_path / "b.cif"
    a.write_text(_mini_cif())
    b.write_text(_mini_cif(shift=(5.0, -3.0, 2.0)))
    out = compare_files(str(a), str(b))
    assert out["matched_chains"] == 3 and out["lddt"] == pytest.approx(1.0) and out["rmsd_all_atom"] < 1e-3


def test_homologous_constructs_match_through_alignment():
    import os

    from test_prepare import EXAMPLES

    from deepfold3_dev_b200.evaluation.compare import compare_files

    a = os.path.join(EXAMPLES, "9m22_msa", "templates", "7v2g_A.cif")
    b = os.path.join(EXAMPLES, "9m22_msa", "templates", "6aq1_B.cif")
    if not (os.path.exists(a) and os.path.exists(b)):
        pytest.skip("reference example files not available")
    out = compare_files(a, b)  # two crystal forms of one protein whose constructs differ at the termini
    assert out["matched_chains"] >= 1 and out["tm_score"] > 0.9 and out["lddt"] > 0.8 and out["matched_atoms"] > 900
