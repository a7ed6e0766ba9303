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


def test_accuracy_sweep_plan_score_and_trajectory(tmp_path):
    """The sweep harness on fabricated predictions: balanced shards, per-GPU command lines, scores per structure,
    mean / oracle / top-ranked per target, category rows, trajectory over two checkpoint steps, fold classes."""
    import csv
    import json

    from click.testing import CliRunner
    from test_prepare import _mini_cif

    from deepfold3_dev_b200.cli.main import cli
    from deepfold3_dev_b200.evaluation import sweep

    inputs, truth, run = tmp_path / "inputs", tmp_path / "truth", tmp_path / "run"
    lengths = {"t1": 900, "t2": 300, "t3": 250, "t4": 200, "t5": 120}
    for cat, names in (("monomer_protein", ["t1", "t2", "t3"]), ("interface_protein_protein", ["t4", "t5"])):
        (inputs / cat).mkdir(parents=True)
        for n in names:
            (inputs / cat / f"{n}.json").write_text(json.dumps({"name": n, "sequences": [{"protein": {"id": ["A"], "sequence": "G" * lengths[n]}}]}))
    truth.mkdir()
    for n in lengths:
        (truth / f"{n}.cif").write_text(_mini_cif())
    targets = sweep.discover_targets(str(inputs), str(truth), max_tokens=1024)
    assert [t.tokens for t in targets if t.name == "t1"] == [900] and all(t.truth for t in targets) and len(targets) == 5
    assert len(sweep.discover_targets(str(inputs), str(truth), max_tokens=280)) == 3
    shards = sweep.plan_shards(targets, 2)
    assert [t.name for t in shards[0]] == ["t1"] and sorted(t.name for t in shards[1]) == ["t2", "t3", "t4", "t5"]
    jobs = sweep.sweep_commands(targets, str(run / "pred" / "step_10"), "w.safetensors", [0, 3], [42, 43], num_samples=2, extra=["--num-recycles", "3"])
    assert [env["CUDA_VISIBLE_DEVICES"] for env, _ in jobs] == ["0", "3"] and jobs[0][0]["OMP_NUM_THREADS"] == "8"
    argv = jobs[1][1][0][2]
    assert argv[argv.index("--seed") + 1] == "42" and "--skip-existing" in argv and argv[-2:] == ["--num-recycles", "3"]
    assert len(jobs[1][1]) == 4  # two categories x two seeds on the second GPU
    r = CliRunner().invoke(cli, ["eval-sweep", "run", "--inputs", str(inputs), "--run-dir", str(run), "--gpus", "0,1", "--dry-run",
                                 "--seed", "7", "--", "--num-recycles", "2"])  # fmt: skip
    assert r.exit_code == 0 and "inference-batch" in r.output and "--num-recycles 2" in r.output, r.output

    # fabricated predictions: step 10 is worse (one sample displaced per residue), step 20 is exact
    for step, noise in ((10, 3.0), (20, 0.0)):
        for t in targets:
            tdir = run / "pred" / f"step_{step}" / t.category / t.name
            for sample in (0, 1):
                d = tdir / f"seed-42_sample-{sample}"
                d.mkdir(parents=True)
                text = _mini_cif(shift=(1.0, 2.0, 3.0))
                if noise and sample == 1:  # stretch the chain: x grows with the atom index
                    out = []
                    for line in text.splitlines():
                        f = line.split()
                        if f and f[0] == "ATOM" and len(f) > 11:
                            f[9] = f"{float(f[9]) * (1.0 + noise):.3f}"
                            line = " ".join(f)
                        out.append(line)
                    text = "\n".join(out) + "\n"
                (d / "model.cif").write_text(text)
            with open(tdir / "ranking_scores.csv", "w") as f:
                f.write("seed,sample,ranking_score\n42,0,0.2\n42,1,0.9\n")  # the ranking prefers the distorted sample
    r = CliRunner().invoke(cli, ["eval-sweep", "score", "--inputs", str(inputs), "--truth", str(truth), "--run-dir", str(run)])
    assert r.exit_code == 0, r.output
    with open(run / "eval" / "step_10" / "scores.csv") as f:
        rows = list(csv.DictReader(f))
    assert len(rows) == 10 and {r_["fold_class"] for r_ in rows} <= {"coil", "alpha", "beta", "mixed", "none"}
    with open(run / "eval" / "step_10" / "summary.csv") as f:
        summ = {(r_["category"], r_["fold_class"]): r_ for r_ in csv.DictReader(f)}
    mono = summ[("monomer_protein", "all")]
    assert int(mono["targets"]) == 3 and float(mono["lddt_oracle"]) == pytest.approx(1.0)
    assert float(mono["lddt_mean"]) < float(mono["lddt_oracle"]) and float(mono["lddt_top"]) < float(mono["lddt_oracle"])
    assert float(mono["rmsd_trace_oracle"]) < 1e-2 < float(mono["rmsd_trace_mean"])
    with open(run / "trajectory.csv") as f:
        traj = [r_ for r_ in csv.DictReader(f) if r_["category"] == "monomer_protein"]
    assert [int(float(r_["step"])) for r_ in traj] == [10, 20] and float(traj[1]["lddt_mean"]) == pytest.approx(1.0)
    assert float(traj[0]["lddt_mean"]) < float(traj[1]["lddt_mean"])

    # fold classes from C-alpha geometry: an ideal helix, an extended strand, a helix followed by a strand
    strand = np.stack([3.3 * np.arange(40), 0.9 * (np.arange(40) % 2), np.zeros(40)], 1)
    assert sweep.fold_class(_helix(60))[0] == "alpha" and sweep.fold_class(strand)[0] == "beta"
    assert sweep.fold_class(np.concatenate([_helix(40), strand + [0, 0, 80.0]]))[0] == "mixed"
    assert sweep.fold_class(np.random.default_rng(0).normal(size=(50, 3)) * 8)[0] == "coil"
    (tmp_path / "ck").mkdir()
    (tmp_path / "ck" / "checkpoint_20.pt").write_text("")
    assert sweep.resolve_checkpoint(str(tmp_path / "ck"), 20).endswith("checkpoint_20.pt") and sweep.resolve_checkpoint(str(tmp_path / "ck"), 30) is None


def test_secondary_structure_from_traces_and_helix_recovery():
    import numpy as np

    from deepfold3_dev_b200.evaluation.secondary_structure import assign_ss, runs, ss_agreement

    t = np.arange(20) * np.deg2rad(100.0)
    helix = np.stack([2.3 * np.cos(t), 2.3 * np.sin(t), 1.5 * np.arange(20)], -1)  # ideal alpha helix: 1.5 A rise, 100 degrees
    k = np.arange(12)
    strand = np.stack([3.3 * k, 0.9 * (k % 2), np.zeros(12)], -1) + helix[-1] + np.array([3.8, 0.0, 0.0])
    trace = np.concatenate([helix, strand])
    ss = assign_ss(trace)
    assert "".join(ss) == "H" * 20 + "E" * 12 and runs(ss, "H") == [(0, 20)] and runs(ss, "E") == [(20, 32)]
    walk = np.cumsum(np.random.default_rng(0).normal(size=(32, 3)) * 2.2, 0)
    assert set(assign_ss(walk)) == {"C"}
    same = ss_agreement(trace, trace)
    assert same["q3"] == 1.0 and same["f1_helix"] == 1.0 and same["f1_strand"] == 1.0 and same["helix_recovery"] == [1.0]
    lost = trace.copy()
    lost[:20] = walk[:20]  # the helix is gone, the strand is kept
    got = ss_agreement(lost, trace)
    assert got["f1_helix"] == 0.0 and got["f1_strand"] == 1.0 and got["helix_recovery"] == [0.0] and got["q3"] == 12 / 32
    half = trace.copy()
    half[10:20] = walk[:10] + trace[9]  # the second half of the helix unravels
    part = ss_agreement(half, trace)
    assert 0.3 <= part["helix_recovery_mean"] <= 0.6 and 0 < part["f1_helix"] < 1
