"""The prediction command end to end on CPU with a tiny model: steering flags, outputs, figures."""

import importlib
import importlib.util
import json
import os

import torch
from click.testing import CliRunner
from helpers import tiny_config


def test_inference_command_with_restraints_and_guidance(tmp_path, monkeypatch):
    main = importlib.import_module("deepfold3_dev_b200.cli.main")

    def tiny(params, device, optim, snapshot, allow_missing_keys, det, ccd):
        from deepfold3_dev_b200.models.model import DeepFold3

        cfg = tiny_config()
        cfg.diffusion.steps = 3
        torch.manual_seed(0)
        return DeepFold3(cfg).eval(), cfg, torch.device("cpu")

    monkeypatch.setattr(main, "_prepare_model", tiny)
    job = [{"name": "rjob", "dialect": "deepfold3", "modelSeeds": [1],
            "sequences": [{"protein": {"id": "A", "sequence": "MKTAYIAKQRQISFVKSH"}}, {"protein": {"id": "B", "sequence": "GSHMSEQNNTEMTFQ"}}]}]  # fmt: skip
    (tmp_path / "job.json").write_text(json.dumps(job))
    out = tmp_path / "out"
    res = CliRunner().invoke(main.cli, [
        "inference", "--json", str(tmp_path / "job.json"), "--output", str(out), "--num-recycles", "1", "--num-samples", "2",
        "--precision", "fp32", "--restraint", "A/3-6:B/2-5@8", "--repel", "A/10:B/10@12", "--restraint-pair", "A/1-2:B/1-2",
        "--guidance", "1.5@all@1..100", "--plot-confidences", "--msa-pairing", "none", "--no-bucket"])  # fmt: skip
    assert res.exit_code == 0, res.output + repr(res.exception)
    assert "2 samples" in res.output
    for k in (0, 1):
        files = set(os.listdir(out / f"seed-1_sample-{k}"))
        assert {"confidences.json", "logits.npz", "model.cif"} <= files
        if importlib.util.find_spec("matplotlib") is not None:  # without it the figure is skipped with a warning
            assert any(f.endswith(".png") for f in files)
    manifest = json.loads((out / "run_manifest.json").read_text())
    assert manifest["status"] == "done" and manifest["num_tokens"] == 33
    bad = CliRunner().invoke(main.cli, ["inference", "--json", str(tmp_path / "job.json"), "--output", str(out), "--restraint", "A/3-6"])
    assert bad.exit_code != 0  # a restraint needs two selectors


def test_inference_batch_shards_jobs(tmp_path, monkeypatch):
    main = importlib.import_module("deepfold3_dev_b200.cli.main")

    def tiny(params, device, optim, snapshot, allow_missing_keys, det, ccd):
        from deepfold3_dev_b200.models.model import DeepFold3

        cfg = tiny_config()
        cfg.diffusion.steps = 2
        return DeepFold3(cfg).eval(), cfg, torch.device("cpu")

    monkeypatch.setattr(main, "_prepare_model", tiny)
    paths = []
    for k in range(3):
        job = [{"name": f"j{k}", "dialect": "deepfold3", "modelSeeds": [0], "sequences": [{"protein": {"id": "A", "sequence": "MKTAYIAKQR"}}]}]
        (tmp_path / f"j{k}.json").write_text(json.dumps(job))
        paths.append(str(tmp_path / f"j{k}.json"))
    (tmp_path / "list.txt").write_text("\n".join(paths) + "\n")
    res = CliRunner().invoke(main.cli, ["inference-batch", "--inputs-file", str(tmp_path / "list.txt"), "--output-template",
                                        str(tmp_path / "out" / "{name}"), "--num-recycles", "0", "--num-samples", "1", "--precision", "fp32",
                                        "--no-bucket", "--shard", "1/2"])  # fmt: skip
    assert res.exit_code == 0, res.output + repr(res.exception)
    assert sorted(os.listdir(tmp_path / "out")) == ["j1"] and "1 jobs done" in res.output
    bad = CliRunner().invoke(main.cli, ["inference-batch", "--inputs-file", str(tmp_path / "list.txt"), "--shard", "2/2"])
    assert bad.exit_code != 0


def test_inference_batch_guidance_sweep_and_line_columns(tmp_path, monkeypatch):
    main = importlib.import_module("deepfold3_dev_b200.cli.main")

    trunk_runs = []

    def tiny(params, device, optim, snapshot, allow_missing_keys, det, ccd):
        from deepfold3_dev_b200.models.model import DeepFold3

        cfg = tiny_config()
        cfg.diffusion.steps = 2
        model = DeepFold3(cfg).eval()
        inner = model.run_evoformer
        model.run_evoformer = lambda *a, **k: (trunk_runs.append(k.get("seed")), inner(*a, **k))[1]
        return model, cfg, torch.device("cpu")

    monkeypatch.setattr(main, "_prepare_model", tiny)
    job = [{"name": "ab", "dialect": "deepfold3", "modelSeeds": [0],
            "sequences": [{"protein": {"id": "H", "sequence": "MKTAYIAKQR"}}, {"protein": {"id": "A", "sequence": "GSHMSEQNNT"}}]}]  # fmt: skip
    (tmp_path / "ab.json").write_text(json.dumps(job))
    sweep = {"groups": {"antibody": [{"name": "plain", "guidance": []}, {"name": "iface2", "guidance": ["2.0@{pairs}"]}]}}
    (tmp_path / "sweep.json").write_text(json.dumps(sweep))
    out = tmp_path / "runs" / "{cfg}" / "ab"
    (tmp_path / "list.txt").write_text(f"# json  out  columns\n{tmp_path / 'ab.json'}\t{out}\tgroup=antibody\tpairs=H:A\tseeds=5,6\n")
    lines = main.parse_inputs_file(str(tmp_path / "list.txt"))
    assert lines == [(str(tmp_path / "ab.json"), str(out), {"group": "antibody", "pairs": "H:A", "seeds": "5,6"})]
    args = ["inference-batch", "--inputs-file", str(tmp_path / "list.txt"), "--guidance-sweep", str(tmp_path / "sweep.json"),
            "--num-recycles", "0", "--num-samples", "1", "--precision", "fp32", "--no-bucket", "--no-hoist-sampler"]  # fmt: skip
    res = CliRunner().invoke(main.cli, args)
    assert res.exit_code == 0, res.output + repr(res.exception)
    assert sorted(os.listdir(tmp_path / "runs")) == ["iface2", "plain"]
    assert sorted(trunk_runs) == [5, 6]  # two settings, two seeds: the trunk ran once per seed
    for name in ("iface2", "plain"):
        run = tmp_path / "runs" / name / "ab"
        assert {"seed-5_sample-0", "seed-6_sample-0"} <= set(os.listdir(run))  # the line's seeds, not the job's
        assert json.loads((run / "run_manifest.json").read_text())["guidance_setting"] == name
    # the sweep excludes --guidance, needs {cfg} in the directory, a known group, and pairs= where an entry uses {pairs}
    assert CliRunner().invoke(main.cli, args + ["--guidance", "2.0"]).exit_code != 0
    (tmp_path / "list.txt").write_text(f"{tmp_path / 'ab.json'}\t{tmp_path / 'flat'}\tgroup=antibody\tpairs=H:A\n")
    assert CliRunner().invoke(main.cli, args).exit_code != 0
    (tmp_path / "list.txt").write_text(f"{tmp_path / 'ab.json'}\t{out}\tgroup=other\n")
    assert CliRunner().invoke(main.cli, args).exit_code != 0
    (tmp_path / "list.txt").write_text(f"{tmp_path / 'ab.json'}\t{out}\tgroup=antibody\n")
    assert CliRunner().invoke(main.cli, args).exit_code != 0
