"""Collapse-free softmax family and the single-track probe."""

import json
import os

import pytest
import torch
import torch.nn.functional as F

from deepfold3_dev_b200.training import stable_softmax as ss
from deepfold3_dev_b200.training.single_track_probe import SingleTrackProbe


def test_matches_reference_functions_at_ordinary_margins():
    torch.manual_seed(0)
    z = torch.randn(5, 7, 11, dtype=torch.float64)
    t = torch.randint(0, 11, (5, 7))
    assert torch.allclose(ss.log_softmax(z), F.log_softmax(z, -1)) and torch.allclose(ss.softmax(z, 1), F.softmax(z, 1))
    want = F.cross_entropy(z.reshape(-1, 11), t.reshape(-1), reduction="none").reshape(5, 7)
    assert torch.allclose(ss.cross_entropy(z, t), want)
    m = ss.logit_margin(z, t)
    assert torch.allclose(want, F.softplus(-m))


def test_target_gradient_survives_large_margin_in_fp32():
    z = torch.tensor([[30.0, 0.0, -1.0, 2.0]], requires_grad=True)
    t = torch.tensor([0])
    ss.cross_entropy(z, t).sum().backward()
    g = z.grad.clone()
    assert g[0, 0] < 0 and abs(float(g.sum())) < 1e-18  # gradients still sum to zero
    z2 = z.detach().clone().requires_grad_(True)
    F.cross_entropy(z2, t).backward()
    assert z2.grad[0, 0] == 0  # the standard form has lost the target gradient here
    exact = torch.softmax(z.detach().double(), -1)[0, 0] - 1
    assert abs(float(g[0, 0]) - float(exact)) / abs(float(exact)) < 1e-3


class _Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.single_transition = torch.nn.Linear(8, 8)
        self.use_single_track = True

    def forward(self, s):
        u = self.single_transition(s)
        p = getattr(self, "_probe", None)
        if p is not None and p.enabled:
            p.record_block(self._probe_layer_idx, s, u, 0.5)
        return s + 0.5 * u


class _Model(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.evoformer = torch.nn.Module()
        self.evoformer.trunk_pairformer = torch.nn.ModuleList(_Block() for _ in range(3))

    def forward(self, s):
        for b in self.evoformer.trunk_pairformer:
            s = b(s)
        return s


def test_probe_writes_one_row_per_probed_step(tmp_path):
    torch.manual_seed(0)
    model = _Model()
    probe = SingleTrackProbe(model, str(tmp_path / "probe.jsonl"))
    x = torch.randn(2, 5, 8)
    model(x)  # not probed
    probe.begin_step(7)
    model(x)
    probe.end_step({"loss": 1.5})
    probe.begin_step(8)
    probe.discard_step()
    rows = [json.loads(line) for line in open(tmp_path / "probe.jsonl")]
    assert len(rows) == 1 and rows[0]["step"] == 7 and rows[0]["loss"] == 1.5
    assert rows[0]["rms_s_l0"] > 0 and -1 <= rows[0]["cos_su_mean"] <= 1 and "sum_gamma_alpha" in rows[0]
    assert "w_norm_single_transition_l_last" in rows[0]


def test_checkpoint_report_and_run_status(tmp_path):
    from deepfold3_dev_b200.utils.run_tools import checkpoint_report, run_status

    model = {"evoformer.a.weight": torch.ones(4, 4), "evoformer.a.bias": torch.tensor([float("nan"), 1.0]), "head.w": torch.full((3,), 2.0)}
    torch.save({"model": model, "ema": {"evoformer.a.weight": torch.zeros(4, 4)}, "global_step": 12}, tmp_path / "c.pt")
    rep = checkpoint_report(str(tmp_path / "c.pt"))
    assert rep["total_parameters"] == 21 and rep["meta"]["global_step"] == 12 and rep["non_finite"][0]["name"] == "evoformer.a.bias"
    rows = {r["module"]: r for r in rep["modules"]}
    assert rows["evoformer.a"]["ema_distance"] == 4.0 and abs(rows["head.w"]["norm"] - 12**0.5) < 1e-6
    os_dir = tmp_path / "run" / "logs"
    os_dir.mkdir(parents=True)
    with open(os_dir / "metrics.jsonl", "w") as f:
        for i in range(10):
            f.write(json.dumps({"step": i, "time": 100.0 + 2 * i, "train/loss": 5.0 - 0.3 * i}) + "\n")
        f.write('{"step": 10, "ti')  # a torn last line
    st = run_status(str(tmp_path / "run"))
    assert st["rows"] == 10 and st["last_step"] == 9 and abs(st["steps_per_hour"] - 1800.0) < 1e-6
    assert st["loss_recent_mean"] < st["loss_earlier_mean"] and st["non_finite_losses"] == 0


def test_deploy_recipes_render_and_parse(tmp_path):
    """The cluster recipes: shell files parse, manifests are valid YAML, the multi-node template renders with no token
    left, the RDMA address map resolves an address against a stand-in for kubectl, and the collective check runs on gloo."""
    import json
    import subprocess
    import sys

    import yaml

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    dep = os.path.join(root, "deploy")
    shells = [os.path.join(d, f) for d, _, fs in os.walk(dep) for f in fs if f.endswith((".sh", ".sbatch"))]
    assert len(shells) >= 12
    for path in shells:
        assert subprocess.run(["bash", "-n", path], capture_output=True).returncode == 0, path
    for name in ("trainjob.yaml", "comm-check.yaml", "plm-job.yaml"):
        with open(os.path.join(dep, "k8s", name)) as f:
            assert all(d["kind"] in ("PyTorchJob", "Job") for d in yaml.safe_load_all(f))
    env = dict(os.environ, DRY_RUN="1", NODES="4", EXCLUDE_HOSTS="host-a,host-b", IB_HCA="=mlx5_0,mlx5_1", DF3_COMM_LOG="1")
    out = subprocess.run(["bash", os.path.join(dep, "k8s", "submit.sh"), "My_Run", "--override", "max_steps=5"],
                         capture_output=True, text=True, env=env)  # fmt: skip
    assert out.returncode == 0 and "__" not in out.stdout.replace("__main__", ""), out.stderr
    job = yaml.safe_load(out.stdout)
    assert job["metadata"]["name"] == "my-run" and job["spec"]["pytorchReplicaSpecs"]["Worker"]["replicas"] == 3
    pod = job["spec"]["pytorchReplicaSpecs"]["Master"]["template"]
    terms = pod["spec"]["affinity"]["nodeAffinity"]["requiredDuringSchedulingIgnoredDuringExecution"]["nodeSelectorTerms"]
    assert terms[0]["matchExpressions"][1]["values"] == ["host-a", "host-b"]
    script = pod["spec"]["containers"][0]["args"][0]
    assert "--override max_steps=5" in script and "DF3_NODES=4" in script and "DF3_COMM_LOG=1" in script
    assert pod["spec"]["containers"][0]["resources"]["limits"] == {"nvidia.com/gpu": 8, "rdma/hca": 8}
    # env.sh: several nodes -> NCCL gradient transport, RAS and flight recorder on, verbose logging only on request
    probe = subprocess.run(["bash", "-c", f"DF3_NODES=2 DF3_COMM_LOG=1 source {dep}/env.sh && df3_describe_env"],
                           capture_output=True, text=True)  # fmt: skip
    assert "DF3_COMM=collective" in probe.stdout and "NCCL_RAS_ENABLE=1" in probe.stdout and "NCCL_DEBUG=INFO" in probe.stdout
    quiet = subprocess.run(["bash", "-c", f"unset DF3_COMM; source {dep}/env.sh && df3_describe_env"], capture_output=True, text=True)
    assert "NCCL_DEBUG=WARN" in quiet.stdout and "DF3_COMM=" not in quiet.stdout
    # address map against a stand-in for kubectl
    pods = {"items": [{"metadata": {"name": "my-run-worker-1", "annotations": {"k8s.v1.cni.cncf.io/network-status": json.dumps(
        [{"name": "k8s", "ips": ["192.168.0.4"], "default": True}, {"name": "rdma-net", "ips": ["10.1.2.3"]}])}},
        "spec": {"nodeName": "host-q"}, "status": {"phase": "Running"}}]}  # fmt: skip
    (tmp_path / "pods.json").write_text(json.dumps(pods))
    fake = tmp_path / "kubectl"
    fake.write_text(f"#!/bin/bash\ncat {tmp_path}/pods.json\n")
    fake.chmod(0o755)
    res = subprocess.run(["bash", os.path.join(dep, "k8s", "rdma_ip_map.sh"), "my-run", "10.1.2.3"], capture_output=True,
                         text=True, env=dict(os.environ, KUBECTL=str(fake)))  # fmt: skip
    assert "10.1.2.3: host host-q, pod my-run-worker-1" in res.stdout, res.stdout + res.stderr
    # collective check on two gloo ranks
    table = tmp_path / "cc.json"
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
                          "--nproc-per-node", "2", os.path.join(dep, "comm_check.py"), "--sizes-mib", "1", "--iters", "2",
                          "--warmup", "1", "--json", str(table), "--peer", "--peer-transport", "collective"],
                         capture_output=True, text=True, timeout=300)  # fmt: skip
    assert run.returncode == 0, run.stderr[-2000:]
    rows = json.loads(table.read_text())["rows"]
    assert {r["op"] for r in rows} == {"all_reduce", "all_gather", "peer_all_gather", "peer_transpose", "peer_rows_to_channels"}
    assert all(r["busbw_gbs"] > 0 for r in rows)


def test_every_shipped_config_loads():
    """Each file under configs/ builds: the structure-model recipes (initial, stages 0-4, fine-tuning) through the
    config loader with their `base:` chains, the language-model ones through theirs; the stage-0 family is the wide-pair
    variant without triangle attention and without the Pairformer single track."""
    import glob

    import torch

    from deepfold3_dev_b200.complexlm.config import load_experiment
    from deepfold3_dev_b200.complexlm.model import ComplexLM
    from deepfold3_dev_b200.config.loader import build_configs
    from deepfold3_dev_b200.models.model import DeepFold3

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")
    files = sorted(glob.glob(os.path.join(root, "*.yaml")))
    assert len(files) >= 16
    sizes = {}
    for path in files:
        name = os.path.basename(path)[:-5]
        if name.startswith("plm-"):
            cfg = load_experiment(path)
            with torch.device("meta"):
                sizes[name] = sum(p.numel() for p in ComplexLM(cfg.model).parameters())
        else:
            tc, mc = build_configs([path], [])
            assert tc.max_tokens >= 64 and mc.pairformer.num_layer >= 1, name
            if name.startswith("stage"):
                assert mc.pairformer.pair_channel == 256 and not mc.pairformer.use_single_track
                assert not mc.evoformer.use_triangle_attention and mc.diffusion.conditioning_pair_channel == 256
    assert sizes["plm-8m"] < sizes["plm-35m"] < sizes["plm-150m"] < sizes["plm-base"] and 6.5e8 < sizes["plm-base"] < 7e8
    tc, mc = build_configs([os.path.join(root, "stage4.yaml")], [])
    assert (tc.max_tokens, tc.max_atoms, mc.data.max_chains) == (768, 10368, 50) and tc.extra_datasets[0].format == "of3pdb"
    with torch.device("meta"):
        wide = DeepFold3(mc)
    names = dict(wide.named_parameters())
    assert not any(".pairformer." in n and "single_attn" in n for n in names)


def test_benchmark_plots(tmp_path):
    """Row lists of the three benchmark kinds render to PNG files (needs matplotlib; without it the tool says so)."""
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks"))
    import plot_results

    files = {
        "m.json": [{"module": "a", "tokens": 384, "backward": False, "ours_ms": 0.5, "eager_ms": 2.0, "speedup": 4.0}],
        "p.json": [{"impl": "ours", "regime": "inference", "blocks": 8, "tokens": 384, "ms": 12.7},
                   {"impl": "reference", "regime": "inference", "blocks": 8, "tokens": 384, "ms": 37.7}],
        "v.json": [{"module": "a", "out_err_kernels": 1e-3, "out_err_pytorch_bf16": 2e-3, "grad_err_kernels": 3e-3, "grad_err_pytorch_bf16": 2e-3}],
    }  # fmt: skip
    for name, rows in files.items():
        (tmp_path / name).write_text(json.dumps(rows))
    try:
        import matplotlib  # noqa: F401
    except ImportError:
        with pytest.raises(RuntimeError, match="matplotlib"):
            plot_results.plot_file(str(tmp_path / "m.json"), str(tmp_path / "plots"))
        return
    for name in files:
        assert os.path.getsize(plot_results.plot_file(str(tmp_path / name), str(tmp_path / "plots"))) > 1000
    (tmp_path / "x.json").write_text(json.dumps([{"something": 1}]))
    with pytest.raises(ValueError, match="unknown benchmark"):
        plot_results.plot_file(str(tmp_path / "x.json"), str(tmp_path / "plots"))


def test_guides_name_existing_commands_files_and_switches():
    """Every command, source path and environment switch the guides mention exists in the package."""
    import re
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    listing = subprocess.check_output([sys.executable, "-m", "deepfold3_dev_b200.cli", "--help"], cwd=root, text=True)
    commands = {line.split()[0] for line in listing.split("Commands:")[1].splitlines() if line.startswith("  ") and line.split()}
    sources = ""
    for base, _, names in os.walk(root):
        if any(part in base for part in ("/.git", "/_work", "_out", "/baseline/_ref", "/build")):
            continue
        for n in names:
            if n.endswith((".py", ".cu", ".cuh", ".h", ".sh")):
                with open(os.path.join(base, n), errors="ignore") as f:
                    sources += f.read()
    guides = sorted(os.listdir(os.path.join(root, "docs")))
    assert {"training.md", "inference.md", "data-pipeline.md", "kernels.md", "parallelism.md", "complex-lm.md"} <= set(guides)
    prefixes = "deepfold3_dev_b200/|ops/|data/|models/|training/|parallel/|inference/|utils/|complexlm/|config/|evaluation/|benchmarks/|deploy/|configs/|tests/|profiles/"
    for g in guides:
        with open(os.path.join(root, "docs", g)) as f:
            text = f.read()
        for cmd in re.findall(r"deepfold3_dev_b200\.cli ([a-z][a-z0-9-]+)", text):
            assert cmd in commands, (g, cmd)
        for path in re.findall(rf"`((?:{prefixes})[A-Za-z0-9_./-]+\.(?:py|cu|cuh|h|yaml|md|sh))", text):
            assert os.path.exists(os.path.join(root, path)) or os.path.exists(os.path.join(root, "deepfold3_dev_b200", path)), (g, path)
        for var in set(re.findall(r"\b(DF3_[A-Z_]+|DEEPFOLD3_[A-Z_]+)\b", text)):
            assert var in sources, (g, var)


def test_triage_finds_offender_divergence_gradient_agreement_series_and_mirror(tmp_path):
    import json

    import numpy as np
    import torch
    from click.testing import CliRunner

    from deepfold3_dev_b200.utils import triage as T

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b, self.c = torch.nn.Linear(4, 4), torch.nn.Linear(4, 4), torch.nn.Linear(4, 4)
            self.poison = False

        def forward(self, x):
            h = self.b(self.a(x))
            return self.c(h / 0.0 if self.poison else h)

    net = Net()
    x = torch.randn(3, 4)
    clean = T.activation_trace(net, lambda: net(x))
    assert [r.name for r in clean] == ["a", "b", "c"] and T.first_nonfinite(clean) is None
    net.poison = True
    bad = T.activation_trace(net, lambda: net(x))
    assert T.first_nonfinite(bad).name == "c"  # a and b were still finite
    net.poison = False
    with torch.no_grad():
        net.b.weight.mul_(3.0)
    parted = T.diff_traces(clean, T.activation_trace(net, lambda: net(x)))
    assert parted and parted[0]["name"] == "b"  # the first module whose magnitude moved
    assert T.largest_activations(clean, 1)[0].abs_max == max(r.abs_max for r in clean)

    # gradients that agree, then gradients that are independent
    base = torch.randn(1000)
    same, indep = T.GradientSpread(), T.GradientSpread()
    for k in range(16):
        same.add(base * (1 + 0.1 * k))
        indep.add(torch.randn(1000))
    a, b = same.result(), indep.result()
    assert abs(a["resultant_length"] - 1) < 1e-9 and abs(a["mean_pairwise_cosine"] - 1) < 1e-9
    assert abs(b["mean_pairwise_cosine"]) < 0.1 and b["resultant_length"] < 0.5 and abs(b["independent_baseline"] - 0.25) < 1e-12

    # a growing series floats to the top
    (tmp_path / "logs").mkdir()
    with open(tmp_path / "logs" / "metrics.jsonl", "w") as f:
        for step in range(0, 2000, 100):
            f.write(json.dumps({"step": step, "train/act_rms/pair_max": 1.0 * np.exp(step / 1000), "train/act_rms/single_max": 2.0, "train/loss": 3.0}) + "\n")
    rows = T.series_summary(str(tmp_path), "act_rms", ceiling=3.0)
    assert [r["series"] for r in rows] == ["act_rms/pair_max", "act_rms/single_max"]
    assert abs(rows[0]["log_slope_per_1k_steps"] - 1.0) < 1e-6 and rows[0]["above_ceiling"] and not rows[1]["above_ceiling"]

    # a right-handed helix against itself and against its mirror image
    t = np.arange(30) * np.deg2rad(100.0)
    helix = np.stack([2.3 * np.cos(t), 2.3 * np.sin(t), 1.5 * np.arange(30)], -1)
    rot, _ = np.linalg.qr(np.random.default_rng(0).normal(size=(3, 3)))
    rot *= np.sign(np.linalg.det(rot))
    ok = T.handedness(helix @ rot.T + 5.0, helix)
    flipped = T.handedness((helix * np.array([1.0, 1.0, -1.0])) @ rot.T, helix)
    assert not ok["mirror_image"] and ok["dihedral_sign_match"] == 1.0 and ok["rmsd_proper"] < 1e-6
    assert flipped["mirror_image"] and flipped["dihedral_sign_match"] == 0.0 and flipped["rmsd_mirrored"] < 1e-6 < flipped["rmsd_proper"]

    import importlib

    cli_main = importlib.import_module("deepfold3_dev_b200.cli.main")
    res = CliRunner().invoke(cli_main.cli, ["triage", "series", str(tmp_path), "--prefix", "act_rms"])
    assert res.exit_code == 0 and "act_rms/pair_max" in res.output
    cfg = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "smoke.yaml")
    res = CliRunner().invoke(cli_main.cli, ["triage", "activations", "--config", cfg, "--tokens", "24", "--top", "3"])
    assert res.exit_code == 0, res.output + repr(res.exception)
    report = json.loads(res.output)
    assert report["first_nonfinite"] is None and len(report["largest"]) == 3 and report["modules_called"] > 50
    res = CliRunner().invoke(cli_main.cli, ["triage", "distogram", "--config", cfg, "--tokens", "24", "--save", str(tmp_path / "maps.npz")])
    assert res.exit_code == 0, res.output + repr(res.exception)
    report = json.loads(res.output)
    # the head's output layer starts at zero: every bin equally likely, so the cross-entropy is log(bins)
    assert report["pairs"] == 24 * 23 and abs(report["cross_entropy"] - report["uniform_cross_entropy"]) < 1e-4
    maps = np.load(tmp_path / "maps.npz")
    assert maps["true_distance"].shape == maps["expected_distance"].shape == (24, 24)
