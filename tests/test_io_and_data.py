"""CPU tests of the output layer and the data side; metric formulas are checked against the reference package."""

import json
import os
import struct

import numpy as np
import pytest
import torch

from deepfold3_dev_b200.data import cropper, datasets, pack, samplers
from deepfold3_dev_b200.data.inference_input import InferenceInput
from deepfold3_dev_b200.data.parse.a3m import parse_a3m
from deepfold3_dev_b200.data.parse.json_input import parse_json_input
from deepfold3_dev_b200.data.synthetic import synthetic_complex
from deepfold3_dev_b200.io import confidences as conf
from deepfold3_dev_b200.io import logit_codec, mmcif
from deepfold3_dev_b200.io.background_writer import BackgroundWriter
from deepfold3_dev_b200.models import bucket


def _feats():
    return synthetic_complex([("protein", 14), ("protein", 11), ("ligand", 5)], num_msa=6, num_templates=1, seed=3, with_gt=False)


def test_confidence_metrics_match_reference(reference_package):
    from deepfold3.io import confidences as R

    torch.manual_seed(0)
    f = _feats()
    N = f["res_type"].shape[0]
    pae, pde, plddt = torch.randn(2, N, N, 64) * 2, torch.randn(2, N, N, 64), torch.randn(2, N, 24 * 50)
    seq = f["seq_mask"].float()
    pm = seq[:, None] * seq[None, :]
    am = f["ref_mask"].float()
    torch.testing.assert_close(conf.error_bin_centers(), R._error_bin_centers())
    for mine, ref in zip(conf.compute_plddt(plddt, am), R.compute_plddt(plddt, am)):
        torch.testing.assert_close(mine, ref)
    torch.testing.assert_close(conf.compute_pae(pae, pm), R.compute_pae(pae, pm))
    for mine, ref in zip(conf.compute_pde(pde, pm), R.compute_pde(pde, pm)):
        torch.testing.assert_close(mine, ref)
    assert conf.compute_ptm(pae[0], seq, pm) == pytest.approx(R.compute_ptm(pae[0], seq, pm), rel=1e-5)
    assert conf.compute_iptm(pae[0], seq, pm, f["asym_id"]) == pytest.approx(R.compute_iptm(pae[0], seq, pm, f["asym_id"]), rel=1e-5)
    assert conf.compute_ranking_score(0.5, 0.7, 0.1, True) == pytest.approx(R.compute_ranking_score(0.5, 0.7, 0.1, True))
    assert conf.compute_ranking_score(0.5, float("nan")) == pytest.approx(R.compute_ranking_score(0.5, float("nan")))


def test_clash_and_single_chain_iptm():
    f = synthetic_complex([("protein", 10)], num_msa=2, num_templates=0, seed=1, with_gt=False)
    pae = torch.randn(10, 10, 64)
    assert np.isnan(conf.compute_iptm(pae, f["seq_mask"].float(), torch.ones(10, 10), f["asym_id"]))
    spread = torch.arange(10 * 24 * 3).float().view(10, 24, 3)
    poly = f["mol_type"] != 3
    assert not conf.has_clash(spread, f["ref_mask"].float(), f["residue_index"], f["asym_id"], poly)
    collapsed = torch.zeros(10, 24, 3)
    assert conf.has_clash(collapsed, f["ref_mask"].float(), f["residue_index"], f["asym_id"], poly)


def test_mmcif_text_and_logit_codec(tmp_path):
    f = _feats()
    N = f["res_type"].shape[0]
    txt = mmcif.structure_to_mmcif(torch.randn(2, N, 24, 3), torch.rand(2, N, 24) * 100, f, chain_names=["A", "B", "L"])
    atoms = [ln for ln in txt.splitlines() if ln.startswith(("ATOM", "HETATM"))]
    assert len(atoms) == 2 * int(f["ref_mask"].sum())
    assert atoms[0].split()[3] == "N" and atoms[0].split()[6] == "A" and atoms[-1].split()[-1] == "2"
    assert mmcif.asym_id_to_chain_name(0) == "A" and mmcif.asym_id_to_chain_name(26) == "AA"
    logits = np.random.RandomState(0).randn(5, 7, 64).astype(np.float32) * 4
    for scheme, tol in (("f32", 1e-7), ("f16", 1e-2), ("u8", 3e-2)):
        path = str(tmp_path / f"l_{scheme}.npz")
        logit_codec.save_logits(path, {"pae": logits}, scheme, attrs={"job": "x"})
        back = logit_codec.load_logits(path)
        assert back.attrs["job"] == "x" and logit_codec.head_names(path) == ["pae"]
        assert np.abs(logit_codec.softmax(back["pae"]) - logit_codec.softmax(logits)).max() < tol


def test_background_writer_orders_and_reports_errors(tmp_path):
    seen = []
    with BackgroundWriter() as w:
        for i in range(5):
            w.submit(seen.append, i)
    assert seen == [0, 1, 2, 3, 4]
    w = BackgroundWriter()
    w.submit(lambda: 1 / 0)
    with pytest.raises(RuntimeError, match="background write failed"):
        w.close()


def test_a3m_and_json_dialects(tmp_path):
    m = parse_a3m(">q\nACDE\n>h1\nAC-aaE\n>dup\nACDE\n")
    assert m.sequences == ["ACDE", "AC-E"] and m.deletions.tolist() == [[0, 0, 0, 0], [0, 0, 0, 2]]
    af3 = {"name": "t", "modelSeeds": [4], "sequences": [
        {"protein": {"id": ["A", "B"], "sequence": "ACDEFGHIK", "unpairedMsa": ">q\nACDEFGHIK\n>h\nAC-EFGHaIK\n"}},
        {"rna": {"id": "R", "sequence": "ACGU"}}, {"ligand": {"id": "Z", "ccdCodes": ["ZN"]}}]}  # fmt: skip
    p = tmp_path / "j.json"
    p.write_text(json.dumps(af3))
    (job,) = parse_json_input(str(p))
    assert job.dialect == "alphafold3" and job.num_chains == 4 and job.seeds == [4]
    inp = InferenceInput.from_job(job)
    f = inp.features
    assert inp.num_tokens == 9 + 9 + 4 + 1 and inp.chain_names == ["A", "B", "R", "Z"]
    assert f["entity_id"].tolist() == [0] * 18 + [1] * 4 + [2] and f["sym_id"][9:18].tolist() == [1] * 9
    assert f["msa"].shape == (3, 23) and f["msa"][1, 9:].eq(21).all() and f["deletion_matrix"][1, 7] == 1
    assert f["ref_mask"][0].sum() == 5 and f["ref_mask"][-1].sum() == 1 and int(f["ref_element"][-1, 0]) == 30
    server = [{"name": "s", "sequences": [{"proteinChain": {"sequence": "ACD", "count": 2}}, {"ion": {"ion": "MG", "count": 1}}]}]
    (sjob,) = parse_json_input(server)
    assert sjob.dialect == "alphafoldserver" and sjob.num_chains == 3
    ptx = [{"name": "p", "sequences": [{"proteinChain": {"sequence": "ACD", "count": 1, "msa": {}}}]}]
    assert parse_json_input(ptx)[0].dialect == "protenix"
    with pytest.raises(ValueError, match="conformer"):
        InferenceInput.from_job(parse_json_input({"name": "l", "sequences": [{"ligand": {"id": "L", "ccdCodes": ["ATP"]}}]})[0])


def test_job_dialect_details(tmp_path, caplog):
    """Behaviour of the job parser beyond the happy path: seeds per dialect, key aliases, SMILES against component codes,
    Protenix alignment directories, HHsearch hit files, user dictionaries from a path, the template date cut-off,
    tolerant handling of malformed optional parts, errors for unusable jobs, alignment search on demand."""
    import logging

    from deepfold3_dev_b200.data.parse import json_input as ji

    # seeds: the file formats fall back to 42, the server format draws one
    assert parse_json_input({"sequences": [{"protein": {"id": "A", "sequence": "ACD"}}]})[0].seeds == [42]
    drawn = parse_json_input([{"name": "s", "sequences": [{"proteinChain": {"sequence": "ACD", "count": 1}}]}])[0].seeds
    assert len(drawn) == 1 and 0 <= drawn[0] < 2**32
    # Protenix: chain-key aliases, alignment directory, ligand as component code or SMILES
    pre = tmp_path / "msa" / "0"
    pre.mkdir(parents=True)
    (pre / "non_pairing.a3m").write_text(">q\nACDEF\n>u\nACDEF\n")
    (pre / "pairing.a3m").write_text(">q\nACDEF\n>p\nAC-EF\n")
    ptx = tmp_path / "ptx.json"
    ptx.write_text(json.dumps([{"name": "p", "modelSeeds": [], "sequences": [
        {"proteinChain": {"sequence": "acdef", "count": 2, "msa": {"precomputed_msa_dir": "msa/0"},
                          "modifications": [{"ptmType": "CCD_SEP", "ptmPosition": 3}, {"ptmType": "TPO"}, "junk"]}},
        {"rnaChain": {"sequence": "ACGU", "count": 1, "modifications": [{"modificationType": "2MG", "basePosition": 1}]}},
        {"dnaChain": {"sequence": "ACGT", "count": 1}},
        {"ligand": {"ligand": "CCD_ATP", "count": 1}}, {"ligand": {"ligand": "CC(=O)O", "count": 2}}]}]))  # fmt: skip
    with caplog.at_level(logging.WARNING):
        (job,) = parse_json_input(str(ptx))
    prot, rna, dna, atp, smi = job.chains
    assert job.dialect == "protenix" and job.seeds == [42] and job.num_chains == 7
    assert prot.sequence == "ACDEF" and prot.ids == ["A", "B"] and prot.modifications == [("SEP", 3)]
    assert prot.unpaired_msa.count(">") == 2 and "AC-EF" in prot.paired_msa
    assert rna.mol_type == 2 and rna.modifications == [("2MG", 1)] and dna.mol_type == 1
    assert atp.ccd_codes == ["ATP"] and atp.smiles is None and smi.smiles == "CC(=O)O" and smi.ccd_codes == [] and smi.ids == ["F", "G"]
    assert sum("modification skipped" in r.message for r in caplog.records) == 2
    # the server format names components with or without the prefix
    srv = parse_json_input([{"name": "s", "modelSeeds": ["7"], "sequences": [{"proteinChain": {"sequence": "ACD", "count": 1}},
                            {"ligand": {"ligand": "HEM", "count": 1}}, {"ion": {"ion": "CCD_MG", "count": 2}}]}])[0]  # fmt: skip
    assert srv.dialect == "alphafoldserver" and srv.seeds == [7] and srv.chains[1].ccd_codes == ["HEM"] and srv.chains[2].ccd_codes == ["MG"]

    # AF3: HHsearch hits, dictionary from a path, template date cut-off, malformed bonds
    hhr = tmp_path / "hits.hhr"
    hhr.write_text("Query q\n\nNo 1\n>1abc_B some protein\nProbab=99.0 E-value=1e-20 Score=100 Aligned_cols=4 Identities=50% Similarity=0.5 Sum_probs=3.5\n\n"
                   "Q q 2 CDEF 5 (5)\nQ Consensus 2 cdef 5 (5)\nT Consensus 10 cdxf 13 (90)\nT 1abc_B 10 CD-F 13 (90)\n\n")
    (tmp_path / "my.cif").write_text("data_LIG\n_chem_comp.id LIG\n")
    af3 = tmp_path / "af3.json"
    af3.write_text(json.dumps({"name": "t", "maxTemplateDate": "2020-01-01", "userCCDPath": "my.cif", "description": "demo",
        "bondedAtomPairs": [[["A", 1, "CA"], ["L", 1, "C1"]], [["A", 1], ["L", 1, "C1"]], "x"],
        "sequences": [{"protein": {"id": "A", "sequence": "ACDEF", "templatesPath": "hits.hhr", "description": "chain a"}},
                      {"protein": {"id": "B", "sequence": "GHIKL", "templates": [
                          {"mmcifPath": "old.cif", "queryIndices": [0], "templateIndices": [0], "releaseDate": "2019-05-05"},
                          {"mmcifPath": "new.cif", "queryIndices": [0], "templateIndices": [0], "releaseDate": "2021-02-03"},
                          {"mmcifPath": "undated.cif", "queryIndices": [0], "templateIndices": [0]}]}},
                      {"ligand": {"id": "L", "smiles": "CCO"}}]}))  # fmt: skip
    caplog.clear()
    with caplog.at_level(logging.WARNING):
        (job,) = parse_json_input(str(af3))
    a, b, lig = job.chains
    assert job.max_template_date == "2020-01-01" and job.user_ccd.startswith("data_LIG") and job.description == "demo" and a.description == "chain a"
    assert len(job.bonded_atom_pairs) == 1 and sum("bondedAtomPairs entry skipped" in r.message for r in caplog.records) == 2
    (hit,) = a.templates
    assert (hit["pdbId"], hit["chainId"], hit["queryIndices"], hit["templateIndices"]) == ("1ABC", "B", [1, 2, 4], [9, 10, 11])
    assert [h["mmcifPath"] for h in b.templates] == ["old.cif", "undated.cif"] and b.templates[0]["_base_dir"] == str(tmp_path)
    assert parse_json_input({"maxTemplateDate": "soon", "sequences": [{"protein": {"id": "A", "sequence": "AC"}}]})[0].max_template_date is None

    # unusable jobs and arguments
    with pytest.raises(ValueError, match="no chains"):
        parse_json_input({"name": "empty", "sequences": []})
    with pytest.raises(ValueError, match="unknown sequence entry"):
        parse_json_input({"name": "x", "sequences": [{"peptoid": {"sequence": "AA"}}]})
    with pytest.raises(ValueError, match="msa_pairing"):
        parse_json_input({"sequences": [{"protein": {"id": "A", "sequence": "AC"}}]}, msa_pairing="sometimes")

    # alignment search on demand: once per job, distinct sequences without an alignment only
    calls = []

    def fake_search(seqs):
        calls.append(list(seqs))
        return [{"unpaired": f">q\n{s}\n>h\n{s}\n", "paired": None, "templates": [{"pdbId": "2XYZ", "chainId": "A", "queryIndices": [0],
                 "templateIndices": [0], "releaseDate": "2030-01-01"}]} for s in seqs]  # fmt: skip

    (job,) = parse_json_input({"name": "m", "maxTemplateDate": "2025-01-01", "sequences": [
        {"protein": {"id": ["A", "B"], "sequence": "ACDEF"}}, {"protein": {"id": "C", "sequence": "GHIKL", "unpairedMsa": ">q\nGHIKL\n"}},
        {"protein": {"id": "D", "sequence": "MNPQR"}}]}, msa_search=fake_search)  # fmt: skip
    assert calls == [["ACDEF", "MNPQR"]] and job.chains[0].unpaired_msa.count(">") == 2 and job.chains[1].unpaired_msa.count(">") == 1
    assert job.chains[0].templates == []  # the searched hit is newer than the job's cut-off
    assert ji.detect_dialect({"dialect": "Protenix", "sequences": []}) == "protenix"


def test_modified_residue_keeps_alignment_and_template_columns(tmp_path):
    """A chain with a modified residue is tokenised per atom at that residue; every token still reads the alignment and
    template column of its residue (the chain must not fall back to a query-only alignment)."""
    from test_prepare import _mini_cif

    from deepfold3_dev_b200.data import ref_conformers

    ref_conformers._TABLE["SEP"] = {"atoms": ["N", "CA", "C", "O", "CB", "OG", "P", "O1P", "O2P", "O3P"], "elements": [7, 6, 6, 8, 6, 8, 15, 8, 8, 8],
                                    "charges": [0] * 10, "coords": [[float(i), 0.5 * i, 0.0] for i in range(10)]}  # fmt: skip
    try:
        (tmp_path / "t.cif").write_text(_mini_cif())
        job = {"name": "m", "sequences": [
            {"protein": {"id": "A", "sequence": "GASG", "modifications": [{"ptmType": "SEP", "ptmPosition": 3}],
                         "unpairedMsa": ">q\nGASG\n>h1\nGTSG\n>h2\nG-SaG\n",
                         "templates": [{"mmcifPath": "t.cif", "chainId": "A", "queryIndices": [0, 1, 2], "templateIndices": [0, 1, 2]}]}},
            {"protein": {"id": "B", "sequence": "ACD", "unpairedMsa": ">q\nACD\n>h\nAGD\n"}}]}  # fmt: skip
        p = tmp_path / "job.json"
        p.write_text(json.dumps(job))
        inp = InferenceInput.from_job(parse_json_input(str(p))[0], msa_pairing="none")
        f = inp.features
        # chain A: G, A, ten atom tokens of SEP, G  -> 13 tokens; chain B: 3
        assert inp.num_tokens == 13 + 3 and f["residue_index"][:13].tolist() == [0, 1] + [2] * 10 + [3]
        ser = const_res("SER")
        assert f["msa"].shape[0] == 4  # query + two rows of A + one row of B
        assert f["msa"][1, :13].tolist() == [const_res("GLY"), const_res("THR")] + [ser] * 10 + [const_res("GLY")]
        assert f["msa"][2, 1] == 21 and f["deletion_matrix"][2, 12] == 1 and (f["msa"][1, 13:] == 21).all()
        assert f["template_mask"][0] == 1 and f["template_aatype"][0, :13].tolist() == [const_res("GLY"), const_res("ALA")] + [ser] * 10 + [21]
        assert f["template_pseudo_beta_mask"][0, 2:12].eq(1).all() and (f["template_aatype"][0, 13:] == 21).all()
    finally:
        ref_conformers._TABLE.pop("SEP", None)


def const_res(name):
    from deepfold3_dev_b200.data import const

    return const.RES_TYPE_ORDER[name]


def test_crops_keep_consistency():
    f = synthetic_complex([("protein", 60), ("protein", 50), ("ligand", 6)], num_msa=8, num_templates=2, seed=1)
    for strategy in ("contiguous", "spatial", "spatial_interface"):
        c, used = cropper.crop(f, 48, 300, torch.Generator().manual_seed(3), strategy=strategy)
        n = c["res_type"].shape[0]
        assert used == strategy and n <= 48 and int(c["ref_mask"].sum()) <= 300
        assert c["msa"].shape == (8, n) and c["template_aatype"].shape == (2, n) and c["pair_mask"].shape == (n, n)
        assert c["token_index"].tolist() == list(range(n)) and int(c["frame_token_index"].max()) < n
    inter, _ = cropper.crop(f, 48, 0, torch.Generator().manual_seed(5), strategy="spatial_interface")
    assert len(torch.unique(inter["asym_id"])) >= 2
    same, used = cropper.crop(f, 500)
    assert used == "none" and same is f


def test_crop_seeding_budgets_and_resolved_tokens():
    """Spatial crops on a constructed geometry: unresolved tokens are never selected, the anchor chain / interface
    decides where the seed falls, the atom budget cuts the farthest tokens (not the last by index), a crop with too
    few resolved tokens is redrawn, and the contiguous crop meets its budget."""
    n_a, n_b, n_c = 40, 40, 30
    n = n_a + n_b + n_c
    # three straight chains: A along x at y=0, B parallel at y=8 (touches A everywhere), C far away at y=200
    xyz = torch.zeros(n, 3)
    xyz[:n_a, 0] = torch.arange(n_a) * 3.8
    xyz[n_a : n_a + n_b, 0] = torch.arange(n_b) * 3.8
    xyz[n_a : n_a + n_b, 1] = 8.0
    xyz[n_a + n_b :, 0] = torch.arange(n_c) * 3.8
    xyz[n_a + n_b :, 1] = 200.0
    asym = torch.cat([torch.zeros(n_a), torch.ones(n_b), torch.full((n_c,), 2)]).long()
    resolved = torch.ones(n, dtype=torch.bool)
    resolved[5:15] = False  # an unresolved stretch inside chain A
    atoms = torch.full((n,), 5)
    g = lambda s: torch.Generator().manual_seed(s)  # noqa: E731

    for seed in range(6):
        keep = cropper.spatial_crop(xyz, resolved, asym, 24, g(seed), False, atoms, 0, anchor=("chain", 2, -1))
        assert (asym[keep] == 2).all() and len(keep) == 24  # seeded in the anchor chain, which is far from the others
        keep = cropper.spatial_crop(xyz, resolved, asym, 24, g(seed), True, atoms, 0, anchor=("interface", 0, 1))
        assert set(asym[keep].tolist()) == {0, 1} and resolved[keep].all()
        keep = cropper.spatial_crop(xyz, resolved, asym, 30, g(seed), True, atoms, 0)
        assert 2 not in asym[keep].tolist()  # chain C touches nothing, so it cannot hold an interface seed
    # atom budget: 10 tokens x 5 atoms fit into 50 atoms, and they are the 10 nearest to the seed
    keep = cropper.spatial_crop(xyz, resolved, asym, 24, g(1), False, atoms, 50, anchor=("chain", 2, -1))
    full = cropper.spatial_crop(xyz, resolved, asym, 24, g(1), False, atoms, 0, anchor=("chain", 2, -1))
    assert len(keep) == 10 and set(keep.tolist()) <= set(full.tolist())
    span = xyz[keep, 0].max() - xyz[keep, 0].min()
    assert float(span) <= 3.8 * 9 + 1e-3  # ten consecutive residues around the seed
    # a large token does not get skipped in favour of smaller ones farther away
    order = torch.tensor([3, 1, 2, 0])
    assert cropper._within_budgets(order, torch.tensor([1, 1, 9, 1]), 4, 4).tolist() == [1, 3]
    # contiguous: exactly the budget when the chains can fill it; atom budget in collection order
    for seed in range(4):
        keep = cropper.contiguous_crop(asym, 64, g(seed), atoms, 0)
        assert len(keep) == 64 and keep.tolist() == sorted(keep.tolist())
        assert len(cropper.contiguous_crop(asym, 64, g(seed), atoms, 100)) == 20

    # through crop(): features with a ground truth whose chain B is entirely unresolved
    f = synthetic_complex([("protein", 40), ("protein", 40), ("protein", 30)], num_msa=4, num_templates=0, seed=2)
    f["atom_gt_mask"] = f["atom_gt_mask"].clone()
    f["atom_gt_mask"][40:80] = False
    for seed in range(5):
        c, used, keep = cropper.crop(f, 32, 0, g(seed), strategy="spatial", return_keep=True)
        assert not ((keep >= 40) & (keep < 80)).any() and c["res_type"].shape[0] == 32
    # contiguous crops may land on the unresolved chain; the retry makes sure enough resolved tokens are in the crop
    for seed in range(8):
        c, used, keep = cropper.crop(f, 16, 0, g(seed), weights={"contiguous": 1.0, "spatial": 0.0, "spatial_interface": 0.0}, return_keep=True)
        assert int(f["atom_gt_mask"][keep].any(-1).sum()) >= cropper.MIN_RESOLVED


def test_anchor_weights_follow_cluster_sizes():
    """Chain anchors weigh beta_chain * alpha / |chain cluster|, interface anchors beta_interface * (alpha_1 + alpha_2) /
    |pair of chain clusters|; the record weight is their sum; invalid chains and interfaces offer no anchor."""
    from deepfold3_dev_b200.data import const
    from deepfold3_dev_b200.data.types import ChainInfo, InterfaceInfo, Record

    def chain(i, mol, cluster, valid=True):
        return ChainInfo(i, "ABCDEFG"[i], mol, cluster, f"m{i}", 50, valid=valid)

    P, R, L = const.MOL_PROTEIN, const.MOL_RNA, const.MOL_NONPOLYMER
    recs = [
        Record("r0", [chain(0, P, "c1"), chain(1, P, "c2"), chain(2, L, "lig")], [InterfaceInfo(0, 1), InterfaceInfo(0, 2), InterfaceInfo(1, 2, valid=False)]),
        Record("r1", [chain(0, P, "c1"), chain(1, P, "c2")], [InterfaceInfo(1, 0)]),  # the same pair of clusters, other order
        Record("r2", [chain(0, R, "rna"), chain(1, P, "c1", valid=False)], [InterfaceInfo(0, 1)]),
        Record("r3", [chain(0, P, "c9", valid=False)], []),
    ]
    tables = samplers.anchor_tables(recs)
    a0 = dict(zip(tables[0][0], tables[0][1]))
    assert a0[("chain", 0, -1)] == pytest.approx(0.5 * 3.0 / 2)  # cluster c1 has two valid members (r2's copy is invalid)
    assert a0[("chain", 2, -1)] == pytest.approx(0.5 * 1.0 / 1)
    assert a0[("interface", 0, 1)] == pytest.approx(1.0 * (3.0 + 3.0) / 2)  # {c1, c2} occurs in r0 and r1
    assert a0[("interface", 0, 2)] == pytest.approx(1.0 * (3.0 + 1.0) / 1) and ("interface", 1, 2) not in a0
    assert tables[2][0] == [("chain", 0, -1)] and tables[2][1] == [pytest.approx(0.5 * 3.0)]  # interface with an invalid chain: no anchor
    assert tables[3] == ([], [])
    w = samplers.record_weights(tables)
    assert w[0] == pytest.approx(sum(tables[0][1])) and w[3] < 1e-9 and w[0] > w[1] > w[2] * 0.99


def test_sampler_resume_sharding_collate_pack(tmp_path):
    w = [1.0, 3.0, 0.5, 2.0]
    full = samplers.WeightedClusterSampler(w, seed=2, rank=0, world_size=1, block=8)
    r0 = samplers.WeightedClusterSampler(w, seed=2, rank=0, world_size=2, block=4)
    r1 = samplers.WeightedClusterSampler(w, seed=2, rank=1, world_size=2, block=4)
    stream = [next(full) for _ in range(8)]
    assert [next(r0) for _ in range(4)] == stream[0::2] and [next(r1) for _ in range(4)] == stream[1::2]
    st = full.state_dict()
    nxt = [next(full) for _ in range(10)]
    full.load_state_dict(st)
    assert [next(full) for _ in range(10)] == nxt
    src = tmp_path / "src"
    src.mkdir()
    for i in range(3):
        torch.save(synthetic_complex([("protein", 40 + 5 * i), ("protein", 30)], num_msa=4, num_templates=0, seed=i), src / f"ex{i}.pt")
    assert pack.build_pack(str(src), str(tmp_path / "pk")) == 3
    pk = pack.Pack(str(tmp_path / "pk"))
    assert pk.exists("ex2.pt") and not pk.exists("nope") and pk.read_bytes("ex1.pt") == (src / "ex1.pt").read_bytes()
    assert sorted(os.listdir(tmp_path / "pk")) == ["SHA256SUMS", "_build", "keys.npy", "loc.npy", "meta.json", "shards"]
    ds = datasets.FeatureDirDataset(str(src), max_tokens=48, pack=pk)
    batch = next(datasets.BatchStream(ds, samplers.WeightedClusterSampler(ds.weights(), seed=1), batch_size=2, pad_tokens_to=64))
    assert batch["res_type"].shape == (2, 64) and batch["msa"].shape == (2, 4, 64) and batch["seq_mask"].sum(-1).tolist() == [48, 48]
    assert (batch["msa"][:, :, 48:] == 21).all() and len(batch["_record_id"]) == 2


def test_pack_is_transparent_to_loaders(tmp_path):
    """A dataset root whose bulky subtrees were moved into ``_pack`` reads like the unpacked tree: nested keys, several
    shards, authoritative misses, pass-through for files left outside, resumable build, the earlier index layout."""
    import json
    import shutil

    import numpy as np

    from deepfold3_dev_b200.data import io_cache
    from deepfold3_dev_b200.data.parse.a3m import msa_from_a3m_file

    root = tmp_path / "root"
    (root / "structures" / "ab").mkdir(parents=True)
    (root / "msa").mkdir()
    rng = np.random.default_rng(0)
    for i in range(5):
        np.savez(root / "structures" / "ab" / f"{i}.npz", x=rng.normal(size=(50 + i, 3)))
    (root / "msa" / "q.a3m").write_text(">q\nACDE\n>h\nAC-E\n")
    (root / "manifest.json").write_text("[]")
    try:
        n = pack.build_pack(str(root), str(root / "_pack"), shard_bytes=3000, include=("structures/", "msa/"))
        assert n == 6 and len(os.listdir(root / "_pack" / "shards")) >= 2
        meta = json.loads((root / "_pack" / "meta.json").read_text())
        assert meta["format"] == "deepfold3-pack" and meta["files"] == 6 and meta["include"] == ["structures/", "msa/"]
        want = {i: io_cache.read_npz(str(root / "structures" / "ab" / f"{i}.npz"))["x"] for i in range(5)}
        shutil.rmtree(root / "structures")
        shutil.rmtree(root / "msa")
        assert pack.register(str(root)) is not None
        for i in range(5):
            assert (io_cache.read_npz(str(root / "structures" / "ab" / f"{i}.npz"))["x"] == want[i]).all()
        assert msa_from_a3m_file(str(root / "msa" / "q.a3m"), 0).sequences.shape == (2, 4)
        assert io_cache.exists(str(root / "structures" / "ab" / "3.npz")) and io_cache.exists(str(root / "msa"))
        assert not io_cache.exists(str(root / "structures" / "ab" / "9.npz"))
        assert pack.lookup(str(root / "structures" / "zz.npz"))[2] == "miss" and pack.lookup(str(root / "manifest.json"))[2] == "pass"
        assert io_cache.exists(str(root / "manifest.json"))
        with pytest.raises(FileNotFoundError):
            io_cache.read_bytes(str(root / "structures" / "ab" / "9.npz"))
        # a rerun after the sources are gone keeps what the state file lists; new files go into further shards
        (root / "msa").mkdir()
        (root / "msa" / "r.a3m").write_text(">r\nAC\n")
        assert pack.build_pack(str(root), str(root / "_pack"), shard_bytes=3000, include=("structures/", "msa/")) == 7
        # the index layout of earlier versions of this package is still read
        old = tmp_path / "old"
        old.mkdir()
        import tarfile

        with tarfile.open(old / "shard-00000.tar", "w") as tar:
            info = tar.gettarinfo(str(root / "manifest.json"), arcname="m.json")
            with open(root / "manifest.json", "rb") as f:
                tar.addfile(info, f)
            (old / "index.json").write_text(json.dumps({"m.json": [0, tar.offset - 512, 2]}))
        assert pack.Pack(str(old)).read_bytes("m.json") == b"[]"
    finally:
        pack.unregister_all()


def test_bucket_pad_unpad_preserves_prediction():
    from deepfold3_dev_b200.models.model import DeepFold3
    from tests.helpers import tiny_config, wake_zero_init

    assert bucket.bucket_size(130) == 160 and bucket.bucket_size(4097) == 4608
    torch.manual_seed(0)
    cfg = tiny_config()
    cfg.diffusion.steps = 2
    cfg.diffusion.num_samples = 1
    model = DeepFold3(cfg).eval()
    wake_zero_init(model)
    f = synthetic_complex([("protein", 20), ("protein", 13)], num_msa=5, num_templates=1, seed=2, with_gt=False)
    padded, n = bucket.pad_features(f, 40)
    assert n == 33 and padded["res_type"].shape[0] == 40 and padded["msa"].shape == (5, 40) and not padded["seq_mask"][33:].any()
    with torch.no_grad():
        a = model(f, seed=1, num_recycles=1)
        b = bucket.unpad_output(model(padded, seed=1, num_recycles=1), n)
    assert b.pae.shape == a.pae.shape and b.distogram.shape == a.distogram.shape
    torch.testing.assert_close(b.distogram, a.distogram, atol=2e-4, rtol=1e-3)
    torch.testing.assert_close(b.atom_positions, a.atom_positions, atol=2e-3, rtol=1e-3)


def test_af3_record_reader(tmp_path):
    from deepfold3_dev_b200.convert import af3

    def record(scope, name, arr, dtype=None):
        dt = (dtype or str(arr.dtype)).encode()
        raw = arr.tobytes()
        return struct.pack(f"<5i{len(scope)}s{len(name)}s{len(dt)}s{arr.ndim}i", len(scope), len(name), len(dt), arr.ndim,
                           len(raw), scope.encode(), name.encode(), dt, *arr.shape) + raw  # fmt: skip

    w = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    bf = (np.asarray([1.5, -2.0], dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
    path = tmp_path / "p.bin"
    path.write_bytes(record("trunk/stack/linear", "weights", w) + record("head/norm", "scale", bf, "bfloat16"))
    params = af3.read_af3_params(str(path))
    assert params["head/norm"]["scale"].tolist() == [1.5, -2.0]
    assert params["trunk/stack/linear"]["weights"].shape == (2, 3, 4) and params["trunk/stack/linear"]["weights"][1, 0, 0] == 12


def test_inference_runner_writes_the_output_tree(tmp_path):
    from deepfold3_dev_b200.inference.runner import run_job, sample_chunk_seed, sample_chunks
    from deepfold3_dev_b200.models.model import DeepFold3
    from tests.helpers import tiny_config, wake_zero_init

    assert sample_chunks(5, 2) == [2, 2, 1] and sample_chunks(5, 0) == [5] and sample_chunk_seed(7, 0) == 7
    cfg = tiny_config()
    cfg.diffusion.steps = 2
    model = DeepFold3(cfg).eval()
    wake_zero_init(model)
    inp = InferenceInput.from_sequence("MKTAYIAKQRQISFVK")
    out = str(tmp_path / "o")
    s = run_job(model, inp, out, "cpu", seeds=[1, 2], num_recycles=0, num_samples=2, dtype=torch.float32, use_bucket=False, sample_chunk=1)
    assert len(s) == 4 and os.path.exists(os.path.join(out, "ranking_scores.csv"))
    for seed in (1, 2):
        assert os.path.exists(os.path.join(out, f"seed-{seed}_distogram.npz"))
        for i in (0, 1):
            assert sorted(os.listdir(os.path.join(out, f"seed-{seed}_sample-{i}"))) == ["confidences.json", "logits.npz", "model.cif"]
    man = json.load(open(os.path.join(out, "run_manifest.json")))
    assert man["status"] == "done" and "kernel_census" in man
    again = run_job(model, inp, out, "cpu", seeds=[1, 2], num_recycles=0, num_samples=2, dtype=torch.float32, use_bucket=False, skip_existing=True)
    assert again == []


def test_schedule_free_matches_reference(reference_package):
    from deepfold3.training.schedule_free import AdamWScheduleFree

    from deepfold3_dev_b200.training.schedule_free import FlatAdamWScheduleFree

    torch.manual_seed(0)
    a = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 1))
    b = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 1))
    b.load_state_dict(a.state_dict())
    kw = dict(lr=3e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, warmup_steps=3)
    ref = AdamWScheduleFree(a.parameters(), **kw)
    ref.train()
    mine = FlatAdamWScheduleFree(b, **kw)
    x, y = torch.randn(32, 6), torch.randn(32, 1)
    for _ in range(6):
        for model, opt in ((a, ref), (b, mine)):
            opt.zero_grad()
            ((model(x) - y) ** 2).mean().backward()
            opt.step()
    for pa, pb in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(pb, pa, atol=1e-6, rtol=1e-5)
    ref.eval()
    mine.eval()
    for pa, pb in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(pb, pa, atol=1e-6, rtol=1e-5)


def test_extra_losses_match_reference_and_differentiate(reference_package):
    from deepfold3.training import loss as R

    from deepfold3_dev_b200.training import extra_losses as X

    torch.manual_seed(0)
    f = synthetic_complex([("protein", 12), ("protein", 9)], num_msa=2, num_templates=0, seed=4)
    N = 21
    pred = (f["atom_gt_positions"][None] + 0.5 * torch.randn(3, N, 24, 3)).requires_grad_(True)
    cb = torch.full((N,), 4)
    target = torch.where(f["ref_mask"][:, 4], torch.tensor(1.2), torch.tensor(0.0))
    args = (pred, f["frame_token_index"], f["frame_atom_index"], cb, target)
    torch.testing.assert_close(X.chirality_loss(*args), R.chirality_loss(*args))
    mine, ref = X.chirality_violation_rates(*args), R.chirality_violation_rates(*args)
    for k in ref:
        torch.testing.assert_close(mine[k], ref[k])
    bb = (pred, f["atom_gt_positions"], f["atom_gt_mask"], f["seq_mask"], f["asym_id"], f["mol_type"])
    torch.testing.assert_close(X.backbone_chirality_loss(*bb), R.backbone_chirality_loss(*bb))
    # FAPE: zero at the ground truth, positive and differentiable away from it, chunking does not change it
    tok = torch.arange(N)[:, None].expand(N, 3).contiguous()
    slots = torch.tensor([0, 1, 2]).expand(N, 3).contiguous()
    ok = torch.ones(N, 3, dtype=torch.bool)
    pm = torch.ones(N, N, dtype=torch.bool)
    common = (tok, slots, ok, f["frame_atom_index"], f["frame_token_index"], pm)
    zero, _ = X.fape_loss(f["atom_gt_positions"][None], f["atom_gt_positions"], *common)
    assert float(zero) < 2e-3
    a, _ = X.fape_loss(pred, f["atom_gt_positions"], *common)
    b, _ = X.fape_loss(pred, f["atom_gt_positions"], *common, chunk_size=5)
    torch.testing.assert_close(a, b)
    intra, inter = X.fape_loss(pred, f["atom_gt_positions"], *common, asym_id=f["asym_id"], mode="both")
    assert float(a) > 0 and float(inter) > 0
    sc, parts = X.shape_complementarity_loss(pred, f["atom_gt_positions"], f["atom_gt_mask"], f["token_to_rep_atom"], f["asym_id"],
                                             f["mol_type"], f["seq_mask"])  # fmt: skip
    (a + intra + sc).backward()
    assert torch.isfinite(pred.grad).all() and float(pred.grad.abs().sum()) > 0 and set(parts) >= {"shape_comp_token"}


HHR = """Query         q
Match_columns 10

 No Hit                             Prob E-value P-value  Score    SS Cols Query HMM  Template HMM
  1 1ABC_A some protein             99.9 1.2E-30 1E-34  200.0   0.0   8    2-9      5-12 (100)

No 1
>1ABC_A some protein
Probab=99.90  E-value=1.2e-30  Score=200.00  Aligned_cols=8  Identities=50%  Similarity=0.9  Sum_probs=7.5  Template_Neff=5.0

Q q                 2 ACDE-FGH    8 (10)
Q Consensus         2 acde-fgh    8 (10)
T Consensus         5 ac~eKfgh   12 (100)
T 1ABC_A            5 AC-EKFGH   11 (100)

"""


def test_hhr_hits_and_template_features():
    from deepfold3_dev_b200.data.parse.hhr import parse_hhr
    from deepfold3_dev_b200.data.templates import TemplateChain, template_features

    (hit,) = parse_hhr(HHR)
    assert (hit.pdb_id, hit.chain_id, hit.aligned_cols, hit.sum_probs) == ("1ABC", "A", 8, 7.5)
    assert hit.query_to_hit_mapping == {1: 4, 2: 5, 4: 6, 5: 8, 6: 9, 7: 10}
    rng = np.random.RandomState(0)
    tpl = TemplateChain(["GLY"] * 12, rng.randn(12, 24, 3).astype(np.float32), np.ones((12, 24), bool), hit.query_to_hit_mapping)
    f = template_features(10, [tpl], max_templates=4, token_offset=3, num_tokens=20)
    assert f["template_mask"].tolist() == [1, 0, 0, 0] and f["template_aatype"].shape == (4, 20)
    assert f["template_backbone_mask"][0].nonzero().flatten().tolist() == [4, 5, 7, 8, 9, 10]
    R = f["template_backbone_frame"][0, 4]
    torch.testing.assert_close(R @ R.T, torch.eye(3), atol=1e-5, rtol=0)
    torch.testing.assert_close(f["template_pseudo_beta"][0, 4], f["template_ca"][0, 4])  # glycine: CA stands in for CB


def test_msa_search_cache_and_fake_binary(tmp_path, monkeypatch):
    from deepfold3_dev_b200.data.msa import search

    cache = search.MsaCache(str(tmp_path / "cache"))
    fake = tmp_path / "mmseqs"
    fake.write_text("#!/bin/sh\nif [ \"$1\" = result2msa ]; then printf '>query\\nACDE\\n>hit\\nAC-E\\n' > \"$5\"; fi\nexit 0\n")
    fake.chmod(0o755)
    a3m = search.search_local("ACDE", "/db/uniref", cache, binary=str(fake))
    assert parse_a3m(a3m).sequences == ["ACDE", "AC-E"]
    fake.unlink()  # the second call must come from the cache
    assert search.search_local("ACDE", "/db/uniref", cache, binary=str(fake)) == a3m
    with pytest.raises(RuntimeError, match="not on PATH"):
        search.search_local("WWWW", "/db/uniref", cache, binary=str(fake))


def test_staged_mmseqs_pipeline_with_a_stand_in_binary(tmp_path):
    """The staged local pipeline against a stand-in for the ``mmseqs`` binary that records its calls and fabricates the
    files the next stage reads: stage order, index / load-mode detection, GPU flags, one pass for a batch with
    duplicates, template hits split by query, the cache, paired alignments with a row-count check, the CLI."""
    import json
    import stat

    from click.testing import CliRunner

    from deepfold3_dev_b200.cli.main import cli
    from deepfold3_dev_b200.data.msa import mmseqs_pipeline as mp
    from deepfold3_dev_b200.data.msa.search import MsaCache

    db = tmp_path / "db"
    db.mkdir()
    (db / "uniref30_2302_db.idx").write_text("")  # UniRef has a precomputed index, the environmental database has none
    log = tmp_path / "calls.log"
    fake = tmp_path / "mmseqs"
    fake.write_text(f"""#!/usr/bin/env python3
import os, sys
a = sys.argv[1:]
open({str(log)!r}, "a").write(" ".join(a) + "\\n")
cmd = a[0]
def queries(work):
    return [l[1:].strip() for l in open(os.path.join(work, "query.fasta")) if l.startswith(">")]
if cmd == "unpackdb":
    src, out = a[1], a[2]
    work = os.path.dirname(src)
    os.makedirs(out, exist_ok=True)
    seqs = [l.strip() for l in open(os.path.join(work, "query.fasta")) if not l.startswith(">")]
    for i, (q, s) in enumerate(zip(queries(work), seqs)):
        rows = 3 if "pair" in os.path.basename(src) else 2 + i
        open(os.path.join(out, f"{{i}}.a3m"), "w").write("".join(f">{{q if r == 0 else 'hit%d' % r}}\\n{{s}}\\n" for r in range(rows)) + "\\0")
elif cmd == "convertalis":
    work = os.path.dirname(a[4])
    with open(a[4], "w") as f:
        for q in queries(work):
            f.write("\\t".join([q, "1abc_A", "0.9", "50", "2", "0", "1", "50", "3", "52", "1e-30", "200", "50M"]) + "\\n")
""")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)

    s = mp.MmseqsSettings(str(db), use_env=True, use_templates=True, gpu=True, threads=4, binary=str(fake))
    assert mp.detect_db_mode(str(db), s.uniref_db) == (".idx", "2") and mp.detect_db_mode(str(db), s.env_db) == ("", "0")
    plan = mp.plan_monomer(s, "/w", "/w/query.fasta")
    assert [c[0] for c in plan] == ["createdb", "search", "mvdb", "lndb", "expandaln", "align", "filterresult", "result2msa", "search",
                                    "convertalis", "search", "expandaln", "align", "filterresult", "result2msa", "mergedbs", "unpackdb"]  # fmt: skip
    assert "--gpu" in plan[1] and "-s" not in plan[1] and plan[1][plan[1].index("--db-load-mode") + 1] == "2"
    assert plan[4][2].endswith("uniref30_2302_db.idx") and plan[11][2].endswith("colabfold_envdb_202108_db")
    assert plan[12][1] == "/w/tmp_env/latest/profile_1" and plan[10][1] == "/w/prof_res"
    cpu = mp.plan_monomer(mp.MmseqsSettings(str(db), use_env=False), "/w", "/w/query.fasta")
    assert "-s" in cpu[1] and cpu[-2][0] == "mvdb" and len(cpu) == 10

    cache = MsaCache(str(tmp_path / "cache"))
    res = mp.search_monomer_batch(["ACDEF", "GHIKL", "ACDEF"], s, cache)
    assert [parse_a3m(r["a3m"]).sequences[0] for r in res] == ["ACDEF", "GHIKL", "ACDEF"] and res[0] is res[2]
    assert res[1]["a3m"].count(">") == 3 and "\x00" not in res[1]["a3m"]
    hits = mp.parse_m8(res[0]["m8"] + "broken line\n")
    assert list(hits) == ["0"] and hits["0"][0].target == "1abc_A" and hits["0"][0].cigar == "50M" and hits["0"][0].t_start == 3
    calls = log.read_text().splitlines()
    assert sum(c.startswith("createdb") for c in calls) == 1  # one pass for the whole batch
    log.write_text("")
    again = mp.search_monomer_batch(["GHIKL", "MNPQR"], s, cache)  # the first comes from the cache, only the second is searched
    assert again[0]["a3m"] == res[1]["a3m"] and parse_a3m(again[1]["a3m"]).sequences[0] == "MNPQR"
    assert sum(c.startswith("createdb") for c in log.read_text().splitlines()) == 1

    paired = mp.search_pair_batch([["ACDEF", "GHIKL", "ACDEF"], ["WWWWW"]], s, cache)
    assert len(paired[0]) == 2 and all(b.count(">") == 3 for b in paired[0]) and paired[1] == [">101\nWWWWW\n"]
    pair_plan = mp.plan_pair(s, "/w", "/w/query.fasta")
    assert [c[0] for c in pair_plan].count("pairaln") == 2 and pair_plan[-2][-1] == "5"

    jobs = tmp_path / "jobs.txt"
    job = tmp_path / "cx.json"
    job.write_text(json.dumps({"name": "cx", "sequences": [{"protein": {"id": ["A"], "sequence": "ACDEF"}}, {"protein": {"id": ["B"], "sequence": "GHIKL"}}]}))
    jobs.write_text(f"{job}\n")
    r = CliRunner().invoke(cli, ["msa-batch", "--inputs-file", str(jobs), "--output-dir", str(tmp_path / "out"), "--db-dir", str(db),
                                 "--use-templates", "--paired", "--mmseqs", str(fake), "--cache-dir", str(tmp_path / "c2")])  # fmt: skip
    assert r.exit_code == 0 and "2 sequences searched, 1 complexes paired" in r.output, r.output
    import hashlib

    key = hashlib.sha1(b"GHIKL").hexdigest()
    assert (tmp_path / "out" / f"{key}.a3m").exists() and (tmp_path / "out" / f"{key}.m8").exists()
    assert (tmp_path / "out" / "paired" / "cx" / f"{key}.a3m").read_text().count(">") == 3
    with pytest.raises(RuntimeError, match="not on PATH"):
        mp.run_plan([["version"]], binary=str(tmp_path / "absent"))


def test_tiled_linear_is_transparent():
    from deepfold3_dev_b200.models.tiled_linear import TiledLinear

    lin = torch.nn.Linear(8, 4)
    tiled = TiledLinear(lin, 3).train()
    x = torch.randn(10, 5, 8)
    torch.testing.assert_close(tiled(x), lin(x))
    assert list(tiled.state_dict()) == ["weight", "bias"]
    other = TiledLinear(torch.nn.Linear(8, 4), 0)
    other.load_state_dict(tiled.state_dict())
    torch.testing.assert_close(other.inner.weight, lin.weight)


def test_reference_pickled_config_loads_without_the_reference(reference_package, tmp_path):
    """A blob that pickles the reference's config classes loads in a process that cannot import the reference."""
    import subprocess
    import sys

    import deepfold3.model.config as RC

    path = tmp_path / "ckpt.pt"
    cfg = RC.ModelConfig()
    cfg.num_recycles = 7
    torch.save({"model": {"w": torch.ones(2)}, "model_cfg": cfg, "ema": None}, path)
    code = ("import sys; from deepfold3_dev_b200.inference.weights import load_state; "
            f"s, c = load_state({str(path)!r}); print(type(c).__module__, c.num_recycles, s['w'].tolist())")  # fmt: skip
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root, env={**os.environ, "PYTHONPATH": root})
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.split() == ["deepfold3_dev_b200.config.schema", "7", "[1.0,", "1.0]"]


def test_species_pairing_atomisation_masks_and_io_cache(tmp_path):
    from deepfold3_dev_b200.data import io_cache
    from deepfold3_dev_b200.data.atomize import atomize_tokens, maybe_atomize
    from deepfold3_dev_b200.data.masking import TokenMask
    from deepfold3_dev_b200.data.msa.pairing import pair_by_species, species_id, unpaired_rows_not_in_paired

    a = parse_a3m(">q\nACDE\n>tr|A1|X_HUMAN OX=9606\nACDD\n>tr|A2|X_MOUSE OX=10090\nACEE\n>tr|A3|Y_HUMAN OX=9606\nAADE\n", dedup=False)
    b = parse_a3m(">q\nKLM\n>tr|B1|Z_MOUSE OX=10090\nKLL\n>tr|B2|Z_HUMAN OX=9606\nKMM\n>tr|B3|Z_RAT OX=10116\nKKK\n", dedup=False)
    (pa, pb), res = pair_by_species([a, b])
    assert res.rows.tolist() == [[0, 0], [1, 2], [2, 1]] and res.species == ["query", "9606", "10090"]
    assert pa.sequences == ["ACDE", "ACDD", "ACEE"] and pb.sequences == ["KLM", "KMM", "KLL"]
    assert species_id("sp|P1|ABC_YEAST desc") == "YEAST" and species_id(">x") == ""
    assert unpaired_rows_not_in_paired(a, pa).tolist() == [0, 3]
    job = {"name": "c", "sequences": [
        {"protein": {"id": "A", "sequence": "ACDE", "unpairedMsa": ">q\nACDE\n>tr|A1|X_HUMAN OX=9606\nACDD\n>tr|A2|X_MOUSE OX=10090\nACEE\n"}},
        {"protein": {"id": "B", "sequence": "KLM", "unpairedMsa": ">q\nKLM\n>tr|B1|Z_MOUSE OX=10090\nKLL\n>tr|B2|Z_HUMAN OX=9606\nKMM\n"}}]}  # fmt: skip
    inp = InferenceInput.from_job(parse_json_input(job)[0])
    msa = inp.features["msa"]
    # rows 1-2 are paired across both chains (no gap block), later rows are the per-chain blocks
    assert not (msa[1] == 21).any() and not (msa[2] == 21).any() and (msa[3, 4:] == 21).all()
    f = synthetic_complex([("protein", 10)], num_msa=3, num_templates=1, seed=1)
    g = atomize_tokens(f, torch.tensor([2, 5]))
    k = int(f["ref_mask"][2].sum() + f["ref_mask"][5].sum())
    assert g["res_type"].shape[0] == 8 + k and g["msa"].shape == (3, 8 + k) and int(g["ref_mask"].sum()) == int(f["ref_mask"].sum())
    assert int(g["is_atomized"].sum()) == k and not g["frames_mask"][g["is_atomized"]].any()
    torch.testing.assert_close(g["atom_gt_positions"][g["is_atomized"], 0][0], f["atom_gt_positions"][2, 0])
    assert maybe_atomize(f, torch.Generator().manual_seed(0), p_example=0.0) is f
    from deepfold3_dev_b200.data.atomize import atomize_stored_features

    every = atomize_stored_features(f, torch.Generator().manual_seed(0), 1.0)
    assert int(every["is_atomized"].sum()) == int(f["ref_mask"][(f["mol_type"] != 3) & (f["ref_mask"].sum(-1) > 1)].sum())
    two = atomize_stored_features(f, torch.Generator().manual_seed(0), 1.0, max_residues=2)
    assert len(torch.unique(two["residue_index"][two["is_atomized"]] * 100 + two["asym_id"][two["is_atomized"]])) == 2
    assert atomize_stored_features(f, torch.Generator().manual_seed(0), 0.0) is f
    tm = TokenMask.fixed_from_chains(np.asarray([0, 0, 1, 1, 2]), [1])
    assert tm.loss_weight(5).tolist() == [1, 1, 0, 0, 1] and tm.select(np.asarray([2, 4])).get("fixed").tolist() == [True, False]
    io_cache.set_drop_page_cache(True)
    np.savez(tmp_path / "x.npz", a=np.arange(4))
    assert io_cache.read_npz(str(tmp_path / "x.npz"))["a"].tolist() == [0, 1, 2, 3]
    io_cache.set_drop_page_cache(False)


def test_crop_before_alignment_load_equals_crop_after(tmp_path):
    """Cropping first and reading only the surviving chains' alignments gives the features of the old order
    (featurise with every alignment, then crop), and chains cropped away are never read."""
    from deepfold3_dev_b200.data import cropper
    from deepfold3_dev_b200.data.featurize import attach_cropped_msa, msa_block
    from deepfold3_dev_b200.data.synthetic import synthetic_complex
    from deepfold3_dev_b200.data.types import MSA

    feats = synthetic_complex([("protein", 30), ("protein", 24), ("protein", 20)], num_msa=1, num_templates=0, seed=3)
    feats = {k: v for k, v in feats.items() if k not in ("msa", "msa_mask", "deletion_matrix", "profile", "deletion_mean", "has_deletion", "deletion_value")}
    cols = {0: (0, 30), 1: (30, 54), 2: (54, 74)}
    rng = np.random.default_rng(0)
    msas = {}
    for a, (s, e) in cols.items():
        seq = rng.integers(0, 20, size=(5, e - s)).astype(np.int8)
        seq[0] = feats["res_type"][s:e].numpy()
        msas[a] = MSA(seq, np.ones_like(seq, dtype=bool), rng.integers(0, 3, size=seq.shape).astype(np.int8))
    full = dict(feats)
    full.update(msa_block(full, cols, None, msas, 64))
    gen = torch.Generator().manual_seed(5)
    want, _, keep = cropper.crop(full, 40, 0, gen, strategy="contiguous", return_keep=True)
    gen = torch.Generator().manual_seed(5)
    bare, _, keep2 = cropper.crop(dict(feats), 40, 0, gen, strategy="contiguous", return_keep=True)
    assert torch.equal(keep, keep2)
    opened = []

    def load(a):
        opened.append(a)
        return msas[a]

    got, read, skipped = attach_cropped_msa(bare, keep2, cols, load, max_msa_rows=64)
    alive = {a for a, (s, e) in cols.items() if bool(((keep >= s) & (keep < e)).any())}
    assert set(opened) == alive and read == len(alive) and skipped == 3 - len(alive)
    # rows of chains that were cropped away are all-gap rows in the crop-after features and absent here
    keep_rows = (want["msa"] != 21).any(dim=1)
    for key in ("msa", "deletion_matrix"):
        assert torch.equal(got[key], want[key][keep_rows]), key


def test_batch_stream_counts_drops_by_exception_type():
    from deepfold3_dev_b200.data.datasets import BatchStream

    class Flaky:
        def __getitem__(self, i):
            if i % 3 == 0:
                raise KeyError("missing alignment")
            if i % 5 == 0:
                raise ValueError("no tokens")
            return {"res_type": torch.zeros(4, dtype=torch.long), "x": torch.ones(4)}

    stream = BatchStream(Flaky(), iter(range(100)), batch_size=2)
    for _ in range(5):
        next(stream)
    c = stream.counters()
    assert c["data/served"] == 10 and c["data/dropped"] == c["data/dropped/KeyError"] + c["data/dropped/ValueError"] > 0
    assert c["data/retries"] == c["data/dropped"]


def test_openfold3_atom_array_import_and_columnar_cache(tmp_path):
    from deepfold3_dev_b200.data import of3
    from deepfold3_dev_b200.data.types import Structure, load_manifest

    names = ["N", "CA", "C", "O"]
    rows = []
    for chain, (res, n_res) in {"A": ("ALA", 3), "B": ("GLY", 2)}.items():
        for r in range(n_res):
            for a in names:
                rows.append((chain, r + 1, res, a, a[0]))
    rows += [("C", 1, "HEM", "FE", "FE"), ("C", 1, "HEM", "N1", "N")]
    n = len(rows)
    coord = np.cumsum(np.full((n, 3), 1.3, dtype=np.float32), axis=0)
    src = tmp_path / "of3" / "1abc"
    src.mkdir(parents=True)
    np.savez(src / "1abc.npz", coord=coord, chain_id=np.array([r[0] for r in rows]), res_id=np.array([r[1] for r in rows]),
             res_name=np.array([r[2] for r in rows]), atom_name=np.array([r[3] for r in rows]), element=np.array([r[4] for r in rows]),
             molecule_type_id=np.array([0] * 20 + [3] * 2), bonds=np.array([[20, 21, 1], [0, 1, 1]]))  # fmt: skip
    cache = {"structure_data": {"1abc": {"release_date": "2020-01-05", "resolution": 2.1, "experimental_method": "X-RAY DIFFRACTION",
                                         "chains": {"A": {"cluster_id": "c7", "molecule_type": "PROTEIN", "template_ids": ["2xyz_A"]},
                                                    "B": {"cluster_id": "c9", "molecule_type": "PROTEIN"},
                                                    "C": {"cluster_id": "lig", "molecule_type": "LIGAND"}}}}}  # fmt: skip
    (tmp_path / "cache.json").write_text(json.dumps(cache))
    out = tmp_path / "train"
    assert of3.convert_directory(str(tmp_path / "of3"), str(out), str(tmp_path / "cache.json")) == (1, 0)
    rec = load_manifest(str(out / "manifest.json"))[0]
    assert [c.mol_type for c in rec.chains] == [0, 0, 3] and [c.num_residues for c in rec.chains] == [3, 2, 1]
    assert rec.chains[0].cluster_id == "c7" and rec.structure_info.resolution == 2.1 and rec.structure_info.released == "2020-01-05"
    st = Structure.load(str(out / "structures" / "1abc.npz"))
    assert len(st.atoms) == n and len(st.residues) == 6 and st.chain_canonical_seqs[0] == "AAA" and len(st.bonds) == 1
    entries, chains = of3.build_columnar_cache(str(tmp_path / "cache.json"), str(tmp_path / "col"))
    assert (entries, chains) == (1, 3)
    col = of3.ColumnarCache(str(tmp_path / "col"))
    e = col.entry(col.index_of("1ABC"))
    assert e["resolution"] == pytest.approx(2.1) and e["chains"][0]["template_ids"] == ["2xyz_A"] and col.index_of("9zzz") == -1
    assert list(col.select(max_release_date="2019-12-31")) == [] and list(col.select(max_release_date="2021-01-01", max_resolution=3.0)) == [0]
    assert col.cluster_weights(np.array([0]))[0] == pytest.approx(3.0)


def test_ligand_automorphisms_by_graph_search():
    from deepfold3_dev_b200.data.symmetry import graph_automorphisms

    ring = [(i, (i + 1) % 6) for i in range(6)]
    perms = graph_automorphisms([6] * 6, ring)
    assert len(perms) == 12 and perms[0] == list(range(6)) and all(sorted(p) == list(range(6)) for p in perms)
    assert len(graph_automorphisms([6, 8, 8], [(0, 1), (0, 2)])) == 2                       # the two oxygens swap
    assert len(graph_automorphisms([6, 8, 8], [(0, 1), (0, 2)], orders=[2, 1])) == 1        # not when the bond orders differ
    assert len(graph_automorphisms([15, 8, 8, 8, 8], [(0, 1), (0, 2), (0, 3), (0, 4)])) == 24
    assert len(graph_automorphisms([6] * 6, ring, limit=5)) == 5


def test_logit_files_follow_the_reference_layout(tmp_path):
    """Every scheme round-trips, the file is laid out as the reference documents it (payload per head under its own
    name, ``_meta`` JSON with per-head scheme / shape / scale / clip / bin_axis), a file assembled by hand from that
    description loads, and so does a file in this package's earlier layout."""
    rng = np.random.RandomState(1)
    pae = (rng.randn(3, 6, 6, 9) * 5).astype(np.float32)   # odd bin count: the 4-bit scheme pads a nibble
    plddt = (rng.randn(3, 6, 50) * 3).astype(np.float32)
    tol = {"float32": 1e-7, "float16": 1e-2, "int8": 6e-2, "int8_softmax": 3e-2, "int4_softmax": 0.3}
    for scheme in logit_codec.SCHEMES:
        path = str(tmp_path / f"{scheme}.npz")
        logit_codec.save_logits(path, pae=pae, plddt=plddt, pde=None, scheme=scheme, extra={"token_chain": np.arange(6)},
                                attrs={"seed": 7})  # fmt: skip
        with np.load(path) as z:
            assert set(z.files) == {"pae", "plddt", "token_chain", "_meta"}
            meta = json.loads(bytes(z["_meta"]).decode())
        assert meta["version"] == 1 and meta["attrs"] == {"seed": 7} and set(meta["heads"]) == {"pae", "plddt"}
        assert meta["heads"]["pae"]["shape"] == [3, 6, 6, 9] and meta["heads"]["pae"]["scheme"] == scheme
        back = logit_codec.load_logits(path)
        assert back["token_chain"].tolist() == list(range(6)) and logit_codec.load_attrs(path) == {"seed": 7}
        for name, ref in (("pae", pae), ("plddt", plddt)):
            assert back[name].shape == ref.shape
            assert np.abs(logit_codec.softmax(back[name]) - logit_codec.softmax(ref)).max() < tol[scheme], (scheme, name)
    # a file put together by hand as the format is documented: uint8 levels, level 255 = row maximum, step = clip / 255
    clip, levels = 16.0, 255
    shifted = np.clip(plddt - plddt.max(-1, keepdims=True), -clip, 0)
    payload = np.rint((shifted + clip) / (clip / levels)).astype(np.uint8)
    meta = {"heads": {"plddt": {"scheme": "int8_softmax", "dtype": "float32", "shape": list(plddt.shape), "scale": clip / levels,
                                "clip": clip, "bin_axis": 2}}, "attrs": {"sample": 1}, "version": 1}  # fmt: skip
    hand = str(tmp_path / "hand.npz")
    np.savez_compressed(hand, plddt=payload, _meta=np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8))
    got = logit_codec.load_logits(hand)
    assert got.attrs == {"sample": 1} and np.abs(got["plddt"] - shifted).max() <= clip / levels / 2 + 1e-6
    # the earlier layout of this package
    old = str(tmp_path / "old.npz")
    np.savez_compressed(old, __attrs__=np.frombuffer(json.dumps({"scheme": "f16", "clip": 30.0, "heads": ["pae"]}).encode(), dtype=np.uint8),
                        **{"pae.payload": pae.astype(np.float16)})  # fmt: skip
    assert np.abs(logit_codec.load_logits(old)["pae"] - pae).max() < 2e-2 and logit_codec.head_names(old) == ["pae"]
    with pytest.raises(ValueError):
        logit_codec.save_logits(str(tmp_path / "x.npz"), pae=pae, scheme="int3")


def test_smiles_ligands_without_a_toolkit():
    """SMILES -> heavy-atom graph (charges, bond orders, rings, branches, dots) -> embedded conformer -> a prediction job
    whose ligand has one token per atom and the bonds of the string."""
    from deepfold3_dev_b200.data import smiles as smi
    from deepfold3_dev_b200.data.parse.json_input import parse_json_input

    el, ch, bonds, arom = smi.parse_smiles("CC(=O)Oc1ccccc1C(=O)[O-]")       # aspirin, deprotonated
    assert el.count(6) == 9 and el.count(8) == 4 and sum(ch) == -1 and len(bonds) == 13
    assert sum(1 for *_, o in bonds if o == 4) == 6 and sum(1 for *_, o in bonds if o == 2) == 2 and sum(arom) == 6
    el, ch, bonds, _ = smi.parse_smiles("[NH3+][C@@H](C)C(=O)[O-].[Na+]")     # explicit H counts, stereo mark, a counter-ion
    assert el == [7, 6, 6, 6, 8, 8, 11] and ch == [1, 0, 0, 0, 0, -1, 1] and len(bonds) == 5
    assert len(smi.parse_smiles("C%12CCCCC%12")[2]) == 6 and len(smi.parse_smiles("N#Cc1ccccc1")[0]) == 8
    for bad in ("C1CC", "C(C", "CQ", "C)"):
        with pytest.raises(ValueError):
            smi.parse_smiles(bad)
    code, entry = smi.component_from_smiles("c1ccc2[nH]ccc2c1")               # indole: two fused rings
    assert code == smi.component_from_smiles("c1ccc2[nH]ccc2c1")[0] and entry["atoms"][:2] == ["C1", "C2"]
    x = np.asarray(entry["coords"])
    for a, b, _ in entry["bonds"]:
        assert 1.2 < np.linalg.norm(x[a] - x[b]) < 1.7
    d = np.linalg.norm(x[:, None] - x[None], axis=-1) + 9 * np.eye(len(x))
    assert d.min() > 1.1                                                       # no two atoms on top of each other
    assert np.linalg.svd(x - x.mean(0), compute_uv=False)[2] < 0.5             # the fused ring system is flat
    job = {"name": "lig", "modelSeeds": [1], "sequences": [{"protein": {"id": "A", "sequence": "MKTAYIAKQR"}},
                                                             {"ligand": {"id": "L", "smiles": "CC(=O)Oc1ccccc1C(=O)O"}}]}
    inp = InferenceInput.from_job(parse_json_input(job)[0], msa_crop_size=4)
    f = inp.features
    lig = f["mol_type"] == 3
    assert int(lig.sum()) == 13 and int(f["ref_mask"][lig].sum()) == 13
    assert int(f["bond_matrix"][lig][:, lig].sum()) == 2 * 13                   # 13 bonds, symmetric


def test_permutation_tables_are_built_from_cropped_features():
    """Exchangeable residue atoms and ligand automorphisms, indexed in the example they were computed from, and usable
    by the ground-truth symmetry resolution: a prediction that equals the permuted ground truth costs nothing."""
    from deepfold3_dev_b200.data.symmetry import apply_ligand_token_permutation, apply_token_atom_permutation, symmetry_features

    f = synthetic_complex([("protein", 24), ("ligand", 6)], num_msa=2, num_templates=0, seed=4)
    lig = torch.nonzero(f["mol_type"] == 3).flatten()
    assert len(lig) == 6
    # make the ligand a six-ring of carbons: 12 automorphisms
    f["ref_element"][lig, 0] = 6
    f["bond_matrix"] = torch.zeros(30, 30, 1)
    for k in range(6):
        a, b = int(lig[k]), int(lig[(k + 1) % 6])
        f["bond_matrix"][a, b, 0] = f["bond_matrix"][b, a, 0] = 1.0
    tables = symmetry_features(f)
    perms = tables["ligand_perms"]
    assert perms.shape[1] == 4 and int(perms[:, 1].max()) + 1 == 11 and set(perms[:, 2].tolist()) <= set(lig.tolist())
    swaps = tables["atom_swap_pairs"]
    names = lambda t, a: "".join(chr(int(c) + 32) for c in f["ref_atom_name_chars"][t, a]).strip()  # noqa: E731
    swappable = {"ASP": {"OD1", "OD2"}, "GLU": {"OE1", "OE2"}, "PHE": {"CD1", "CD2", "CE1", "CE2"}, "TYR": {"CD1", "CD2", "CE1", "CE2"},
                 "ARG": {"NH1", "NH2"}, "LEU": {"CD1", "CD2"}, "VAL": {"CG1", "CG2"}}  # fmt: skip
    for t, a, b in swaps.tolist():
        assert f["mol_type"][t] == 0 and {names(t, a), names(t, b)} <= set().union(*swappable.values())
    # ground truth = prediction with the ring rotated by one position: the table finds the rotation and undoes it
    gt = f["atom_gt_positions"].clone()
    pred = gt.clone()
    pred[lig, 0] = gt[lig.roll(1), 0]
    fixed = apply_ligand_token_permutation(pred, gt, f["atom_gt_mask"], perms)
    assert torch.allclose(fixed[lig, 0], pred[lig, 0])
    if len(swaps):
        t, a, b = swaps[0].tolist()
        pred2 = gt.clone()
        pred2[t, a], pred2[t, b] = gt[t, b], gt[t, a]
        fixed2 = apply_token_atom_permutation(pred2, gt, f["atom_gt_mask"], swaps)
        assert torch.allclose(fixed2[t, a], pred2[t, a]) and torch.allclose(fixed2[t, b], pred2[t, b])
