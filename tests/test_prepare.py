"""mmCIF reader, structure containers, filters, clustering, surface targets and the structure featuriser (CPU)."""

import math
import os

import numpy as np
import pytest
import torch

from deepfold3_dev_b200.data import const, sasa
from deepfold3_dev_b200.data.featurize import featurize_structure
from deepfold3_dev_b200.data.parse.cif import parse_cif
from deepfold3_dev_b200.data.parse.mmcif import parse_mmcif, parse_oper_expression
from deepfold3_dev_b200.data.prepare import StructureFilterConfig, cluster_records, filter_structure, prepare_directory
from deepfold3_dev_b200.data.prepare.clustering import greedy_kmer_clusters
from deepfold3_dev_b200.data.prepare.filters import filter_structure_metadata, select_interface_chains
from deepfold3_dev_b200.data.templates import cigar_to_index_pairs, parse_m8
from deepfold3_dev_b200.data.types import ATOM_DTYPE, MSA, Record, Structure, StructureInfo, load_manifest

# example jobs of the reference distribution (JSON + alignments + template mmCIF files); tests that need them are skipped
# when DF3_REFERENCE_EXAMPLES does not point at a copy
EXAMPLES = os.environ.get("DF3_REFERENCE_EXAMPLES", os.path.join(os.path.dirname(__file__), "..", "..", "reference", "examples"))


def _mini_cif(shift=(0.0, 0.0, 0.0), second_far=True) -> str:
    """Two copies of GLY-ALA-SER-GLY (chains A, B), one zinc ion (chain C), a water, an altloc, a two-operator assembly."""
    seq = ["GLY", "ALA", "SER", "GLY"]
    lines = ["data_TEST", "_entry.id TEST", "_exptl.method 'X-RAY DIFFRACTION'", "_refine.ls_d_res_high 1.8",
             "_pdbx_database_status.recvd_initial_deposition_date 2020-01-02",
             "loop_", "_entity.id", "_entity.type", "1 polymer", "2 non-polymer", "3 water",
             "loop_", "_entity_poly.entity_id", "_entity_poly.type", "_entity_poly.pdbx_seq_one_letter_code_can",
             "1 'polypeptide(L)'", ";GASG", ";",
             "loop_", "_entity_poly_seq.entity_id", "_entity_poly_seq.num", "_entity_poly_seq.mon_id"]  # fmt: skip
    lines += [f"1 {i + 1} {r}" for i, r in enumerate(seq)]
    lines += ["loop_", "_struct_asym.id", "_struct_asym.entity_id", "A 1", "B 1", "C 2", "D 3"]
    lines += ["loop_", "_pdbx_struct_assembly_gen.assembly_id", "_pdbx_struct_assembly_gen.oper_expression",
              "_pdbx_struct_assembly_gen.asym_id_list", "1 1 A,B,C,D"]  # fmt: skip
    lines += ["loop_", "_pdbx_struct_oper_list.id"] + [f"_pdbx_struct_oper_list.matrix[{i}][{j}]" for i in (1, 2, 3) for j in (1, 2, 3)]
    lines += [f"_pdbx_struct_oper_list.vector[{i}]" for i in (1, 2, 3)] + ["1 1 0 0 0 1 0 0 0 1 0 0 0"]
    cols = ["group_PDB", "id", "type_symbol", "label_atom_id", "label_alt_id", "label_comp_id", "label_asym_id",
            "label_entity_id", "label_seq_id", "Cartn_x", "Cartn_y", "Cartn_z", "occupancy", "B_iso_or_equiv",
            "auth_seq_id", "auth_asym_id", "pdbx_PDB_model_num"]  # fmt: skip
    lines += ["loop_"] + [f"_atom_site.{c}" for c in cols]
    k = 0
    for chain, off in (("A", 0.0), ("B", 30.0 if second_far else 0.3)):
        for i, r in enumerate(seq[:3]):  # the 4th residue is unresolved
            for name in const.RESIDUE_ATOMS[r]:
                k += 1
                x, y, z = 3.8 * i + shift[0] + off, 1.2 * (k % 5) + shift[1], 0.9 * (k % 3) + shift[2]
                alt = "A" if (name == "CB" and r == "ALA") else "."
                lines.append(f"ATOM {k} {name[0]} {name} {alt} {r} {chain} 1 {i + 1} {x:.3f} {y:.3f} {z:.3f} 0.6 10.0 {i + 1} {chain} 1")
                if alt == "A":
                    k += 1
                    lines.append(f"ATOM {k} C CB B ALA {chain} 1 {i + 1} 99.0 99.0 99.0 0.4 10.0 {i + 1} {chain} 1")
            k += 1
            lines.append(f"ATOM {k} H H . {r} {chain} 1 {i + 1} 0 0 0 1.0 10.0 {i + 1} {chain} 1")
    lines.append(f"HETATM {k + 1} ZN ZN . ZN C 2 . {2.0 + shift[0]:.3f} {2.0 + shift[1]:.3f} {4.0 + shift[2]:.3f} 1.0 10.0 101 A 1")
    lines.append(f"HETATM {k + 2} O O . HOH D 3 . 9.0 9.0 9.0 1.0 10.0 201 A 1")
    return "\n".join(lines) + "\n"


def test_cif_grammar():
    text = "data_x\n_a.b 'it''s ok'\n_a.c \"q r\"\nloop_\n_t.i\n_t.v\n1 'a b'\n2 ?\n# comment\n_z.text\n;line one\nline two\n;\n"
    b = parse_cif(text)[0]
    assert b.name == "x" and b.value("a", "c") == "q r"
    assert b.column("t", "v") == ["a b", "?"] and b.rows("t") == 2
    assert b.value("z", "text") == "line one\nline two"


def test_oper_expression():
    assert parse_oper_expression("1") == [["1"]]
    assert parse_oper_expression("(1-3)") == [["1"], ["2"], ["3"]]
    assert len(parse_oper_expression("(1,2)(3-5)")) == 6


def test_parse_mmcif_and_roundtrip(tmp_path):
    p = tmp_path / "test.cif"
    p.write_text(_mini_cif())
    st, rec = parse_mmcif(str(p))
    assert [c["name"] for c in st.chains] == [b"A", b"B", b"C"]  # water dropped
    assert [int(c["entity_id"]) for c in st.chains] == [0, 0, 1] and [int(c["sym_id"]) for c in st.chains] == [0, 1, 0]
    a = st.chains[0]
    assert int(a["res_num"]) == 4 and not st.residues[3]["is_present"]  # unresolved residue kept from the sequence
    assert int(a["atom_num"]) == 4 + 5 + 6 + 4
    ala_cb = st.atoms[4 + 4]
    assert ala_cb["name"] == b"CB" and ala_cb["x"] < 50  # the higher-occupancy alternate location was taken
    assert st.chain_canonical_seqs[0] == "GASG"
    assert rec.structure_info.resolution == pytest.approx(1.8) and rec.structure_info.method == "X-RAY DIFFRACTION"
    assert rec.chains[0].msa_id == rec.chains[1].msa_id and rec.chains[2].res_name == "ZN"
    assert {(i.chain_1, i.chain_2) for i in rec.interfaces} == {(0, 2)}
    st.save(tmp_path / "s.npz")
    back = Structure.load(tmp_path / "s.npz")
    assert back.atoms.dtype == ATOM_DTYPE and np.array_equal(back.atoms, st.atoms) and back.chain_canonical_seqs == st.chain_canonical_seqs
    st.save_split(tmp_path / "split")
    split = Structure.load_split(tmp_path / "split")
    assert np.allclose(split.coords(), st.coords()) and np.array_equal(split.residues, st.residues)
    sub = st.select_chains([1, 2])
    assert len(sub.chains) == 2 and int(sub.chains[1]["atom_idx"]) == int(sub.chains[0]["atom_num"])
    assert Record.from_dict(rec.to_dict()).to_dict() == rec.to_dict()


def test_filters(tmp_path):
    p = tmp_path / "clash.cif"
    p.write_text(_mini_cif(second_far=False))  # chain B sits on chain A
    st, rec = parse_mmcif(str(p))
    rec, why = filter_structure(st, rec, StructureFilterConfig(min_residues=2))
    assert sum(c.valid for c in rec.chains[:2]) == 1 and "chain clashing" in why.values()
    assert not any(f.valid for f in rec.interfaces if not (rec.chains[f.chain_1].valid and rec.chains[f.chain_2].valid))
    st2, rec2 = parse_mmcif(str(p))
    rec2, why2 = filter_structure(st2, rec2, StructureFilterConfig(min_residues=4))
    assert not rec2.chains[0].valid and why2["A"].startswith("length 3")
    cfg = StructureFilterConfig(max_resolution=1.5, max_release_date="2021-01-01")
    assert "resolution" in filter_structure_metadata(StructureInfo(resolution=1.8, released="2020-01-01"), cfg)
    assert "released" in filter_structure_metadata(StructureInfo(resolution=1.0, released=None), cfg)
    assert filter_structure_metadata(StructureInfo(resolution=1.0, released="2020-05-05"), cfg) is None


def test_interface_chain_selection(tmp_path):
    p = tmp_path / "t.cif"
    p.write_text(_mini_cif())
    st, _ = parse_mmcif(str(p))
    assert select_interface_chains(st, ("chain", 0, 0), max_chains=5) == {0, 1, 2}
    keep = select_interface_chains(st, ("chain", 0, 0), max_chains=1)
    assert keep == {0, 2}  # the far copy is dropped, the ion next to chain A comes back in


def test_clustering():
    seqs = {"a": "MKTAYIAKQRQISFVKSHFSRQ", "b": "MKTAYIAKQRQISFVKSHFSRA", "c": "GGGGSGGGGSGGGGSGGGGSGG"}
    rep = greedy_kmer_clusters(seqs, 0.4)
    assert rep["a"] == rep["b"] and rep["c"] != rep["a"]


def test_prepare_directory_and_cluster(tmp_path):
    src = tmp_path / "src"
    src.mkdir()
    (src / "one.cif").write_text(_mini_cif())
    (src / "bad.cif").write_text("data_bad\n_entry.id bad\n")
    counts = prepare_directory(str(src), str(tmp_path / "out"), StructureFilterConfig(min_residues=2))
    assert counts == {"ok": 1, "rejected": 0, "error": 1}
    recs = load_manifest(str(tmp_path / "out" / "manifest.json"))
    cluster_records(recs, {str(recs[0].chains[0].msa_id): "GASG"})
    assert recs[0].chains[2].cluster_id == "lig:ZN" and recs[0].chains[0].cluster_id == recs[0].chains[1].cluster_id
    assert os.path.exists(tmp_path / "out" / "structures" / "test.npz")


def test_sasa_sphere_and_burial():
    r = sasa.VDW_BY_Z[6]
    one = sasa.atom_sasa(np.zeros((1, 3)), np.array([r]))
    assert one[0] == pytest.approx(4 * math.pi * (r + sasa.PROBE) ** 2)
    two = sasa.atom_sasa(np.array([[0.0, 0, 0], [2.0, 0, 0]]), np.array([r, r]), n_points=400)
    # two equal spheres of radius R at distance d each lose a cap of height R - d/2
    R = r + sasa.PROBE
    assert two[0] == pytest.approx(4 * math.pi * R * R - 2 * math.pi * R * (R - 1.0), rel=0.03)
    pos = np.zeros((2, 1, 3))
    pos[1, 0, 0] = 3.0
    t = sasa.burial_targets(pos, np.ones((2, 1), bool), np.full((2, 1), 6), np.array([0, 1]), np.ones(2, bool))
    assert t.dsasa[0, 1] > 1.0 and t.dsasa[0, 0] == 0 and t.n_contact[0, 1] == 1
    assert list(t.buried_area()) == [(0, 1)]


def test_featurize_structure(tmp_path):
    p = tmp_path / "t.cif"
    p.write_text(_mini_cif())
    st, rec = parse_mmcif(str(p))
    msa = MSA(np.array([[7, 0, 15, 7], [7, 0, 21, 7]], np.int8), np.ones((2, 4), bool), np.zeros((2, 4), np.int8))
    f = featurize_structure(st, rec, unpaired_msa={0: msa})
    N = 4 + 4 + 1
    assert f["res_type"].shape == (N,) and f["msa"].shape == (2, N) and int(f["msa"][1, 2]) == const.MSA_GAP
    assert f["bond_matrix"].shape == (N, N, 1) and f["profile"].shape == (N, const.RES_TYPE_COUNT)
    assert f["atom_gt_mask"][3].sum() == 0 and f["atom_gt_mask"][0].sum() == 4  # unresolved residue, glycine
    assert int(f["mol_type"][-1]) == const.MOL_NONPOLYMER and f["ref_mask"][-1].sum() == 1
    assert torch.allclose(f["atom_gt_positions"][-1, 0], torch.tensor([2.0, 2.0, 4.0]))


def test_cigar_pairs_and_m8():
    q, t = cigar_to_index_pairs("3M2I2M1D1M", 1, 5)
    assert q == [0, 1, 2, 5, 6, 7] and t == [4, 5, 6, 7, 8, 10]
    hits = parse_m8("101\t7yf1_A\t0.856\t132\t19\t0\t1\t132\t2\t133\t6.1E-53\t183\t132M\n")
    assert hits[0]["chainId"] == "A" and hits[0]["templateIndices"][0] == 1 and len(hits[0]["queryIndices"]) == 132


@pytest.mark.skipif(not os.path.isdir(EXAMPLES), reason="reference example files not mounted")
def test_reference_example_job_features():
    from deepfold3_dev_b200.data.inference_input import InferenceInput

    inp = InferenceInput.from_json(os.path.join(EXAMPLES, "9j1y.json"))[0]
    f = inp.features
    assert inp.num_tokens == 245 and f["msa"].shape[1] == 245 and f["msa"].shape[0] > 1000
    assert f["template_mask"].sum() == 4 and f["template_backbone_mask"][0].sum() > 100


def test_structure_dataset_on_the_fly(tmp_path):
    from deepfold3_dev_b200.data.datasets import StructureDataset, collate, open_dataset

    src = tmp_path / "src"
    src.mkdir()
    (src / "one.cif").write_text(_mini_cif())
    prepare_directory(str(src), str(tmp_path / "out"), StructureFilterConfig(min_residues=2))
    recs = load_manifest(str(tmp_path / "out" / "manifest.json"))
    os.makedirs(tmp_path / "out" / "msa")
    MSA(np.array([[7, 0, 15, 7], [7, 0, 21, 7], [7, 1, 15, 7]], np.int8), np.ones((3, 4), bool), np.zeros((3, 4), np.int8)).save(
        tmp_path / "out" / "msa" / f"{recs[0].chains[0].msa_id}.npz")
    d = open_dataset(str(tmp_path / "out"), max_tokens=6)
    assert isinstance(d, StructureDataset) and len(d) == 1 and len(d.weights()) == 1
    x = d[0]
    assert x["res_type"].shape == (6,) and x["msa"].shape[1] == 6 and x["_record_id"] == "test"
    assert x["msa"].shape[0] == 5  # query + two alignment rows for each of the two copies
    b = collate([x, d[1]])
    assert b["res_type"].shape == (2, 6) and b["bond_matrix"].shape == (2, 6, 6, 1)

    # stochastic atomisation (training regulariser): every standard residue split into atom tokens that keep their
    # residue's alignment column, residue index and reference frame; the crop budget counts the extra tokens
    full = open_dataset(str(tmp_path / "out"), max_tokens=64, atomize_prob=1.0)[0]
    plain = open_dataset(str(tmp_path / "out"), max_tokens=64)[0]
    # per chain: GLY ALA SER resolved (4 + 5 + 6 atoms) and one unresolved GLY, which has no atoms to split and stays a
    # residue token; plus the zinc ion
    n_other = int((plain["mol_type"] != 0).sum())
    assert plain["res_type"].shape[0] == 2 * 4 + n_other and full["res_type"].shape[0] == 2 * (15 + 1) + n_other
    prot = (full["mol_type"] == 0) & (full["ref_mask"].sum(-1) == 1)
    assert int(prot.sum()) == 30 and (full["res_type"][prot] == 20).all() and not full["frames_mask"][prot].any()
    # chain A of the entry is GLY ALA SER (resolved part): 4 + 5 + 6 atom tokens reading alignment columns 0, 1, 2
    first = full["asym_id"] == full["asym_id"][0]
    assert full["msa"][1][first].tolist() == [7] * 4 + [0] * 5 + [21] * 6 + [7] and full["msa"][2][first].tolist() == [7] * 4 + [1] * 5 + [15] * 6 + [7]
    assert full["residue_index"][first].unique_consecutive().numel() == 4
    assert len(full["ref_space_uid"][first][:, 0].unique()) == 4  # one reference frame per residue
    # bonds between the atom tokens of the chain: 3 (GLY) + 4 (ALA) + 5 (SER) inside the residues, two peptide links
    inside = full["bond_matrix"][..., 0][first][:, first]
    assert int(inside.sum()) == 2 * (3 + 4 + 5 + 2 + 1) and bool((inside == inside.T).all())  # + SER 3 to the residue token of GLY 4
    assert inside[2, 4] == 1  # C of GLY 1 (third atom) to N of ALA 2 (first atom of the next residue)
    capped = open_dataset(str(tmp_path / "out"), max_tokens=64, atomize_prob=1.0, atomize_max_residues=1)[0]
    assert capped["res_type"].shape[0] < full["res_type"].shape[0] and int((capped["ref_mask"].sum(-1) == 1).sum()) > n_other
    cropped = open_dataset(str(tmp_path / "out"), max_tokens=10, atomize_prob=1.0)[0]
    assert cropped["res_type"].shape[0] == 10 and cropped["msa"].shape[1] == 10
    with pytest.raises(ValueError, match="atomize_source"):
        open_dataset(str(tmp_path / "out"), max_tokens=64, atomize_prob=0.5, atomize_source="sideways")[0]


def test_training_stream_id_lists_and_evaluation_split(tmp_path):
    """The stream builder behind ``train``: include / exclude lists, the release-date split into training and evaluation
    sets, the extended dataset spec, and an evaluation loader that yields the same examples on every pass."""
    from deepfold3_dev_b200.cli.main import _read_id_list, build_training_stream
    from deepfold3_dev_b200.config.schema import ModelConfig, TrainingConfig
    from deepfold3_dev_b200.parallel.dist import DistInfo

    src = tmp_path / "src"
    src.mkdir()
    for name, date in (("aaa1", "2019-05-01"), ("bbb2", "2020-06-01"), ("ccc3", "2022-03-01"), ("ddd4", "2023-01-01")):
        (src / f"{name}.cif").write_text(_mini_cif().replace("data_TEST", f"data_{name.upper()}").replace("_entry.id TEST", f"_entry.id {name.upper()}")
                                         .replace("2020-01-02", date))  # fmt: skip
    out = tmp_path / "out"
    prepare_directory(str(src), str(out), StructureFilterConfig(min_residues=2))
    tc, mc = TrainingConfig(max_tokens=16, max_atoms=0, batch_size_per_rank=1, num_workers=0, eval_samples=8), ModelConfig()
    spec = [f"pdb:{out}:1.0:weighted:0:df3"]

    stream, sampler = build_training_stream(tc, mc, DistInfo(), spec)
    batch = next(iter(stream))
    assert batch["res_type"].shape == (1, 16) and batch["_record_id"][0] in ("aaa1", "bbb2", "ccc3", "ddd4")  # padded to the token budget

    (tmp_path / "inc.txt").write_text("# ids\nAAA1\nbbb2 extra columns are ignored\n\nccc3\n")
    (tmp_path / "exc.txt").write_text("bbb2\n")
    inc, exc = _read_id_list(str(tmp_path / "inc.txt")), _read_id_list(str(tmp_path / "exc.txt"))
    assert inc == {"aaa1", "bbb2", "ccc3"} and _read_id_list(None) is None
    stream, _ = build_training_stream(tc, mc, DistInfo(), spec, include=inc, exclude=exc)
    seen = {next(stream)["_record_id"][0] for _ in range(12)}
    assert seen == {"aaa1", "ccc3"}

    stream, _, loader = build_training_stream(tc, mc, DistInfo(), spec, eval_cutoff_date="2021-01-01", return_eval=True)
    assert {next(stream)["_record_id"][0] for _ in range(12)} == {"aaa1", "bbb2"}
    first = [b["_record_id"][0] for b in loader]
    assert sorted(first) == ["ccc3", "ddd4"] and [b["_record_id"][0] for b in loader] == first  # re-iterable, same order
    a, b = next(iter(loader)), next(iter(loader))
    assert torch.equal(a["res_type"], b["res_type"]) and torch.equal(a["ref_pos"], b["ref_pos"])  # the same crop every time
    # two ranks split the evaluation set; without a date split and without configured sets there is nothing to evaluate
    halves = [build_training_stream(tc, mc, DistInfo(rank=r, world_size=2), spec, eval_cutoff_date="2021-01-01", return_eval=True)[2] for r in (0, 1)]
    assert sorted(len(h) for h in halves) == [1, 1]
    assert build_training_stream(tc, mc, DistInfo(), spec, return_eval=True)[2] is None


def test_crystallization_aids_are_dropped_from_xray_entries(tmp_path):
    sulfate = _mini_cif().replace(" ZN ZN . ZN C 2", " S S . SO4 C 2")
    (tmp_path / "s.cif").write_text(sulfate)
    (tmp_path / "n.cif").write_text(sulfate.replace("X-RAY DIFFRACTION", "SOLUTION NMR"))
    (tmp_path / "z.cif").write_text(_mini_cif())
    kept = lambda name, drop: [c.res_name for c in parse_mmcif(str(tmp_path / name), use_assembly=False, drop_crystallization_aids=drop)[1].chains]  # noqa: E731
    assert kept("s.cif", False)[-1] == "SO4" and "SO4" not in kept("s.cif", True) and len(kept("s.cif", True)) == 2
    assert kept("n.cif", True)[-1] == "SO4"  # only diffraction entries carry crystallisation additives
    assert kept("z.cif", True)[-1] == "ZN"  # a real ligand stays


def test_training_templates_respect_dates_and_sampling(tmp_path):
    """Templates of training examples: per-sequence hit list under the dataset root, coordinates from the per-chain
    cache, release-date cut-off relative to the example (fail-closed), self-hits dropped, k = min(U{0..n}, max) sampled,
    features placed on the surviving tokens of the chain."""
    import json
    import random

    from deepfold3_dev_b200.data import templates as tpl
    from deepfold3_dev_b200.data.datasets import StructureDataset

    src = tmp_path / "src"
    src.mkdir()
    (src / "one.cif").write_text(_mini_cif())
    out = tmp_path / "out"
    prepare_directory(str(src), str(out), StructureFilterConfig(min_residues=2))
    rec = load_manifest(str(out / "manifest.json"))[0]
    assert rec.structure_info.released == "2020-01-02"
    # the template entry: the same small structure under another id, moved in space
    mirror = tmp_path / "mirror"
    mirror.mkdir()
    (mirror / "1abc.cif").write_text(_mini_cif(shift=(3.0, 0.0, 0.0)).replace("data_TEST", "data_1ABC").replace("_entry.id TEST", "_entry.id 1ABC"))
    cache = tmp_path / "cache"
    assert tpl.build_chain_cache(str(mirror), str(cache)) == 2
    msa_id = str(rec.chains[0].msa_id)
    hit = {"template_pdb_id": "1abc", "template_chain_id": "A", "identity": 0.5, "evalue": 1e-9, "qstart": 1, "qend": 3, "tstart": 1, "tend": 3, "cigar": "3M"}
    hits = [dict(hit, release_date="2015-06-01"), dict(hit, template_pdb_id="test", release_date="2010-01-01"),
            dict(hit, template_chain_id="B", release_date="2019-12-25"), dict(hit, template_chain_id="B", release_date=None)]
    index = out / "monomer_templates" / msa_id[:2].lower() / f"{msa_id}.json"
    index.parent.mkdir(parents=True)
    index.write_text(json.dumps(hits))

    # cut-off arithmetic: 60 days before the example, capped by the recipe's hard limit; nothing known -> no templates
    assert tpl.template_cutoff("2020-01-02", 60) == "2019-11-03" and tpl.template_cutoff("2020-01-02", 60, "2018-01-01") == "2018-01-01"
    assert tpl.template_cutoff(None, 60, None, "2017-05-05") == "2017-05-05" and tpl.template_cutoff(None, 60) is None
    rng = random.Random(0)
    picks = [tpl.sample_training_templates(hits, "test", "2019-11-03", rng, 4) for _ in range(40)]
    assert {len(p) for p in picks} == {0, 1} and all(p[0]["release_date"] == "2015-06-01" for p in picks if p)
    assert tpl.sample_training_templates(hits, "test", None, rng, 4) == []  # fail closed
    assert {len(tpl.sample_training_templates(hits, "other", "2021-01-01", rng, 2)) for _ in range(60)} == {0, 1, 2}
    assert tpl.passes_hit_filters(dict(hit, qend=50, tend=50), 100) and not tpl.passes_hit_filters(hit, 100)  # 3 residues: too short
    assert not tpl.passes_hit_filters(dict(hit, qend=99, tend=99, identity=1.0), 100)  # a copy of the query

    # the index builder: m8 rows -> filtered, dated hit lists in the sharded layout
    m8 = tmp_path / "m8"
    m8.mkdir()
    row = lambda t, ident, q2, t2, cigar: "\t".join(["q", t, str(ident), "50", "0", "0", "1", str(q2), "1", str(t2), "1e-9", "100", cigar])  # noqa: E731
    (m8 / "seqx.m8").write_text("\n".join([row("2xyz_A", 0.4, 40, 40, "40M"), row("3abc_B", 1.0, 50, 50, "50M"), row("4def_C", 0.3, 4, 4, "4M"),
                                            row("5ghi_A", 0.5, 30, 30, "30M")]) + "\n")
    built = tmp_path / "built"
    built.mkdir()
    assert tpl.build_monomer_template_index(str(built), str(m8), {"2XYZ": "2001-02-03"}, {"seqx": 50}) == (1, 2)
    got = json.loads((built / "monomer_templates" / "se" / "seqx.json").read_text())
    assert [(h["template_pdb_id"], h["template_chain_id"], h["release_date"]) for h in got] == [("2xyz", "A", "2001-02-03"), ("5ghi", "A", None)]
    assert tpl.hit_index_pairs(got[0]) == (list(range(40)), list(range(40)))

    d = StructureDataset(str(out), max_tokens=64, pdb_chain_cache_dir=str(cache))
    seen, placed = [], 0
    for i in range(0, 24, 2):
        x = d[i]
        assert x["template_aatype"].shape == (4, x["res_type"].shape[0]) and x["template_mask"].shape == (4,)
        seen.append(int(x["template_mask"].sum()))
        for c in (0, 1):  # the two copies of the chain draw their templates independently and share the template rows
            cols = x["asym_id"] == c
            if bool((x["template_aatype"][0][cols] != 21).any()):
                placed += 1
                assert x["template_aatype"][0][cols].tolist()[:3] == [7, 0, 15] and x["template_pseudo_beta_mask"][0][cols][:3].eq(1).all()
                assert (x["template_aatype"][0][cols][3:] == 21).all()  # the fourth residue is not aligned
                assert x["template_backbone_mask"][0][cols][:3].eq(1).all() and seen[-1] == 1
    assert set(seen) == {0, 1} and placed >= 2 and d.templates_used == placed
    # an example without a release date and no configured fallback gets no template
    for r in d.records:
        r.structure_info.released = None
    assert all(int(d[i]["template_mask"].sum()) == 0 for i in range(6))
    # an example slower than the configured threshold is reported with the time of every phase
    import logging

    slow = StructureDataset(str(out), max_tokens=64, pdb_chain_cache_dir=str(cache), slow_sample_log_threshold_s=1e-9)
    lines = []
    handler = logging.Handler()
    handler.emit = lambda record: lines.append(record.getMessage())
    logging.getLogger("deepfold3_dev_b200.data.datasets").addHandler(handler)
    try:
        slow[0]
    finally:
        logging.getLogger("deepfold3_dev_b200.data.datasets").removeHandler(handler)
    assert len(lines) == 1 and lines[0].startswith("SLOW_SAMPLE ") and all(k in lines[0] for k in ("featurize=", "crop=", "msa=", "templates="))
    d.default_template_cutoff_date = "2016-01-01"
    assert any(int(d[i]["template_mask"].sum()) == 1 for i in range(12))


_PLM_CIF = """data_ZZ1
_chem_comp.id ZZ1
_chem_comp.name 'TEST ACID'
loop_
_chem_comp_atom.comp_id
_chem_comp_atom.atom_id
_chem_comp_atom.type_symbol
_chem_comp_atom.charge
_chem_comp_atom.pdbx_leaving_atom_flag
_chem_comp_atom.model_Cartn_x
_chem_comp_atom.model_Cartn_y
_chem_comp_atom.model_Cartn_z
_chem_comp_atom.pdbx_model_Cartn_x_ideal
_chem_comp_atom.pdbx_model_Cartn_y_ideal
_chem_comp_atom.pdbx_model_Cartn_z_ideal
ZZ1 C1  C 0  N 9.0 9.0 9.0 0.000 0.000 0.000
ZZ1 O1  O -1 N 9.0 9.0 9.0 1.250 0.000 0.000
ZZ1 O2  O 0  Y 9.0 9.0 9.0 -0.600 1.100 0.000
ZZ1 "C1'" C 0 N 9.0 9.0 9.0 -0.800 -1.200 0.300
ZZ1 H1  H 0  N 9.0 9.0 9.0 -1.800 -1.200 0.300
loop_
_chem_comp_bond.comp_id
_chem_comp_bond.atom_id_1
_chem_comp_bond.atom_id_2
_chem_comp_bond.value_order
ZZ1 C1 O1 SING
ZZ1 C1 O2 DOUB
ZZ1 C1 "C1'" SING
ZZ1 "C1'" H1 SING
data_ZZ2
_chem_comp.id ZZ2
loop_
_chem_comp_atom.comp_id
_chem_comp_atom.atom_id
_chem_comp_atom.type_symbol
_chem_comp_atom.charge
_chem_comp_atom.model_Cartn_x
_chem_comp_atom.model_Cartn_y
_chem_comp_atom.model_Cartn_z
ZZ2 MG MG 2 1.0 2.0 3.0
"""


def test_component_dictionary_lookup(tmp_path):
    from deepfold3_dev_b200.data import ccd, ref_conformers
    from deepfold3_dev_b200.data.inference_input import InferenceInput
    from deepfold3_dev_b200.data.parse.json_input import JobInput, LigandChainInput, ProteinChainInput

    path = tmp_path / "components.cif"
    path.write_text(_PLM_CIF)
    comps = ccd.load_components(str(path), {"zz1"})
    assert list(comps) == ["ZZ1"]
    c = comps["ZZ1"]
    assert c.atoms == ["C1", "O1", "O2", "C1'"] and c.elements == [6, 8, 8, 6] and c.charges == [0, -1, 0, 0]
    assert c.leaving == [False, False, True, False] and c.bonds == [(0, 1, 1), (0, 2, 2), (0, 3, 1)]
    assert np.allclose(c.coords[1], [1.25, 0, 0])  # ideal coordinates, not the model ones
    assert ccd.leaving_atom_sets(comps)["ZZ1"] == {"O2"} and ccd.atom_name_sets(comps)["ZZ1"] == {"C1", "O1", "O2", "C1'"}
    assert np.allclose(ccd.load_components(str(path))["ZZ2"].coords[0], [1, 2, 3])  # model coordinates as the fallback
    # an entry without any coordinates is embedded from its bond graph: bonded atoms at bond length, none coincide
    bare = _PLM_CIF.split("data_ZZ2")[0].replace("data_ZZ1", "data_ZZ7").replace("ZZ1 ", "ZZ7 ")
    for number in ("9.0 9.0 9.0", "0.000 0.000 0.000", "1.250 0.000 0.000", "-0.600 1.100 0.000", "-0.800 -1.200 0.300", "-1.800 -1.200 0.300"):
        bare = bare.replace(number, "? ? ?")
    emb = ccd.parse_component(bare)
    dist = np.linalg.norm(emb.coords[:, None] - emb.coords[None], axis=-1)
    assert emb.atoms == c.atoms and all(1.1 < dist[i, j] < 1.7 for i, j, _ in emb.bonds) and dist[np.triu_indices(4, 1)].min() > 1.0
    ref_conformers.set_ccd_source(str(path))
    try:
        job = JobInput("lig", [ProteinChainInput(["A"], "GASG"), LigandChainInput(["L"], ["ZZ1"])])
        inp = InferenceInput.from_job(job)
        assert inp.num_tokens == 4 + 4 and int(inp.features["ref_element"][-3, 0]) == 8
        bm = inp.features["bond_matrix"][..., 0]
        assert bm.shape == (8, 8) and bm[4, 5] == 1 and bm[5, 4] == 1 and bm[4, 6] == 1 and bm[4, 7] == 1 and bm.sum() == 6
        from deepfold3_dev_b200.data.parse.json_input import BondedAtomPair

        job.bonded_atom_pairs = [BondedAtomPair(("A", 3, "OG"), ("L", 1, "O1"))]
        bm2 = InferenceInput.from_job(job).features["bond_matrix"][..., 0]
        assert bm2[2, 5] == 1 and bm2[5, 2] == 1 and bm2.sum() == 8
        assert ccd.export_table(str(path), str(tmp_path / "t.json")) == 2
    finally:
        ref_conformers.set_ccd_source(None)
        ref_conformers._TABLE.pop("ZZ1", None)
        ref_conformers._TABLE.pop("ZZ2", None)


@pytest.mark.skipif(not os.path.isdir(EXAMPLES), reason="reference example files not mounted")
def test_prepare_job_templates_from_hits(tmp_path):
    from deepfold3_dev_b200.data.templates import build_chain_cache, load_json_templates, load_template_chain, prepare_job_templates

    src = tmp_path / "pdb"
    src.mkdir()
    import shutil

    for name in ("7yf1_A.cif", "5hz8_A.cif"):
        shutil.copy(os.path.join(EXAMPLES, "9m22_msa", "templates", name), src / (name.split("_")[0] + ".cif"))
    m8 = open(os.path.join(EXAMPLES, "9m22_msa", "pdb70.m8")).read()
    hits = prepare_job_templates(m8, str(src), str(tmp_path / "out"), max_release_date="2022-12-31")
    assert [h["name"] for h in hits] == ["7yf1_A.cif", "5hz8_A.cif"]  # the two entries on disk, best first
    assert prepare_job_templates(m8, str(src), str(tmp_path / "old"), max_release_date="2020-01-01")[0]["name"] == "5hz8_A.cif"
    chains = load_json_templates(hits, str(tmp_path / "out"))
    assert len(chains) == 2 and chains[0].atom_mask.sum() > 500
    assert build_chain_cache(str(src), str(tmp_path / "cache")) >= 2
    cached = load_template_chain(str(tmp_path / "cache" / "7yf1_A.npz"), hits[0]["queryIndices"], hits[0]["templateIndices"])
    assert cached.res_names == chains[0].res_names and np.allclose(cached.coords, chains[0].coords)


def test_structure_mmcif_write_read_cycle(tmp_path):
    from deepfold3_dev_b200.data.featurize import tokenize_structure
    from deepfold3_dev_b200.io.structure_mmcif import with_coordinates, write_structure

    p = tmp_path / "t.cif"
    p.write_text(_mini_cif())
    st, _ = parse_mmcif(str(p))
    write_structure(st, str(tmp_path / "w.cif"))
    back, _ = parse_mmcif(str(tmp_path / "w.cif"), use_assembly=False)
    assert len(back.chains) == len(st.chains) and np.array_equal(back.residues["name"], st.residues["name"])
    assert np.array_equal(back.atoms["is_present"], st.atoms["is_present"])
    ok = st.atoms["is_present"]
    assert np.allclose(back.coords()[ok], st.coords()[ok], atol=2e-3) and back.chain_canonical_seqs[0] == "GASG"
    tok, rows, _ = tokenize_structure(st)
    moved = with_coordinates(st, np.ones((len(rows), 24, 3), np.float32), rows, np.full((len(rows), 24), 77.0))
    assert moved.atoms["is_present"].all() and float(moved.atoms["b_factor"].min()) == 77.0 and float(moved.coords().max()) == 1.0


def test_date_cutoff_is_fail_closed():
    from deepfold3_dev_b200.data.datasets import apply_date_cutoff
    from deepfold3_dev_b200.data.types import ChainInfo

    def rec(i, date):
        return Record(str(i), [ChainInfo(0, "A", 0, "c", "m", 10)], [], StructureInfo(released=date) if date != "none" else None)

    recs = [rec(0, "2020-01-01"), rec(1, "2022-05-05"), rec(2, None), rec(3, "none"), rec(4, "2021-09-30")]
    assert [r.id for r in apply_date_cutoff(recs, "2021-09-30")] == ["0", "4"]
    assert [r.id for r in apply_date_cutoff(recs, "2021-09-30", keep_after=True)] == ["1"]
    assert len(apply_date_cutoff(recs, "")) == 5


def test_component_dictionary_gz_and_json_table(tmp_path):
    import gzip

    from deepfold3_dev_b200.data import ccd, ref_conformers

    gz = tmp_path / "components.cif.gz"
    with gzip.open(gz, "wt") as f:
        f.write(_PLM_CIF)
    assert [c for c, _ in ccd.iter_blocks(str(gz), {"ZZ2"})] == ["ZZ2"]
    assert sorted(ccd.load_components(str(gz))) == ["ZZ1", "ZZ2"]
    table = tmp_path / "t.json"
    assert ccd.export_table(str(gz), str(table), {"ZZ1"}) == 1
    try:
        ref_conformers.set_ccd_source(str(table))  # a JSON table is loaded at once
        names, elements, charges, coords = ref_conformers.get_ref_atoms("zz1")
        assert names == ["C1", "O1", "O2", "C1'"] and charges[1] == -1 and coords.shape == (4, 3)
        assert ref_conformers.load_component_text(_PLM_CIF) == 2 and ref_conformers.get_ref_atoms("ZZ2")[0] == ["MG"]
    finally:
        ref_conformers._TABLE.pop("ZZ1", None)
        ref_conformers._TABLE.pop("ZZ2", None)


def test_dataset_tool_commands(tmp_path):
    """The dataset maintenance commands on a one-entry prepared directory, through the command line."""
    import json

    from click.testing import CliRunner

    from deepfold3_dev_b200.cli.main import cli
    from deepfold3_dev_b200.data.types import Structure

    src = tmp_path / "src"
    src.mkdir()
    (src / "one.cif").write_text(_mini_cif())
    out = tmp_path / "out"
    prepare_directory(str(src), str(out), StructureFilterConfig(min_residues=2))
    rec = load_manifest(str(out / "manifest.json"))[0]
    st = Structure.load(str(out / "structures" / "test.npz"))
    seq = st.chain_canonical_seqs[rec.chains[0].chain_id]
    run = CliRunner().invoke

    # export-complexes: two protein copies -> one multimer entry
    r = run(cli, ["export-complexes", "--data-dir", str(out), "--output", str(tmp_path / "cx.json")])
    assert r.exit_code == 0, r.output
    assert json.loads((tmp_path / "cx.json").read_text()) == {"test": [seq, seq]}

    # import-msa: an A3M named anything, matched by its query sequence
    a3m = tmp_path / "a3m" / "deep" / "whatever.a3m"
    a3m.parent.mkdir(parents=True)
    a3m.write_text(f">query\n{seq}\n>hit1\n{seq[:-1]}-\n>hit2\n{seq[0].lower()}{seq}\n")
    r = run(cli, ["import-msa", "--data-dir", str(out), "--msa-dir", str(tmp_path / "a3m")])
    assert r.exit_code == 0 and "1 written" in r.output, r.output
    stored = MSA.load(str(out / "msa" / f"{rec.chains[0].msa_id}.npz"))
    assert stored.sequences.shape == (2, len(seq))  # hit2 equals the query once its insertion is dropped: de-duplicated
    r = run(cli, ["import-msa", "--data-dir", str(out), "--msa-dir", str(tmp_path / "a3m")])
    assert "0 written" in r.output  # resume-safe: existing files stay

    # import-paired-msa: <record>/<msa_id>.paired.a3m
    paired = tmp_path / "paired" / "test"
    paired.mkdir(parents=True)
    (paired / f"{rec.chains[0].msa_id}.paired.a3m").write_text(f">query\n{seq}\n>p1\n{seq}\n")
    r = run(cli, ["import-paired-msa", "--data-dir", str(out), "--paired-dir", str(tmp_path / "paired")])
    assert r.exit_code == 0, r.output
    after = load_manifest(str(out / "manifest.json"))[0]
    assert after.chains[0].paired_msa_id == f"test/{rec.chains[0].msa_id}"
    assert os.path.exists(out / "msa_paired" / "test" / f"{rec.chains[0].msa_id}.npz")

    # enrich-manifest from an entries.idx line (id, header, date mm/dd/yy, compound, source, authors, resolution, method)
    idx = tmp_path / "entries.idx"
    idx.write_text("IDCODE, HEADER...\n-----\nTEST\tHYDROLASE\t03/15/99\tX\tY\tZ\t1.85\tX-RAY DIFFRACTION\n")
    m = json.loads((out / "manifest.json").read_text())
    m[0]["structure_info"].update(resolution=None, method=None, deposited=None)
    (out / "manifest.json").write_text(json.dumps(m))
    r = run(cli, ["enrich-manifest", "--data-dir", str(out), "--idx", str(idx)])
    assert r.exit_code == 0 and "3 fields filled" in r.output, r.output
    info = load_manifest(str(out / "manifest.json"))[0].structure_info
    assert info.resolution == 1.85 and info.deposited == "1999-03-15" and info.method == "X-RAY DIFFRACTION"

    # stamp-template-index-space: dry run changes nothing, the real run is idempotent
    (out / "templates").mkdir()
    (out / "templates" / "abc.json").write_text(json.dumps([{"pdb": "1abc", "chain": "A"}]))
    r = run(cli, ["stamp-template-index-space", "--data-dir", str(out), "--dry-run"])
    assert "1 would be stamped" in r.output and isinstance(json.loads((out / "templates" / "abc.json").read_text()), list)
    r = run(cli, ["stamp-template-index-space", "--data-dir", str(out), "--space", "seqres"])
    assert json.loads((out / "templates" / "abc.json").read_text())["index_space"] == "seqres"
    r = run(cli, ["stamp-template-index-space", "--data-dir", str(out), "--space", "seqres"])
    assert "0 stamped" in r.output
    r = run(cli, ["stamp-template-index-space", "--data-dir", str(out), "--space", "struct"])
    assert r.exit_code != 0  # already stamped with the other frame

    # pack + pack-verify, then a corrupted source is caught
    r = run(cli, ["pack", str(out / "structures"), str(tmp_path / "pk")])
    assert r.exit_code == 0
    assert run(cli, ["pack-verify", str(out / "structures"), str(tmp_path / "pk")]).exit_code == 0
    with open(out / "structures" / "test.npz", "ab") as f:
        f.write(b"x")
    assert run(cli, ["pack-verify", str(out / "structures"), str(tmp_path / "pk")]).exit_code != 0

    # drop-obsolete with a local id list, deleting the files
    r = run(cli, ["drop-obsolete", "--data-dir", str(out), "--ids-file", str(tmp_path / "ids.json")])
    assert r.exit_code != 0  # the id file has to exist
    (tmp_path / "ids.json").write_text(json.dumps(["TEST"]))
    r = run(cli, ["drop-obsolete", "--data-dir", str(out), "--ids-file", str(tmp_path / "ids.json"), "--delete-files"])
    assert r.exit_code == 0 and "1 obsolete records dropped" in r.output
    assert load_manifest(str(out / "manifest.json")) == [] and not os.path.exists(out / "structures" / "test.npz")

    # the chemical component cache with automorphisms, and fetch-ccd from a local file
    (tmp_path / "comp.cif").write_text(_PLM_CIF)
    r = run(cli, ["fetch-ccd", "--output", str(tmp_path / "ccd"), "--from-file", str(tmp_path / "comp.cif")])
    assert r.exit_code == 0 and os.path.exists(tmp_path / "ccd" / "comp.cif")
    r = run(cli, ["build-ccd-cache", "--components-cif", str(tmp_path / "comp.cif"), "--output", str(tmp_path / "ccd.json"),
                  "--automorphisms"])  # fmt: skip
    assert r.exit_code == 0, r.output
    table = json.loads((tmp_path / "ccd.json").read_text())
    assert set(table) == {"ZZ1", "ZZ2"} and "automorphisms" not in table["ZZ1"]  # C(-O-)(=O)C: the two oxygens differ in bond order


def test_template_hit_is_reconciled_with_the_structure_sequence(tmp_path):
    from deepfold3_dev_b200.data import const
    from deepfold3_dev_b200.data.templates import reconcile_hit_with_chain, template_chain_from_mmcif

    # the docstring case of the purpose: database sequence differs from the chain at the ends and in one stretch
    chain = "XDEFGHKLMNPQRS"
    db = "ABCDEFGHIJKLMNPQ"  # 3 extra residues in front of D, "IJ" where the chain has nothing
    hit, start = db[3:], 3  # the hit covers db positions 3..15
    mapping = {q: t for q, t in zip(range(10, 23), range(3, 16))}
    moved = reconcile_hit_with_chain(mapping, hit, start, chain)
    assert all(chain[moved[q]] == db[mapping[q]] for q in moved)  # every kept position points at the same residue
    assert set(mapping) - set(moved) == {15, 16}  # the queries aligned to I and J have no residue in the chain
    assert reconcile_hit_with_chain(mapping, hit, start, "WWWWWWWWWWWWWWWW") is None  # the wrong chain
    same = reconcile_hit_with_chain({0: 1, 1: 2}, "DE", 1, chain)
    assert same == {0: 1, 1: 2}  # already in place: untouched

    # through the file reader: a hit whose database sequence lacks the chain's first three residues
    path = os.path.join(EXAMPLES, "9m22_msa", "templates", "7yf1_A.cif")
    full = template_chain_from_mmcif(path, "A", list(range(20)), list(range(20)))
    letters = "".join(const.PROTEIN_3TO1.get(n, "X") for n in full.res_names)
    shifted = template_chain_from_mmcif(path, "A", list(range(20)), list(range(20)), hit_sequence=letters[3:43], hit_start=0)
    assert shifted.query_to_hit == {q: q + 3 for q in range(20)}
    assert template_chain_from_mmcif(path, "A", list(range(20)), list(range(20)), hit_sequence="W" * 40, hit_start=0) is None


def test_template_date_backfill_and_alignment_worklist(tmp_path):
    import importlib
    import json

    from click.testing import CliRunner

    cli = importlib.import_module("deepfold3_dev_b200.cli.main").cli
    src = tmp_path / "src"
    src.mkdir()
    (src / "one.cif").write_text(_mini_cif())
    out = tmp_path / "out"
    prepare_directory(str(src), str(out), StructureFilterConfig(min_residues=2))
    # hit lists without dates: one plain list, one wrapped with its index space
    (out / "monomer_templates" / "ab").mkdir(parents=True)
    hits = [{"template_pdb_id": "1abc", "template_chain_id": "A", "release_date": None}, {"template_pdb_id": "9zzz", "release_date": None},
            {"template_pdb_id": "2def", "release_date": "1999-01-01"}]  # fmt: skip
    (out / "monomer_templates" / "ab" / "abcd.json").write_text(json.dumps(hits))
    (out / "monomer_templates" / "ab" / "abce.json").write_text(json.dumps({"index_space": "struct", "hits": hits[:1]}))
    (tmp_path / "dates.json").write_text(json.dumps({"1ABC": "2001-02-03", "2def": "2010-10-10"}))
    args = ["backfill-template-dates", "--data-dir", str(out), "--release-dates", str(tmp_path / "dates.json")]
    dry = CliRunner().invoke(cli, args + ["--dry-run"])
    assert dry.exit_code == 0 and "2 dates would be filled in 2 files, 1 hits without a known date" in dry.output
    assert json.loads((out / "monomer_templates" / "ab" / "abcd.json").read_text())[0]["release_date"] is None
    assert CliRunner().invoke(cli, args).exit_code == 0
    got = json.loads((out / "monomer_templates" / "ab" / "abcd.json").read_text())
    assert [h["release_date"] for h in got] == ["2001-02-03", None, "1999-01-01"]  # present dates are kept
    wrapped = json.loads((out / "monomer_templates" / "ab" / "abce.json").read_text())
    assert wrapped["index_space"] == "struct" and wrapped["hits"][0]["release_date"] == "2001-02-03"

    # nothing has an alignment yet: every distinct protein sequence is on the list; with one attached it drops off
    res = CliRunner().invoke(cli, ["msa-worklist", "--data-dir", str(out), "--output", str(tmp_path / "todo")])
    assert res.exit_code == 0, res.output + repr(res.exception)
    stats = json.loads((tmp_path / "todo" / "stats.json").read_text())
    fasta = (tmp_path / "todo" / "combined.fasta").read_text().split()
    assert stats["with_alignment"] == 0 and stats["sequences_to_search"] == stats["protein_sequences"] == len(fasta) // 2 >= 1
    msa_id = fasta[0][1:]
    (out / "msa").mkdir(exist_ok=True)
    (out / "msa" / f"{msa_id}.a3m").write_text(f">query\n{fasta[1]}\n")
    CliRunner().invoke(cli, ["msa-worklist", "--data-dir", str(out), "--output", str(tmp_path / "todo")])
    again = json.loads((tmp_path / "todo" / "stats.json").read_text())
    assert again["with_alignment"] == 1 and again["sequences_to_search"] == stats["sequences_to_search"] - 1
