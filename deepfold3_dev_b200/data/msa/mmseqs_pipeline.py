"""Local MMseqs2 searches in the ColabFold manner: staged pipelines over UniRef30, an environmental database and a
PDB sequence database, for single chains (batched) and for paired alignments of complexes.

The reference drives the same binary with the same stages (data/msa/mmseqs2.py:564-1863: ``_search_monomer``,
``_search_pair``, ``search_monomer_batch``, ``search_pair_batch``; shell forms in scripts/mmseqs_msa.sh and
scripts/mmseqs_pair.sh). Here the stages are data: ``plan_monomer`` / ``plan_pair`` return the list of ``mmseqs``
command lines for a work directory, ``run_plan`` executes it, and the batch functions put all distinct query sequences of
many jobs into one query database so that the (expensive) database load is paid once per batch.

Stages for unpaired alignments (per target database):
  search (3 iterations, profile kept) -> expandaln (cluster members) -> align (re-align against the profile)
  -> filterresult -> result2msa (A3M, diversity filter in identity bins)
then the UniRef and environmental alignments are merged per query. Templates: one more search of the UniRef profile
against the PDB sequences, reported as an m8 table with CIGAR strings. Paired alignments: search + expandaln + align as
above on the chains of one complex, ``pairaln`` keeps hits whose taxonomy occurs for every chain, a second align +
``pairaln`` pass orders them, ``result2msa`` writes row-aligned A3M blocks.

GPU: with ``gpu=True`` the prefilter runs on the GPU (databases built with ``makepaddedseqdb``); with
``gpu_server=True`` it is delegated to an already running ``mmseqs gpuserver`` that keeps the database resident
(``deploy/msa/gpuserver.sh``), which removes the per-search start-up cost.
"""

from __future__ import annotations

import dataclasses
import hashlib
import os
import shutil
import subprocess
import tempfile

UNIREF_DB = "uniref30_2302_db"
ENV_DB = "colabfold_envdb_202108_db"
TEMPLATE_DB = "pdb100_230517"
M8_COLUMNS = "query,target,fident,alnlen,mismatch,gapopen,qstart,qend,tstart,tend,evalue,bits,cigar"


@dataclasses.dataclass
class MmseqsSettings:
    db_dir: str
    uniref_db: str = UNIREF_DB
    env_db: str = ENV_DB
    template_db: str = TEMPLATE_DB
    use_env: bool = True
    use_templates: bool = False
    gpu: bool = False
    gpu_server: bool = False
    threads: int = 32
    sensitivity: float = 8.0
    max_seqs: int = 10000
    pairing_mode: int = 0  # 0: a hit must occur for every chain (complete pairing), 1: greedy
    binary: str = "mmseqs"


def detect_db_mode(db_dir: str, name: str) -> tuple[str, str]:
    """``(suffix, load mode)``: with a precomputed index (``<name>.idx``) the index is used and memory-mapped
    (``--db-load-mode 2``); without one the plain database is read (``--db-load-mode 0``)."""
    if os.path.exists(os.path.join(db_dir, f"{name}.idx")) or os.path.exists(os.path.join(db_dir, f"{name}.idx.dbtype")):
        return ".idx", "2"
    return "", "0"


def _search_flags(s: MmseqsSettings, load: str) -> list[str]:
    flags = ["--num-iterations", "3", "--db-load-mode", load, "-a", "-e", "0.1", "--max-seqs", str(s.max_seqs),
             "--threads", str(s.threads)]  # fmt: skip
    if s.gpu or s.gpu_server:
        flags += ["--gpu", "1", "--prefilter-mode", "1"]  # ungapped GPU prefilter: no k-mer sensitivity setting
        if s.gpu_server:
            flags += ["--gpu-server", "1"]
    else:
        flags += ["-s", f"{s.sensitivity:g}"]
    return flags


_FILTER_MSA = ["--filter-msa", "1", "--filter-min-enable", "1000", "--diff", "3000", "--qid", "0.0,0.2,0.4,0.6,0.8,1.0",
               "--qsc", "0", "--max-seq-id", "0.95"]  # fmt: skip


def _expand_align_filter(work, qdb, expand_from, realign_with, db, tag, load, threads) -> list[list[str]]:
    """expandaln -> align -> filterresult -> result2msa for one target database; the A3M database is ``<tag>.a3m``.
    ``expand_from`` is the query side of the search that produced ``res_<tag>``; ``realign_with`` the profile the
    expanded hits are re-aligned against."""
    j = lambda n: os.path.join(work, n)  # noqa: E731
    return [
        ["expandaln", expand_from, db, j(f"res_{tag}"), db, j(f"res_{tag}_exp"), "--db-load-mode", load, "--threads", threads,
         "--expansion-mode", "0", "-e", "inf", "--expand-filter-clusters", "1", "--max-seq-id", "0.95"],
        ["align", realign_with, db, j(f"res_{tag}_exp"), j(f"res_{tag}_exp_realign"), "--db-load-mode", load, "--threads", threads,
         "-e", "10", "--max-accept", "1000000", "--alt-ali", "10", "-a"],
        ["filterresult", qdb, db, j(f"res_{tag}_exp_realign"), j(f"res_{tag}_exp_realign_filter"), "--db-load-mode", load,
         "--threads", threads, "--qid", "0", "--qsc", "0.8", "--diff", "0", "--max-seq-id", "1.0", "--filter-min-enable", "100"],
        ["result2msa", qdb, db, j(f"res_{tag}_exp_realign_filter"), j(f"{tag}.a3m"), "--msa-format-mode", "6",
         "--db-load-mode", load, "--threads", threads, *_FILTER_MSA],
    ]  # fmt: skip


def plan_monomer(s: MmseqsSettings, work: str, fasta: str) -> list[list[str]]:
    """Command lines (without the binary) that turn ``fasta`` into ``work/out/<index>.a3m`` (and ``work/pdb.m8``)."""
    j = lambda n: os.path.join(work, n)  # noqa: E731
    threads = str(s.threads)
    suf, load = detect_db_mode(s.db_dir, s.uniref_db)
    uniref = os.path.join(s.db_dir, s.uniref_db)
    qdb, prof = j("qdb"), j("prof_res")
    plan = [
        ["createdb", fasta, qdb, "--shuffle", "0"],
        ["search", qdb, uniref, j("res_uniref"), j("tmp"), *_search_flags(s, load)],
        ["mvdb", j("tmp/latest/profile_1"), prof],     # the profile of the last iteration: query side of everything below
        ["lndb", j("qdb_h"), j("prof_res_h")],
        *_expand_align_filter(work, qdb, qdb, prof, uniref + suf, "uniref", load, threads),
    ]
    merged = [j("uniref.a3m")]
    if s.use_templates:
        tsuf, tload = detect_db_mode(s.db_dir, s.template_db)
        tdb = os.path.join(s.db_dir, s.template_db)
        plan += [
            ["search", prof, tdb, j("res_pdb"), j("tmp_pdb"), "--db-load-mode", tload, "--threads", threads, "-s", "7.5", "-a", "-e", "0.1"],
            ["convertalis", prof, tdb + tsuf, j("res_pdb"), j("pdb.m8"), "--format-output", M8_COLUMNS, "--db-load-mode", tload,
             "--threads", threads],
        ]  # fmt: skip
    if s.use_env:
        esuf, eload = detect_db_mode(s.db_dir, s.env_db)
        env = os.path.join(s.db_dir, s.env_db)
        # the environmental search starts from the UniRef profile; its hits are re-aligned against its own last profile
        plan += [
            ["search", prof, env, j("res_env"), j("tmp_env"), *_search_flags(s, eload)],
            *_expand_align_filter(work, qdb, prof, j("tmp_env/latest/profile_1"), env + esuf, "env", eload, threads),
        ]
        merged.append(j("env.a3m"))
    plan += [["mergedbs", qdb, j("final.a3m"), *merged] if len(merged) > 1 else ["mvdb", merged[0], j("final.a3m")],
             ["unpackdb", j("final.a3m"), j("out"), "--unpack-name-mode", "0", "--unpack-suffix", ".a3m"]]  # fmt: skip
    return plan


def plan_pair(s: MmseqsSettings, work: str, fasta: str, env: bool = False) -> list[list[str]]:
    """Paired alignment of the chains in ``fasta`` (one complex): ``work/pair_out/<chain index>.a3m`` hold the same
    number of rows in the same taxon order."""
    j = lambda n: os.path.join(work, n)  # noqa: E731
    threads = str(s.threads)
    name = s.env_db if env else s.uniref_db
    suf, load = detect_db_mode(s.db_dir, name)
    db = os.path.join(s.db_dir, name)
    qdb = j("qdb")
    pair = ["--db-load-mode", load, "--threads", threads, "--pairing-mode", str(s.pairing_mode), "--pairing-dummy-mode", "0"]
    return [
        ["createdb", fasta, qdb, "--shuffle", "0"],
        ["search", qdb, db, j("res"), j("tmp"), *_search_flags(s, load)],
        ["expandaln", qdb, db + suf, j("res"), db + suf, j("res_exp"), "--db-load-mode", load, "--threads", threads,
         "--expansion-mode", "0", "-e", "inf"],
        ["align", qdb, db + suf, j("res_exp"), j("res_exp_realign"), "--db-load-mode", load, "--threads", threads, "-e", "0.001",
         "--max-accept", "1000000", "-c", "0.5", "--cov-mode", "1"],
        ["pairaln", qdb, db, j("res_exp_realign"), j("res_exp_realign_pair"), *pair],
        ["align", qdb, db + suf, j("res_exp_realign_pair"), j("res_exp_realign_pair_bt"), "--db-load-mode", load, "--threads", threads,
         "-e", "inf", "-a"],
        ["pairaln", qdb, db, j("res_exp_realign_pair_bt"), j("res_final"), *pair],
        ["result2msa", qdb, db + suf, j("res_final"), j("pair.a3m"), "--db-load-mode", load, "--threads", threads,
         "--msa-format-mode", "5"],
        ["unpackdb", j("pair.a3m"), j("pair_out"), "--unpack-name-mode", "0", "--unpack-suffix", ".a3m"],
    ]  # fmt: skip


def run_plan(plan: list[list[str]], binary: str = "mmseqs", log=None) -> None:
    exe = shutil.which(binary) or (binary if os.path.isfile(binary) and os.access(binary, os.X_OK) else None)
    if exe is None:
        raise RuntimeError(f"{binary!r} is not on PATH: install MMseqs2, use the MSA server, or give precomputed alignments")
    for argv in plan:
        if log:
            log(" ".join([binary, *argv]))
        done = subprocess.run([exe, *argv], capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"mmseqs {argv[0]} failed ({done.returncode}): {done.stderr[-2000:]}")


@dataclasses.dataclass
class TemplateHit:
    query: str
    target: str
    identity: float
    aln_len: int
    q_start: int
    q_end: int
    t_start: int
    t_end: int
    evalue: float
    bits: float
    cigar: str


def parse_m8(text: str) -> dict[str, list[TemplateHit]]:
    """Template hits per query id from an m8 table in ``M8_COLUMNS`` order; malformed lines are skipped."""
    out: dict[str, list[TemplateHit]] = {}
    for line in text.splitlines():
        f = line.rstrip("\n").split("\t")
        if len(f) < 13:
            continue
        try:
            hit = TemplateHit(f[0], f[1], float(f[2]), int(f[3]), int(f[6]), int(f[7]), int(f[8]), int(f[9]), float(f[10]),
                              float(f[11]), f[12])  # fmt: skip
        except ValueError:
            continue
        out.setdefault(hit.query, []).append(hit)
    return out


def _clean(a3m: str) -> str:
    return a3m.replace("\x00", "")


def sequence_key(sequences: list[str], tag: str) -> str:
    return hashlib.sha1((tag + "|" + "|".join(sequences)).encode()).hexdigest()


def search_monomer_batch(sequences: list[str], settings: MmseqsSettings, cache=None, work_dir: str | None = None, log=None):
    """Unpaired alignments (and template hits) for many sequences with one pass over the databases.

    Returns ``[{"a3m": text, "m8": text or ""}]`` in the order of ``sequences``; duplicates are searched once; cached
    sequences are not searched at all.
    """
    tag = f"mono:{settings.uniref_db}:{int(settings.use_env)}:{int(settings.use_templates)}"
    results: dict[str, dict] = {}
    todo = []
    for seq in dict.fromkeys(sequences):
        hit = cache.get(sequence_key([seq], tag)) if cache else None
        if hit is not None:
            a3m, _, m8 = hit.partition("\x01")
            results[seq] = {"a3m": a3m, "m8": m8}
        else:
            todo.append(seq)
    if todo:
        with tempfile.TemporaryDirectory(dir=work_dir) as work:
            fasta = os.path.join(work, "query.fasta")
            with open(fasta, "w") as f:
                f.writelines(f">{i}\n{seq}\n" for i, seq in enumerate(todo))
            run_plan(plan_monomer(settings, work, fasta), settings.binary, log)
            m8_by_query: dict[str, list[str]] = {}
            if settings.use_templates and os.path.exists(os.path.join(work, "pdb.m8")):
                with open(os.path.join(work, "pdb.m8")) as f:
                    for line in f:
                        m8_by_query.setdefault(line.split("\t", 1)[0], []).append(line)
            for i, seq in enumerate(todo):
                path = os.path.join(work, "out", f"{i}.a3m")
                if os.path.exists(path):
                    with open(path) as f:
                        a3m = _clean(f.read())
                else:  # no hit at all: the query alone
                    a3m = f">{i}\n{seq}\n"
                m8 = "".join(m8_by_query.get(str(i), []))
                results[seq] = {"a3m": a3m, "m8": m8}
                if cache:
                    cache.put(sequence_key([seq], tag), a3m + "\x01" + m8)
    return [results[seq] for seq in sequences]


def search_pair_batch(complexes: list[list[str]], settings: MmseqsSettings, cache=None, work_dir: str | None = None, env: bool = False,
                      log=None) -> list[list[str]]:
    """Paired alignments: for every complex one A3M per distinct chain sequence, row-aligned across the chains.

    A complex with a single distinct sequence (monomer or homomer) needs no pairing and gets query-only blocks.
    """
    tag = f"pair:{settings.env_db if env else settings.uniref_db}:{settings.pairing_mode}"
    out = []
    for chains in complexes:
        distinct = list(dict.fromkeys(chains))
        if len(distinct) < 2:
            out.append([f">101\n{s}\n" for s in distinct])
            continue
        key = sequence_key(distinct, tag)
        hit = cache.get(key) if cache else None
        if hit is not None:
            out.append(hit.split("\x01"))
            continue
        with tempfile.TemporaryDirectory(dir=work_dir) as work:
            fasta = os.path.join(work, "query.fasta")
            with open(fasta, "w") as f:
                f.writelines(f">{101 + i}\n{seq}\n" for i, seq in enumerate(distinct))
            run_plan(plan_pair(settings, work, fasta, env), settings.binary, log)
            blocks = []
            for i, seq in enumerate(distinct):
                path = os.path.join(work, "pair_out", f"{i}.a3m")
                if os.path.exists(path):
                    with open(path) as f:
                        blocks.append(_clean(f.read()))
                else:
                    blocks.append(f">{101 + i}\n{seq}\n")
        rows = [b.count(">") for b in blocks]
        if len(set(rows)) != 1:  # pairing must give the same number of rows per chain; fall back to the queries alone
            blocks = [f">{101 + i}\n{seq}\n" for i, seq in enumerate(distinct)]
        if cache:
            cache.put(key, "\x01".join(blocks))
        out.append(blocks)
    return out
