"""MSA search back ends: a local ``mmseqs`` pipeline and the ColabFold MMseqs2 API
(reference: data/msa/mmseqs2.py:452-1863).

Both are process boundaries: the local search shells out to the ``mmseqs`` binary, the remote one talks HTTP.
Results (A3M text per query) are cached on disk by the SHA-1 of the query, so a repeated query never searches twice.
"""

from __future__ import annotations

import hashlib
import io
import json
import os
import shutil
import subprocess
import tarfile
import tempfile
import time
import urllib.request

DEFAULT_HOST = "https://api.colabfold.com"


def _key(seqs: list[str], tag: str) -> str:
    return hashlib.sha1((tag + "|" + "|".join(seqs)).encode()).hexdigest()


class MsaCache:
    def __init__(self, root: str):
        self.root = root
        os.makedirs(root, exist_ok=True)

    def get(self, key: str) -> str | None:
        path = os.path.join(self.root, key + ".a3m")
        if os.path.exists(path):
            with open(path) as f:
                return f.read()
        return None

    def put(self, key: str, a3m: str) -> None:
        tmp = os.path.join(self.root, key + ".a3m.tmp")
        with open(tmp, "w") as f:
            f.write(a3m)
        os.replace(tmp, os.path.join(self.root, key + ".a3m"))


def search_local(sequence: str, db: str, cache: MsaCache | None = None, binary: str = "mmseqs", threads: int = 8,
                 sensitivity: float = 8.0, extra_args: tuple = ()) -> str:  # fmt: skip
    """``mmseqs createdb / search / result2msa`` for one sequence against ``db``; returns A3M text."""
    key = _key([sequence], "local:" + os.path.basename(db))
    if cache and (hit := cache.get(key)) is not None:
        return hit
    exe = shutil.which(binary)
    if exe is None:
        raise RuntimeError(f"{binary!r} is not on PATH: install MMseqs2 or give precomputed alignments")
    with tempfile.TemporaryDirectory() as tmp:
        fasta = os.path.join(tmp, "q.fasta")
        with open(fasta, "w") as f:
            f.write(f">query\n{sequence}\n")
        run = lambda *a: subprocess.run([exe, *a], check=True, capture_output=True, text=True)  # noqa: E731
        qdb, res, msa = (os.path.join(tmp, n) for n in ("qdb", "res", "msa.a3m"))
        run("createdb", fasta, qdb)
        run("search", qdb, db, res, os.path.join(tmp, "tmp"), "--threads", str(threads), "-s", str(sensitivity), "--num-iterations", "3", *extra_args)
        run("result2msa", qdb, db, res, msa, "--msa-format-mode", "6", "--threads", str(threads))
        with open(msa) as f:
            a3m = f.read().replace("\x00", "")
    if cache:
        cache.put(key, a3m)
    return a3m


def search_server(sequences: list[str], cache: MsaCache | None = None, host: str = DEFAULT_HOST, pairing: bool = False,
                  poll_s: float = 5.0, timeout_s: float = 3600.0, opener=urllib.request.urlopen) -> list[str]:  # fmt: skip
    """Submit to the ColabFold API (``ticket/msa`` or ``ticket/pair``), poll, download; one A3M per input sequence."""
    key = _key(sequences, "server:pair" if pairing else "server:msa")
    if cache and (hit := cache.get(key)) is not None:
        return hit.split("\x00")[: len(sequences)]
    query = "".join(f">{101 + i}\n{s}\n" for i, s in enumerate(sequences))
    endpoint = "pair" if pairing else "msa"
    data = urllib.parse.urlencode({"q": query, "mode": "pairgreedy" if pairing else "env"}).encode()
    ticket = json.load(opener(urllib.request.Request(f"{host}/ticket/{endpoint}", data=data), timeout=60))
    t0 = time.time()
    while ticket.get("status") in ("PENDING", "RUNNING", "UNKNOWN"):
        if time.time() - t0 > timeout_s:
            raise TimeoutError("MSA server did not finish in time")
        time.sleep(poll_s)
        ticket = json.load(opener(f"{host}/ticket/{ticket['id']}", timeout=60))
    if ticket.get("status") != "COMPLETE":
        raise RuntimeError(f"MSA server returned {ticket.get('status')!r}")
    blob = opener(f"{host}/result/download/{ticket['id']}", timeout=600).read()
    per_query: dict[int, list[str]] = {}
    with tarfile.open(fileobj=io.BytesIO(blob)) as tar:
        for member in tar.getmembers():
            if not member.name.endswith(".a3m"):
                continue
            text = tar.extractfile(member).read().decode().replace("\x00", "")
            current = None
            for line in text.splitlines():
                if line.startswith(">") and line[1:].split()[0].isdigit() and int(line[1:].split()[0]) >= 101:
                    current = int(line[1:].split()[0]) - 101
                if current is not None:
                    per_query.setdefault(current, []).append(line)
    out = ["\n".join(per_query.get(i, [f">{101 + i}", s])) + "\n" for i, s in enumerate(sequences)]
    if cache:
        cache.put(key, "\x00".join(out))
    return out
