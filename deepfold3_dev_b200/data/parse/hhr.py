"""HHsearch / HHblits result files (``.hhr``) -> template hits (reference: data/parse/hhr.py).

An ``.hhr`` file has a summary table followed by one block per hit: a ``>`` header line, a statistics line
(``Probab=.. E-value=.. Aligned_cols=.. Sum_probs=..``) and alignment chunks with ``Q <name> <start> <seq> <end>``
and ``T <name> <start> <seq> <end>`` lines (consensus / ss lines are skipped).
"""

from __future__ import annotations

import dataclasses
import re


@dataclasses.dataclass(frozen=True)
class TemplateHit:
    index: int
    pdb_id: str
    chain_id: str
    aligned_cols: int
    sum_probs: float
    e_value: float
    query_sequence: str
    hit_sequence: str
    indices_query: list
    indices_hit: list

    @property
    def query_to_hit_mapping(self) -> dict:
        return {q: h for q, h in zip(self.indices_query, self.indices_hit) if q != -1 and h != -1}


_STATS = re.compile(r"(\w[\w-]*)=\s*([^\s]+)")
_NAME = re.compile(r">\s*(\w{4})_(\w+)")


def _indices(seq: str, start: int) -> list[int]:
    out, pos = [], start
    for c in seq:
        if c == "-":
            out.append(-1)
        else:
            out.append(pos)
            pos += 1
    return out


def parse_hhr(text: str) -> list[TemplateHit]:
    blocks = re.split(r"^No (\d+)\s*$", text, flags=re.M)
    hits = []
    for k in range(1, len(blocks) - 1, 2):
        number, body = int(blocks[k]), blocks[k + 1]
        lines = [ln for ln in body.splitlines() if ln.strip()]
        if not lines or not lines[0].startswith(">"):
            continue
        m = _NAME.match(lines[0])
        pdb_id, chain = (m.group(1).upper(), m.group(2)) if m else (lines[0][1:5].upper(), "A")
        stats = dict(_STATS.findall(lines[1])) if len(lines) > 1 else {}
        q_seq, t_seq, q_start, t_start = [], [], None, None
        for ln in lines[2:]:
            parts = ln.split()
            if len(parts) >= 5 and parts[0] in ("Q", "T") and parts[1] not in ("Consensus", "ss_pred", "ss_dssp", "ss_conf"):
                start, seq = int(parts[2]), parts[3]
                if parts[0] == "Q":
                    q_seq.append(seq)
                    q_start = start if q_start is None else q_start
                else:
                    t_seq.append(seq)
                    t_start = start if t_start is None else t_start
        q, t = "".join(q_seq), "".join(t_seq)
        if not q or len(q) != len(t):
            continue
        hits.append(TemplateHit(number, pdb_id, chain, int(float(stats.get("Aligned_cols", 0))),
                                float(stats.get("Sum_probs", 0.0)), float(stats.get("E-value", 0.0)), q, t,
                                _indices(q, (q_start or 1) - 1), _indices(t, (t_start or 1) - 1)))  # fmt: skip
    return hits
