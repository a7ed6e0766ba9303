"""A small STAR/CIF reader: text -> blocks -> categories -> columns.

The reference reads mmCIF through gemmi (data/prepare/structure.py:47-125); this module is a dependency-free reader for
the subset of the grammar that the PDB and ModelCIF archives use: ``data_`` blocks, ``loop_`` tables, single items,
quoted values, ``;`` text fields and ``#`` comments. A category that appears twice in one block (seen in some ModelCIF
files) keeps its first occurrence, which is what the reference's lenient fallback does.
"""

from __future__ import annotations

import gzip
import re
from dataclasses import dataclass, field

_QUOTED = re.compile(r"""\s*(?:'((?:[^']|'(?=\S))*)'|"((?:[^"]|"(?=\S))*)"|(\#.*)|(\S+))""")
MISSING = ("?", ".")


@dataclass
class CifBlock:
    name: str
    categories: dict[str, dict[str, list[str]]] = field(default_factory=dict)

    def table(self, category: str) -> dict[str, list[str]]:
        """Columns of ``_category.*`` keyed by item name (empty dict when absent)."""
        return self.categories.get(category.lstrip("_"), {})

    def rows(self, category: str) -> int:
        t = self.table(category)
        return len(next(iter(t.values()))) if t else 0

    def column(self, category: str, item: str, default: str | None = None) -> list[str]:
        t = self.table(category)
        if item in t:
            return t[item]
        return [default] * self.rows(category) if default is not None else []

    def value(self, category: str, item: str) -> str | None:
        col = self.table(category).get(item)
        if not col or col[0] in MISSING:
            return None
        return col[0]


def _tokens(text: str):
    """Yield ``(is_quoted, token)``; a quoted token is always a value, never a keyword or tag."""
    lines = text.splitlines()
    i, n = 0, len(lines)
    while i < n:
        line = lines[i]
        if line.startswith(";"):
            buf = [line[1:]]
            i += 1
            while i < n and not lines[i].startswith(";"):
                buf.append(lines[i])
                i += 1
            yield True, "\n".join(buf).strip()
            i += 1
            continue
        i += 1
        if not line or line[0] == "#":
            continue
        if "'" not in line and '"' not in line and "#" not in line:
            for tok in line.split():
                yield False, tok
            continue
        for m in _QUOTED.finditer(line):
            if m.group(3) is not None:
                break
            if m.group(4) is not None:
                yield False, m.group(4)
            else:
                yield True, m.group(1) if m.group(1) is not None else m.group(2)


def parse_cif(text: str) -> list[CifBlock]:
    blocks: list[CifBlock] = []
    block: CifBlock | None = None
    loop_tags: list[tuple[str, str]] | None = None
    loop_cols: list[list[str]] = []
    loop_pos = 0
    pending: tuple[str, str] | None = None
    skip_loop = False

    def split_tag(tag: str) -> tuple[str, str]:
        cat, _, item = tag[1:].partition(".")
        return cat, item

    def close_loop():
        nonlocal loop_tags, loop_cols, loop_pos, skip_loop
        loop_tags, loop_cols, loop_pos, skip_loop = None, [], 0, False

    for quoted, tok in _tokens(text):
        low = tok.lower() if not quoted else ""
        if not quoted and low.startswith("data_"):
            close_loop()
            block = CifBlock(tok[5:])
            blocks.append(block)
            continue
        if block is None:
            continue
        if not quoted and low == "loop_":
            close_loop()
            loop_tags = []
            continue
        if not quoted and tok.startswith("_"):
            cat, item = split_tag(tok)
            if loop_tags is not None and not loop_pos and (not loop_cols or len(loop_cols[0]) == 0):
                # still in the header of a loop
                if not loop_tags:
                    skip_loop = cat in block.categories
                loop_tags.append((cat, item))
                col: list[str] = []
                loop_cols.append(col)
                if not skip_loop:
                    block.categories.setdefault(cat, {})[item] = col
                continue
            close_loop()
            pending = (cat, item)
            continue
        # a value
        if pending is not None:
            cat, item = pending
            table = block.categories.setdefault(cat, {})
            table.setdefault(item, [tok])
            pending = None
        elif loop_tags:
            loop_cols[loop_pos].append(tok)
            loop_pos = (loop_pos + 1) % len(loop_tags)
    return blocks


def read_cif(path: str) -> list[CifBlock]:
    """Read ``.cif`` or ``.cif.gz`` (``.zst`` needs the zstandard package and raises a clear error without it)."""
    p = str(path)
    if p.endswith(".gz"):
        with gzip.open(p, "rt", encoding="utf-8", errors="replace") as f:
            return parse_cif(f.read())
    if p.endswith(".zst"):
        try:
            import zstandard
        except ImportError as exc:
            raise RuntimeError(f"{p}: reading .zst files needs the 'zstandard' package") from exc
        with open(p, "rb") as f:
            return parse_cif(zstandard.ZstdDecompressor().stream_reader(f).read().decode("utf-8", "replace"))
    with open(p, encoding="utf-8", errors="replace") as f:
        return parse_cif(f.read())
