"""Vocabulary and chemistry tables of the feature pipeline (AF3 conventions; reference: data/const.py)."""

from __future__ import annotations

MOL_PROTEIN, MOL_DNA, MOL_RNA, MOL_NONPOLYMER = 0, 1, 2, 3
MOL_TYPE_NAMES = {MOL_PROTEIN: "PROTEIN", MOL_DNA: "DNA", MOL_RNA: "RNA", MOL_NONPOLYMER: "NONPOLYMER"}
MOL_TYPE_IDS = {v: k for k, v in MOL_TYPE_NAMES.items()}

RES_TYPE_COUNT = 31
PROTEIN_RES3 = ("ALA", "ARG", "ASN", "ASP", "CYS", "GLN", "GLU", "GLY", "HIS", "ILE", "LEU", "LYS", "MET", "PHE",
                "PRO", "SER", "THR", "TRP", "TYR", "VAL")  # fmt: skip
RES_TYPE_ORDER: dict[str, int] = {name: i for i, name in enumerate(PROTEIN_RES3)}
RES_TYPE_ORDER.update({"UNK": 20, "-": 21, "A": 22, "G": 23, "C": 24, "U": 25, "DA": 26, "DG": 27, "DC": 28,
                       "DT": 29, "N": 30})  # fmt: skip
RES_TYPE_INDEX_TO_NAME = {v: k for k, v in RES_TYPE_ORDER.items()}
PROTEIN_1TO3 = dict(zip("ARNDCQEGHILKMFPSTWYV", PROTEIN_RES3)) | {"X": "UNK"}
PROTEIN_3TO1 = {v: k for k, v in PROTEIN_1TO3.items()}
RNA_1TO3 = {"A": "A", "G": "G", "C": "C", "U": "U", "N": "N"}
DNA_1TO3 = {"A": "DA", "G": "DG", "C": "DC", "T": "DT", "N": "N"}

MSA_GAP = 21
MSA_VOCAB_SIZE = 32
MSA_MASK = 31
MAX_ATOMS_PER_TOKEN = 24
MAX_MSA_ROWS = 16_384
NUM_ELEMENTS = 128
RESOLUTION_UNKNOWN = 0.0

_BB = ("N", "CA", "C", "O", "CB")  # chemical-component order: O at slot 3, CB at slot 4
# heavy atoms per residue in dense order; GLY has no CB
RESIDUE_ATOMS: dict[str, tuple[str, ...]] = {
    "ALA": _BB,
    "ARG": _BB + ("CG", "CD", "NE", "CZ", "NH1", "NH2"),
    "ASN": _BB + ("CG", "OD1", "ND2"),
    "ASP": _BB + ("CG", "OD1", "OD2"),
    "CYS": _BB + ("SG",),
    "GLN": _BB + ("CG", "CD", "OE1", "NE2"),
    "GLU": _BB + ("CG", "CD", "OE1", "OE2"),
    "GLY": ("N", "CA", "C", "O"),
    "HIS": _BB + ("CG", "ND1", "CD2", "CE1", "NE2"),
    "ILE": _BB + ("CG1", "CG2", "CD1"),
    "LEU": _BB + ("CG", "CD1", "CD2"),
    "LYS": _BB + ("CG", "CD", "CE", "NZ"),
    "MET": _BB + ("CG", "SD", "CE"),
    "PHE": _BB + ("CG", "CD1", "CD2", "CE1", "CE2", "CZ"),
    "PRO": _BB + ("CG", "CD"),
    "SER": _BB + ("OG",),
    "THR": _BB + ("OG1", "CG2"),
    "TRP": _BB + ("CG", "CD1", "CD2", "NE1", "CE2", "CE3", "CZ2", "CZ3", "CH2"),
    "TYR": _BB + ("CG", "CD1", "CD2", "CE1", "CE2", "CZ", "OH"),
    "VAL": _BB + ("CG1", "CG2"),
    "UNK": _BB,
}
_RIBOSE = ("P", "OP1", "OP2", "O5'", "C5'", "C4'", "O4'", "C3'", "O3'", "C2'", "C1'")
_PURINE_A = ("N9", "C8", "N7", "C5", "C6", "N6", "N1", "C2", "N3", "C4")
_PURINE_G = ("N9", "C8", "N7", "C5", "C6", "O6", "N1", "C2", "N2", "N3", "C4")
_PYR_C = ("N1", "C2", "O2", "N3", "C4", "N4", "C5", "C6")
_PYR_U = ("N1", "C2", "O2", "N3", "C4", "O4", "C5", "C6")
_PYR_T = ("N1", "C2", "O2", "N3", "C4", "O4", "C5", "C7", "C6")
RESIDUE_ATOMS.update(
    {
        "A": _RIBOSE + ("O2'",) + _PURINE_A,
        "G": _RIBOSE + ("O2'",) + _PURINE_G,
        "C": _RIBOSE + ("O2'",) + _PYR_C,
        "U": _RIBOSE + ("O2'",) + _PYR_U,
        "DA": _RIBOSE + _PURINE_A,
        "DG": _RIBOSE + _PURINE_G,
        "DC": _RIBOSE + _PYR_C,
        "DT": _RIBOSE + _PYR_T,
        "N": _RIBOSE,
    }
)
# Covalent bonds between the heavy atoms of the standard residues (textbook chemistry; the component dictionary lists
# the same). Needed when a standard residue is tokenised per atom: its atom tokens are then joined in the token bond
# matrix like those of a ligand. Linking atoms to the neighbouring residues: C -> N (peptides), O3' -> P (nucleic acids).
_BACKBONE_BONDS = (("N", "CA"), ("CA", "C"), ("C", "O"))
_SIDE_CHAIN_BONDS: dict[str, tuple[tuple[str, str], ...]] = {
    "ALA": (), "GLY": (), "UNK": (),
    "ARG": (("CB", "CG"), ("CG", "CD"), ("CD", "NE"), ("NE", "CZ"), ("CZ", "NH1"), ("CZ", "NH2")),
    "ASN": (("CB", "CG"), ("CG", "OD1"), ("CG", "ND2")),
    "ASP": (("CB", "CG"), ("CG", "OD1"), ("CG", "OD2")),
    "CYS": (("CB", "SG"),),
    "GLN": (("CB", "CG"), ("CG", "CD"), ("CD", "OE1"), ("CD", "NE2")),
    "GLU": (("CB", "CG"), ("CG", "CD"), ("CD", "OE1"), ("CD", "OE2")),
    "HIS": (("CB", "CG"), ("CG", "ND1"), ("CG", "CD2"), ("ND1", "CE1"), ("CD2", "NE2"), ("CE1", "NE2")),
    "ILE": (("CB", "CG1"), ("CB", "CG2"), ("CG1", "CD1")),
    "LEU": (("CB", "CG"), ("CG", "CD1"), ("CG", "CD2")),
    "LYS": (("CB", "CG"), ("CG", "CD"), ("CD", "CE"), ("CE", "NZ")),
    "MET": (("CB", "CG"), ("CG", "SD"), ("SD", "CE")),
    "PHE": (("CB", "CG"), ("CG", "CD1"), ("CG", "CD2"), ("CD1", "CE1"), ("CD2", "CE2"), ("CE1", "CZ"), ("CE2", "CZ")),
    "PRO": (("CB", "CG"), ("CG", "CD"), ("CD", "N")),
    "SER": (("CB", "OG"),),
    "THR": (("CB", "OG1"), ("CB", "CG2")),
    "TRP": (("CB", "CG"), ("CG", "CD1"), ("CG", "CD2"), ("CD1", "NE1"), ("NE1", "CE2"), ("CD2", "CE2"), ("CD2", "CE3"),
            ("CE2", "CZ2"), ("CE3", "CZ3"), ("CZ2", "CH2"), ("CZ3", "CH2")),
    "TYR": (("CB", "CG"), ("CG", "CD1"), ("CG", "CD2"), ("CD1", "CE1"), ("CD2", "CE2"), ("CE1", "CZ"), ("CE2", "CZ"), ("CZ", "OH")),
    "VAL": (("CB", "CG1"), ("CB", "CG2")),
}  # fmt: skip
_SUGAR_BONDS = (("P", "OP1"), ("P", "OP2"), ("P", "O5'"), ("O5'", "C5'"), ("C5'", "C4'"), ("C4'", "O4'"), ("C4'", "C3'"),
                ("C3'", "O3'"), ("C3'", "C2'"), ("C2'", "C1'"), ("C1'", "O4'"))  # fmt: skip
_PURINE_BONDS = (("C1'", "N9"), ("N9", "C8"), ("C8", "N7"), ("N7", "C5"), ("C5", "C6"), ("C6", "N1"), ("N1", "C2"), ("C2", "N3"),
                 ("N3", "C4"), ("C4", "C5"), ("C4", "N9"))  # fmt: skip
_PYRIMIDINE_BONDS = (("C1'", "N1"), ("N1", "C2"), ("C2", "O2"), ("C2", "N3"), ("N3", "C4"), ("C4", "C5"), ("C5", "C6"), ("C6", "N1"))
_BASE_BONDS = {"A": _PURINE_BONDS + (("C6", "N6"),), "G": _PURINE_BONDS + (("C6", "O6"), ("C2", "N2")),
               "C": _PYRIMIDINE_BONDS + (("C4", "N4"),), "U": _PYRIMIDINE_BONDS + (("C4", "O4"),),
               "T": _PYRIMIDINE_BONDS + (("C4", "O4"), ("C5", "C7"))}  # fmt: skip
RESIDUE_BONDS: dict[str, tuple[tuple[str, str], ...]] = {
    name: _BACKBONE_BONDS + ((("CA", "CB"),) if name != "GLY" else ()) + side for name, side in _SIDE_CHAIN_BONDS.items()
}
for _base in "AGCU":
    RESIDUE_BONDS[_base] = _SUGAR_BONDS + (("C2'", "O2'"),) + _BASE_BONDS[_base]
for _base in "AGCT":
    RESIDUE_BONDS["D" + _base] = _SUGAR_BONDS + _BASE_BONDS[_base]
RESIDUE_BONDS["N"] = _SUGAR_BONDS
POLYMER_LINK = {MOL_PROTEIN: ("C", "N"), MOL_RNA: ("O3'", "P"), MOL_DNA: ("O3'", "P")}  # (atom of residue i, atom of residue i + 1)

# Buffer, cryo-protectant and precipitant molecules that are dropped from X-ray entries (AF3 supplement 2.5.4, table 9):
# they are not part of the biological assembly and would otherwise become spurious ligand tokens.
CRYSTALLIZATION_AIDS = frozenset({"SO4", "GOL", "EDO", "PO4", "ACT", "PEG", "DMS", "TRS", "PGE", "PG4", "FMT", "EPE", "MPD",
                                  "MES", "CD", "IOD"})  # fmt: skip

ELEMENT_NUMBER = {"H": 1, "C": 6, "N": 7, "O": 8, "F": 9, "P": 15, "S": 16, "CL": 17, "SE": 34, "BR": 35, "I": 53,
                  "MG": 12, "ZN": 30, "FE": 26, "CA": 20, "NA": 11, "K": 19, "MN": 25, "CU": 29, "CO": 27, "NI": 28}  # fmt: skip


def atom_element(atom_name: str) -> int:
    """Atomic number of a standard-residue atom from the first letter of its name."""
    return ELEMENT_NUMBER.get(atom_name[0], 6)


def encode_atom_name(name: str, length: int = 4) -> list[int]:
    """AF3 atom-name characters: ``ord(c) - 32`` padded with 0 to ``length``."""
    codes = [ord(c) - 32 for c in name[:length]]
    return codes + [0] * (length - len(codes))


def representative_atom(res_name: str, mol_type: int) -> str:
    """Token-centre atom: CA for proteins, C1' for nucleic acids."""
    return "CA" if mol_type == MOL_PROTEIN else "C1'"


def frame_atoms(mol_type: int) -> tuple[str, str, str]:
    """Atoms ``(a, b, c)`` of the token frame: (N, CA, C) for proteins, (C1', C3', C4') for nucleic acids."""
    return ("N", "CA", "C") if mol_type == MOL_PROTEIN else ("C1'", "C3'", "C4'")
