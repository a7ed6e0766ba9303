"""Structure-accuracy metrics and the predicted-vs-experimental comparison (reference: repo-root scripts
struct_accuracy.py, gdt_ts.py, usalign_tm.py, check_chirality.py and the FoldBench harness under bench/)."""

from .metrics import dockq, gdt_ts, kabsch, lddt, rmsd, tm_score  # noqa: F401
