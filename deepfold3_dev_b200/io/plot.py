"""Confidence plots (reference: io/plot.py): per-token pLDDT trace and PAE heat map of one sample."""

from __future__ import annotations

import json
import os


def plot_confidences(confidences_json: str, output: str | None = None) -> str:
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError as exc:
        raise RuntimeError("plotting needs matplotlib") from exc
    import numpy as np

    with open(confidences_json) as f:
        c = json.load(f)
    output = output or os.path.splitext(confidences_json)[0] + ".png"
    fig, (a, b) = plt.subplots(1, 2, figsize=(11, 4.5))
    plddt = np.asarray(c["token_plddts"], dtype=float)
    a.plot(plddt, lw=1.0)
    chains = np.asarray(c.get("token_chain_ids", []))
    for edge in np.nonzero(np.diff(chains))[0] if len(chains) else []:
        a.axvline(edge + 0.5, color="k", lw=0.5, alpha=0.4)
    a.set(ylim=(0, 100), xlabel="token", ylabel="pLDDT", title=f"pTM {c.get('ptm', float('nan')):.2f}  ipTM {c.get('iptm') or float('nan'):.2f}")
    im = b.imshow(np.asarray(c["pae"], dtype=float), cmap="Greens_r", vmin=0, vmax=31.75)
    b.set(xlabel="aligned token", ylabel="scored token", title="PAE (Angstrom)")
    fig.colorbar(im, ax=b, fraction=0.046)
    fig.tight_layout()
    fig.savefig(output, dpi=130)
    plt.close(fig)
    return output
