"""Evaluation-time diagnostics of the complex language model (reference: complexlm/diagnostics.py:1-310).

``permutation_sensitivity``: how much the per-token hidden states and the loss move when the chains of a complex are
re-ordered (zero for pattern ``cg``: chain-scoped layers do not see the order, complex-scoped layers have no positions;
non-zero for the global-rotary baseline ``r``). ``attention_sink_stats``: per layer, how concentrated attention is,
reported against the uniform baseline of each query's own scope (a chain-scoped query can give a key at most the share
its chain allows, so raw maxima are not comparable between kinds).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .data import Example, pack
from .model import IGNORE_INDEX, ComplexLM, PackedBatch


@torch.no_grad()
def permutation_sensitivity(model: ComplexLM, example: Example, order: list[int]) -> dict[str, float]:
    """Compare one complex with its chains in the given order against the original order."""
    was_training = model.training
    model.eval()

    def run(ex: Example):
        b = pack([ex]).to(next(model.parameters()).device)
        out = model(b, return_hidden=True)
        loss = F.cross_entropy(out.logits.float(), b.labels, ignore_index=IGNORE_INDEX) if (b.labels != IGNORE_INDEX).any() else out.logits.sum() * 0
        return out.hidden[-1].float(), float(loss), b

    h0, l0, b0 = run(example)
    pick = lambda xs: [xs[i] for i in order]  # noqa: E731
    shuffled = Example(pick(example.tokens), pick(example.labels), pick(example.starts), example.entity[order], pick(example.iface),
                       example.iface_known, example.source)  # fmt: skip
    h1, l1, _ = run(shuffled)
    # bring the permuted run back to the original token order
    lens = [len(t) for t in example.tokens]
    starts0 = [sum(lens[:i]) for i in range(len(lens))]
    back = torch.cat([torch.arange(starts0[i], starts0[i] + lens[i]) for i in order]).to(h0.device)
    h1_aligned = torch.empty_like(h1)
    h1_aligned[back] = h1
    cos = F.cosine_similarity(h0, h1_aligned, dim=-1)
    pooled = F.cosine_similarity(h0.mean(0), h1_aligned.mean(0), dim=0)
    model.train(was_training)
    return {"loss_change": l1 - l0, "token_cosine_mean": float(cos.mean()), "token_cosine_min": float(cos.min()),
            "pooled_cosine": float(pooled)}  # fmt: skip


@torch.no_grad()
def attention_sink_stats(model: ComplexLM, batch: PackedBatch) -> list[dict]:
    """Per layer: mean over heads and queries of the largest key weight, of the top-5 mass, and the largest weight as a
    multiple of the uniform weight of the query's scope (``x_uniform``) and as a fraction of 1 (``frac_of_ceiling``)."""
    was_training = model.training
    model.eval()
    out = model(batch, return_attn=True)
    rows = []
    for blk, w in zip(model.blocks, out.attentions or []):
        allowed = blk.attn.allowed(batch)  # [T, T]
        scope = allowed.sum(-1).clamp(min=1).float()  # keys each query may see
        top = w.amax(-1)  # [H, T]
        top5 = w.topk(min(5, w.shape[-1]), dim=-1).values.sum(-1)
        rows.append({"kind": blk.kind, "max_mass": float(top.mean()), "top5_mass": float(top5.mean()),
                     "x_uniform": float((top * scope).mean()), "frac_of_ceiling": float(top.mean())})  # fmt: skip
    model.train(was_training)
    return rows
