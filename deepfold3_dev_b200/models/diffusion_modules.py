"""Diffusion-head building blocks: schedules, augmentation, conditioning, the 24-block transformer.

Reference: model/diffusion.py:96-900. Tensors that vary per diffusion sample
carry an explicit sample axis ``S`` after the batch axis (``[B, S, N, ...]``);
state shared by the samples of one molecule stays ``[B, ...]`` and broadcasts.
"""

from __future__ import annotations

import dataclasses
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .atom_attention import AtomEncoderStatic
from .primitives import (
    LayerNorm,
    LinearNoBias,
    biased_linear,
    budget_rows,
    gemm_itemsize,
    make_transition_block,
    map_pair_rows,
    map_row_chunks,
    small_normal_init_,
)

FOURIER_INIT_SEED = 314159  # fixed basis for the noise-level embedding, same across runs and ranks


@dataclasses.dataclass
class DiffusionStatic:
    """Noise-independent state for one batch of (molecule, trunk output) pairs."""

    encoder_static: AtomEncoderStatic
    pair_cond: torch.Tensor  # [B, N, N, c_pair]
    single_cond_pre_noise: torch.Tensor  # [B, N, c_single]
    ref_pos: torch.Tensor  # [B, N, M, 3]
    ref_mask: torch.Tensor  # [B, N, M]
    seq_mask: torch.Tensor  # [B, N]
    pair_logits: tuple[torch.Tensor, ...] | None = None  # per super-block [B, sbs*H, N, N], padding mask folded in


@dataclasses.dataclass(frozen=True)
class GuidanceTerm:
    """One classifier-free-guidance term: ``D += (scale - 1) * (D_cond - D_uncond)`` inside ``sigma_range``."""

    scale: float
    pair_keep: torch.Tensor | None = None
    sigma_range: tuple[float, float] | None = None


def noise_schedule(t, sigma_data=16.0, smin=0.0004, smax=160.0, p=7.0):
    """``sigma_data * (smax^(1/p) + t (smin^(1/p) - smax^(1/p)))^p``."""
    return sigma_data * (smax ** (1 / p) + t * (smin ** (1 / p) - smax ** (1 / p))) ** p


def random_rigid_transforms(shape, device, generator=None):
    """Rotations ``[*shape, 3, 3]`` by Gram-Schmidt of two normal vectors, and translations ``[*shape, 3]``.

    Draw order (v0 block, v1 block, translation block) follows the reference's
    batched sampler (diffusion.py:352-382) so a seeded generator gives the same
    transforms.
    """
    v0 = torch.randn(*shape, 3, device=device, generator=generator)
    v1 = torch.randn(*shape, 3, device=device, generator=generator)
    trans = torch.randn(*shape, 3, device=device, generator=generator)
    e0 = v0 / v0.norm(dim=-1, keepdim=True).clamp(min=1e-10)
    v1 = v1 - e0 * (v1 * e0).sum(-1, keepdim=True)
    e1 = v1 / v1.norm(dim=-1, keepdim=True).clamp(min=1e-10)
    e2 = torch.linalg.cross(e0, e1)
    return torch.stack([e0, e1, e2], dim=-2), trans


def augment(positions: torch.Tensor, mask: torch.Tensor, generator=None) -> torch.Tensor:
    """Centre each sample on its masked mean, rotate and translate it at random, zero masked atoms (fp32 math).

    ``positions``: ``[B, S, N, M, 3]``; ``mask``: ``[B, N, M]``. One batched
    expression replaces the reference's per-sample Python loop.
    """
    B, S = positions.shape[:2]
    rot, trans = random_rigid_transforms((B, S), positions.device, generator)
    m = mask.float()[:, None, :, :, None]
    p32 = positions.float()
    center = (p32 * m).sum(dim=(2, 3), keepdim=True) / m.sum(dim=(2, 3), keepdim=True).clamp(min=1e-6)
    out = torch.einsum("bsnmi,bsij->bsnmj", p32 - center, rot) + trans[:, :, None, None, :]
    return (out * m).to(positions.dtype)


def build_diffusion_clean_mask(asym_id, seq_mask, num_samples, *, prob, mode="chain", min_frac=0.25, max_frac=0.75):
    """``[B, S, N]`` bool of tokens handed to the denoiser clean (masked / partial diffusion), or ``None``.

    Each sample fires with probability ``prob``; a fired sample keeps a random
    proper subset of chains (``mode='chain'``) or a contiguous span clean
    (reference: diffusion.py:155-209).
    """
    if prob <= 0.0 or num_samples <= 0:
        return None
    B, N = asym_id.shape
    dev = asym_id.device
    fire = torch.rand(B, num_samples, device=dev) < prob
    if not bool(fire.any()):
        return None
    out = torch.zeros(B, num_samples, N, dtype=torch.bool, device=dev)
    for b in range(B):
        valid = seq_mask[b].bool()
        n_valid = int(valid.sum())
        if n_valid < 4:
            continue
        chains = asym_id[b][valid].unique()
        valid_idx = valid.nonzero(as_tuple=True)[0]
        for s in range(num_samples):
            if not bool(fire[b, s]):
                continue
            frac = min_frac + float(torch.rand((), device=dev)) * (max_frac - min_frac)
            if mode == "chain" and chains.numel() >= 2:
                perm = chains[torch.randperm(chains.numel(), device=dev)]
                k = max(1, min(int(chains.numel()) - 1, int(round(frac * float(chains.numel())))))
                out[b, s] = (asym_id[b].unsqueeze(-1) == perm[:k]).any(-1) & valid
            else:
                ln = max(1, min(n_valid - 1, int(round(frac * n_valid))))
                start = int(torch.randint(0, n_valid - ln + 1, (), device=dev))
                out[b, s, valid_idx[start : start + ln]] = True
    return out


def interface_pair_keep(asym_id):
    """``[.., N, N]`` bool, True on intra-chain pairs."""
    return asym_id.unsqueeze(-1) == asym_id.unsqueeze(-2)


def draw_interface_pair_keep(asym_id, seq_mask, generator=None):
    """Random drop of inter-chain pair blocks, at least one; ``None`` if some element has a single chain."""
    B, N = asym_id.shape
    dev = asym_id.device
    keep = torch.ones(B, N, N, dtype=torch.bool, device=dev)
    for b in range(B):
        valid = seq_mask[b].bool()
        chains = asym_id[b][valid].unique()
        C = chains.numel()
        if C < 2:
            return None
        r = torch.rand((), generator=generator, device=dev)
        drop = torch.triu(torch.rand(C, C, generator=generator, device=dev) < r, diagonal=1)
        if not bool(drop.any()):
            iu = torch.triu_indices(C, C, offset=1, device=dev)
            pick = int(torch.randint(iu.shape[1], (), generator=generator, device=dev))
            drop[iu[0, pick], iu[1, pick]] = True
        drop = drop | drop.T
        idx = torch.searchsorted(chains, asym_id[b]).clamp_(max=C - 1)
        keep[b] = ~drop[idx.unsqueeze(-1), idx.unsqueeze(-2)] | ~(valid.unsqueeze(-1) & valid.unsqueeze(-2))
    return keep


def cond_drop_stats(asym_id, seq_mask, *, use_conditioning: bool, pair_keep):
    """0-d indicator tensors describing this forward's conditioning drop, for logging."""
    dev = seq_mask.device
    interface, full = pair_keep is not None, not use_conditioning
    out = {
        "none": torch.tensor(float(not full and not interface), device=dev),
        "full": torch.tensor(float(full), device=dev),
        "interface": torch.tensor(float(interface), device=dev),
    }
    if asym_id is not None:
        valid = seq_mask.bool()
        multi = all(asym_id[b][valid[b]].unique().numel() >= 2 for b in range(asym_id.shape[0]))
        out["multichain"] = torch.tensor(float(multi), device=dev)
        if interface:
            inter = (valid.unsqueeze(-1) & valid.unsqueeze(-2)) & ~interface_pair_keep(asym_id)
            out["interface_pair_frac"] = (~pair_keep & inter).sum() / inter.sum().clamp(min=1)
    return out


@torch.no_grad()
def null_pair_stats(null_pair, pair, asym_id, seq_mask):
    """Norm and cosine diagnostics of the learned fill vector against the trunk pair."""
    v, z = null_pair.detach().float(), pair.detach().float()
    valid = seq_mask.bool()
    pv = valid.unsqueeze(-1) & valid.unsqueeze(-2)
    out = {"norm": v.norm()}
    out["norm_ratio"] = out["norm"] / z.norm(dim=-1)[pv].mean().clamp(min=1e-12)
    same = interface_pair_keep(asym_id) if asym_id is not None else torch.ones_like(pv)
    for name, m in (("intra", pv & same), ("inter", pv & ~same)):
        if bool(m.any()):
            out[f"cos_{name}"] = F.cosine_similarity(v, z[m].mean(0), dim=0)
    return out


def mask_trunk_pair(embeddings: dict, pair_keep, fill=None) -> dict:
    """Copy of ``embeddings`` whose pair is zero (or ``fill``) where ``pair_keep`` is False."""
    pair = embeddings["pair"]
    keep = pair_keep.unsqueeze(-1)
    if fill is None:
        return {**embeddings, "pair": pair * keep.to(pair.dtype)}
    return {**embeddings, "pair": torch.where(keep, pair, fill.to(pair.dtype))}


class DiffusionTransformerBlock(nn.Module):
    """AdaLN-zero attention + AdaLN-zero SwiGLU feed-forward (reference: diffusion.py:385-594)."""

    def __init__(self, c, c_single_cond, num_heads=16, key_dim=None, value_dim=None, num_intermediate_factor=2,
                 optim=None, cond_bias_init_beta=None):  # fmt: skip
        super().__init__()
        key_dim = c if key_dim is None else key_dim
        value_dim = c if value_dim is None else value_dim
        assert key_dim % num_heads == 0 and value_dim % num_heads == 0
        self.num_heads = num_heads
        self.key_dim_per_head = key_dim // num_heads
        self.val_dim_per_head = value_dim // num_heads
        self.scale = self.key_dim_per_head**-0.5
        hidden = c * num_intermediate_factor
        self.attn_norm = LayerNorm(c, elementwise_affine=False)
        self.attn_cond_norm_w = nn.Parameter(torch.ones(c_single_cond))
        self.attn_cond_scale = biased_linear(c_single_cond, c, "zeros")
        self.attn_cond_bias = LinearNoBias(c_single_cond, c, initializer="zeros")
        self.to_q = biased_linear(c, key_dim, "linear")
        self.to_k = LinearNoBias(c, key_dim)
        self.to_v = LinearNoBias(c, value_dim)
        self.to_g = LinearNoBias(c, value_dim, initializer="zeros")
        self.out_proj = LinearNoBias(value_dim, c)
        self.zero_cond = biased_linear(c_single_cond, c, "zeros", bias_value=-2.0)
        self.ffn_norm = LayerNorm(c, elementwise_affine=False)
        self.ffn_cond_norm_w = nn.Parameter(torch.ones(c_single_cond))
        self.ffn_cond_scale = biased_linear(c_single_cond, c, "zeros")
        self.ffn_cond_bias = LinearNoBias(c_single_cond, c, initializer="zeros")
        self.ffn_linear1 = LinearNoBias(c, hidden * 2, initializer="relu")
        self.ffn_linear2 = LinearNoBias(hidden, c)
        self.ffn_zero_cond = biased_linear(c_single_cond, c, "zeros", bias_value=-2.0)
        if cond_bias_init_beta is not None:
            if cond_bias_init_beta <= 0:
                raise ValueError(f"cond_bias_init_beta must be > 0, got {cond_bias_init_beta}")
            small_normal_init_(self.attn_cond_bias.weight, cond_bias_init_beta)
            small_normal_init_(self.ffn_cond_bias.weight, cond_bias_init_beta)

    def run(self, x, cond_norm, single_cond, pair_logits):
        """``x`` ``[B, S, N, c]``; ``cond_norm`` = parameter-free LN of ``single_cond`` ``[B, S|1, N, cs]``;
        ``pair_logits`` ``[B, H, N, N]`` with the padding mask already added."""
        B, S, N, _ = x.shape
        H, Dk, Dv = self.num_heads, self.key_dim_per_head, self.val_dim_per_head
        # adaptive LayerNorm and the gated residual updates go through ops.ada_norm / ops.gated_residual: one kernel each
        # way under bf16 autocast on a GPU (the result of ada_norm is then the bf16 tensor the projections read), the
        # same arithmetic written out in PyTorch everywhere else
        # the conditioning LayerNorm's weight is folded into the two projections that read it ((c * w) W^T = c (W * w)^T):
        # a [c, cs] product instead of an element-wise pass over the [B, S, N, cs] activations, forward and backward
        wa = self.attn_cond_norm_w
        xn = ops.ada_norm(x, ops.linear(cond_norm, self.attn_cond_scale.weight * wa, self.attn_cond_scale.bias),
                          ops.linear(cond_norm, self.attn_cond_bias.weight * wa), self.attn_norm.eps)
        q = self.to_q(xn).view(B, S, N, H, Dk).transpose(2, 3)
        kv = ops.stacked_linear(xn, self.to_k.weight, self.to_v.weight)  # keys and values: one product
        k = kv[..., : H * Dk].view(B, S, N, H, Dk).transpose(2, 3)
        v = kv[..., H * Dk :].view(B, S, N, H, Dv).transpose(2, 3)
        out = ops.pair_bias_attention(q, k, v, pair_logits, None, self.scale, fp32_qk=True)
        out = ops.sigmoid_gate_mul(xn, self.to_g.weight, out.transpose(2, 3).reshape(B, S, N, H * Dv))  # gate in the GEMM epilogue
        x = ops.gated_residual(x, self.zero_cond(single_cond), self.out_proj(out))
        wf = self.ffn_cond_norm_w
        xn = ops.ada_norm(x, ops.linear(cond_norm, self.ffn_cond_scale.weight * wf, self.ffn_cond_scale.bias),
                          ops.linear(cond_norm, self.ffn_cond_bias.weight * wf), self.ffn_norm.eps)
        ff = self.ffn_linear2(ops.swiglu(self.ffn_linear1(xn)))
        return ops.gated_residual(x, self.ffn_zero_cond(single_cond), ff)

    def forward(self, x, mask, single_cond, pair_logits):
        """Reference-shaped call: ``x`` ``[B?, N, c]``, ``mask`` ``[B?, N]``, ``pair_logits`` ``[B?, H, N, N]``."""
        squeeze = x.dim() == 2
        if squeeze:
            x, mask, single_cond = x.unsqueeze(0), mask.unsqueeze(0), single_cond.unsqueeze(0)
            pair_logits = None if pair_logits is None else pair_logits.unsqueeze(0)
        B, N, _ = x.shape
        bias = (1e9 * (mask.float() - 1.0)).view(B, 1, 1, N)
        logits = bias.expand(B, self.num_heads, N, N) if pair_logits is None else pair_logits.float() + bias
        out = self.run(x.unsqueeze(1), ops.layer_norm(single_cond).unsqueeze(1), single_cond.unsqueeze(1), logits)
        out = out.squeeze(1)
        return out.squeeze(0) if squeeze else out


class DiffusionTransformer(nn.Module):
    """24 blocks in super-blocks of 4; each super-block projects its own pair logits (reference: :597-730)."""

    def __init__(self, c, c_single_cond, num_blocks=24, num_heads=16, key_dim=None, value_dim=None,
                 num_intermediate_factor=2, super_block_size=4, c_pair=128, optim=None,
                 cond_bias_init_beta=None):  # fmt: skip
        super().__init__()
        assert num_blocks % super_block_size == 0
        self.num_blocks, self.super_block_size = num_blocks, super_block_size
        self.pair_norm_w = nn.Parameter(torch.ones(c_pair))
        self.pair_logits_proj = nn.ModuleList(
            LinearNoBias(c_pair, super_block_size * num_heads) for _ in range(num_blocks // super_block_size)
        )
        self.layers = nn.ModuleList(
            DiffusionTransformerBlock(c, c_single_cond, num_heads, key_dim, value_dim, num_intermediate_factor,
                                      optim=optim, cond_bias_init_beta=cond_bias_init_beta)  # fmt: skip
            for _ in range(num_blocks)
        )
        self.output_norm_w = nn.Parameter(torch.ones(c))
        self.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0

    def hoist_pair_logits(self, pair_cond, mask) -> tuple[torch.Tensor, ...]:
        """Per super-block ``[B, sbs*H, N, N]`` logits with ``1e9 (mask - 1)`` added along keys, as contiguous head
        planes. They keep the dtype the projection produces (bf16 under autocast: widening them would add no
        information, and the attention kernel stages bf16 bias tiles by TMA), fp32 otherwise."""
        rows = budget_rows(self.pair_chunk_budget, pair_cond.shape[-2], 4 * pair_cond.shape[-1])
        if torch.is_grad_enabled():
            rows = 0
        N = pair_cond.shape[-3]

        parts: list[list[torch.Tensor]] = [[] for _ in self.pair_logits_proj]
        for lo in range(0, N, rows or N):
            pn = ops.layer_norm(pair_cond[..., lo : lo + (rows or N), :, :], self.pair_norm_w, None)
            for got, proj in zip(parts, self.pair_logits_proj):
                got.append(ops.head_bias_planes(pn, proj.weight))  # [B, sbs*H, rows, N]
        out = []
        for got in parts:
            logits = got[0] if len(got) == 1 else torch.cat(got, dim=-2)
            dtype = logits.dtype if logits.dtype == torch.bfloat16 else torch.float32
            bias = (1e9 * (mask.float() - 1.0))[:, None, None, :].to(dtype)
            out.append((logits.to(dtype) + bias).contiguous())
        return tuple(out)

    # ---- inference fast path -----------------------------------------------------------------------------------
    # Without autograd the conditioning terms of all blocks (two AdaLN scale / shift pairs and two output gates per
    # block, functions of the single conditioning only) come from two stacked products per denoiser call instead of six
    # small ones per block, the q / k / v projections are one product, the output gate and SwiGLU ride in GEMM epilogues
    # and every "a * b + c" is one addcmul: about 12 kernels per block instead of about 32 (the sampler at 1024 tokens
    # is bound by kernel count, not by arithmetic). Same arithmetic as ``DiffusionTransformerBlock.run``; the AdaLN
    # norm weights are folded into the stacked conditioning weights.
    def _fast_weights(self):
        from ..ops import autograd_ops as ao

        layers = list(self.layers)
        names = ("attn_cond_norm_w", "ffn_cond_norm_w")
        mods = ("attn_cond_scale", "attn_cond_bias", "ffn_cond_scale", "ffn_cond_bias", "zero_cond", "ffn_zero_cond", "to_q",
                "to_k", "to_v", "to_g", "out_proj", "ffn_linear1", "ffn_linear2")  # fmt: skip
        sig = sum(getattr(ly, n)._version for ly in layers for n in names)
        sig += sum(p._version for ly in layers for m in mods for p in getattr(ly, m).parameters())
        hit = self.__dict__.get("_fast_cache")
        if hit is not None and hit[0] == sig and hit[1]["wc"].device == layers[0].to_k.weight.device:
            return hit[1]
        bf = torch.bfloat16
        with torch.no_grad():
            c = layers[0].to_k.weight.shape[1]
            wc, bc, wz, bz, per = [], [], [], [], []
            for ly in layers:
                wa, wf = ly.attn_cond_norm_w.float(), ly.ffn_cond_norm_w.float()
                wc += [ly.attn_cond_scale.weight.float() * wa, ly.attn_cond_bias.weight.float() * wa,
                       ly.ffn_cond_scale.weight.float() * wf, ly.ffn_cond_bias.weight.float() * wf]  # fmt: skip
                zero = torch.zeros(c, device=wa.device)
                bc += [ly.attn_cond_scale.bias.float(), zero, ly.ffn_cond_scale.bias.float(), zero]
                wz += [ly.zero_cond.weight.float(), ly.ffn_zero_cond.weight.float()]
                bz += [ly.zero_cond.bias.float(), ly.ffn_zero_cond.bias.float()]
                qkv = torch.cat([ly.to_q.weight, ly.to_k.weight, ly.to_v.weight], 0).to(bf).contiguous()
                qkv_b = torch.cat([ly.to_q.bias.float(), torch.zeros(ly.to_k.weight.shape[0] + ly.to_v.weight.shape[0], device=wa.device)])
                per.append({"qkv": qkv, "qkv_b": qkv_b, "g": ly.to_g.weight.to(bf).contiguous(), "o": ly.out_proj.weight.to(bf).contiguous(),
                            "w1": ly.ffn_linear1.weight.to(bf).contiguous(), "w2": ly.ffn_linear2.weight.to(bf).contiguous()})  # fmt: skip
            out = {"wc": torch.cat(wc, 0).to(bf).contiguous(), "bc": torch.cat(bc).contiguous(), "wz": torch.cat(wz, 0).to(bf).contiguous(),
                   "bz": torch.cat(bz).contiguous(), "per": per, "c": c}  # fmt: skip
        if not torch.cuda.is_current_stream_capturing():  # tensors made inside a graph capture belong to that graph's pool
            self.__dict__["_fast_cache"] = (sig, out)
        return out

    def _run_fast(self, act, single_cond, pair_logits):
        from ..ops import autograd_ops as ao

        W = self._fast_weights()
        L, c = len(self.layers), W["c"]
        ly0 = self.layers[0]
        H, Dk, Dv, sbs = ly0.num_heads, ly0.key_dim_per_head, ly0.val_dim_per_head, self.super_block_size
        B, S, N, _ = act.shape
        bf = torch.bfloat16
        cond16 = single_cond.to(bf)
        cond = ao.K.gemm(ops.layer_norm(cond16).contiguous(), W["wc"], W["bc"], None, None, 0, False).view(*single_cond.shape[:-1], L, 4, c)
        cond[..., 0::2, :].sigmoid_()                       # the two AdaLN scales of every block
        gates = ao.K.gemm(cond16.contiguous(), W["wz"], W["bz"], None, None, 0, False).view(*single_cond.shape[:-1], L, 2, c).sigmoid_()
        x = act.to(bf)
        for i, ly in enumerate(self.layers):
            w = W["per"][i]
            logits = pair_logits[i // sbs][:, (i % sbs) * H : (i % sbs + 1) * H]
            xn = torch.addcmul(cond[..., i, 1, :], cond[..., i, 0, :], ops.layer_norm(x))
            qkv = ao.K.gemm(xn, w["qkv"], w["qkv_b"], None, None, 0, False)
            q = qkv[..., : H * Dk].view(B, S, N, H, Dk).transpose(2, 3)
            k = qkv[..., H * Dk : 2 * H * Dk].view(B, S, N, H, Dk).transpose(2, 3)
            v = qkv[..., 2 * H * Dk :].view(B, S, N, H, Dv).transpose(2, 3)
            out = ops.pair_bias_attention(q, k, v, logits, None, ly.scale, fp32_qk=True)
            out = out.transpose(2, 3).reshape(B, S, N, H * Dv)
            gated = ao.K.gemm(xn, w["g"], None, None, out.contiguous(), 3, False)          # sigmoid(xn Wg^T) * out
            x = torch.addcmul(x, gates[..., i, 0, :], ao.K.gemm(gated, w["o"], None, None, None, 0, False))
            xn = torch.addcmul(cond[..., i, 3, :], cond[..., i, 2, :], ops.layer_norm(x))
            hidden = ao.K.gemm(xn, w["w1"], None, None, None, 2, False)                    # SwiGLU in the epilogue
            x = torch.addcmul(x, gates[..., i, 1, :], ao.K.gemm(hidden, w["w2"], None, None, None, 0, False))
        return ops.layer_norm(x, self.output_norm_w, None).to(act.dtype)

    def _fast_ok(self, act, pair_logits) -> bool:
        import os

        if torch.is_grad_enabled() or not act.is_cuda or not ops.bf16_mode(act) or os.environ.get("DF3_DIFFUSION_FAST", "1") == "0":
            return False
        ly = self.layers[0]
        nat = ops.fused(act.to(torch.bfloat16) if act.dtype != torch.bfloat16 else act, "gemm")
        return (nat is not None and ly.to_k.weight.shape[1] % 64 == 0 and (ly.num_heads * ly.key_dim_per_head) % 8 == 0
                and all(t.dtype == torch.bfloat16 for t in pair_logits))

    def run(self, act, single_cond, pair_logits):
        """``act`` ``[B, S, N, c]``, ``single_cond`` ``[B, S|1, N, cs]``, hoisted ``pair_logits``."""
        if self._fast_ok(act, pair_logits):
            return self._run_fast(act, single_cond, pair_logits)
        H, sbs = self.layers[0].num_heads, self.super_block_size
        cond_norm = ops.layer_norm(single_cond)
        for sb, logits in enumerate(pair_logits):
            for j in range(sbs):
                act = self.layers[sb * sbs + j].run(act, cond_norm, single_cond, logits[:, j * H : (j + 1) * H])
        return ops.layer_norm(act, self.output_norm_w, None)

    def forward(self, act, mask, single_cond, pair_cond):
        """Reference-shaped call on ``[B?, N, ...]`` tensors."""
        squeeze = act.dim() == 2
        if squeeze:
            act, mask, single_cond, pair_cond = (t.unsqueeze(0) for t in (act, mask, single_cond, pair_cond))
        out = self.run(act.unsqueeze(1), single_cond.unsqueeze(1), self.hoist_pair_logits(pair_cond, mask)).squeeze(1)
        return out.squeeze(0) if squeeze else out


class DiffusionConditioningBlock(nn.Module):
    """Trunk outputs + features + noise level → conditioning vectors (reference: diffusion.py:733-900)."""

    def __init__(self, c_pair_in, c_single_in, rel_feat_dim, c_pair_out, c_single_out, target_feat_dim=447,
                 use_trunk_single=True, sigma_data=16.0, fourier_dim=256, num_intermediate_factor=2,
                 optim=None):  # fmt: skip
        super().__init__()
        self.sigma_data = sigma_data
        pair_in = c_pair_in + rel_feat_dim
        self.pair_cond_norm_w = nn.Parameter(torch.ones(pair_in))
        self.pair_cond_proj = LinearNoBias(pair_in, c_pair_out)
        self.pair_trans0 = make_transition_block(c_pair_out, num_intermediate_factor, config=optim)
        self.pair_trans1 = make_transition_block(c_pair_out, num_intermediate_factor, config=optim)
        self.num_intermediate_factor = num_intermediate_factor
        self.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0
        self.use_trunk_single = bool(use_trunk_single)
        single_in = (c_single_in if self.use_trunk_single else 0) + target_feat_dim
        self.single_cond_norm_w = nn.Parameter(torch.ones(single_in))
        self.single_cond_proj = LinearNoBias(single_in, c_single_out)
        gen = torch.Generator().manual_seed(FOURIER_INIT_SEED)
        self.register_buffer("fourier_weight", torch.randn(fourier_dim, generator=gen))
        self.register_buffer("fourier_bias", torch.rand(fourier_dim, generator=gen))
        self.noise_emb_norm_w = nn.Parameter(torch.ones(fourier_dim))
        self.noise_emb_proj = LinearNoBias(fourier_dim, c_single_out)
        self.single_trans0 = make_transition_block(c_single_out, num_intermediate_factor, config=optim)
        self.single_trans1 = make_transition_block(c_single_out, num_intermediate_factor, config=optim)

    def _fourier_noise_embedding(self, sigma):
        x = 0.25 * torch.log(sigma.float())
        return torch.cos(2 * math.pi * (x.unsqueeze(-1) * self.fourier_weight.float() + self.fourier_bias.float()))

    def _pair_cond(self, pair_emb, rel_feat):
        x = torch.cat([pair_emb, rel_feat.to(pair_emb.dtype)], dim=-1)
        x = self.pair_cond_proj(ops.layer_norm(x, self.pair_cond_norm_w, None))
        x = x + self.pair_trans0(x)
        return x + self.pair_trans1(x)

    def compute_static(self, single_emb, pair_emb, target_feat, rel_feat):
        """``(single_cond_pre_noise [.., N, cs], pair_cond [.., N, N, cp])``."""
        widest = max(
            4 * (pair_emb.shape[-1] + rel_feat.shape[-1]),
            2 * self.num_intermediate_factor * self.pair_cond_proj.out_features * gemm_itemsize(pair_emb),
        )
        pair_cond = map_pair_rows(self._pair_cond, pair_emb, self.pair_chunk_budget, widest, rel_feat)
        s_in = torch.cat([single_emb, target_feat], dim=-1) if self.use_trunk_single else target_feat
        return self.single_cond_proj(ops.layer_norm(s_in, self.single_cond_norm_w, None)), pair_cond

    def add_noise(self, single_cond_pre_noise, noise_level):
        """Add the noise-level embedding and run the two single transitions.

        ``noise_level`` broadcasts against the leading axes of
        ``single_cond_pre_noise`` once a token axis and a channel axis are
        appended (e.g. ``[B, S]`` against ``[B, 1, N, c]``).
        """
        emb = self._fourier_noise_embedding(noise_level / self.sigma_data)
        emb = ops.layer_norm(emb, self.noise_emb_norm_w, None)
        proj = self.noise_emb_proj(emb.to(single_cond_pre_noise.dtype))
        while proj.dim() < single_cond_pre_noise.dim():
            proj = proj.unsqueeze(-2)
        x = single_cond_pre_noise + proj
        x = x + self.single_trans0(x)
        return x + self.single_trans1(x)

    def forward(self, single_emb, pair_emb, target_feat, rel_feat, noise_level):
        pre, pair_cond = self.compute_static(single_emb, pair_emb, target_feat, rel_feat)
        return self.add_noise(pre, noise_level), pair_cond
