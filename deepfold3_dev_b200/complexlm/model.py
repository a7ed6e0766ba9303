"""The complex language model and its packed batch (reference: complexlm/model.py:116-466, batch.py, vocab.py).

One token axis holds many complexes back to back. A layer of kind ``c`` attends inside a chain with rotary positions that
restart per chain; ``g`` attends inside a complex with no positions; ``r`` inside a complex with rotary positions over the
concatenation; ``x`` to the other chains of the complex only. Blocks are pre-norm with bias-free projections, q/k norms,
SwiGLU at 8/3 expansion rounded up to 256, residual scaling sqrt(layers / 36). Parameter names equal the reference's so
checkpoints interchange. Under ``mup`` hidden matrices take init variance and Adam step scaled by the width multiple,
attention logits scale 1/d_head and the readout is divided by the width multiple.

Segment attention: on CUDA in half precision the packed path hands cumulative segment offsets to torch's variable-length
attention; elsewhere a dense masked attention gives the same numbers (and is the only path that returns weights).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, fields

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from .config import ComplexLMConfig

# --- vocabulary: ESM-2's ids, so an ESM-2 embedding table copies over --------------------------------------------------
ESM2_TOKENS = "LAGVSERTIDPKQNFYMHWCXBUZO"
CLS_ID, PAD_ID, EOS_ID, UNK_ID, MASK_ID, VOCAB_SIZE = 0, 1, 2, 3, 32, 33
STANDARD_TOKENS = "ACDEFGHIKLMNPQRSTVWY"
IGNORE_INDEX = -100


def ascii_to_id_table() -> np.ndarray:
    table = np.full(256, UNK_ID, dtype=np.uint8)
    for i, ch in enumerate(ESM2_TOKENS):
        table[ord(ch)] = 4 + i
    return table


def encode(seq: str) -> np.ndarray:
    return ascii_to_id_table()[np.frombuffer(seq.upper().encode("ascii", "replace"), dtype=np.uint8)]


def decode(ids) -> str:
    chars = {4 + i: c for i, c in enumerate(ESM2_TOKENS)} | {CLS_ID: "^", PAD_ID: ".", EOS_ID: "$", UNK_ID: "X", MASK_ID: "#"}
    return "".join(chars.get(int(i), "?") for i in ids)


def standard_token_ids() -> np.ndarray:
    t = ascii_to_id_table()
    return np.sort(np.array([t[ord(c)] for c in STANDARD_TOKENS], dtype=np.int64))


@dataclass
class PackedBatch:
    """``tokens``/``labels``/``positions``/``global_positions``/``chain_index``/``complex_index``/``entity_index``/
    ``iface``/``iface_known`` are ``[T]``; ``chain_cu`` ``[chains + 1]`` and ``complex_cu`` ``[complexes + 1]`` are int32
    segment offsets; ``source`` is ``[complexes]``. Labels are ``IGNORE_INDEX`` where a position is not scored."""

    tokens: torch.Tensor
    labels: torch.Tensor
    positions: torch.Tensor
    global_positions: torch.Tensor
    chain_cu: torch.Tensor
    complex_cu: torch.Tensor
    chain_index: torch.Tensor
    complex_index: torch.Tensor
    entity_index: torch.Tensor
    iface: torch.Tensor
    iface_known: torch.Tensor
    source: torch.Tensor
    max_chain_len: int
    max_complex_len: int

    @property
    def n_tokens(self) -> int:
        return int(self.tokens.numel())

    @property
    def n_chains(self) -> int:
        return int(self.chain_cu.numel() - 1)

    @property
    def n_complexes(self) -> int:
        return int(self.complex_cu.numel() - 1)

    def _map(self, fn) -> "PackedBatch":
        return PackedBatch(**{f.name: fn(getattr(self, f.name)) if torch.is_tensor(getattr(self, f.name)) else getattr(self, f.name)
                              for f in fields(self)})  # fmt: skip

    def to(self, device, non_blocking: bool = False) -> "PackedBatch":
        return self._map(lambda t: t.to(device, non_blocking=non_blocking))

    def pin_memory(self) -> "PackedBatch":
        return self._map(lambda t: t.pin_memory())

    def chains_only(self) -> "PackedBatch":
        """The same tokens with every chain made its own complex (what ``*_single`` metrics score)."""
        out = self._map(lambda t: t)
        out.complex_cu, out.complex_index = self.chain_cu, self.chain_index
        out.global_positions, out.max_complex_len = self.positions, self.max_chain_len
        return out


class RMSNorm(nn.Module):
    """Root-mean-square normalisation with a learned gain, evaluated in fp32 whatever the activation dtype."""

    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return F.rms_norm(x.float(), self.weight.shape, self.weight.float(), self.eps).to(x.dtype)


def build_norm(cfg: ComplexLMConfig, dim: int, bias: bool | None = None) -> nn.Module:
    """The normalisation layer the configuration names; ``bias`` overrides the configured bias switch of a LayerNorm
    (the ESM-C compatible layout wants some norms with and some without)."""
    makers = {
        "rmsnorm": lambda: RMSNorm(dim, cfg.norm_eps),
        "layernorm": lambda: nn.LayerNorm(dim, eps=cfg.norm_eps, bias=cfg.bias if bias is None else bias),
    }
    return makers.get(cfg.norm, makers["layernorm"])()


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """``x`` [T, H, D] rotated (rotate-half form) by per-token integer positions [T]."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device).float() / d))
    ang = positions.float()[:, None] * inv[None]
    cos, sin = torch.cat([ang.cos()] * 2, -1)[:, None], torch.cat([ang.sin()] * 2, -1)[:, None]
    a, b = x.float().chunk(2, -1)
    return (x.float() * cos + torch.cat([-b, a], -1) * sin).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, cfg: ComplexLMConfig, kind: str):
        super().__init__()
        self.cfg, self.kind = cfg, kind
        self.n_heads, self.head_dim = cfg.n_heads, cfg.head_dim
        self.scale = (cfg.base_head_dim**0.5) / self.head_dim if cfg.mup else self.head_dim**-0.5
        self.norm = build_norm(cfg, cfg.d_model, bias=True if cfg.esmc_compat else None)
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model, bias=cfg.bias)
        self.out_proj = nn.Linear(cfg.d_model, cfg.d_model, bias=cfg.bias)
        self.q_norm = build_norm(cfg, cfg.d_model, bias=False) if cfg.qk_layernorm else nn.Identity()
        self.k_norm = build_norm(cfg, cfg.d_model, bias=False) if cfg.qk_layernorm else nn.Identity()

    def allowed(self, batch: PackedBatch) -> torch.Tensor:
        """[T, T] bool of permitted (query, key) pairs; a query with no key sees itself."""
        if self.kind == "c":
            ok = batch.chain_index[:, None] == batch.chain_index[None]
        else:
            ok = batch.complex_index[:, None] == batch.complex_index[None]
            if self.kind == "x":
                ok = ok & (batch.chain_index[:, None] != batch.chain_index[None])
        eye = torch.eye(ok.shape[0], dtype=torch.bool, device=ok.device)
        return ok | (~ok.any(-1, keepdim=True) & eye)

    def forward(self, x, batch: PackedBatch, return_attn: bool = False):
        T = x.shape[0]
        q, k, v = self.qkv(self.norm(x)).chunk(3, dim=-1)
        q, k = self.q_norm(q).to(v.dtype), self.k_norm(k).to(v.dtype)
        q, k, v = (t.reshape(T, self.n_heads, self.head_dim) for t in (q, k, v))
        if self.kind in ("c", "r"):
            pos = batch.positions if self.kind == "c" else batch.global_positions
            q, k = rope(q, pos, self.cfg.rope_theta), rope(k, pos, self.cfg.rope_theta)
        packed = (self.cfg.attn_impl == "varlen" and self.kind != "x" and v.is_cuda and not return_attn
                  and v.dtype in (torch.bfloat16, torch.float16))  # fmt: skip
        attn = None
        if packed:
            from torch.nn.attention.varlen import varlen_attn

            cu, longest = (batch.chain_cu, batch.max_chain_len) if self.kind == "c" else (batch.complex_cu, batch.max_complex_len)
            out = varlen_attn(q.contiguous(), k.contiguous(), v.contiguous(), cu, cu, longest, longest, scale=self.scale)
        else:
            ok = self.allowed(batch)[None, None]
            qh, kh, vh = (t.transpose(0, 1)[None] for t in (q, k, v))
            if return_attn:
                s = (qh.float() @ kh.float().transpose(-1, -2)) * self.scale
                w = s.masked_fill(~ok, float("-inf")).softmax(-1)
                out, attn = (w.to(vh.dtype) @ vh)[0].transpose(0, 1), w[0]
            else:
                out = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=ok, scale=self.scale)[0].transpose(0, 1)
        return self.out_proj(out.reshape(T, -1)), attn


def swiglu_hidden(d_model: int, expansion_ratio: float) -> int:
    """Hidden width of the gated feed-forward: ``expansion_ratio * d_model`` rounded up to a multiple of 256."""
    return 256 * math.ceil(expansion_ratio * d_model / 256)


class SwiGLUFFN(nn.Module):
    """Pre-norm gated feed-forward: ``w_out(silu(g) * u)`` with ``[g, u] = w_in(norm(x))``."""

    def __init__(self, cfg: ComplexLMConfig):
        super().__init__()
        self.hidden = swiglu_hidden(cfg.d_model, cfg.expansion_ratio)
        self.norm = build_norm(cfg, cfg.d_model, bias=True if cfg.esmc_compat else None)
        self.w_in = nn.Linear(cfg.d_model, 2 * self.hidden, bias=cfg.bias)
        self.w_out = nn.Linear(self.hidden, cfg.d_model, bias=cfg.bias)

    def forward(self, x):
        h = self.w_in(self.norm(x))
        return self.w_out(F.silu(h[..., : self.hidden]) * h[..., self.hidden :])


class Block(nn.Module):
    def __init__(self, cfg: ComplexLMConfig, kind: str):
        super().__init__()
        self.kind = kind
        self.attn = Attention(cfg, kind)
        self.ffn = SwiGLUFFN(cfg)
        self.residue_scale = math.sqrt(cfg.n_layers / 36) if cfg.scale_residue else 1.0

    def forward(self, x, batch, return_attn=False):
        delta, attn = self.attn(x, batch, return_attn)
        x = x + delta / self.residue_scale
        return x + self.ffn(x) / self.residue_scale, attn


class MLMHead(nn.Module):
    """Masked-token read-out: dense + GELU + norm, then the vocabulary projection."""

    def __init__(self, cfg: ComplexLMConfig):
        super().__init__()
        width = cfg.d_model
        self.dense = nn.Linear(width, width, bias=cfg.bias or cfg.esmc_compat)
        self.norm = build_norm(cfg, width, bias=True if cfg.esmc_compat else None)
        self.out = nn.Linear(width, cfg.vocab_size, bias=True)

    def forward(self, x):
        hidden = self.norm(F.gelu(self.dense(x)))
        return self.out(hidden)


@dataclass
class ComplexLMOutput:
    logits: torch.Tensor
    hidden: list | None = None
    attentions: list | None = None


def mup_role(name: str, param: torch.Tensor) -> str:
    """``embedding`` / ``readout`` (one width dimension), ``hidden`` (two: the only rescaled kind), ``vector`` (none)."""
    if param.dim() < 2:
        return "vector"
    if name.startswith("embed."):
        return "embedding"
    if name.startswith("head.out."):
        return "readout"
    return "hidden"


class ComplexLM(nn.Module):
    def __init__(self, cfg: ComplexLMConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.embed_dropout = nn.Dropout(cfg.embed_dropout) if cfg.embed_dropout else nn.Identity()
        self.chain_gate = nn.Parameter(torch.zeros(1)) if cfg.chain_signal == "random" else None
        self.blocks = nn.ModuleList(Block(cfg, k) for k in cfg.kinds)
        self.norm = build_norm(cfg, cfg.d_model, bias=False if cfg.esmc_compat else None)
        self.head = MLMHead(cfg)
        self.readout_mult = 1.0 / cfg.width_mult
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=cfg.init_std)
                if getattr(m, "bias", None) is not None:
                    nn.init.zeros_(m.bias)
        if cfg.mup:
            with torch.no_grad():
                for name, p in self.named_parameters():
                    if mup_role(name, p) == "hidden":
                        p.div_(cfg.width_mult**0.5)

    @property
    def n_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def forward(self, batch: PackedBatch, return_hidden: bool = False, return_attn: bool = False) -> ComplexLMOutput:
        x = self.embed_dropout(self.embed(batch.tokens))
        if self.chain_gate is not None:  # a per-chain random vector breaks the exact-homomer symmetry
            noise = torch.randn(batch.n_chains, x.shape[-1], device=x.device, dtype=x.dtype)
            x = x + self.chain_gate * noise[batch.chain_index.long()]
        hidden = [x] if return_hidden else None
        attns = []
        for blk in self.blocks:
            x, a = blk(x, batch, return_attn)
            if hidden is not None:
                hidden.append(x)
            if a is not None:
                attns.append(a)
        x = self.norm(x)
        if hidden is not None:
            hidden[-1] = x
        return ComplexLMOutput(self.head(x) * self.readout_mult, hidden, attns or None)

    def param_groups(self, weight_decay: float) -> list[dict]:
        """Optimizer groups by muP role. Hidden matrices step with ``lr / width_mult`` and decay with
        ``weight_decay * width_mult`` (so lr x decay does not depend on the width); matrices of the other roles decay
        plainly; vectors (gains, biases) and the embedding table do not decay."""
        mult = float(self.cfg.width_mult)
        groups: dict[tuple[str, bool], dict] = {}
        for name, param in self.named_parameters():
            if not param.requires_grad:
                continue
            role = mup_role(name, param)
            decays = role in ("hidden", "readout")
            group = groups.get((role, decays))
            if group is None:
                scale = 1.0 / mult if role == "hidden" else 1.0
                decay = 0.0 if not decays else weight_decay * (mult if role == "hidden" else 1.0)
                group = groups[(role, decays)] = {"params": [], "role": role, "lr_scale": scale, "weight_decay": decay}
            group["params"].append(param)
        return list(groups.values())

    @torch.no_grad()
    def warm_start_from_esm2(self, embedding: torch.Tensor) -> None:
        """Copy an ESM-2 token embedding table (same ids) when the widths agree."""
        if embedding.shape == self.embed.weight.shape:
            self.embed.weight.copy_(embedding)
