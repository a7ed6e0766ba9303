"""Optional protein-language-model frontend: a frozen ESM-2 encoder, chain packing and the pair projection.

Reference: model/esm2.py:68-354 (own ESM-2 implementation with rotary attention and a loader for the Hub's
``model.safetensors``), model/plm.py:47-318 (frozen wrapper, ``per_chain`` / ``joined`` packing, scatter back onto
the trunk's tokens), model/lm_pair.py:36-114 (learned layer mixture -> outer product/difference -> pair track).
As in the reference it is not wired into ``ModelConfig``; the side language model and the ``plm-*`` commands use it.

Differences in construction: q, k and v are one fused projection (the loader concatenates the three Hub tensors);
``per_chain`` mode runs the chains as rows of one padded batch, so no attention is computed across chains at all
instead of being masked out of a packed sequence. Outputs equal the packed, block-diagonal formulation.
``LMPairShim`` keeps the reference's parameter names, which do live in checkpoints.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..data import const

ESM2_ALPHABET = "LAGVSERTIDPKQNFYMHWCXBUZO"  # ids 4.. in this order; 0 cls, 1 pad, 2 eos, 3 unk, 32 mask


@dataclass(frozen=True)
class PLMTokenizer:
    """Special ids and the residue-type -> token-id table of one language model."""

    pad_id: int
    unk_id: int
    mask_id: int
    res_type_to_id: torch.Tensor
    cls_id: int | None = None
    eos_id: int | None = None


def esm2_tokenizer() -> PLMTokenizer:
    table = torch.full((const.RES_TYPE_COUNT,), 3, dtype=torch.long)
    for three, one in const.PROTEIN_3TO1.items():
        if one in ESM2_ALPHABET:
            table[const.RES_TYPE_ORDER[three]] = 4 + ESM2_ALPHABET.index(one)
    return PLMTokenizer(pad_id=1, unk_id=3, mask_id=32, res_type_to_id=table, cls_id=0, eos_id=2)


@dataclass
class ESM2Config:
    hidden_size: int = 1280
    num_hidden_layers: int = 33
    num_attention_heads: int = 20
    intermediate_size: int = 5120
    vocab_size: int = 33
    layer_norm_eps: float = 1e-5
    pad_token_id: int = 1
    mask_token_id: int = 32
    token_dropout: bool = True
    emb_layer_norm_before: bool = False

    @classmethod
    def from_json(cls, path: str) -> "ESM2Config":
        with open(path) as f:
            raw = json.load(f)
        return cls(**{k: v for k, v in raw.items() if k in cls.__dataclass_fields__})


def rotary(x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Rotate-half rotary embedding of ``x`` [B, H, L, D] at integer ``positions`` [B, L] (base 10000)."""
    d = x.shape[-1]
    inv = 1.0 / (10000 ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = positions.float().unsqueeze(-1) * inv  # [B, L, D/2]
    cos, sin = torch.cat([ang.cos()] * 2, -1).unsqueeze(1), torch.cat([ang.sin()] * 2, -1).unsqueeze(1)
    x1, x2 = x.float().chunk(2, dim=-1)
    return (x.float() * cos + torch.cat([-x2, x1], -1) * sin).to(x.dtype)


class ESM2Block(nn.Module):
    def __init__(self, cfg: ESM2Config):
        super().__init__()
        h = cfg.hidden_size
        self.heads = cfg.num_attention_heads
        self.norm_attn = nn.LayerNorm(h, eps=cfg.layer_norm_eps)
        self.qkv = nn.Linear(h, 3 * h)
        self.proj = nn.Linear(h, h)
        self.norm_ffn = nn.LayerNorm(h, eps=cfg.layer_norm_eps)
        self.up = nn.Linear(h, cfg.intermediate_size)
        self.down = nn.Linear(cfg.intermediate_size, h)

    def forward(self, x, bias, positions):
        B, L, h = x.shape
        q, k, v = self.qkv(self.norm_attn(x)).view(B, L, 3, self.heads, h // self.heads).permute(2, 0, 3, 1, 4)
        q, k = rotary(q, positions), rotary(k, positions)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=bias)
        x = x + self.proj(a.transpose(1, 2).reshape(B, L, h))
        return x + self.down(F.gelu(self.up(self.norm_ffn(x))))


class ESM2Encoder(nn.Module):
    """Returns every hidden state: ``[B, L, layers + 1, hidden]`` (embedding output first, final LayerNorm on the last)."""

    tokenizer = staticmethod(esm2_tokenizer)

    def __init__(self, cfg: ESM2Config):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size, padding_idx=cfg.pad_token_id)
        self.norm_in = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps) if cfg.emb_layer_norm_before else None
        self.blocks = nn.ModuleList(ESM2Block(cfg) for _ in range(cfg.num_hidden_layers))
        self.norm_out = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)

    def forward(self, input_ids, sequence_id=None, position_ids=None):
        cfg = self.cfg
        real = input_ids != cfg.pad_token_id
        x = self.embed(input_ids)
        if cfg.token_dropout:
            # ESM-2 was trained with masked positions zeroed and the rest rescaled; without masks this is a constant
            # factor (1 - 0.15 * 0.8) that has to stay for the embeddings to match
            masked = input_ids == cfg.mask_token_id
            x = x.masked_fill(masked.unsqueeze(-1), 0.0)
            seen = masked.sum(-1).float() / real.sum(-1).clamp(min=1)
            x = (x * (1 - 0.15 * 0.8) / (1 - seen)[:, None, None]).to(x.dtype)
        if self.norm_in is not None:
            x = self.norm_in(x)
        x = x * real.unsqueeze(-1).to(x.dtype)
        L = input_ids.shape[1]
        allow = real[:, None, :].expand(-1, L, -1)
        if sequence_id is not None:
            allow = allow & (sequence_id[:, :, None] == sequence_id[:, None, :]) & (sequence_id[:, :, None] >= 0)
        eye = torch.eye(L, dtype=torch.bool, device=x.device)
        allow = allow | (~allow.any(-1, keepdim=True) & eye)  # a row without keys attends to itself (no NaN rows)
        bias = torch.zeros(allow.shape, dtype=x.dtype, device=x.device).masked_fill_(~allow, float("-inf")).unsqueeze(1)
        if position_ids is None:
            position_ids = torch.arange(L, device=x.device).unsqueeze(0).expand_as(input_ids)
        states = [x]
        for blk in self.blocks:
            x = blk(x, bias, position_ids)
            states.append(x)
        states[-1] = self.norm_out(x)
        return torch.stack(states, dim=-2)

    @torch.no_grad()
    def load_hf_safetensors(self, path: str) -> None:
        """``model.safetensors`` of a ``facebook/esm2_*`` snapshot (keys with or without the ``esm.`` prefix)."""
        from safetensors.torch import load_file

        sd = load_file(str(path))
        pre = "esm." if any(k.startswith("esm.") for k in sd) else ""
        g = lambda k: sd[pre + k]  # noqa: E731

        def put(mod, key):
            mod.weight.copy_(g(key + ".weight"))
            mod.bias.copy_(g(key + ".bias"))

        self.embed.weight.copy_(g("embeddings.word_embeddings.weight"))
        if self.norm_in is not None:
            put(self.norm_in, "embeddings.layer_norm")
        put(self.norm_out, "encoder.emb_layer_norm_after")
        for i, b in enumerate(self.blocks):
            p = f"encoder.layer.{i}."
            put(b.norm_attn, p + "attention.LayerNorm")
            b.qkv.weight.copy_(torch.cat([g(p + f"attention.self.{n}.weight") for n in ("query", "key", "value")]))
            b.qkv.bias.copy_(torch.cat([g(p + f"attention.self.{n}.bias") for n in ("query", "key", "value")]))
            put(b.proj, p + "attention.output.dense")
            put(b.norm_ffn, p + "LayerNorm")
            put(b.up, p + "intermediate.dense")
            put(b.down, p + "output.dense")


class FrozenPLM(nn.Module):
    """Frozen backend + packing: trunk token features in, ``[..., N, layers + 1, d_model]`` hidden states out.

    Only protein tokens take part; atomised residues collapse to one input position per residue and every atom token
    of the residue receives that residue's states. The backend never appears in ``state_dict``.
    """

    def __init__(self, model_dir: str | None = None, backend: str = "esm2", join: str = "per_chain", cfg: ESM2Config | None = None):
        super().__init__()
        if backend != "esm2":
            raise ValueError(f"unknown language-model backend {backend!r}")
        if join not in ("per_chain", "joined"):
            raise ValueError("join must be 'per_chain' or 'joined'")
        self.model_dir, self.join = model_dir, join
        if cfg is None and model_dir is not None:
            cfg = ESM2Config.from_json(os.path.join(model_dir, "config.json"))
        self.cfg = cfg or ESM2Config()
        self.tok = esm2_tokenizer()
        object.__setattr__(self, "_backbone", None)  # kept out of the module registry: frozen, never checkpointed

    def load(self, device, dtype=torch.bfloat16, random_init: bool = False) -> None:
        enc = ESM2Encoder(self.cfg)
        if not random_init:
            if self.model_dir is None:
                raise ValueError("no snapshot directory given")
            enc.load_hf_safetensors(os.path.join(self.model_dir, "model.safetensors"))
        object.__setattr__(self, "_backbone", enc.to(device=device, dtype=dtype).eval().requires_grad_(False))

    @property
    def d_model(self) -> int:
        return self.cfg.hidden_size

    @property
    def num_layers(self) -> int:
        return self.cfg.num_hidden_layers

    def _chains(self, res_type, asym_id, residue_index, mol_type, mask):
        """Per protein chain: ``(token ids per residue, residue numbers, residue slot of every token, token indices)``."""
        out = []
        ok = (mol_type == const.MOL_PROTEIN) & mask.bool()
        for a in torch.unique(asym_id[ok]).tolist():
            idx = torch.nonzero(ok & (asym_id == a)).flatten()
            res = residue_index[idx]
            first = torch.ones_like(res, dtype=torch.bool)
            first[1:] = res[1:] != res[:-1]
            slot = torch.cumsum(first.long(), 0) - 1
            ids = self.tok.res_type_to_id.to(res_type.device)[res_type[idx][first]]
            out.append((ids, res[first], slot, idx))
        return out

    @torch.no_grad()
    def forward(self, res_type, asym_id, residue_index, mol_type, mask):
        """Unbatched ``[N]`` inputs or batched ``[B, N]`` (looped); returns detached hidden states on the tokens."""
        if self._backbone is None:
            raise RuntimeError("call load() first")
        if res_type.dim() == 2:
            return torch.stack([self.forward(res_type[b], asym_id[b], residue_index[b], mol_type[b], mask[b])
                                for b in range(res_type.shape[0])])  # fmt: skip
        enc, tok, dev = self._backbone, self.tok, res_type.device
        N = res_type.shape[0]
        dtype = next(enc.parameters()).dtype
        out = torch.zeros(N, self.num_layers + 1, self.d_model, device=dev, dtype=dtype)
        chains = self._chains(res_type, asym_id, residue_index, mol_type, mask)
        if not chains:
            return out
        if self.join == "per_chain":
            L = max(len(c[0]) for c in chains) + 2
            ids = torch.full((len(chains), L), tok.pad_id, device=dev, dtype=torch.long)
            pos = torch.zeros(len(chains), L, device=dev, dtype=torch.long)
            for r, (t, num, _, _) in enumerate(chains):
                n = len(t)
                ids[r, 0], ids[r, 1 : n + 1], ids[r, n + 1] = tok.cls_id, t, tok.eos_id
                rel = num - num[0] + 1  # true numbering keeps gaps of unresolved regions or crops
                pos[r, 1 : n + 1], pos[r, n + 1] = rel, rel[-1] + 1
            h = enc(ids, None, pos)
            for r, (t, _, slot, idx) in enumerate(chains):
                out[idx] = h[r, 1 : len(t) + 1][slot]
            return out
        parts, poss, spans, at = [], [], [], 0
        for t, num, _, _ in chains:  # [CLS] c1 [EOS] [CLS] c2 [EOS] ... as one sequence, attention across chains
            rel = num - num[0] + 1
            parts.append(torch.cat([t.new_tensor([tok.cls_id]), t, t.new_tensor([tok.eos_id])]))
            poss.append(torch.cat([rel.new_tensor([0]), rel, rel[-1:] + 1]) + at)
            spans.append((sum(len(p) for p in parts[:-1]) + 1, len(t)))
            at = int(poss[-1][-1]) + 1
        h = enc(torch.cat(parts).unsqueeze(0), None, torch.cat(poss).unsqueeze(0))[0]
        for (s, n), (_, _, slot, idx) in zip(spans, chains):
            out[idx] = h[s : s + n][slot]
        return out


class SingleToPair(nn.Module):
    """[..., N, d_in] -> [..., N, N, d_out] from the outer product and the (antisymmetric) outer difference."""

    def __init__(self, input_dim: int, downproject_dim: int, output_dim: int):
        super().__init__()
        self.downproject = nn.Linear(input_dim, downproject_dim, bias=False)
        self.output_mlp = nn.Sequential(nn.Linear(2 * downproject_dim, output_dim), nn.GELU(), nn.Linear(output_dim, output_dim))

    def forward(self, x):
        x = self.downproject(x)
        a, b = x.unsqueeze(-2), x.unsqueeze(-3)
        return self.output_mlp(torch.cat([a * b, a - b], dim=-1))


class LMPairShim(nn.Module):
    """Learned softmax mixture over the backend's hidden states (uniform at start), projected to the pair track."""

    def __init__(self, d_pair: int, d_model: int, num_layers: int):
        super().__init__()
        self.d_pair, self.num_states = d_pair, num_layers + 1
        self.to_pair_channels = nn.Sequential(nn.LayerNorm(d_model), nn.Linear(d_model, d_pair, bias=False))
        self.layer_combine = nn.Parameter(torch.zeros(self.num_states))
        self.to_pair = nn.Sequential(SingleToPair(d_pair, d_pair, d_pair), nn.LayerNorm(d_pair))

    def forward(self, hidden_states, *, dropout: float = 0.0):
        if hidden_states.shape[-2] != self.num_states:
            raise ValueError(f"expected {self.num_states} hidden states, got {hidden_states.shape[-2]}")
        w = self.layer_combine.softmax(0).to(hidden_states.dtype)
        mixed = (self.to_pair_channels(hidden_states) * w.view(-1, 1)).sum(-2)
        z = self.to_pair(mixed)
        return F.dropout(z, p=dropout, training=True) if dropout > 0 else z  # dropout stays on at inference by design
