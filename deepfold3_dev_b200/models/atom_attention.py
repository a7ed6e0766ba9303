"""Atom-level modules: per-atom conditioning, windowed cross-attention transformer, encoders, decoder.

Reference: model/atom_cross_attn.py:451-1307; parameter names are identical.

Layout decision that differs from the reference: activations carry an explicit
diffusion-sample axis, ``[B, S, W, Q, c]``, while everything derived from the
conditioning alone (AdaLN scales and shifts, zero-gates, pair logits with the
key mask folded in) is computed once per molecule at ``[B, 1, W, ...]`` and
broadcast over ``S``. The reference materialises ``S`` copies of that state in
training (``expand_for_samples``) and only broadcasts in its hoisted sampler;
here the broadcast form is the only form, for training and inference alike,
and it is differentiable.
"""

from __future__ import annotations

import dataclasses

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .atom_layout import AtomLayout, build_atom_layout, queries_to_keys, queries_to_slots, slots_to_queries
from .primitives import LayerNorm, LinearNoBias, biased_linear, map_pair_rows


@dataclasses.dataclass
class AtomBlockTerms:
    """Conditioning-only terms of one transformer block, each ``[B, 1, W, ...]``."""

    logit_bias: torch.Tensor  # [B, 1, W, H, Q, K] pair logits + key mask
    q_scale: torch.Tensor
    q_bias: torch.Tensor
    k_scale: torch.Tensor  # key-side AdaLN scale and shift per QUERY slot [B, 1, W, Q, c]: a key is some window's query atom,
    k_bias: torch.Tensor  # so keys and values are projected once per atom and gathered into the windows afterwards
    attn_gate: torch.Tensor
    ffn_scale: torch.Tensor
    ffn_bias: torch.Tensor
    ffn_gate: torch.Tensor


@dataclasses.dataclass
class AtomEncoderStatic:
    """Noise-independent state of the atom encoder for a batch of molecules (all ``[B, ...]``)."""

    layout: AtomLayout
    queries_single: torch.Tensor  # [B, W, Q, c]
    queries_mask: torch.Tensor  # [B, W, Q]
    keys_single: torch.Tensor  # [B, W, K, c]
    keys_mask: torch.Tensor  # [B, W, K]
    atom_pair: torch.Tensor  # [B, W, Q, K, cp]
    ref_mask: torch.Tensor  # [B, N, M]
    encoder_terms: tuple | None = None
    decoder_terms: tuple | None = None

    @property
    def subsets(self):
        return self.layout


@dataclasses.dataclass
class AtomEncoderOutput:
    token_act: torch.Tensor  # [B, S, N, ct]
    skip_connection: torch.Tensor  # [B, S, W, Q, c]
    static: AtomEncoderStatic


class AtomPerAtomConditioning(nn.Module):
    """Per-atom embedding of the reference conformer (reference: atom_cross_attn.py:451-570)."""

    def __init__(self, per_atom_channels, per_atom_pair_channels, num_element_classes=128, num_atom_name_chars=64,
                 atom_name_length=4, ref_element_zero_index=False):  # fmt: skip
        super().__init__()
        c, cp = per_atom_channels, per_atom_pair_channels
        self.num_element_classes = num_element_classes
        self.num_atom_name_chars = num_atom_name_chars
        self.ref_element_zero_index = ref_element_zero_index
        self.embed_ref_pos = LinearNoBias(3, c)
        self.embed_ref_mask = LinearNoBias(1, c)
        self.embed_ref_element = LinearNoBias(num_element_classes, c)
        self.embed_ref_charge = LinearNoBias(1, c)
        self.embed_ref_atom_name = LinearNoBias(num_atom_name_chars * atom_name_length, c)
        self.single_to_pair_row = LinearNoBias(c, cp)
        self.single_to_pair_col = LinearNoBias(c, cp)
        self.embed_pair_offsets = LinearNoBias(3, cp)
        self.embed_pair_distances = LinearNoBias(1, cp)
        self.pair_mlp1 = LinearNoBias(cp, cp, initializer="relu")
        self.pair_mlp2 = LinearNoBias(cp, cp, initializer="relu")
        self.pair_mlp3 = LinearNoBias(cp, cp, initializer="zeros")

    def single_cond(self, ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars):
        """``[..., N, M, c]``. One-hot inputs are applied as embedding lookups (same sums, no one-hot tensor)."""
        m = ref_mask.unsqueeze(-1)
        act = self.embed_ref_pos(ref_pos) + self.embed_ref_mask(m.to(ref_pos.dtype))
        elem = (ref_element - 1).clamp(min=0) if self.ref_element_zero_index else ref_element
        act = act + F.embedding(elem, self.embed_ref_element.weight.t().to(act.dtype))
        act = act + self.embed_ref_charge(torch.arcsinh(ref_charge).unsqueeze(-1).to(act.dtype))
        L = ref_atom_name_chars.shape[-1]
        table = self.embed_ref_atom_name.weight.t().to(act.dtype)  # [L * chars, c]
        offs = torch.arange(L, device=ref_atom_name_chars.device) * self.num_atom_name_chars
        act = act + F.embedding(ref_atom_name_chars + offs, table).sum(-2)
        return act * m.to(act.dtype)

    def apply_pair_mlp(self, pair):
        h = self.pair_mlp1(F.relu(pair))
        h = self.pair_mlp2(F.relu(h))
        return pair + self.pair_mlp3(F.relu(h))

    def forward(self, ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars):
        """``(atom_single [.., N, M, c], intra_token_pair [.., N, M, M, cp])``."""
        act = self.single_cond(ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars)
        row, col = self.single_to_pair_row(F.relu(act)), self.single_to_pair_col(F.relu(act))
        pair = row.unsqueeze(-2) + col.unsqueeze(-3)
        off = ref_pos.unsqueeze(-2) - ref_pos.unsqueeze(-3)
        pair = pair + self.embed_pair_offsets(off)
        pair = pair + self.embed_pair_distances(1.0 / (1.0 + off.pow(2).sum(-1, keepdim=True)))
        return act, self.apply_pair_mlp(pair)


class AtomCrossAttTransformer(nn.Module):
    """Blocks of windowed cross-attention + feed-forward with AdaLN-zero conditioning.

    Keys of every block are re-gathered from the current query activations
    (reference: atom_cross_attn.py:573-869).
    """

    def __init__(self, per_atom_channels, per_atom_pair_channels, num_blocks=3, num_heads=4,
                 num_intermediate_factor=2):  # fmt: skip
        super().__init__()
        c, cp, H = per_atom_channels, per_atom_pair_channels, num_heads
        assert c % H == 0
        self.num_heads, self.head_dim, self.num_blocks = H, c // H, num_blocks
        hidden = c * num_intermediate_factor
        self.pair_norm_w = nn.Parameter(torch.ones(cp))
        self.pair_logits_proj = LinearNoBias(cp, num_blocks * H)
        self.attn_blocks = nn.ModuleList(
            nn.ModuleDict(
                {
                    "to_q": biased_linear(c, c, "linear"),
                    "to_k": LinearNoBias(c, c),
                    "to_v": LinearNoBias(c, c),
                    "to_g": LinearNoBias(c, c, initializer="zeros"),
                    "out_proj": LinearNoBias(c, c),
                    "zero_cond": biased_linear(c, c, "zeros", bias_value=-2.0),
                }
            )
            for _ in range(num_blocks)
        )
        self.ffn_blocks = nn.ModuleList(
            nn.ModuleDict(
                {
                    "linear1": LinearNoBias(c, hidden * 2, initializer="relu"),
                    "linear2": LinearNoBias(hidden, c),
                    "zero_cond": biased_linear(c, c, "zeros", bias_value=-2.0),
                }
            )
            for _ in range(num_blocks)
        )
        self.attn_norms = nn.ModuleList(LayerNorm(c, elementwise_affine=False) for _ in range(num_blocks))
        self.ffn_norms = nn.ModuleList(LayerNorm(c, elementwise_affine=False) for _ in range(num_blocks))

        def plist():
            return nn.ParameterList(nn.Parameter(torch.ones(c)) for _ in range(num_blocks))

        def scales():
            return nn.ModuleList(biased_linear(c, c, "zeros") for _ in range(num_blocks))

        def shifts():
            return nn.ModuleList(LinearNoBias(c, c, initializer="zeros") for _ in range(num_blocks))

        self.attn_cond_w, self.attn_cond_scale, self.attn_cond_bias = plist(), scales(), shifts()
        self.k_cond_w, self.k_cond_scale, self.k_cond_bias = plist(), scales(), shifts()
        self.ffn_cond_w, self.ffn_cond_scale, self.ffn_cond_bias = plist(), scales(), shifts()

    def block_terms(self, queries_single, keys_single, keys_mask, pair_cond) -> tuple[AtomBlockTerms, ...]:
        """Everything the blocks derive from conditioning alone; inputs ``[B, W, ...]``, outputs ``[B, 1, W, ...]``."""
        B, W, Q, K = pair_cond.shape[:4]
        H, nb = self.num_heads, self.num_blocks
        logits = self.pair_logits_proj(ops.layer_norm(pair_cond, self.pair_norm_w, None))  # [B, W, Q, K, nb*H]
        logits = logits.reshape(B, W, Q, K, nb, H).permute(4, 0, 1, 5, 2, 3)  # [nb, B, W, H, Q, K]
        key_bias = 1e9 * (keys_mask.to(logits.dtype) - 1.0)[:, :, None, None, :]
        # ``keys_single`` is ``queries_single`` gathered into the windows (``queries_to_keys``), and everything derived
        # from it is row-wise, so the key-side terms are computed per atom and the gather is left to ``run``
        qn = ops.layer_norm(queries_single)
        terms = []
        for i, (attn, ffn) in enumerate(zip(self.attn_blocks, self.ffn_blocks, strict=True)):
            cq, ck, cf = qn * self.attn_cond_w[i], qn * self.k_cond_w[i], qn * self.ffn_cond_w[i]
            vals = (
                logits[i] + key_bias,
                torch.sigmoid(self.attn_cond_scale[i](cq)),
                self.attn_cond_bias[i](cq),
                torch.sigmoid(self.k_cond_scale[i](ck)),
                self.k_cond_bias[i](ck),
                torch.sigmoid(attn["zero_cond"](queries_single)),
                torch.sigmoid(self.ffn_cond_scale[i](cf)),
                self.ffn_cond_bias[i](cf),
                torch.sigmoid(ffn["zero_cond"](queries_single)),
            )
            terms.append(AtomBlockTerms(*(v.unsqueeze(1) for v in vals)))
        return tuple(terms)

    def run(self, queries_act: torch.Tensor, terms: tuple[AtomBlockTerms, ...], layout: AtomLayout) -> torch.Tensor:
        """``queries_act`` ``[B, S, W, Q, c]`` through all blocks."""
        B, S, W, Q, C = queries_act.shape
        H, D, K = self.num_heads, self.head_dim, layout.K
        scale = D**-0.5
        for i, (attn, ffn, t) in enumerate(zip(self.attn_blocks, self.ffn_blocks, terms, strict=True)):
            # LayerNorm and the key / value projections act on rows, and the keys of a window are a gather of query
            # atoms (masked slots get a -1e9 logit bias), so they run once per atom (a quarter of the window-key rows)
            # and the gather moves the projected keys and values: gather(f(x)) = f(gather(x)) for row-wise f
            normed = self.attn_norms[i](queries_act)
            xq = t.q_scale * normed + t.q_bias
            xk = t.k_scale * normed + t.k_bias
            q = attn["to_q"](xq).view(B, S, W, Q, H, D).transpose(-2, -3)
            kv = queries_to_keys(layout, ops.stacked_linear(xk, attn["to_k"].weight, attn["to_v"].weight), sample_axis=True)
            k = kv[..., :C].view(B, S, W, K, H, D).transpose(-2, -3)
            v = kv[..., C:].view(B, S, W, K, H, D).transpose(-2, -3)
            out = ops.window_attention(q, k, v, t.logit_bias, scale)  # [B, S, W, H, Q, D]
            out = out.transpose(-2, -3).reshape(B, S, W, Q, C)
            out = out * torch.sigmoid(attn["to_g"](xq))
            queries_act = queries_act + t.attn_gate * attn["out_proj"](out)
            xf = t.ffn_scale * self.ffn_norms[i](queries_act) + t.ffn_bias
            queries_act = queries_act + t.ffn_gate * ffn["linear2"](ops.swiglu(ffn["linear1"](xf)))
        return queries_act

    def forward(self, queries_act, queries_mask, queries_single_cond, keys_single_cond, keys_mask, pair_cond,
                layout: AtomLayout):  # fmt: skip
        """Convenience form: ``queries_act`` ``[B, W, Q, c]`` (no sample axis)."""
        terms = self.block_terms(queries_single_cond, keys_single_cond, keys_mask, pair_cond)
        return self.run(queries_act.unsqueeze(1), terms, layout).squeeze(1)


def _offsets_valid(layout: AtomLayout, ref_space_uid):
    """``[B, W, Q, K]``: the two atoms share a reference conformer (token identity if no uid given)."""
    if ref_space_uid is None:
        return layout.token_of_query.unsqueeze(-1) == layout.token_of_key.unsqueeze(-2)
    uq = slots_to_queries(layout, ref_space_uid.unsqueeze(-1))
    uk = queries_to_keys(layout, uq)
    return uq.squeeze(-1).unsqueeze(-1) == uk.squeeze(-1).unsqueeze(-2)


class _WindowPairMixin:
    """Cross-window pair conditioning shared by the two encoders."""

    def _window_pair(self, layout, queries_single, keys_single, ref_pos, ref_space_uid, extra=None):
        q_pos = slots_to_queries(layout, ref_pos)
        k_pos = queries_to_keys(layout, q_pos)
        valid = _offsets_valid(layout, ref_space_uid).unsqueeze(-1)
        pair = self.single_to_pair_row_enc(F.relu(queries_single)).unsqueeze(-2)
        pair = pair + self.single_to_pair_col_enc(F.relu(keys_single)).unsqueeze(-3)
        off = q_pos.unsqueeze(-2) - k_pos.unsqueeze(-3)
        v = valid.to(pair.dtype)
        pair = pair + self.enc_embed_pair_offsets(off.to(pair.dtype)) * v
        inv = 1.0 / (1.0 + off.pow(2).sum(-1, keepdim=True))
        pair = pair + self.enc_embed_pair_distances(inv.to(pair.dtype)) * v
        pair = pair + self.enc_embed_offsets_valid(v)
        if extra is not None:
            pair = pair + extra
        return self.per_atom.apply_pair_mlp(pair)

    def _aggregate(self, layout, queries_act, ref_mask, sample_axis):
        """Masked mean over a token's atoms of ``relu(proj(queries_act))``."""
        atoms = queries_to_slots(layout, self.proj_for_aggr(queries_act), sample_axis=sample_axis)
        m = ref_mask.unsqueeze(1) if sample_axis else ref_mask
        denom = m.sum(-1, keepdim=True).clamp(min=1e-6)
        return (F.relu(atoms) * m.unsqueeze(-1).to(atoms.dtype)).sum(-2) / denom.to(atoms.dtype)


class EvoformerConditioningEncoder(nn.Module, _WindowPairMixin):
    """Reference conformer → per-token features ``[.., N, 384]`` fed to the trunk (reference: :872-998)."""

    def __init__(self, per_atom_channels=128, per_token_channels=384, per_atom_pair_channels=16, num_blocks=3, Q=32,
                 K=128, num_element_classes=128, num_atom_name_chars=64, atom_name_length=4,
                 ref_element_zero_index=False):  # fmt: skip
        super().__init__()
        c, cp = per_atom_channels, per_atom_pair_channels
        self.Q, self.K = Q, K
        self.per_atom = AtomPerAtomConditioning(
            c, cp, num_element_classes, num_atom_name_chars, atom_name_length, ref_element_zero_index
        )
        self.single_to_pair_row_enc = LinearNoBias(c, cp)
        self.single_to_pair_col_enc = LinearNoBias(c, cp)
        self.enc_embed_pair_offsets = LinearNoBias(3, cp)
        self.enc_embed_pair_distances = LinearNoBias(1, cp)
        self.enc_embed_offsets_valid = LinearNoBias(1, cp)
        self.atom_transformer = AtomCrossAttTransformer(c, cp, num_blocks=num_blocks)
        self.proj_for_aggr = LinearNoBias(c, per_token_channels)

    def forward(self, ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars, ref_space_uid=None):
        squeeze = ref_pos.dim() == 3
        if squeeze:
            ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars = (
                t.unsqueeze(0) for t in (ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars)
            )
            ref_space_uid = None if ref_space_uid is None else ref_space_uid.unsqueeze(0)
        layout = build_atom_layout(ref_mask.bool(), self.Q, self.K).trim()
        atom_single = self.per_atom.single_cond(ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars)
        q_single = slots_to_queries(layout, atom_single)
        k_single = queries_to_keys(layout, q_single)
        q_mask = layout.query_mask.to(atom_single.dtype)
        k_mask = layout.key_mask.to(atom_single.dtype)
        pair = self._window_pair(layout, q_single, k_single, ref_pos, ref_space_uid)
        act = self.atom_transformer(q_single, q_mask, q_single, k_single, k_mask, pair, layout)
        act = act * q_mask.unsqueeze(-1)
        tok = self._aggregate(layout, act, ref_mask, sample_axis=False)
        return tok.squeeze(0) if squeeze else tok


class AtomEncoder(nn.Module, _WindowPairMixin):
    """Diffusion atom encoder: conformer + trunk conditioning + noisy positions → token activations (:1001-1234)."""

    def __init__(self, per_atom_channels, per_token_channels, per_atom_pair_channels, atom_transformer_num_blocks=3,
                 Q=32, K=128, num_element_classes=128, num_atom_name_chars=64, atom_name_length=4,
                 ref_element_zero_index=False, c_trunk_single=384, c_trunk_pair=128):  # fmt: skip
        super().__init__()
        c, cp = per_atom_channels, per_atom_pair_channels
        self.Q, self.K = Q, K
        self.per_atom = AtomPerAtomConditioning(
            c, cp, num_element_classes, num_atom_name_chars, atom_name_length, ref_element_zero_index
        )
        self.lnorm_trunk_single_w = nn.Parameter(torch.ones(c_trunk_single))
        self.embed_trunk_single = LinearNoBias(c_trunk_single, c, initializer="zeros")
        self.lnorm_trunk_pair_w = nn.Parameter(torch.ones(c_trunk_pair))
        self.embed_trunk_pair = LinearNoBias(c_trunk_pair, cp, initializer="zeros")
        self.pair_chunk_budget = 0
        self.single_to_pair_row_enc = LinearNoBias(c, cp)
        self.single_to_pair_col_enc = LinearNoBias(c, cp)
        self.enc_embed_pair_offsets = LinearNoBias(3, cp)
        self.enc_embed_pair_distances = LinearNoBias(1, cp)
        self.enc_embed_offsets_valid = LinearNoBias(1, cp)
        self._pos_proj = LinearNoBias(3, c)
        self.atom_transformer = AtomCrossAttTransformer(c, cp, num_blocks=atom_transformer_num_blocks)
        self.proj_for_aggr = LinearNoBias(c, per_token_channels)

    def compute_static(self, ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars, trunk_single,
                       trunk_pair, ref_space_uid=None, decoder: "AtomDecoder | None" = None) -> AtomEncoderStatic:  # fmt: skip
        """All noise-independent state, inputs ``[B, ...]``. ``decoder`` also gets its block terms cached."""
        B, N = ref_pos.shape[0], ref_pos.shape[1]
        layout = build_atom_layout(ref_mask.bool(), self.Q, self.K).trim()
        atom_single = self.per_atom.single_cond(ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars)
        ts = self.embed_trunk_single(ops.layer_norm(trunk_single, self.lnorm_trunk_single_w, None))
        atom_single = atom_single + ts.unsqueeze(-2)
        q_single = slots_to_queries(layout, atom_single)
        k_single = queries_to_keys(layout, q_single)
        q_mask = layout.query_mask.to(atom_single.dtype)
        k_mask = layout.key_mask.to(atom_single.dtype)
        tp = map_pair_rows(
            lambda rows: self.embed_trunk_pair(ops.layer_norm(rows, self.lnorm_trunk_pair_w, None)), trunk_pair,
            self.pair_chunk_budget, 4 * trunk_pair.shape[-1],
        )  # fmt: skip
        pair_idx = layout.token_of_query.unsqueeze(-1) * N + layout.token_of_key.unsqueeze(-2)  # [B, W, Q, K]
        pair_ok = layout.query_mask.unsqueeze(-1) & layout.key_mask.unsqueeze(-2)
        cp = tp.shape[-1]
        contrib = torch.gather(tp.reshape(B, N * N, cp), 1, pair_idx.reshape(B, -1, 1).expand(B, -1, cp))
        contrib = contrib.reshape(*pair_idx.shape, cp) * pair_ok.unsqueeze(-1).to(tp.dtype)
        pair = self._window_pair(layout, q_single, k_single, ref_pos, ref_space_uid, extra=contrib)
        static = AtomEncoderStatic(layout, q_single, q_mask, k_single, k_mask, pair, ref_mask)
        static.encoder_terms = self.atom_transformer.block_terms(q_single, k_single, k_mask, pair)
        if decoder is not None:
            static.decoder_terms = decoder.atom_transformer.block_terms(q_single, k_single, k_mask, pair)
        return static

    def forward(self, noisy_atom_pos, static: AtomEncoderStatic) -> AtomEncoderOutput:
        """``noisy_atom_pos`` ``[B, S, N, M, 3]`` (or ``None``) → token activations ``[B, S, N, ct]``."""
        layout = static.layout
        q0 = static.queries_single.unsqueeze(1)
        if noisy_atom_pos is not None:
            nq = slots_to_queries(layout, noisy_atom_pos, sample_axis=True)
            act = q0 + self._pos_proj(nq.to(q0.dtype)) * static.queries_mask[:, None, :, :, None]
        else:
            act = q0
        act = self.atom_transformer.run(act, static.encoder_terms, layout)
        act = act * static.queries_mask[:, None, :, :, None]
        tok = self._aggregate(layout, act, static.ref_mask, sample_axis=True)
        return AtomEncoderOutput(token_act=tok, skip_connection=act, static=static)


class AtomDecoder(nn.Module):
    """Token activations → per-atom position update (reference: atom_cross_attn.py:1237-1307)."""

    def __init__(self, per_atom_channels, per_token_channels, per_atom_pair_channels, atom_transformer_num_blocks=3):
        super().__init__()
        c = per_atom_channels
        self.proj_tokens = LinearNoBias(per_token_channels, c)
        self.atom_transformer = AtomCrossAttTransformer(
            c, per_atom_pair_channels, num_blocks=atom_transformer_num_blocks
        )
        self.atom_norm_w = nn.Parameter(torch.ones(c))
        self.pos_update = LinearNoBias(c, 3, initializer="zeros")

    def forward(self, token_act: torch.Tensor, enc: AtomEncoderOutput) -> torch.Tensor:
        """``token_act`` ``[B, S, N, ct]`` → ``[B, S, N, M, 3]``."""
        static, layout = enc.static, enc.static.layout
        B, S = token_act.shape[:2]
        tok = self.proj_tokens(token_act)  # [B, S, N, c]
        qmask = static.queries_mask[:, None, :, :, None]
        # broadcast token → its atoms: gather rows by the token index of each query slot
        idx = layout.token_of_query.reshape(B, 1, -1, 1).expand(B, S, -1, tok.shape[-1])
        act = torch.gather(tok, 2, idx).reshape(B, S, layout.num_windows, layout.Q, -1) * qmask.to(tok.dtype)
        act = (act + enc.skip_connection) * qmask.to(tok.dtype)
        terms = static.decoder_terms
        if terms is None:
            terms = self.atom_transformer.block_terms(
                static.queries_single, static.keys_single, static.keys_mask, static.atom_pair
            )
        act = self.atom_transformer.run(act, terms, layout) * qmask.to(tok.dtype)
        upd = self.pos_update(ops.layer_norm(act, self.atom_norm_w, None))
        return queries_to_slots(layout, upd, sample_axis=True)
