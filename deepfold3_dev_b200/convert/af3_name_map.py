"""The table that relates AlphaFold 3's Haiku parameter scopes to this model's state-dict keys, and the two
converters it drives (``haiku_to_torch``, ``torch_to_haiku``).

An AF3 parameter file is ``{scope: {name: array}}``. A scope holds one Haiku module's arrays; a module built under
``hk.experimental.layer_stack`` stores every array with the layer index as leading axis (two leading axes for the
diffusion transformer: super-block, block). The table below says, per scope,

* the module here that owns the arrays (a state-dict prefix, with ``{i}`` for the layer index),
* the *kind* of the scope, which fixes how arrays are renamed and re-laid-out:

    ``lin``   Haiku Linear storing ``weights [in, *out]`` (+ ``bias``)       -> ``.weight [prod(out), in]``, ``.bias``
    ``lint``  Haiku Linear with transposed storage ``weights [*out, in]``    -> ``.weight [prod(out), in]``
    ``ln``    LayerNorm ``scale`` / ``offset``                               -> ``.weight`` / ``.bias``
    ``gain``  LayerNorm without offset, kept here as a bare parameter       -> the key itself
    ``scal``  Linear on a scalar input, ``weights [out]``                    -> ``.weight [out, 1]``
    ``raw``   arrays created with ``hk.get_parameter`` under given names     -> given keys, unchanged

* the number of leading stack axes.

Composite modules (triangle multiply, grid attention, Pairformer block, ...) are written once as
``{sub-scope: (kind, key suffix)}`` dictionaries and instantiated wherever they occur. The same table read backwards
re-stacks a state dict into AF3's layout, which is how the map is tested without the published checkpoint: a random
state dict of this model goes to the Haiku layout and back, and the reference implementation's converter
(convert/af3.py:274-913) must produce the same tensors from the same Haiku arrays.
"""

from __future__ import annotations

import re
import warnings
from dataclasses import dataclass

import numpy as np
import torch

# ---- composite modules: {haiku sub-scope: (kind, torch suffix)} ------------------------------------------------------------
TRI_MUL = {
    "left_norm_input": ("ln", "norm_left"), "projection": ("lin", "proj"), "gate": ("lin", "gate"),
    "center_norm": ("ln", "norm_center"), "output_projection": ("lin", "out_proj"), "gating_linear": ("lin", "out_gate"),
}  # fmt: skip
GRID_ATTN = {  # q, k and the gate are stored output-major in AF3's GridSelfAttention
    "act_norm": ("ln", "norm"), "pair_bias_projection": ("lin", "pair_bias"), "q_projection": ("lint", "to_q"),
    "k_projection": ("lint", "to_k"), "v_projection": ("lin", "to_v"), "gating_query": ("lint", "to_g"),
    "output_projection": ("lin", "out_proj"),
}  # fmt: skip
MSA_ATTN = {
    "act_norm": ("ln", "norm"), "pair_norm": ("ln", "pair_norm"), "pair_logits": ("lin", "pair_logits"),
    "v_projection": ("lin", "to_v"), "gating_query": ("lin", "to_g"), "output_projection": ("lin", "out_proj"),
}  # fmt: skip
TRANSITION = {"input_layer_norm": ("ln", "norm"), "transition1": ("lin", "linear1"), "transition2": ("lin", "linear2")}
OUTER_PRODUCT = {
    "": ("raw", {"output_w": "out_w", "output_b": "out_b"}), "layer_norm_input": ("ln", "norm"),
    "left_projection": ("lin", "proj_a"), "right_projection": ("lin", "proj_b"),
}  # fmt: skip
SINGLE_TRACK = {  # stored flat in the Pairformer scope, names prefixed "single_attention_"
    "single_attention_layer_norm": ("ln", "single_attn.norm"), "single_attention_q_projection": ("lin", "single_attn.to_q"),
    "single_attention_k_projection": ("lin", "single_attn.to_k"), "single_attention_v_projection": ("lin", "single_attn.to_v"),
    "single_attention_gating_query": ("lin", "single_attn.to_g"), "single_attention_transition2": ("lin", "single_attn.out_proj"),
    "single_pair_logits_norm": ("ln", "single_to_pair_norm"), "single_pair_logits_projection": ("lin", "single_to_pair"),
}  # fmt: skip


def _nest(prefix_h: str, prefix_t: str, block: dict) -> dict:
    """``block`` placed under Haiku sub-scope ``prefix_h`` and state-dict sub-module ``prefix_t``."""
    out = {}
    for sub, (kind, suffix) in block.items():
        scope = prefix_h + ("/" + sub if sub and prefix_h else sub)
        out[scope] = (kind, suffix if kind == "raw" else (f"{prefix_t}.{suffix}" if prefix_t else suffix), prefix_t)
    return out


def _pair_stack(with_single: bool) -> dict:
    block = {}
    block.update(_nest("triangle_multiplication_outgoing", "tri_mul_out", TRI_MUL))
    block.update(_nest("triangle_multiplication_incoming", "tri_mul_in", TRI_MUL))
    block.update(_nest("pair_attention1", "pair_attn_row", GRID_ATTN))
    block.update(_nest("pair_attention2", "pair_attn_col", GRID_ATTN))
    block.update(_nest("pair_transition", "pair_transition", TRANSITION))
    if with_single:
        block.update(_nest("", "", SINGLE_TRACK))
        block.update(_nest("single_transition", "single_transition", TRANSITION))
    return block


PAIRFORMER_BLOCK = _pair_stack(with_single=True)
TEMPLATE_BLOCK = _pair_stack(with_single=False)
EVOFORMER_BLOCK = {
    **_nest("msa_attention1", "row_attn", MSA_ATTN), **_nest("outer_product_mean", "outer_product", OUTER_PRODUCT),
    **_nest("msa_transition", "msa_transition", TRANSITION), **_pair_stack(with_single=False),
}  # fmt: skip

# per-atom conditioning, shared by the diffusion atom encoder and the trunk's conditioning encoder
PER_ATOM = {
    "embed_ref_pos": "per_atom.embed_ref_pos", "embed_ref_mask": "per_atom.embed_ref_mask",
    "embed_ref_element": "per_atom.embed_ref_element", "embed_ref_charge": "per_atom.embed_ref_charge",
    "embed_ref_atom_name": "per_atom.embed_ref_atom_name", "single_to_pair_cond_row": "per_atom.single_to_pair_row",
    "single_to_pair_cond_col": "per_atom.single_to_pair_col", "embed_pair_offsets": "per_atom.embed_pair_offsets",
    "embed_pair_distances": "per_atom.embed_pair_distances", "pair_mlp_1": "per_atom.pair_mlp1", "pair_mlp_2": "per_atom.pair_mlp2",
    "pair_mlp_3": "per_atom.pair_mlp3",
    # the encoder's own second set
    "single_to_pair_cond_row_1": "single_to_pair_row_enc", "single_to_pair_cond_col_1": "single_to_pair_col_enc",
    "embed_pair_offsets_1": "enc_embed_pair_offsets", "embed_pair_distances_1": "enc_embed_pair_distances",
    "embed_pair_offsets_valid": "enc_embed_offsets_valid", "project_atom_features_for_aggr": "proj_for_aggr",
}  # fmt: skip

# one block of an atom cross-attention transformer; Haiku glues the module name in front of these names without a
# separator ("diffusion_atom_transformer_encoderq_projection"). Values: (kind, key template with {p} = transformer
# prefix and {i} = block index).
ATOM_BLOCK = {
    "qsingle_cond_layer_norm": ("gain", "{p}.attn_cond_w.{i}"), "qsingle_cond_scale": ("lin", "{p}.attn_cond_scale.{i}"),
    "qsingle_cond_bias": ("lin", "{p}.attn_cond_bias.{i}"), "ksingle_cond_layer_norm": ("gain", "{p}.k_cond_w.{i}"),
    "ksingle_cond_scale": ("lin", "{p}.k_cond_scale.{i}"), "ksingle_cond_bias": ("lin", "{p}.k_cond_bias.{i}"),
    "q_projection": ("lin", "{p}.attn_blocks.{i}.to_q"), "k_projection": ("lin", "{p}.attn_blocks.{i}.to_k"),
    "v_projection": ("lin", "{p}.attn_blocks.{i}.to_v"), "gating_query": ("lin", "{p}.attn_blocks.{i}.to_g"),
    "transition2": ("lin", "{p}.attn_blocks.{i}.out_proj"), "adaptive_zero_cond": ("lin", "{p}.attn_blocks.{i}.zero_cond"),
    "ffw_single_cond_layer_norm": ("gain", "{p}.ffn_cond_w.{i}"), "ffw_single_cond_scale": ("lin", "{p}.ffn_cond_scale.{i}"),
    "ffw_single_cond_bias": ("lin", "{p}.ffn_cond_bias.{i}"), "ffw_transition1": ("lin", "{p}.ffn_blocks.{i}.linear1"),
    "ffw_transition2": ("lin", "{p}.ffn_blocks.{i}.linear2"), "ffw_adaptive_zero_cond": ("lin", "{p}.ffn_blocks.{i}.zero_cond"),
}  # fmt: skip
# one block of the diffusion transformer (two stack axes: layer = super-block * blocks per super-block + block)
DIFFUSION_BLOCK = {
    "single_cond_layer_norm": ("gain", "attn_cond_norm_w"), "single_cond_scale": ("lin", "attn_cond_scale"),
    "single_cond_bias": ("lin", "attn_cond_bias"), "q_projection": ("lin", "to_q"), "k_projection": ("lin", "to_k"),
    "v_projection": ("lin", "to_v"), "gating_query": ("lin", "to_g"), "transition2": ("lin", "out_proj"),
    "adaptive_zero_cond": ("lin", "zero_cond"), "ffw_single_cond_layer_norm": ("gain", "ffn_cond_norm_w"),
    "ffw_single_cond_scale": ("lin", "ffn_cond_scale"), "ffw_single_cond_bias": ("lin", "ffn_cond_bias"),
    "ffw_transition1": ("lin", "ffn_linear1"), "ffw_transition2": ("lin", "ffn_linear2"), "ffw_adaptive_zero_cond": ("lin", "ffn_zero_cond"),
}  # fmt: skip
TEMPLATE_EMBEDS = (("embed_dgram", "lin"), ("embed_pseudo_beta", "scal"), ("embed_aatype_row", "lin"), ("embed_aatype_col", "lin"),
                   ("embed_unit_vec_x", "scal"), ("embed_unit_vec_y", "scal"), ("embed_unit_vec_z", "scal"),
                   ("embed_backbone_mask", "scal"), ("embed_query", "lin"))  # fmt: skip


@dataclass(frozen=True)
class Entry:
    scope: str      # full Haiku scope
    kind: str
    key: object     # state-dict key (template with {i}); for "raw": {haiku name: key template}
    stack: int = 0  # leading layer axes


def _entries() -> list[Entry]:
    E: list[Entry] = []

    def add(scope, kind, key, stack=0):
        E.append(Entry(scope, kind, key, stack))

    def add_block(base_scope: str, base_key: str, block: dict, stack: int):
        for sub, (kind, suffix, owner) in block.items():
            if kind == "raw":
                prefix = f"{base_key}.{owner}" if owner else base_key
                add(base_scope + sub, kind, {h: f"{prefix}.{t}" for h, t in suffix.items()}, stack)
            else:
                add(base_scope + sub, kind, f"{base_key}.{suffix}", stack)

    evo = "diffuser/evoformer/"
    for name in ("left_single", "right_single", "bond_embedding", "prev_embedding", "prev_single_embedding", "single_activations",
                 "msa_activations", "extra_msa_target_feat"):  # fmt: skip
        add(evo + name, "lin", f"evoformer.{name}")
    add(evo + "~_relative_encoding/position_activations", "lin", "evoformer.position_activations")
    add(evo + "prev_embedding_layer_norm", "ln", "evoformer.prev_embedding_layer_norm")
    add(evo + "prev_single_embedding_layer_norm", "ln", "evoformer.prev_single_embedding_layer_norm")
    add_block(evo + "__layer_stack_no_per_layer/msa_stack/", "evoformer.msa_stack.{i}", EVOFORMER_BLOCK, 1)
    add_block(evo + "__layer_stack_no_per_layer_1/trunk_pairformer/", "evoformer.trunk_pairformer.{i}", PAIRFORMER_BLOCK, 1)

    conf = "diffuser/confidence_head/"
    add_block(conf + "__layer_stack_no_per_layer/confidence_pairformer/", "confidence_head.layers.{i}", PAIRFORMER_BLOCK, 1)
    for name in ("left_target_feat_project", "right_target_feat_project", "distogram_feat_project"):
        add(conf + "~_embed_features/" + name, "lin", f"confidence_head.{name}")
    for haiku, here in (("plddt_logits", "plddt_logits"), ("pae_logits", "pae_logits"), ("left_half_distance_logits", "pde_half_logits"),
                        ("experimentally_resolved_logits", "exp_resolved_logits")):  # fmt: skip
        add(conf + haiku, "lin", f"confidence_head.{here}")
    for haiku, here in (("plddt_logits_ln", "plddt_logits_ln"), ("pae_logits_ln", "pae_logits_ln"), ("logits_ln", "pde_logits_ln"),
                        ("experimentally_resolved_ln", "exp_resolved_ln")):  # fmt: skip
        add(conf + haiku, "ln", f"confidence_head.{here}")
    add("diffuser/distogram_head/half_logits", "lin", "distogram_head.half_logits")

    dh, dk = "diffuser/~/diffusion_head/", "diffusion_head"
    for what in ("pair_cond", "single_cond", "noise_embedding"):
        short = "noise_emb" if what == "noise_embedding" else what
        add(dh + f"{what}_initial_norm", "gain", f"{dk}.conditioning.{short}_norm_w")
        add(dh + f"{what}_initial_projection", "lin", f"{dk}.conditioning.{short}_proj")
    for idx in (0, 1):
        for track, here in (("pair_transition", "pair_trans"), ("single_transition", "single_trans")):
            base = dh + f"{track}_{idx}"
            add(base + "ffw_layer_norm", "ln", f"{dk}.conditioning.{here}{idx}.norm")
            add(base + "ffw_transition1", "lin", f"{dk}.conditioning.{here}{idx}.linear1")
            add(base + "ffw_transition2", "lin", f"{dk}.conditioning.{here}{idx}.linear2")
    add(dh + "single_cond_embedding_norm", "gain", f"{dk}.single_cond_emb_norm_w")
    add(dh + "single_cond_embedding_projection", "lin", f"{dk}.single_cond_embedding_projection")
    add(dh + "transformer/pair_input_layer_norm", "gain", f"{dk}.transformer.pair_norm_w")
    add(dh + "output_norm", "gain", f"{dk}.transformer.output_norm_w")
    stack = dh + "transformer/__layer_stack_with_per_layer/"
    add(stack + "pair_logits_projection", "lin", f"{dk}.transformer.pair_logits_proj.{{i}}", 1)
    for name, (kind, suffix) in DIFFUSION_BLOCK.items():
        add(stack + "__layer_stack_with_per_layer/transformer" + name, kind, f"{dk}.transformer.layers.{{i}}.{suffix}", 2)

    for scope_prefix, here in ((dh + "diffusion_", f"{dk}.atom_encoder"), ("diffuser/evoformer_conditioning_", "evo_cond_encoder")):
        for haiku, suffix in PER_ATOM.items():
            add(scope_prefix + haiku, "lin", f"{here}.{suffix}")
    enc = dh + "diffusion_"
    add(enc + "lnorm_trunk_single_cond", "gain", f"{dk}.atom_encoder.lnorm_trunk_single_w")
    add(enc + "embed_trunk_single_cond", "lin", f"{dk}.atom_encoder.embed_trunk_single")
    add(enc + "lnorm_trunk_pair_cond", "gain", f"{dk}.atom_encoder.lnorm_trunk_pair_w")
    add(enc + "embed_trunk_pair_cond", "lin", f"{dk}.atom_encoder.embed_trunk_pair")
    add(enc + "atom_positions_to_features", "lin", f"{dk}.atom_encoder._pos_proj")
    add(enc + "project_token_features_for_broadcast", "lin", f"{dk}.atom_decoder.proj_tokens")
    add(enc + "atom_features_layer_norm", "gain", f"{dk}.atom_decoder.atom_norm_w")
    add(enc + "atom_features_to_position_update", "lin", f"{dk}.atom_decoder.pos_update")
    for module, here in (("diffusion_atom_transformer_encoder", f"{dk}.atom_encoder.atom_transformer"),
                         ("diffusion_atom_transformer_decoder", f"{dk}.atom_decoder.atom_transformer"),
                         ("evoformer_conditioning_atom_transformer_encoder", "evo_cond_encoder.atom_transformer")):  # fmt: skip
        outer = ("diffuser/" if module.startswith("evoformer") else dh) + module + "/"
        add(outer + "pair_input_layer_norm", "gain", f"{here}.pair_norm_w")
        add(outer + "pair_logits_projection", "lin", f"{here}.pair_logits_proj")
        for name, (kind, template) in ATOM_BLOCK.items():
            add(outer + "__layer_stack_with_per_layer/" + module + name, kind, template.replace("{p}", here), 1)

    te, tk = evo + "template_embedding/", "evoformer.template_embedding"
    ste, sk = te + "single_template_embedding/", f"{tk}.single_template_emb"
    add(te + "output_linear", "lin", f"{tk}.output_proj")
    add(ste + "query_embedding_norm", "ln", f"{sk}.query_norm")
    add(ste + "output_layer_norm", "ln", f"{sk}.output_norm")
    for n, (name, kind) in enumerate(TEMPLATE_EMBEDS):
        add(ste + f"template_pair_embedding_{n}", kind, f"{sk}.{name}")
    add_block(ste + "__layer_stack_no_per_layer/template_embedding_iteration/", f"{sk}.pairformer.{{i}}", TEMPLATE_BLOCK, 1)
    return E


ENTRIES = _entries()
BY_SCOPE = {e.scope: e for e in ENTRIES}


# ---- array conversions --------------------------------------------------------------------------------------------------------
def _t(a) -> torch.Tensor:
    return torch.from_numpy(np.array(a, dtype=np.float32, copy=True))


def _forward(kind: str, key, arrays: dict) -> dict[str, torch.Tensor]:
    """One layer's arrays of one scope -> state-dict entries."""
    out = {}
    if kind in ("lin", "lint", "scal"):
        if "weights" in arrays:
            w = np.asarray(arrays["weights"])
            if kind == "lin":
                w = w.reshape(w.shape[0], -1).T
            elif kind == "lint":
                w = w.reshape(-1, w.shape[-1])
            else:
                w = w.reshape(-1, 1)
            out[f"{key}.weight"] = _t(w)
        if "bias" in arrays and kind != "scal":
            out[f"{key}.bias"] = _t(np.asarray(arrays["bias"]).reshape(-1))
    elif kind == "ln":
        if "scale" in arrays:
            out[f"{key}.weight"] = _t(np.asarray(arrays["scale"]).reshape(-1))
        if "offset" in arrays:
            out[f"{key}.bias"] = _t(np.asarray(arrays["offset"]).reshape(-1))
    elif kind == "gain":
        if "scale" in arrays:
            out[key] = _t(np.asarray(arrays["scale"]).reshape(-1))
    elif kind == "raw":
        for haiku_name, torch_key in key.items():
            if haiku_name in arrays:
                out[torch_key] = _t(arrays[haiku_name])
    else:
        raise ValueError(f"unknown array kind {kind!r}")
    return out


def _backward(kind: str, key, sd: dict) -> dict[str, np.ndarray]:
    """State-dict entries of one layer -> that scope's Haiku arrays (2-D weights: the reader reshapes trailing axes)."""
    get = lambda k: sd[k].detach().float().cpu().numpy() if k in sd else None  # noqa: E731
    out = {}
    if kind in ("lin", "lint", "scal"):
        w = get(f"{key}.weight")
        if w is not None:
            out["weights"] = w.T.copy() if kind == "lin" else (w.copy() if kind == "lint" else w.reshape(-1).copy())
        b = get(f"{key}.bias")
        if b is not None and kind != "scal":
            out["bias"] = b
    elif kind == "ln":
        for haiku_name, suffix in (("scale", "weight"), ("offset", "bias")):
            v = get(f"{key}.{suffix}")
            if v is not None:
                out[haiku_name] = v
    elif kind == "gain":
        v = get(key)
        if v is not None:
            out["scale"] = v
    elif kind == "raw":
        for haiku_name, torch_key in key.items():
            v = get(torch_key)
            if v is not None:
                out[haiku_name] = v
    return out


def _fmt(key, i: int):
    return {h: k.replace("{i}", str(i)) for h, k in key.items()} if isinstance(key, dict) else key.replace("{i}", str(i))


def haiku_to_torch(params: dict) -> dict[str, torch.Tensor]:
    sd: dict[str, torch.Tensor] = {}
    for scope, arrays in params.items():
        entry = BY_SCOPE.get(scope)
        if entry is None:
            if not scope.startswith("__meta__"):
                warnings.warn(f"AF3 conversion: scope {scope!r} is not in the name map and was left out", stacklevel=2)
            continue
        if entry.stack == 0:
            sd.update(_forward(entry.kind, entry.key, arrays))
            continue
        lead = next(iter(arrays.values())).shape[: entry.stack]
        for index in np.ndindex(*lead):
            layer = int(np.ravel_multi_index(index, lead))
            sd.update(_forward(entry.kind, _fmt(entry.key, layer), {n: np.asarray(a)[index] for n, a in arrays.items()}))
    return sd


_LAYER = re.compile(r"\.(\d+)(?=\.|$)")


def torch_to_haiku(state_dict: dict, blocks_per_super: int | None = None) -> dict:
    """Re-stack a state dict into AF3's ``{scope: {name: array}}``. ``blocks_per_super`` (default: read from the number of
    ``pair_logits_proj`` entries) splits the diffusion transformer's layer index into its two stack axes."""
    params: dict = {}
    n_super = len({k for k in state_dict if re.fullmatch(r"diffusion_head\.transformer\.pair_logits_proj\.\d+\.weight", k)})
    for entry in ENTRIES:
        if entry.stack == 0:
            arrays = _backward(entry.kind, entry.key, state_dict)
            if arrays:
                params[entry.scope] = arrays
            continue
        layers = []
        while True:
            arrays = _backward(entry.kind, _fmt(entry.key, len(layers)), state_dict)
            if not arrays:
                break
            layers.append(arrays)
        if not layers:
            continue
        stacked = {n: np.stack([layer[n] for layer in layers]) for n in layers[0]}
        if entry.stack == 2:
            per = blocks_per_super or (len(layers) // max(n_super, 1))
            stacked = {n: a.reshape(len(layers) // per, per, *a.shape[1:]) for n, a in stacked.items()}
        params[entry.scope] = stacked
    return params
