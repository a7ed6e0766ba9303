"""Shared builders for the tests: small configs, synthetic batches, zero-init wake-up."""

import torch


def small_full_width(C):
    """Depth-1 model at the full AF3 channel widths (the reference only supports those widths)."""
    cfg = C.ModelConfig()
    cfg.evoformer.num_layer = 1
    cfg.pairformer.num_layer = 1
    cfg.confidence.num_layer = 1
    cfg.template.pairformer.num_layer = 1
    cfg.diffusion.transformer.num_blocks = 2
    cfg.diffusion.transformer.super_block_size = 2
    cfg.diffusion.atom_cross_att.atom_transformer.num_blocks = 1
    cfg.diffusion.steps = 3
    cfg.diffusion.num_samples = 2
    cfg.num_recycles = 1
    cfg.msa_crop_size = 8
    return cfg


def tiny_config():
    """Narrow model of BASELINE config 1: c_m 16, c_s 64, c_z 32, 1 MSA block, 2 Pairformer blocks, 2 diffusion blocks."""
    from deepfold3_dev_b200.config.schema import ModelConfig

    c = ModelConfig()
    c.evoformer.num_layer = 1
    c.evoformer.msa_channel = 16
    c.evoformer.seq_channel = 64
    c.evoformer.pair_channel = 32
    c.evoformer.msa_attention.num_head = 4
    c.evoformer.outer_product_num_channel = 8
    c.pairformer.num_layer = 2
    c.pairformer.pair_channel = 32
    c.pairformer.seq_channel = 64
    c.pairformer.single_attention_num_head = 4
    c.pairformer.single_key_dim = 64
    c.pairformer.single_value_dim = 64
    c.diffusion.transformer.num_blocks = 2
    c.diffusion.transformer.super_block_size = 2
    c.diffusion.transformer.num_head = 4
    c.diffusion.atom_cross_att.per_token_channels = 64
    c.diffusion.atom_cross_att.per_atom_channels = 32
    c.diffusion.atom_cross_att.atom_transformer.num_blocks = 1
    c.diffusion.conditioning_pair_channel = 32
    c.diffusion.conditioning_seq_channel = 64
    c.diffusion.fourier_dim = 32
    c.confidence.num_layer = 1
    c.confidence.pair_channel = 32
    c.confidence.seq_channel = 64
    c.confidence.single_attention_num_head = 4
    c.template.pair_channel = 32
    c.template.num_channels = 16
    c.template.pairformer.num_layer = 1
    c.template.pairformer.num_channels = 16
    c.msa_crop_size = 16
    return c


def wake_zero_init(model, seed=1, scale=0.05):
    """Perturb zero-initialised and 1-D parameters so wiring mistakes cannot hide behind zero outputs."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            if p.abs().sum() == 0 or p.dim() < 2:
                p.add_(torch.randn(p.shape, generator=g).to(p.device) * scale)
