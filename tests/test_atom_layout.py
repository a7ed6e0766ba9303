import torch

from deepfold3_dev_b200.models.atom_layout import (
    build_atom_layout,
    queries_to_keys,
    queries_to_slots,
    slots_to_queries,
)


def test_roundtrip_and_trim():
    torch.manual_seed(0)
    mask = torch.rand(2, 13, 24) < 0.3
    layout = build_atom_layout(mask, 32, 128)
    x = torch.randn(2, 13, 24, 5) * mask.unsqueeze(-1)
    q = slots_to_queries(layout, x)
    assert q.shape == (2, layout.num_windows, 32, 5)
    torch.testing.assert_close(queries_to_slots(layout, q), x)
    trimmed = layout.trim()
    assert trimmed.num_windows == max(1, -(-int(mask.flatten(1).sum(1).max()) // 32))
    qt = slots_to_queries(trimmed, x)
    torch.testing.assert_close(queries_to_slots(trimmed, qt), x)
    k_full = queries_to_keys(layout, q)[:, : trimmed.num_windows]
    torch.testing.assert_close(queries_to_keys(trimmed, qt), k_full)


def test_sample_axis():
    mask = torch.rand(1, 9, 24) < 0.5
    layout = build_atom_layout(mask).trim()
    x = torch.randn(1, 3, 9, 24, 4) * mask[:, None, :, :, None]
    q = slots_to_queries(layout, x, sample_axis=True)
    for s in range(3):
        torch.testing.assert_close(q[:, s], slots_to_queries(layout, x[:, s]))
    torch.testing.assert_close(queries_to_slots(layout, q, sample_axis=True), x)


def test_matches_reference(reference_package):
    from deepfold3.model.atom_cross_attn import build_atom_subsets

    mask = torch.rand(2, 11, 24, generator=torch.Generator().manual_seed(1)) < 0.4
    ref, mine = build_atom_subsets(mask, 32, 128), build_atom_layout(mask, 32, 128)
    for a, b in (("ta_to_q_idx", "slot_of_query"), ("ta_to_q_mask", "query_mask"), ("q_to_k_mask", "key_mask"),
                 ("token_for_query", "token_of_query"), ("token_for_key", "token_of_key"),
                 ("q_to_ta_idx", "query_of_slot"), ("q_to_ta_mask", "slot_mask")):  # fmt: skip
        assert torch.equal(getattr(ref, a), getattr(mine, b)), a
    assert torch.equal(ref.q_to_k_idx[0], mine.key_of_window)
