"""CPU checks of the DeepSeek-V4 operator oracles (`ferrule_b200.models.v4`): golden vectors of the
hyper-connection math, compressor window semantics, indexer ordering, window selection."""
import torch

from ferrule_b200.models import v4
from ferrule_b200.ops import reference as ref

TINY = v4.HcConfig(hc=2, hidden=2, eps=1e-6, norm_eps=1e-6, sinkhorn_iters=3)


def test_split_zero_mixes_gives_half_pre_unit_post_and_normalised_columns():
    pre, post, comb = v4.hc_split_sinkhorn(torch.zeros(1, TINY.mix), torch.ones(3), torch.zeros(TINY.mix), TINY)
    assert torch.allclose(pre, torch.full((1, 2), 0.5 + TINY.eps))
    assert torch.equal(post, torch.ones(1, 2))
    assert torch.allclose(comb.sum(1), torch.ones(1, 2), atol=1e-5)


def test_post_mixes_residual_through_comb_columns():
    out = v4.hc_post(torch.tensor([[10.0, 20.0]]), torch.tensor([[[5.0, 7.0], [11.0, 13.0]]]),
                     torch.zeros(1, 2), torch.tensor([[[0.0, 1.0], [2.0, 3.0]]]))
    assert out.flatten().tolist() == [22.0, 26.0, 38.0, 46.0]


def test_head_reduces_copies_with_half_weights():
    state = torch.tensor([[[1.0, 2.0], [3.0, 4.0]]])
    out = v4.hc_head(state, torch.zeros(2, 4), torch.ones(1), torch.zeros(2), TINY)
    assert torch.allclose(out, torch.tensor([[(0.5 + 1e-6) * 4.0, (0.5 + 1e-6) * 6.0]]))


def test_pre_then_post_roundtrip_shapes():
    state = torch.tensor([[[1.0, 2.0], [3.0, 4.0]]])
    hidden, (pre, post, comb) = v4.hc_pre(state, torch.zeros(TINY.mix, 4), torch.ones(3), torch.zeros(TINY.mix), TINY)
    out = v4.hc_post(hidden, state, post, comb)
    assert hidden.shape == (1, 2) and out.shape == state.shape and out[0, 0, 0] > state[0, 0, 0]


def test_compressor_window_and_overlap_masking():
    torch.manual_seed(0)
    kv, gate = torch.randn(8, 4), torch.randn(8, 4)
    plain = v4.compressor_pool(kv, gate, torch.zeros(4, 4), ratio=4, overlap=False)
    want = (torch.softmax(gate[:4], 0) * kv[:4]).sum(0)
    assert torch.allclose(plain[0], ref.bf16_round(want))
    # overlap: projection rows are [previous-window half | current-window half]
    kv2, gate2 = torch.randn(8, 8), torch.randn(8, 8)
    over = v4.compressor_pool(kv2, gate2, torch.zeros(4, 8), ratio=4, overlap=True)
    want0 = (torch.softmax(gate2[:4, 4:], 0) * kv2[:4, 4:]).sum(0)          # nothing before the sequence start
    assert torch.allclose(over[0], ref.bf16_round(want0))
    sc = torch.cat([gate2[:4, :4], gate2[4:, 4:]])
    vals = torch.cat([kv2[:4, :4], kv2[4:, 4:]])
    assert torch.allclose(over[1], ref.bf16_round((torch.softmax(sc, 0) * vals).sum(0)))


def test_indexer_topk_is_stable_and_marks_unused_slots():
    q = torch.ones(2, 4)
    rows = torch.tensor([[1.0] * 4, [2.0] * 4, [1.0] * 4, [float("nan")] * 4, [3.0] * 4])
    idx, score = v4.indexer_topk(q, rows, torch.ones(2), k=6, n_visible=4)
    assert idx.tolist() == [1, 0, 2, -1, -1, -1]                # row 4 is not visible, row 3 is not finite
    assert score[1] == 16.0


def test_sliding_window_indices_clip_at_sequence_start():
    assert v4.sliding_window_indices(2, 4).tolist() == [-1, 0, 1, 2]
    assert v4.sliding_window_indices(9, 4).tolist() == [6, 7, 8, 9]


def test_sparse_attention_ignores_masked_rows_and_honours_sink():
    torch.manual_seed(1)
    table = torch.randn(10, 12)
    q = torch.randn(1, 2, 12)
    sel = torch.tensor([[3, -1, 7]], dtype=torch.int32)
    out = v4.sparse_sink_attention(q, table, sel, kv_lora=8, scale=0.3)
    kv = table[[3, 7]]
    want = torch.softmax(q[0] @ kv.T * 0.3, -1) @ kv[:, :8]
    assert torch.allclose(out[0], want, atol=1e-6)
    sunk = v4.sparse_sink_attention(q, table, sel, kv_lora=8, scale=0.3, sink=torch.tensor([50.0, 50.0]))
    assert sunk.abs().max() < 1e-6                                # a huge sink absorbs the mass


def test_markov_head_chains_drafts_and_breaks_ties_low():
    vocab, rank = 12, 4
    w1 = torch.zeros(vocab, rank)
    w2 = torch.zeros(vocab, rank)
    w1[3, 0] = 1.0          # after token 3 ...
    w2[7, 0] = 5.0          # ... token 7 gets a bonus
    logits = torch.zeros(3, vocab)
    logits[0, 3] = 1.0      # first draft: 3
    logits[2, 5] = logits[2, 9] = 2.0
    ids, vals = v4.markov_head(logits, w1, w2, anchor=0)
    assert ids == [3, 7, 5] and vals[1] == 5.0 and vals[2] == 2.0


def test_hc_mean_taps_concatenates_layer_means():
    a = torch.arange(24, dtype=torch.float32).view(1, 4, 6)
    taps = v4.hc_mean_taps([a, 2 * a], 4)
    assert taps.shape == (1, 12) and torch.allclose(taps[0, :6], a[0].mean(0)) and torch.allclose(taps[0, 6:], 2 * a[0].mean(0))
