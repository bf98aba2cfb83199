"""Decisions that the engine and the attention mixer make on the host about a decode step: the classes of
sequence lengths that a decode graph is captured for, and the number of key ranges per sequence."""
from types import SimpleNamespace

import pytest

from quicknn_b200.engine.engine import Engine
from quicknn_b200.parts import MIXERS, PartSpec


def mixer(n_kv=4, head_dim=256, window=None, resident=296):
    pos = PartSpec("rotary", {"head_dim": head_dim, "theta": 1e4, "rotary_dim": head_dim})
    m = MIXERS.get("attention")(PartSpec("attention", {
        "hidden_size": 64, "n_heads": 2 * n_kv, "n_kv_heads": n_kv, "head_dim": head_dim, "scale": 0.1,
        "softcap": None, "window": window, "position": pos}))
    m._resident = resident
    return m


def step(n_seqs, longest, spread, max_seq=8192, tuning=None):
    return SimpleNamespace(n_seqs=n_seqs, longest=longest, spread=spread, max_seq=max_seq, tuning=tuning or {},
                           mode="decode")


def test_length_classes_are_coarse_and_bound_the_longest_sequence():
    assert Engine.length_classes([1]) == (256, 1.0)
    assert Engine.length_classes([256, 250]) == (256, 1.0)
    assert Engine.length_classes([257, 250]) == (512, 1.0)
    assert Engine.length_classes([8192] * 8) == (8192, 1.0)
    assert Engine.length_classes([2048, 1024, 1024, 1024]) == (2048, 1.6)       # 2048 / 1280
    assert Engine.length_classes([1000, 800, 700]) == (1024, 1.25)
    assert Engine.length_classes([4000] + [100] * 15) == (4096, 2.2)
    # a batch that decodes 300 tokens from prompts of 600..900 changes class once
    seen = {Engine.length_classes([600 + t, 750 + t, 900 + t]) for t in range(300)}
    assert len(seen) == 2


def test_key_ranges_at_equal_lengths_fill_whole_rounds_of_blocks():
    """What was measured at context 8192 with equal lengths: batch 1 takes 64 ranges, 8 nine, 12 six, 24 three (one
    round of blocks each); 28 sequences take five ranges (two rounds of 560 blocks on 296 places: faster than
    one round of two long ranges, while six ranges would need a third round)."""
    m = mixer()
    got = {b: m.decode_splits(step(b, 8192, 1.0)) for b in (1, 2, 4, 8, 12, 16, 24, 28, 32)}
    assert got == {1: 64, 2: 37, 4: 18, 8: 9, 12: 6, 16: 9, 24: 3, 28: 5, 32: 9}
    # all blocks fit the device at once up to 12 sequences and at 24
    assert all(got[b] * b * 4 <= 296 for b in (1, 2, 4, 8, 12, 24))
    # whole rounds: 16 x 4 x 9 = 576 blocks are two rounds of 296 places, 32 x 4 x 9 four
    assert -(-16 * 4 * 9 // 296) == 2 and -(-32 * 4 * 9 // 296) == 4
    assert {b: m.decode_splits(step(b, 2048, 1.0)) for b in (16, 32, 64)} == {16: 4, 32: 2, 64: 1}
    # a windowed layer sees at most its window
    assert mixer(window=4096).decode_splits(step(8, 8192, 1.0)) == 9
    assert mixer(window=128).decode_splits(step(8, 8192, 1.0)) == 4
    # short sequences: no range shorter than 32 keys
    assert m.decode_splits(step(1, 256, 1.0)) <= 8


def test_key_ranges_with_unequal_lengths_take_more_than_one_round():
    """64 sequences of very unequal lengths: one range each would let the longest set the pace; equal lengths
    at the same batch stay with few, long blocks."""
    m = mixer()
    assert m.decode_splits(step(64, 2048, 1.6)) == 4
    assert m.decode_splits(step(64, 2048, 1.0)) == 1
    assert m.decode_splits(step(32, 2048, 1.6)) == 4
    # the caller's fixed number wins
    assert m.decode_splits(step(64, 2048, 1.6, tuning={"decode_splits": 7})) == 7
    # lengths unknown (a step built by hand): the cache's longest sequence stands in
    assert m.decode_splits(step(8, 0, 0.0, max_seq=8192)) == 9


@pytest.mark.parametrize("n_kv,hd,resident", [(1, 64, 1184), (16, 128, 592), (8, 256, 296)])
def test_key_ranges_stay_within_what_the_kernels_take(n_kv, hd, resident):
    m = mixer(n_kv=n_kv, head_dim=hd, resident=resident)
    for b in (1, 3, 8, 40, 128, 256):
        for longest in (256, 1024, 8192):
            for spread in (1.0, 1.25, 1.6, 2.2):
                s = m.decode_splits(step(b, longest, spread))
                assert 1 <= s <= 64 and s <= max(1, longest // 32)


def test_rows_cut_off_a_prompt_product_only_where_a_round_of_tiles_is_saved():
    """The decision is a host function of the sizes: at the 2B layer sizes only the down product (inner size 9216),
    only just beyond a multiple of 2048 rows (72 -> 81 tiles of 256 x 256 on 74 pairs of SMs), and only up to 64 rows."""
    import torch
    from quicknn_b200.kernels import ops
    cpu = torch.device("cpu")                         # stands for 148 SMs
    down = lambda m: ops._rows_for_the_small_kernel(m, 2304, 9216, ops.EPI_NONE, cpu)            # noqa: E731
    assert [down(m) for m in (2048, 2049, 2112, 2113, 2304, 4096, 4097, 6145, 257, 100)] == [0, 1, 64, 0, 0, 0, 1, 1, 0, 0]
    for n_out, k, epi in ((4096, 2304, ops.EPI_NONE), (2304, 2048, ops.EPI_NONE), (9216, 2304, ops.EPI_GATED)):
        assert all(ops._rows_for_the_small_kernel(m, n_out, k, epi, cpu) == 0 for m in (2049, 4097, 6145, 8193))
