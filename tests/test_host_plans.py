"""Host-side planning that needs no device: the step's packed arrays and tile list, the product's
tile/split/stage plan, the decode attention's split count (no GPU)."""

import numpy as np
import pytest

from starter_b200.engine.batch import StepEntry, plan_step


def test_plan_step_packs_sequences_and_lists_query_tiles():
    entries = [StepEntry(3, [5, 6, 7], [0, 2]), StepEntry(0, list(range(130)), [129]), StepEntry(7, [9], [])]
    arrays = plan_step(entries, starts=[10, 0, 64], vocab_size=200)
    assert arrays["tokens"].tolist() == [5, 6, 7] + list(range(130)) + [9]
    assert arrays["tok_pos"].tolist() == [10, 11, 12] + list(range(130)) + [64]
    assert arrays["tok_slot"].tolist() == [3] * 3 + [0] * 130 + [7]
    assert arrays["seq_q_start"].tolist() == [0, 3, 133] and arrays["seq_q_len"].tolist() == [3, 130, 1]
    assert arrays["seq_kv_len"].tolist() == [13, 130, 65]
    assert arrays["want_rows"].tolist() == [0, 2, 3 + 129]
    tiles = list(zip(arrays["tile_seq"].tolist(), arrays["tile_first"].tolist()))
    assert sorted(tiles) == [(0, 0), (1, 0), (1, 64), (1, 128), (2, 0)]
    # the tiles with most keys to walk come first
    keys = [arrays["seq_kv_len"][s] - arrays["seq_q_len"][s] + f for s, f in tiles]
    assert keys == sorted(keys, reverse=True)
    assert all(a.dtype == np.int32 for a in arrays.values())
    # the same list in blocks of 256 queries (what the tensor-core prompt attention launches)
    more = plan_step([StepEntry(0, list(range(600)), []), StepEntry(1, list(range(100)), [])], [0, 300], 1000)
    blocks = list(zip(more["block_seq"].tolist(), more["block_first"].tolist()))
    assert blocks == [(0, 512), (1, 0), (0, 256), (0, 0)]      # most keys first: 512, 300, 256, 0 before them


@pytest.mark.parametrize("entries,starts,message", [
    ([], [], "at least one"),
    ([StepEntry(1, [1], []), StepEntry(1, [2], [])], [0, 1], "twice"),
    ([StepEntry(1, [], [])], [0], "no token"),
    ([StepEntry(1, [1, 2], [2])], [0], "place 2"),
    ([StepEntry(1, [300], [])], [0], "outside the vocabulary"),
])
def test_plan_step_refuses_what_makes_no_sense(entries, starts, message):
    with pytest.raises(ValueError, match=message):
        plan_step(entries, starts, vocab_size=200)


def test_product_plan_keeps_every_cta_resident_and_the_tile_in_the_ring():
    from starter_b200.ops import gemm_plan

    shapes = [(6144, 2560, False), (2560, 4096, False), (9728, 2560, True), (2560, 9728, False),
              (151936, 2560, False), (300, 72, False), (64, 8, True)]
    for rows in (1, 8, 16, 17, 33, 64, 65, 200, 256):
        for n, k, gated in shapes:
            bm, splits, stages = gemm_plan(rows, n, k, gated)
            assert bm in (16, 32, 64, 128) and bm >= min(rows, 128)     # more rows: several row tiles
            assert 1 <= splits <= 8 and 2 <= stages <= 8
            stage_bytes = 16384 + bm * 128
            assert stages * stage_bytes + 1024 <= 227 * 1024
            tiles = (n // 64 if gated else -(-n // 128)) * -(-rows // bm)
            if rows <= 64 and splits > 1:
                per_sm = (227 * 1024) // (stages * stage_bytes + 2048)
                assert tiles * splits <= 148 * per_sm          # one wave


def test_decode_attention_splits_fit_one_wave_and_respect_the_length():
    from starter_b200.ops import decode_splits

    assert decode_splits(1, 8, 4, 16) == 8                       # never more parts than a cluster merges
    assert decode_splits(1, 8, 4, 16, kv_hint=3073) == 8
    assert decode_splits(2, 8, 4, 16, kv_hint=3073) == 8
    assert decode_splits(4, 8, 4, 16, kv_hint=3073) == 7         # 224 blocks rather than 256
    assert decode_splits(5, 8, 4, 16, kv_hint=3073) == 6         # 240 blocks, not 280
    assert decode_splits(6, 8, 4, 16, kv_hint=3073) == 5
    assert decode_splits(8, 8, 4, 16, kv_hint=3073) == 4
    assert decode_splits(12, 8, 4, 16, kv_hint=3073) == 2        # 192 blocks, not 288
    assert decode_splits(1, 8, 4, 16, kv_hint=513) == 8
    assert decode_splits(1, 8, 4, 16, kv_hint=16384) == 32       # one long row: many parts through scratch
    assert decode_splits(1, 8, 4, 16, kv_hint=6000) == 8
    assert decode_splits(2, 8, 4, 16, kv_hint=16384) == 8        # two rows fill the SMs from a cluster
    assert decode_splits(8, 8, 4, 16, kv_hint=130) == 3          # a part is a page at least
    assert decode_splits(64, 8, 4, 16) == 1
    assert decode_splits(1, 8, 4, 16, kv_hint=10) == 1
    assert decode_splits(1, 8, 4, 4, kv_hint=513) == 3           # CUDA-core kernel: three pages a part
    for rows in (1, 2, 3, 5, 7, 8, 9, 10, 30, 64):
        for keys in (0, 700, 3073, 20000):
            assert rows * 8 * decode_splits(rows, 8, 4, 16, kv_hint=keys) <= max(256, rows * 8)


def test_decode_graph_length_classes_never_exceed_the_length():
    """A graph captured for a class assumes the class's shortest length: the class of a length is the
    largest one not above it, so every part of the attention keeps a page or more."""
    from starter_b200.engine.graphs import HINT_PAGES, hint_pages

    assert HINT_PAGES[:8] == (1, 2, 3, 4, 6, 8, 12, 16)
    for tokens in (0, 1, 64, 65, 128, 129, 200, 3073, 4096, 100_000):
        pages = max(1, -(-tokens // 64))
        got = hint_pages(tokens)
        assert got in HINT_PAGES and got <= pages
        assert all(p > pages for p in HINT_PAGES if p > got)
    assert [hint_pages(t) for t in (1, 65, 130, 3073)] == [1, 2, 3, 48]
