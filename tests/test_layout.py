"""Closed-form ragged layout vs a brute-force per-element oracle."""

import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from yafsdp_b200.layout import FlatLayout, reshard_ranges


def _oracle(numels, world, align):
    total = sum(numels)
    padded = -(-max(total, 1) // (world * align)) * (world * align)
    shard = padded // world
    owner_of = []
    for i, n in enumerate(numels):
        owner_of += [(i, e) for e in range(n)]
    per = {}
    for flat, (i, e) in enumerate(owner_of):
        r = flat // shard
        per.setdefault((i, r), []).append((e, flat - r * shard))
    return padded, shard, per


@settings(max_examples=150, deadline=None)
@given(st.lists(st.integers(1, 97), min_size=1, max_size=7), st.integers(1, 6), st.sampled_from([1, 2, 8]))
def test_layout_matches_oracle(numels, world, align):
    lay = FlatLayout(numels, world, align)
    padded, shard, per = _oracle(numels, world, align)
    assert lay.padded_numel == padded and lay.shard_numel == shard
    for i, n in enumerate(numels):
        counts = lay.shard_numels(i)
        assert sum(counts) == n
        for r in range(world):
            pl = lay.placement(i, r)
            elems = per.get((i, r), [])
            assert pl.local_numel == len(elems) == counts[r]
            if elems:
                assert pl.global_offset == elems[0][0]
                assert pl.shard_offset == elems[0][1]
                assert [e for e, _ in elems] == list(range(elems[0][0], elems[0][0] + len(elems)))
            else:
                assert pl.global_offset == n  # empty shard marker


def test_layout_examples_from_the_reference_probe():
    # a 768-element parameter fully owned by the second of two ranks: empty shard offset == numel
    lay = FlatLayout([768, 768], 2, 8)
    assert lay.placement(1, 0).local_numel == 0 and lay.placement(1, 0).global_offset == 768
    assert lay.shard_numels(1) == (0, 768)
    # Llama-2-7B layer: padded size and shard size at 8 ranks
    d, f = 4096, 11008
    lay = FlatLayout([d, d * d, d * d, d * d, d * d, d, f * d, f * d, d * f], 8, 8)
    assert lay.total_numel == 202383360 and lay.padded_numel % 64 == 0 and lay.shard_numel * 8 == lay.padded_numel


def test_reshard_ranges_cover_exactly():
    pieces = reshard_ranges(100, [30, 0, 50, 20], 25, 90)
    assert pieces == [(0, 25, 5), (2, 0, 50), (3, 0, 10)]
    assert sum(n for _, _, n in pieces) == 65


def test_invalid_arguments():
    with pytest.raises(ValueError):
        FlatLayout([4], 0)
    with pytest.raises(ValueError):
        FlatLayout([4], 2, 0)
