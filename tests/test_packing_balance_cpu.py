"""Exact global batches over a world size that does not divide them; repacking keeps the historical row order."""
import itertools

import pytest
import torch

from archlab_b200.data.packing import BestFitPacker, balanced_global_batch, balanced_slice


def docs():
    for i in itertools.count():
        yield [2 + (i * 7 + k) % 17 for k in range(3 + i % 9)]


def test_balanced_slices_cover_the_batch_exactly():
    slices = [balanced_slice(192, r, 15) for r in range(15)]
    assert [a for _, a, _ in slices] == [13] * 12 + [12] * 3 and {l for *_, l in slices} == {13}
    assert [s for s, *_ in slices][:4] == [0, 13, 26, 39] and slices[-1][0] + slices[-1][1] == 192
    assert balanced_slice(8, 3, 4) == (6, 2, 2)
    for bad in ((0, 0, 1), (4, 4, 4), (4, 0, 0)):
        with pytest.raises(ValueError):
            balanced_slice(*bad)


def test_ranks_rebuild_one_global_batch_with_ignored_rows_only_as_padding():
    world, B, T = 5, 12, 8
    parts = [balanced_global_batch(BestFitPacker(docs(), B, T, buffer_size=8, bos_token=1), r, world) for r in range(world)]
    whole_x, whole_y, _ = BestFitPacker(docs(), B, T, buffer_size=8, bos_token=1).next_batch()
    assert {p[0].shape for p in parts} == {(3, T)}
    active_x = torch.cat([p[0][:p[2]["active_rows"]] for p in parts])
    active_y = torch.cat([p[1][:p[2]["active_rows"]] for p in parts])
    assert torch.equal(active_x, whole_x) and torch.equal(active_y, whole_y)
    assert sum(int((p[1] >= 0).all(1).sum()) for p in parts) == B and all(bool((p[1][p[2]["active_rows"]:] == -1).all()) for p in parts)


def test_one_large_batch_equals_the_concatenated_small_ones_and_seek_replays():
    small = BestFitPacker(docs(), 4, 8, buffer_size=8, bos_token=1)
    xs, ys = zip(*[(x, y) for x, y, _ in (small.next_batch() for _ in range(3))])
    x12, y12, _ = BestFitPacker(docs(), 12, 8, buffer_size=8, bos_token=1).next_batch()
    assert torch.equal(x12, torch.cat(xs)) and torch.equal(y12, torch.cat(ys))
    run = BestFitPacker(docs(), 2, 8, buffer_size=8, bos_token=1)
    history = [run.next_batch() for _ in range(7)]
    resumed = BestFitPacker(docs(), 2, 8, buffer_size=8, bos_token=1)
    resumed.seek(history[4][2]["batch_index"])
    x, y, state = resumed.next_batch()
    assert torch.equal(x, history[4][0]) and torch.equal(y, history[4][1]) and state == history[4][2]
    assert torch.equal(resumed.next_batch()[0], history[5][0])
