"""The pre-training text corpus as a directory of parquet shards (column ``text``), read row group by row group.

* ``list_shards(dir)``: sorted ``*.parquet`` files (half-written ``*.tmp`` downloads are ignored); an empty directory is an
  error, not an empty epoch.
* The LAST shard is the validation split, all others are training data (so adding shards never moves a validation
  document into training).
* ``document_batches(dir, split, rank, world, resume=...)``: yields ``(texts, cursor)`` per row group.  Within every shard a
  rank takes row groups ``rank, rank + world, ...``; the stream repeats for further epochs.  ``cursor = (shard index, row
  group, epoch)`` is enough to resume: a resumed stream starts at the row group AFTER the cursor's (the one already
  consumed), on the same epoch.
There is no downloader here: this framework runs without network access; shards are staged by the data job.
(Reference: src/archlab/speedrun/dataset.py:38-100 and the cursor of speedrun/dataloader.py's document stream.)
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterator


def list_shards(data_dir) -> list[Path]:
    shards = sorted(p for p in Path(data_dir).iterdir() if p.suffix == ".parquet")
    if not shards:
        raise FileNotFoundError(f"no parquet shards under {data_dir}")
    return shards


def split_shards(data_dir, split: str) -> list[Path]:
    if split not in ("train", "val"):
        raise ValueError("split must be 'train' or 'val'")
    shards = list_shards(data_dir)
    if len(shards) < 2:
        raise ValueError("at least two shards are needed: the last one is the validation split")
    return shards[:-1] if split == "train" else shards[-1:]


def document_batches(data_dir, split: str, *, rank: int = 0, world: int = 1, resume: tuple[int, int, int] | None = None, epochs: int | None = None,
                     column: str = "text") -> Iterator[tuple[list[str], tuple[int, int, int]]]:
    import pyarrow.parquet as pq

    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank must lie inside a positive world size")
    shards = split_shards(data_dir, split)
    first_shard, after_group, epoch = resume if resume is not None else (0, None, 1)
    while epochs is None or epoch <= epochs:
        for index in range(first_shard, len(shards)):
            reader = pq.ParquetFile(shards[index])
            start = rank
            if after_group is not None:
                start = after_group + world                      # the cursor's row group was consumed before the stop
                after_group = None
            for group in range(start, reader.num_row_groups, world):
                yield reader.read_row_group(group, columns=[column]).column(column).to_pylist(), (index, group, epoch)
        first_shard, epoch = 0, epoch + 1
