"""Datasets, samplers and loaders.

* torch-like ``Dataset`` / ``IterableDataset`` / ``DataLoader`` (reference: python_refactor/hetu/utils/data)
* ``LlamaJsonDataset``: jsonl -> BPE token ids with a pickle cache beside the file
  (reference: hotspa/data_utils/llama_dataset.py; sequences are kept at their true length instead of being padded
  to ``max_seq_len + 1``: the hot-switch trainer buckets by real length and packs without padding documents)
* ``NormalSampler`` (whole global batches) and ``DistBatchSampler`` (this data-parallel rank's slice of every
  micro-batch), resumable from ``consumed_samples`` (reference: hotspa/data_utils/llama_dataloader.py)
* ``Dataloader``: the graph-level in-memory batcher (reference: hetu/graph/data/dataloader.{h,cc})
"""
from __future__ import annotations

import json
import os
import pickle

import numpy as np


class Dataset:
    def __getitem__(self, idx):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError


class IterableDataset(Dataset):
    def __iter__(self):
        raise NotImplementedError


class NormalSampler:
    """Index lists of whole global batches, starting after `consumed_samples`."""

    def __init__(self, total_samples: int, consumed_samples: int, global_batch_size: int, drop_last: bool = True):
        if total_samples <= 0 or consumed_samples >= total_samples:
            raise ValueError(f"no samples left to consume: {consumed_samples} of {total_samples}")
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.global_batch_size, self.drop_last = global_batch_size, drop_last

    def __len__(self):
        return self.total_samples

    def __iter__(self):
        batch = []
        for idx in range(self.consumed_samples, self.total_samples):
            batch.append(idx)
            if len(batch) == self.global_batch_size:
                yield batch
                batch = []
        if batch and not self.drop_last:
            yield batch


class DistBatchSampler:
    """Of every group of ``micro_batch_size * dp`` consecutive samples, the slice of data-parallel rank `dp_rank`."""

    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int, data_parallel_rank: int,
                 data_parallel_size: int, drop_last: bool = True):
        if total_samples <= 0 or consumed_samples >= total_samples:
            raise ValueError(f"no samples left to consume: {consumed_samples} of {total_samples}")
        if not 0 <= data_parallel_rank < data_parallel_size:
            raise ValueError("data_parallel_rank out of range")
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.mbs, self.rank, self.dp, self.drop_last = micro_batch_size, data_parallel_rank, data_parallel_size, drop_last

    def __len__(self):
        return self.total_samples

    def __iter__(self):
        batch, full = [], self.mbs * self.dp
        lo = self.rank * self.mbs
        for idx in range(self.consumed_samples, self.total_samples):
            batch.append(idx)
            if len(batch) == full:
                yield batch[lo:lo + self.mbs]
                batch = []
        if batch and not self.drop_last:
            yield batch[lo:lo + self.mbs]


class DataLoader:
    """Minimal loader: iterates a batch sampler (or fixed-size batches) and collates with `collate_fn`."""

    def __init__(self, dataset, batch_size: int = 1, shuffle: bool = False, batch_sampler=None, collate_fn=None,
                 drop_last: bool = False, seed: int = 0):
        self.dataset, self.batch_size, self.shuffle, self.drop_last = dataset, batch_size, shuffle, drop_last
        self.batch_sampler, self.collate_fn, self.seed, self.epoch = batch_sampler, collate_fn or (lambda x: x), seed, 0

    def __iter__(self):
        if self.batch_sampler is not None:
            for idxs in self.batch_sampler:
                yield self.collate_fn([self.dataset[i] for i in idxs])
            return
        order = np.arange(len(self.dataset))
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(order)
        self.epoch += 1
        for s in range(0, len(order), self.batch_size):
            idxs = order[s:s + self.batch_size]
            if len(idxs) < self.batch_size and self.drop_last:
                break
            yield self.collate_fn([self.dataset[int(i)] for i in idxs])

    def __len__(self):
        n = len(self.dataset)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size


class Dataloader:
    """In-memory batcher over one array (graph-level loader of the reference): ``get_arr()`` returns the current
    batch, ``get_next_arr()`` advances; ``set_dp_rank`` / ``set_mp_parts`` select this rank's slice."""

    def __init__(self, raw_data, batch_size: int, name: str = "default", shuffle: bool = False, drop_last: bool = True,
                 seed: int = 0):
        self.raw = np.asarray(raw_data)
        self.batch_size, self.name, self.shuffle, self.drop_last = batch_size, name, shuffle, drop_last
        self.dp_rank, self.dp_nrank = 0, 1
        self.parts, self.slices = None, None
        self.seed, self.epoch = seed, 0
        self._init_states()

    def _init_states(self):
        n = self.raw.shape[0]
        lo, hi = n * self.dp_rank // self.dp_nrank, n * (self.dp_rank + 1) // self.dp_nrank
        self.data = self.raw[lo:hi]
        if self.slices is not None:
            self.data = self.data[(slice(None),) + tuple(self.slices)]
        self.samples_num = self.data.shape[0]
        self.batch_num = self.samples_num // self.batch_size if self.drop_last else \
            (self.samples_num + self.batch_size - 1) // self.batch_size
        self.order = np.arange(self.samples_num)
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(self.order)
        self.batch_index = 0

    def set_dp_rank(self, dp_rank: int, dp_nrank: int):
        self.dp_rank, self.dp_nrank = dp_rank, dp_nrank
        self._init_states()

    def set_mp_parts(self, cur_part, parts):
        """Model-parallel slicing of the non-batch dims: `parts[d]` pieces along dim d+1, keep piece `cur_part[d]`."""
        sl = []
        for d, (c, p) in enumerate(zip(cur_part, parts)):
            size = self.raw.shape[d + 1] // p
            sl.append(slice(c * size, (c + 1) * size))
        self.slices = sl
        self._init_states()

    def get_arr(self):
        s = self.batch_index * self.batch_size
        return self.data[self.order[s:s + self.batch_size]]

    def get_next_arr(self):
        arr = self.get_arr()
        self.batch_index += 1
        if self.batch_index >= self.batch_num:
            self.epoch += 1
            self._init_states()
        return arr

    def __iter__(self):
        for _ in range(self.batch_num):
            yield self.get_next_arr()

    # spellings of the reference's bound Dataloader (python_refactor/hetu/_binding/graph/dataloader.cc)
    @property
    def sample_num(self) -> int:
        return self.samples_num

    @property
    def num_workers(self) -> int:
        return 0

    def get_data(self):
        return self.get_arr()

    def get_next_data(self):
        return self.get_next_arr()


class LlamaJsonDataset(Dataset):
    def __init__(self, json_file: str, key: str, max_seq_len: int, vocab_file: str, merge_file: str,
                 tokenizer=None, use_cache: bool = True):
        from .tokenizer import GPT2BPETokenizer
        self.tokenizer = tokenizer or GPT2BPETokenizer(vocab_file, merge_file)
        self.max_seq_len = max_seq_len
        cache_path = os.path.splitext(json_file)[0] + "_cache.pkl"
        if use_cache and os.path.exists(cache_path):
            with open(cache_path, "rb") as f:
                self.data = pickle.load(f)
        else:
            self.data = []
            with open(json_file, encoding="utf-8") as f:
                for line in f:
                    line = line.strip()
                    if not line:
                        continue
                    ids = self.tokenizer.tokenize(json.loads(line)[key])
                    if ids:                              # empty documents would make empty micro-batches
                        self.data.append(ids)
            if use_cache:
                with open(cache_path, "wb") as f:
                    pickle.dump(self.data, f)
        cap = max_seq_len + 1                            # n + 1 tokens give n (input, label) pairs
        self.data = [np.asarray(d[:cap], dtype=np.int64) for d in self.data]

    def pad_id(self) -> int:
        return self.tokenizer.pad

    def __len__(self):
        return len(self.data)

    def __getitem__(self, idx):
        return self.data[idx]


LLaMAJsonDataset = LlamaJsonDataset


def get_mask_and_position_ids(tokens: np.ndarray, pad: int):
    """[batch, seq] token ids -> (attention mask of non-pad tokens, positions 0..seq-1 per row)."""
    b, s = tokens.shape
    return np.not_equal(tokens, pad), np.tile(np.arange(s, dtype=np.int64), [b, 1])


def global_batches(dataset, global_batch_size: int, num_batches: int, consumed_samples: int = 0, seed: int = 0):
    """Yields `num_batches` global batches (lists of token arrays), wrapping around the dataset."""
    n = len(dataset)
    pos = consumed_samples % n
    for _ in range(num_batches):
        idxs = [(pos + i) % n for i in range(global_batch_size)]
        pos = (pos + global_batch_size) % n
        yield [dataset[i] for i in idxs]


def build_normal_data_loader(dataset, consumed_samples: int, global_batch_size: int):
    return DataLoader(dataset, batch_sampler=NormalSampler(len(dataset), consumed_samples, global_batch_size))


def build_dist_data_loader(dataset, consumed_samples: int, micro_batch_size: int, dp_rank: int, dp_size: int):
    return DataLoader(dataset, batch_sampler=DistBatchSampler(len(dataset), consumed_samples, micro_batch_size,
                                                              dp_rank, dp_size))


def parquet_to_jsonl(parquet_file: str, json_file: str, columns=None, limit: int | None = None) -> int:
    """Dataset preparation: one JSON object per row of a parquet shard (the form `LlamaJsonDataset` reads;
    reference: hotspa/data_utils/create_web_dataset.py).  Streams row groups instead of materialising the table.
    Returns the number of rows written."""
    import pyarrow.parquet as pq
    pf = pq.ParquetFile(parquet_file)
    n = 0
    os.makedirs(os.path.dirname(os.path.abspath(json_file)), exist_ok=True)
    with open(json_file, "w") as f:
        for batch in pf.iter_batches(batch_size=4096, columns=columns):
            for row in batch.to_pylist():
                f.write(json.dumps(row, ensure_ascii=False, default=str) + "\n")
                n += 1
                if limit is not None and n >= limit:
                    return n
    return n


def _main(argv=None) -> int:
    """`python -m hotspa_ae_b200.utils.dataset`: convert a parquet shard and / or build the token cache of a json
    dataset and print a few batches (reference: the __main__ of hotspa/data_utils/llama_dataset.py)."""
    import argparse
    ap = argparse.ArgumentParser(description=_main.__doc__)
    ap.add_argument("--parquet", default="", help="parquet shard to convert into --json_file first")
    ap.add_argument("--json_file", required=True)
    ap.add_argument("--json_key", default="content")
    ap.add_argument("--vocab_file", default="")
    ap.add_argument("--merge_file", default="")
    ap.add_argument("--max_seq_len", type=int, default=4096)
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--show", type=int, default=5, help="batches to print")
    a = ap.parse_args(argv)
    if a.parquet:
        rows = parquet_to_jsonl(a.parquet, a.json_file, limit=a.limit or None)
        print(f"wrote {rows} rows to {a.json_file}")
    if not (a.vocab_file and a.merge_file):
        return 0
    ds = LlamaJsonDataset(a.json_file, a.json_key, a.max_seq_len, a.vocab_file, a.merge_file)
    print(f"{len(ds)} documents, token cache next to {a.json_file}")
    for i, batch in enumerate(global_batches(ds, 4, a.show)):
        print(i, [len(s) for s in batch])
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
