"""Tokenizer, datasets, samplers, bucket packing and token-budget micro-batches (CPU)."""
import json

import numpy as np

from hotspa_ae_b200.utils import data as D
from hotspa_ae_b200.utils.dataset import (Dataloader, DistBatchSampler, LlamaJsonDataset, NormalSampler,
                                          get_mask_and_position_ids)
from hotspa_ae_b200.utils.tokenizer import GPT2BPETokenizer, byte_to_unicode


def _toy_tokenizer():
    b2u = byte_to_unicode()
    vocab = {b2u[b]: b for b in range(256)}
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), (b2u[ord(" ")], "w")]
    for a, b in merges:
        vocab[a + b] = len(vocab)
    vocab["<|endoftext|>"] = len(vocab)
    return GPT2BPETokenizer(vocab=vocab, merges=merges)


def test_bpe_roundtrip_and_merges():
    tok = _toy_tokenizer()
    ids = tok.tokenize("hello world, héllo!")
    assert tok.detokenize(ids) == "hello world, héllo!"
    assert ids[0] == tok.encoder["hello"]                       # merged through he + ll + o
    assert tok.pad == tok.vocab_size and tok.eod == tok.encoder["<|endoftext|>"]


def test_json_dataset_and_samplers(tmp_path):
    tok = _toy_tokenizer()
    path = tmp_path / "docs.json"
    with open(path, "w") as f:
        for i in range(10):
            f.write(json.dumps({"content": "hello " * (i + 1)}) + "\n")
        f.write(json.dumps({"content": ""}) + "\n")
    ds = LlamaJsonDataset(str(path), "content", 8, None, None, tokenizer=tok)
    assert len(ds) == 10 and max(len(d) for d in ds.data) <= 9
    assert (tmp_path / "docs_cache.pkl").exists()
    assert [b for b in NormalSampler(10, 2, 4)] == [[2, 3, 4, 5], [6, 7, 8, 9]]
    assert [b for b in DistBatchSampler(12, 0, 2, 1, 2)] == [[2, 3], [6, 7], [10, 11]]
    mask, pos = get_mask_and_position_ids(np.array([[5, 6, 0], [7, 0, 0]]), 0)
    assert mask.tolist() == [[True, True, False], [True, False, False]] and pos.tolist() == [[0, 1, 2], [0, 1, 2]]
    dl = Dataloader(np.arange(40).reshape(20, 2), 4)
    dl.set_dp_rank(1, 2)
    assert dl.batch_num == 2 and dl.get_next_arr()[0, 0] == 20


def test_bucketing_and_token_budget_micro_batches():
    lens = D.lognormal_lengths(40000, seed=3, max_len=8192)
    assert lens.sum() == 40000
    seqs = D.synthetic_sequences(lens, 1000, seed=3)
    packed = D.bucket_and_pack(lens, [8192, 2048, 0], 1, False)
    members = sorted(i for b in packed for r in b.rows for i in r)
    assert members == list(range(len(lens)))                    # nothing dropped, nothing duplicated
    for b in packed:
        for r in b.rows:
            assert sum(lens[i] for i in r) <= b.max_len + 1
    short = [i for r in packed[1].rows for i in r]
    seen, n_mb = [], None
    for rank in range(4):
        mb = D.token_budget_micro_batches(seqs, short, 4, rank, 4096, 0, 256)
        n_mb = mb["num_micro_batches"] if n_mb is None else n_mb
        assert mb["num_micro_batches"] == n_mb
        for ids, lab, cu, L in zip(mb["input_ids"], mb["labels"], mb["cu_seqlens"], mb["row_len"]):
            assert ids.shape == (1, L) and L % 256 == 0 and cu[0, -1] == L
            seen.append(int((lab != -1).sum()))
    assert sum(seen) == sum(lens[i] - 1 for i in short)         # every target token appears exactly once


def test_token_budget_micro_batches_follow_replica_shares():
    from hotspa_ae_b200.utils import data as D
    lens = D.lognormal_lengths(20000, seed=3, median=200, max_len=2048)
    seqs = D.synthetic_sequences(lens, 1000, seed=3)
    members = list(range(len(seqs)))
    tok = []
    for r in range(2):
        mb = D.token_budget_micro_batches(seqs, members, 2, r, 4096, 0, 8, shares=[0.75, 0.25])
        tok.append(sum(int((a != 0).sum()) for a in mb["position_ids"]) + len(mb["position_ids"]))
        nmb = mb["num_micro_batches"]
    total = sum(len(s) for s in seqs)
    carried = [sum(len(seqs[i]) for i in part) for part in D.balance_by_share([len(s) for s in seqs], [0.75, 0.25])]
    assert sum(carried) == total and abs(carried[0] / total - 0.75) < 0.03
    assert nmb >= 3                      # the heavy replica needs ~15000 / 4096 micro-batches; the light one pads up
    even = D.balance_by_share([len(s) for s in seqs], [0.5, 0.5])
    assert abs(sum(len(seqs[i]) for i in even[0]) / total - 0.5) < 0.03
    import pytest
    with pytest.raises(ValueError):
        D.token_budget_micro_batches(seqs, members, 2, 0, 4096, 0, 8, shares=[1.0])


def test_parquet_to_jsonl(tmp_path):
    import json
    import pyarrow as pa
    import pyarrow.parquet as pq
    from hotspa_ae_b200.utils import dataset as DSM
    rows = [{"content": f"document {i} " * (i + 1), "url": f"http://x/{i}"} for i in range(10)]
    pq.write_table(pa.Table.from_pylist(rows), tmp_path / "shard.parquet")
    n = DSM.parquet_to_jsonl(str(tmp_path / "shard.parquet"), str(tmp_path / "out" / "web.json"))
    lines = (tmp_path / "out" / "web.json").read_text().splitlines()
    assert n == 10 == len(lines) and json.loads(lines[3]) == rows[3]
    assert DSM.parquet_to_jsonl(str(tmp_path / "shard.parquet"), str(tmp_path / "few.json"), columns=["content"],
                                limit=4) == 4
    assert set(json.loads((tmp_path / "few.json").read_text().splitlines()[0])) == {"content"}
    assert DSM._main(["--parquet", str(tmp_path / "shard.parquet"), "--json_file", str(tmp_path / "cli.json")]) == 0
