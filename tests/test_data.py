"""Data pipeline: packing expectations and checkpoint/resume equivalence of every stateful stage."""
import copy
import random

import pytest
import torch

from prime_b200.config import DataConfig
from prime_b200.data import (FakeTokenizedDataset, InterleaveDataset, ParquetDataset, PrefetchDataLoader, SequencePackingDataSet,
                             StatefulLoader, UniformTokenDataset, collate_fn, get_dataloader, load_all_datasets,
                             seq_start_from_collated)
from prime_b200.utils import FakeTokenizer


class CharTokenizer:
    eos_token_id = 1

    def encode(self, text):
        return [3 + (ord(c) % 200) for c in text]


class ListDataset:
    def __init__(self, samples):
        self.samples = samples

    def __iter__(self):
        for s in self.samples:
            yield {"input_ids": s}

    def state_dict(self):
        return {}

    def load_state_dict(self, sd):
        pass


def test_sequence_packing_exact():
    ds = ListDataset([[6, 1, 2, 3, 4], [6, 3, 3, 4, 1, 7], [3, 2], [1, 2], [1, 4, 5, 3, 4, 1, 7, 8]])
    out = list(SequencePackingDataSet(ds, max_seq_length=8, eos_token=0))
    assert out[0]["input_ids"].tolist() == [6, 1, 2, 3, 4, 6, 3, 3]
    assert out[0]["labels"].tolist() == [1, 2, 3, 4, 0, 3, 3, 4]
    assert out[0]["seqlens"] == [5, 3]
    assert out[1]["input_ids"].tolist() == [3, 2, 1, 2, 1, 4, 5, 3]
    assert out[1]["labels"].tolist() == [2, 0, 2, 0, 4, 5, 3, 4]
    assert out[1]["seqlens"] == [2, 2, 4]
    for o in out:
        assert sum(o["seqlens"]) == 8


def test_fake_dataset_and_collate_and_seq_start():
    ds = SequencePackingDataSet(FakeTokenizedDataset(16, 100, seed=1), 16, eos_token=1)
    it = iter(ds)
    batch = collate_fn([next(it) for _ in range(3)])
    assert batch["input_ids"].shape == (3, 16) and batch["labels"].shape == (3, 16)
    ss = seq_start_from_collated(batch["seqlens"], 16)
    assert ss.shape == (48,) and ss.dtype == torch.int32
    for b, lens in enumerate(batch["seqlens"]):
        pos = b * 16
        for n in lens.tolist():
            assert (ss[pos:pos + n] == pos).all()
            pos += n


@pytest.fixture()
def parquet_files(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq
    rng = random.Random(0)
    files = []
    for i in range(6):
        rows = ["".join(rng.choice("abcdefgh ") for _ in range(rng.randint(5, 60))) for _ in range(23 + i)]
        path = tmp_path / f"part_{i}.parquet"
        pq.write_table(pa.table({"text": rows}), path)
        files.append(str(path))
    return files


def _take(it, n):
    return [next(it) for _ in range(n)]


def _same(a, b):
    for x, y in zip(a, b):
        if isinstance(x, dict):
            for k in x:
                xv, yv = x[k], y[k]
                if isinstance(xv, torch.Tensor):
                    assert torch.equal(xv, yv)
                else:
                    assert xv == yv
        else:
            assert x == y


@pytest.mark.parametrize("shard", [None, (1, 2), (2, 8)])
def test_parquet_resume(parquet_files, shard):
    ds = ParquetDataset(parquet_files, CharTokenizer(), shard=shard)
    it = iter(ds)
    _take(it, 100)
    state = copy.deepcopy(ds.state_dict())
    expect = _take(it, 200)
    ds2 = ParquetDataset(parquet_files, CharTokenizer(), shard=shard)
    ds2.load_state_dict(state)
    _same(expect, _take(iter(ds2), 200))


def test_parquet_shards_are_disjoint_and_infinite(parquet_files):
    a = _take(iter(ParquetDataset(parquet_files, CharTokenizer(), shard=(0, 2))), 80)
    b = _take(iter(ParquetDataset(parquet_files, CharTokenizer(), shard=(1, 2))), 80)
    assert a[0] != b[0]
    single = ParquetDataset(parquet_files[:1], CharTokenizer())
    got = _take(iter(single), 60)           # 23 rows: wraps around
    assert got[0] == got[23] and got[1] == got[24]


def test_interleave_and_packing_resume(parquet_files):
    def build():
        d1 = ParquetDataset(parquet_files[:3], CharTokenizer())
        d2 = ParquetDataset(parquet_files[3:], CharTokenizer())
        return SequencePackingDataSet(InterleaveDataset([d1, d2], [0.7, 0.3], seed=3), 64, eos_token=1)
    ds = build()
    it = iter(ds)
    _take(it, 50)
    state = copy.deepcopy(ds.state_dict())
    expect = _take(it, 100)
    ds2 = build()
    ds2.load_state_dict(state)
    _same(expect, _take(iter(ds2), 100))


def test_loader_and_prefetch_resume(parquet_files):
    cfg = DataConfig(seq_length=32, sequence_packing=True)

    def build():
        packed = SequencePackingDataSet(ParquetDataset(parquet_files, CharTokenizer()), 32, eos_token=1)
        return PrefetchDataLoader(StatefulLoader(packed, batch_size=4), cfg, device="cpu")
    dl = build()
    it = iter(dl)
    _take(it, 7)
    state = copy.deepcopy(dl.state_dict())
    expect = _take(it, 10)
    dl2 = build()
    dl2.load_state_dict(state)
    got = _take(iter(dl2), 10)
    for e, g in zip(expect, got):
        assert torch.equal(e["input_ids"], g["input_ids"]) and torch.equal(e["labels"], g["labels"])
        assert torch.equal(e["seq_start"], g["seq_start"])


def test_get_dataloader_fake_and_uniform():
    cfg = DataConfig(seq_length=64, fake=True, num_workers=0)
    dl = get_dataloader(FakeTokenizer(), world_size=1, rank=0, batch_size=2, data_config=cfg, device="cpu")
    b = next(iter(dl))
    assert b["input_ids"].shape == (2, 64) and b["seq_start"].shape == (128,)
    assert int(b["input_ids"].max()) < 1024
    cfg2 = DataConfig(seq_length=32, sequence_packing=False)
    d1 = get_dataloader(None, 1, 0, 3, cfg2, device="cpu", uniform_vocab=500)
    d2 = get_dataloader(None, 1, 0, 3, cfg2, device="cpu", uniform_vocab=500)
    x, y = next(iter(d1)), next(iter(d2))
    assert torch.equal(x["input_ids"], y["input_ids"]) and x["seq_start"] is None
    assert torch.equal(x["input_ids"][:, 1:], x["labels"][:, :-1])


def test_load_all_datasets_striping(parquet_files, tmp_path):
    import os
    d = os.path.dirname(parquet_files[0])
    cfg = DataConfig(dataset_name_or_paths=f"{d},{d}", dataset_ratio="3:1", data_rank=1, data_world_size=2)
    ds = load_all_datasets(cfg, "train", CharTokenizer(), rank=0, world_size=1)
    assert isinstance(ds, InterleaveDataset) and abs(ds.probabilities[0] - 0.75) < 1e-9
    assert ds.datasets[0].arg_files == sorted(parquet_files)[1::2]
    with pytest.raises(ValueError):
        load_all_datasets(DataConfig(dataset_name_or_paths=f"{d},{d}", dataset_ratio="1"), "train", CharTokenizer(), 0, 1)
