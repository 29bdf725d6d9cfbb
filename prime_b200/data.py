"""Data pipeline: fake / parquet / interleaved sources, sequence packing, a stateful loader and a
prefetcher that stages batches on the GPU (reference: src/zeroband/data.py:25-533).

Differences from the reference, by design:
  * Packed batches carry ``seq_start`` (int32 row -> first attendable row), the input the attention
    kernels take, instead of a FlexAttention BlockMask; the prefetch thread builds it with the batch
    and copies tokens from pinned host memory on a side stream.
  * The loader is an in-process iterator with explicit, picklable state (``state_dict`` /
    ``load_state_dict``) — the same resume contract the reference gets from torchdata's
    ``StatefulDataLoader``. Parquet files are still striped across loader shards the way the
    reference stripes them across worker processes (files ``i::n``, or rows ``i::n`` when there are
    fewer files than shards).
  * A ``UniformTokenDataset`` provides the seeded fixed-length uniform-random samples the benchmark
    configurations name.
"""
from __future__ import annotations

import random
import threading
from dataclasses import asdict, dataclass
from typing import Any, Generator, Iterable, Optional

import torch

from .config import DataConfig
from .utils.logger import get_logger

TEST_VOCAB_SIZE = 1024


class Stateful:
    def state_dict(self) -> dict[str, Any]:
        raise NotImplementedError

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        raise NotImplementedError


class FakeTokenizedDataset(Stateful):
    """Infinite random samples of length ``randint(1, seq_len)`` with ids in ``[3, vocab_size)``."""

    def __init__(self, seq_len: int, vocab_size: int, seed: int | None = None):
        assert vocab_size > 3, "Vocab size must be greater than 3"
        self.seq_len, self.vocab_size = seq_len, vocab_size
        self.step = 0
        self.seed = seed
        self._rng = random.Random(seed) if seed is not None else random
        self._gen = torch.Generator().manual_seed(seed) if seed is not None else None

    def __iter__(self) -> Generator[dict[str, Any], Any, None]:
        while True:
            n = self._rng.randint(1, self.seq_len)
            ids = torch.randint(3, self.vocab_size, (n,), generator=self._gen).tolist()
            self.step += 1
            yield {"input_ids": ids}

    def state_dict(self):
        return {"step": self.step}

    def load_state_dict(self, state_dict):
        target = state_dict["step"]
        if self.seed is not None:   # replay the seeded stream so the continuation is identical
            self.__init__(self.seq_len, self.vocab_size, self.seed)
            it = iter(self)
            for _ in range(target):
                next(it)
        self.step = target


class UniformTokenDataset(Stateful):
    """Seeded uniform-random token ids of fixed length ``seq_len + 1`` (one full sample per item,
    no packing needed): the synthetic data of the benchmark configurations."""

    def __init__(self, seq_len: int, vocab_size: int, seed: int = 0):
        self.seq_len, self.vocab_size, self.seed = seq_len, vocab_size, seed
        self.step = 0

    def __iter__(self):
        while True:
            g = torch.Generator().manual_seed(self.seed * 1_000_003 + self.step)
            ids = torch.randint(0, self.vocab_size, (self.seq_len + 1,), generator=g)
            self.step += 1
            yield {"input_ids": ids[:-1].clone(), "labels": ids[1:].clone(), "seqlens": [self.seq_len]}

    def state_dict(self):
        return {"step": self.step}

    def load_state_dict(self, state_dict):
        self.step = state_dict["step"]


@dataclass
class SequencePackingDataSetState:
    inputs_ids: list[int]
    labels: list[int]
    seqlens: list[int]


class SequencePackingDataSet(Stateful):
    """Packs variable-length samples into rows of exactly ``max_seq_length`` tokens.

    Each sample gets an EOS appended; ``labels`` is the sample shifted left by one; a sample that
    does not fit is truncated to fill the row (its remainder is dropped); ``seqlens`` lists the
    document lengths of the row and sums to ``max_seq_length``."""

    def __init__(self, dataset, max_seq_length: int, eos_token: int):
        self.dataset, self.max_seq_length, self.eos_token = dataset, max_seq_length, eos_token
        self.state = SequencePackingDataSetState([], [], [])

    def __iter__(self):
        st = self.state
        for sample in self.dataset:
            ids = list(sample["input_ids"]) + [self.eos_token]
            inp, lab = ids[:-1], ids[1:]
            room = self.max_seq_length - len(st.inputs_ids)
            if len(inp) < room:
                st.inputs_ids.extend(inp)
                st.labels.extend(lab)
                st.seqlens.append(len(inp))
                continue
            st.inputs_ids.extend(inp[:room])
            st.labels.extend(lab[:room])
            st.seqlens.append(room)
            out = {"input_ids": torch.tensor(st.inputs_ids, dtype=torch.long), "labels": torch.tensor(st.labels, dtype=torch.long),
                   "seqlens": [s for s in st.seqlens if s > 0]}
            self.state = st = SequencePackingDataSetState([], [], [])
            yield out

    def state_dict(self):
        return {"dataset": self.dataset.state_dict(), "state": asdict(self.state)}

    def load_state_dict(self, state_dict):
        self.dataset.load_state_dict(state_dict["dataset"])
        self.state = SequencePackingDataSetState(**state_dict["state"])


def collate_fn(samples: list[dict[str, Any]]) -> dict[str, Any]:
    assert set(samples[0].keys()) == {"input_ids", "labels", "seqlens"}
    return {"input_ids": torch.stack([s["input_ids"] for s in samples], 0),
            "labels": torch.stack([s["labels"] for s in samples], 0),
            "seqlens": [torch.tensor(s["seqlens"], dtype=torch.long) for s in samples]}


@dataclass
class PQDatasetState:
    files: list[str]
    file_index: int
    row_index: int
    increment: int
    init_row_index: int


class ParquetDataset(Stateful):
    """Infinite, resumable reader of the ``text`` column of a list of parquet files, tokenised on the
    fly. ``shard = (index, count)`` splits the work between loader shards: whole files when there
    are enough of them, otherwise interleaved rows of every file."""

    def __init__(self, files: list[str], tokenizer, shard: tuple[int, int] | None = None):
        self.arg_files = list(files)
        self.tokenizer = tokenizer
        self.shard = shard
        self.state: PQDatasetState | None = None

    def _lazy_init(self):
        idx, cnt = self.shard if self.shard is not None else (0, 1)
        if cnt > 1 and cnt > len(self.arg_files):
            get_logger().warning(f"loader shard {idx}: {cnt} shards for only {len(self.arg_files)} files; splitting by rows")
            self.state = PQDatasetState(self.arg_files, 0, idx, cnt, idx)
            return
        files = self.arg_files[idx::cnt] if cnt > 1 else self.arg_files
        self.state = PQDatasetState(files, 0, 0, 1, 0)

    def __iter__(self):
        import pyarrow.parquet as pq
        if self.state is None:
            self._lazy_init()
        st = self.state
        while True:
            table = pq.ParquetFile(st.files[st.file_index]).read()["text"]
            n = len(table)
            next_file = False
            while not next_file:
                if st.row_index >= n:               # file shorter than this shard's first row
                    st.row_index = st.init_row_index
                    st.file_index = (st.file_index + 1) % len(st.files)
                    break
                row = table[st.row_index]
                # the state is advanced before the sample is handed out, so a snapshot taken after
                # sample k resumes at sample k+1
                st.row_index += st.increment
                if st.row_index >= n:
                    st.row_index = st.init_row_index
                    st.file_index = (st.file_index + 1) % len(st.files)
                    next_file = True
                yield {"input_ids": self.tokenizer.encode(str(row))}

    @property
    def is_empty(self) -> bool:
        return len(self.arg_files) == 0

    def state_dict(self):
        return asdict(self.state) if self.state is not None else {}

    def load_state_dict(self, state_dict):
        if state_dict:
            self.state = PQDatasetState(**state_dict)


@dataclass
class InterleaveDatasetState:
    current_index: int
    seed: int


class InterleaveDataset(Stateful):
    """Draws each next sample from one of several datasets with the given probabilities. The choice
    sequence comes from a seeded generator that is replayed to ``current_index`` on resume."""

    def __init__(self, datasets: list, probabilities: list[float] | None, seed: int = 42):
        assert len(datasets) > 0, "At least one dataset is required"
        probabilities = probabilities if probabilities is not None else [1.0 / len(datasets)] * len(datasets)
        assert len(datasets) == len(probabilities), "The number of datasets and probabilities must be the same"
        self.datasets, self.probabilities = [], []
        for ds, p in zip(datasets, probabilities):
            if getattr(ds, "is_empty", False):
                get_logger().warning(f"Dataset {ds} is empty. Skipping.")
                continue
            self.datasets.append(ds)
            self.probabilities.append(p)
        self.state = InterleaveDatasetState(0, seed)
        self._init_random_state()

    def _init_random_state(self):
        self.random_generator = random.Random(self.state.seed)
        for _ in range(self.state.current_index):
            self._pick()

    def _pick(self) -> int:
        return self.random_generator.choices(range(len(self.datasets)), weights=self.probabilities, k=1)[0]

    def __iter__(self):
        iters = [iter(d) for d in self.datasets]
        while True:
            i = self._pick()
            sample = next(iters[i])
            self.state.current_index += 1
            yield sample

    def state_dict(self):
        out = {"interleave_state": asdict(self.state)}
        for i, d in enumerate(self.datasets):
            out[f"dataset_{i}"] = d.state_dict()
        return out

    def load_state_dict(self, state_dict):
        self.state = InterleaveDatasetState(**state_dict["interleave_state"])
        for i, d in enumerate(self.datasets):
            d.load_state_dict(state_dict[f"dataset_{i}"])
        self._init_random_state()


class StatefulLoader(Stateful):
    """Batches an iterable, stateful dataset. ``state_dict`` describes the position *after the last
    batch handed out*, so ``load_state_dict`` on a fresh loader continues with the next batch."""

    def __init__(self, dataset, batch_size: int, collate=collate_fn):
        self.dataset, self.batch_size, self.collate = dataset, batch_size, collate
        self._it = None
        self.batches_yielded = 0

    def __iter__(self):
        if self._it is None:
            self._it = iter(self.dataset)
        return self

    def __next__(self):
        if self._it is None:
            self._it = iter(self.dataset)
        samples = [next(self._it) for _ in range(self.batch_size)]
        self.batches_yielded += 1
        return self.collate(samples)

    def state_dict(self):
        return {"dataset": self.dataset.state_dict(), "batches_yielded": self.batches_yielded}

    def load_state_dict(self, state_dict):
        self.dataset.load_state_dict(state_dict["dataset"])
        self.batches_yielded = state_dict.get("batches_yielded", 0)
        self._it = None


def seq_start_from_collated(seqlens: list[torch.Tensor], seq_len: int) -> torch.Tensor:
    """int32 ``[B*seq_len]``: for every token row, the row where its document starts."""
    out = torch.empty(len(seqlens) * seq_len, dtype=torch.int32)
    for b, lens in enumerate(seqlens):
        pos = b * seq_len
        for n in lens.tolist():
            out[pos: pos + n] = pos
            pos += n
        if pos < (b + 1) * seq_len:          # tolerate rows whose listed lengths fall short
            out[pos: (b + 1) * seq_len] = pos
    return out


class PrefetchDataLoader(Stateful):
    """Hides batch preparation behind compute: a background thread pulls the next batch, pins it,
    copies it to the device on a side stream and builds ``seq_start`` for packed batches. Yields
    ``{"input_ids", "labels", "seq_start" | None, "ready": cuda event | None}``; the consumer waits on
    the event (stream wait, no host sync) before using the tensors."""

    def __init__(self, loader: StatefulLoader, data_config: DataConfig, device: torch.device | str | None = None):
        self.loader, self.config = loader, data_config
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self._thread: threading.Thread | None = None
        self._ready: Any = None
        self._stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._started = False

    def _task(self):
        try:
            batch = next(self.loader)
        except StopIteration:
            self._ready = StopIteration
            return
        T = batch["input_ids"].shape[1]
        ss = seq_start_from_collated(batch["seqlens"], T) if self.config.sequence_packing else None
        if self.device.type != "cuda":
            self._ready = {"input_ids": batch["input_ids"], "labels": batch["labels"], "seq_start": ss, "ready": None}
            return
        torch.cuda.set_device(self.device)
        with torch.cuda.stream(self._stream):
            ids = batch["input_ids"].pin_memory().to(self.device, non_blocking=True)
            lab = batch["labels"].pin_memory().to(self.device, non_blocking=True)
            ssd = ss.pin_memory().to(self.device, non_blocking=True) if ss is not None else None
            ev = torch.cuda.Event()
            ev.record(self._stream)
        self._ready = {"input_ids": ids, "labels": lab, "seq_start": ssd, "ready": ev}

    def _prefetch(self):
        self._thread = threading.Thread(target=self._task, daemon=True)
        self._thread.start()

    def _await(self):
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def __iter__(self):
        if not self._started:
            iter(self.loader)
            self._started = True
            if self._ready is None:
                self._prefetch()
        return self

    def __next__(self):
        if not self._started:
            iter(self)
        self._await()
        if self._ready is StopIteration:
            raise StopIteration
        batch, self._ready = self._ready, None
        self._prefetch()
        if batch["ready"] is not None:
            torch.cuda.current_stream(self.device).wait_event(batch["ready"])
        return batch

    def state_dict(self):
        """Loader position plus the already-prefetched batch (kept on the host), so that a resumed
        run sees exactly the batches the interrupted one would have seen."""
        self._await()
        ready = None
        if isinstance(self._ready, dict):
            ready = {k: (v.cpu() if isinstance(v, torch.Tensor) else None) for k, v in self._ready.items() if k != "ready"}
        return {"loader": self.loader.state_dict(), "ready_batch": ready, "started": self._started}

    def load_state_dict(self, state_dict):
        self._await()
        self.loader.load_state_dict(state_dict["loader"])
        rb = state_dict.get("ready_batch")
        self._started = False
        self._ready = None
        if rb is not None:
            self._ready = {k: (v.to(self.device) if isinstance(v, torch.Tensor) else None) for k, v in rb.items()}
            self._ready["ready"] = None

    def __del__(self):
        try:
            self._await()
        except Exception:
            pass


def _get_datafiles(path: str, name: Optional[str] = None, split: str = "train") -> list[str]:
    """Parquet files of a dataset: a local directory / glob is listed directly; anything else goes
    through the HF ``datasets`` builder (needs its cache or network)."""
    import glob
    import os
    if os.path.isdir(path):
        files = sorted(glob.glob(os.path.join(path, "**", "*.parquet"), recursive=True))
        if files:
            return files
    if any(ch in path for ch in "*?["):
        return sorted(glob.glob(path))
    from datasets import load_dataset_builder
    cfgs = load_dataset_builder(path=path, name=name or None).builder_configs
    if not name:
        if "default" not in cfgs:
            get_logger().warning(f"Default config not found for {path}. Using first config.")
            name = next(iter(cfgs.keys()))
        else:
            name = "default"
    return list(cfgs[name].data_files[split])


def _get_probabilities(data_config: DataConfig) -> Optional[list[float]]:
    if data_config.dataset_ratio is None:
        return None
    if len(data_config.dataset_name_or_paths.split(",")) != len(data_config.dataset_ratio.split(":")):
        raise ValueError("Number of datasets and dataset ratios must be the same")
    nums = [float(i) for i in data_config.dataset_ratio.split(":")]
    return [n / sum(nums) for n in nums]


def _load_datasets(dataset_names: str, split: str, tokenizer, data_rank: Optional[int] = None, data_world_size: Optional[int] = None,
                   probabilities: Optional[list[float]] = None, reverse_data_files: bool = False):
    datasets = []
    for spec in dataset_names.split(","):
        name, _, cfg = spec.partition(":")
        files = _get_datafiles(name, cfg, split)
        if reverse_data_files:
            files = files[::-1]
        if data_rank is not None and data_world_size is not None:
            files = files[data_rank::data_world_size]
        datasets.append(ParquetDataset(files=files, tokenizer=tokenizer))
    ds = InterleaveDataset(datasets, probabilities) if len(datasets) > 1 else datasets[0]
    get_logger().info(f"Loaded datasets ({split})")
    return ds


def load_all_datasets(data_config: DataConfig, split: str, tokenizer, rank: int, world_size: int):
    """All configured datasets, interleaved; files are striped by ``data_rank * world + rank`` out of
    ``data_world_size * world`` so every GPU of every worker reads distinct shards."""
    if data_config.split_by_data_rank and data_config.data_rank is not None and data_config.data_world_size is not None:
        split_rank = data_config.data_rank * world_size + rank
        split_world = data_config.data_world_size * world_size
    else:
        split_rank, split_world = rank, world_size
    get_logger().info("Loading Train dataset(s)")
    return _load_datasets(data_config.dataset_name_or_paths, split, tokenizer, split_rank, split_world,
                          _get_probabilities(data_config), data_config.reverse_data_files)


def get_dataloader(tokenizer, world_size: int, rank: int, batch_size: int, data_config: DataConfig,
                   device: torch.device | str | None = None, uniform_vocab: int | None = None) -> PrefetchDataLoader:
    """Batches of ``batch_size`` rows of ``seq_length`` tokens for this rank, prefetched to ``device``."""
    if uniform_vocab is not None:
        loader = StatefulLoader(UniformTokenDataset(data_config.seq_length, uniform_vocab, seed=rank), batch_size)
        return PrefetchDataLoader(loader, data_config, device)
    if data_config.fake:
        # seeded per (worker, rank): a resumed run replays the same stream and workers see different data
        train = FakeTokenizedDataset(data_config.seq_length, TEST_VOCAB_SIZE, seed=1234 + rank + 1000 * (data_config.data_rank or 0))
    else:
        train = load_all_datasets(data_config, "train", tokenizer, rank, world_size)
    packed = SequencePackingDataSet(train, data_config.seq_length, eos_token=tokenizer.eos_token_id)
    return PrefetchDataLoader(StatefulLoader(packed, batch_size), data_config, device)
