"""Migrate a dataloader checkpoint written by the reference (``data/_{rank}.pt`` holding a torchdata
``StatefulDataLoader`` snapshot) to this package's dataloader state, so a run can be resumed here at
(approximately) the same data position (reference: scripts/convert_dl_state.py:33-62, convert_dl_ckpt.sh).

    python -m prime_b200.cli.convert_dl_state @cfg.toml --input-path step_49200/diloco_0/data/_3.pt \
        --output-path out/data/_3.pt --rank 3 --world-size 8

Two source layouts are understood, both per torchdata worker (``_snapshot._worker_snapshots.worker_k``):
the HF-streaming one (``dataset_state.ex_iterable.ex_iterables[i].ex_iterable`` with ``shard_idx`` /
``shard_example_idx``) and the reference's own ParquetDataset one (``dataset_state.dataset.dataset_{i}`` with
``file_index`` / ``row_index``). This package reads every dataset with one stream per rank, so the position of
dataset i is taken from the worker that is furthest ahead: HF-streaming states resume at the start of the next
shard (as the reference's own migration does), Parquet states keep their file and row.
"""
from __future__ import annotations

import os
from typing import Any

import torch

from ..config import Config, parse_argv
from ..data import get_dataloader


class ConvertConfig(Config):
    input_path: str
    output_path: str
    rank: int = 0
    world_size: int = 1


def _walk(d: Any, pred, out: list, path: str = "") -> list:
    """All sub-dicts satisfying ``pred`` in deterministic (sorted-key) order, with their key path."""
    if isinstance(d, dict):
        if pred(d):
            out.append((path, d))
        for k in sorted(d, key=str):
            _walk(d[k], pred, out, f"{path}.{k}" if path else str(k))
    elif isinstance(d, (list, tuple)):
        for i, v in enumerate(d):
            _walk(v, pred, out, f"{path}[{i}]")
    return out


def source_positions(old_loader_state: dict) -> list[dict]:
    """Per dataset index i: {"file_index", "row_index" | None}; the furthest-ahead worker wins."""
    workers = old_loader_state.get("_snapshot", {}).get("_worker_snapshots")
    if not workers:
        workers = {"worker_0": {"dataset_state": old_loader_state}}
    per_ds: dict[int, dict] = {}
    for name in sorted(workers):
        ds_state = workers[name].get("dataset_state", workers[name])
        streaming = _walk(ds_state, lambda x: "shard_idx" in x, [])
        parquet = _walk(ds_state, lambda x: "file_index" in x and "row_index" in x, [])
        if streaming:
            cands = [{"file_index": int(s["shard_idx"]) + 1, "row_index": None} for _, s in streaming]
        else:
            cands = [{"file_index": int(s["file_index"]), "row_index": int(s["row_index"])} for _, s in parquet]
        for i, c in enumerate(cands):
            best = per_ds.get(i)
            key = (c["file_index"], c["row_index"] or 0)
            if best is None or key > (best["file_index"], best["row_index"] or 0):
                per_ds[i] = c
    return [per_ds[i] for i in sorted(per_ds)]


def transfer(old_loader_state: dict, new_state: dict) -> int:
    """Writes the source positions into ``new_state`` (this package's loader state, in place); returns the
    number of datasets positioned."""
    targets = _walk(new_state, lambda x: "file_index" in x and "row_index" in x, [])
    src = source_positions(old_loader_state)
    n = 0
    for (_, tgt), pos in zip(targets, src):
        n_files = len(tgt["files"]) if "files" in tgt else None
        fi = pos["file_index"]
        tgt["file_index"] = fi % n_files if n_files else fi
        tgt["row_index"] = pos["row_index"] if pos["row_index"] is not None else tgt.get("init_row_index", 0)
        n += 1
    return n


def convert(config: ConvertConfig) -> str:
    from ..train import _get_tokenizer
    old = torch.load(config.input_path, map_location="cpu", weights_only=False)
    old = old.get("data_loader", old)
    dl = get_dataloader(_get_tokenizer(config), world_size=config.world_size, rank=config.rank, batch_size=config.train.micro_bs,
                        data_config=config.data, device="cpu")
    next(iter(dl))                       # dataset states are created lazily
    new_state = dl.state_dict()
    new_state["ready_batch"] = None      # the batch prefetched above belongs to the old position
    new_state["started"] = False
    n = transfer(old, new_state)
    os.makedirs(os.path.dirname(os.path.abspath(config.output_path)), exist_ok=True)
    torch.save({"data_loader": new_state}, config.output_path)
    print(f"positioned {n} dataset(s); wrote {config.output_path}")
    return config.output_path


def main(argv=None):
    convert(ConvertConfig(**parse_argv(argv)))


if __name__ == "__main__":
    main()
