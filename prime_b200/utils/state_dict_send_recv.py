"""Ship a (nested) state dict between two ranks of a process group with point-to-point ops
(reference: src/zeroband/utils/state_dict_send_recv.py:1-165).

The dict is split into a tensor-free skeleton, in which every tensor is replaced by a placeholder
string ``zeroband_tensor_{i}_{shape}_{dtype}``, and the list of tensors. On the wire: an int64 with
the pickled skeleton's size, the pickled bytes, then every tensor with ``tag = index``.
"""
from __future__ import annotations

import io
import pickle

import torch

_PREFIX = "zeroband_tensor_"


def _local(t: torch.Tensor) -> torch.Tensor:
    return t.to_local() if hasattr(t, "to_local") else t


def _object_to_tensor(obj) -> tuple[torch.Tensor, torch.Tensor]:
    buf = io.BytesIO()
    pickle.Pickler(buf).dump(obj)
    data = torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8)
    return data, torch.tensor([data.numel()], dtype=torch.long)


def _tensor_to_object(tensor: torch.Tensor, size: int):
    return pickle.Unpickler(io.BytesIO(tensor.cpu().numpy().tobytes()[:size])).load()


def _tensor_to_placeholder(idx: int, tensor: torch.Tensor) -> str:
    return f"{_PREFIX}{idx}_{tensor.shape}_{tensor.dtype}"


def _validate_placeholder_to_tensor(placeholder: str, tensors: list[torch.Tensor]) -> torch.Tensor:
    try:
        idx, shape, dtype = placeholder.split("_")[2:]
    except ValueError as e:
        raise ValueError(f"Invalid tensor placeholder {placeholder}") from e
    t = tensors[int(idx)]
    if shape != str(t.shape):
        raise ValueError(f"tensor {idx} try to load a tensor with shape {shape} but the tensor has shape {t.shape}")
    if dtype != str(t.dtype):
        raise ValueError(f"tensor {idx} try to load a tensor with dtype {dtype} but the tensor has dtype {t.dtype}")
    return t


def _get_sendable_state_dict(state_dict: dict) -> tuple[dict, list[torch.Tensor]]:
    """Deterministic split of a nested dict / list structure into (skeleton, tensors)."""
    tensors: list[torch.Tensor] = []

    def strip(obj):
        if isinstance(obj, torch.Tensor):
            t = _local(obj)
            tensors.append(t)
            return _tensor_to_placeholder(len(tensors) - 1, t)
        if isinstance(obj, dict):
            return {k: strip(v) for k, v in obj.items()}
        if isinstance(obj, (list, tuple)):
            return type(obj)(strip(v) for v in obj)
        return obj

    return strip(state_dict), tensors


def _load_sendable_state_dict(tensors: list[torch.Tensor], state_dict: dict) -> dict:
    """Inverse of ``_get_sendable_state_dict``."""
    def fill(obj):
        if isinstance(obj, str) and obj.startswith(_PREFIX):
            return _validate_placeholder_to_tensor(obj, tensors)
        if isinstance(obj, dict):
            return {k: fill(v) for k, v in obj.items()}
        if isinstance(obj, (list, tuple)):
            return type(obj)(fill(v) for v in obj)
        return obj

    return fill(state_dict)


def send_state_dict(pg, state_dict: dict, dest_rank: int) -> None:
    skeleton, tensors = _get_sendable_state_dict(state_dict)
    send_tensor_and_state_dict(pg, dest_rank, skeleton, tensors)


def send_tensor_and_state_dict(pg, dest_rank: int, state_dict: dict, tensors: list[torch.Tensor]) -> None:
    data, size = _object_to_tensor(state_dict)
    pg.send([size], dest_rank, 0).wait()
    pg.send([data], dest_rank, 0).wait()
    jobs = []
    for i, t in enumerate(tensors):
        buf = _local(t).detach()
        buf = buf.cpu().contiguous() if buf.is_cuda or not buf.is_contiguous() else buf
        jobs.append(pg.send([buf], dest_rank, i))
    for j in jobs:
        j.wait()


def recv_state_dict(pg, src_rank: int, og_state_dict: dict) -> dict:
    """Receive a state dict shaped like ``og_state_dict`` (used only to size the receive buffers)."""
    size = torch.tensor([0], dtype=torch.long)
    pg.recv([size], src_rank, 0).wait()
    data = torch.empty(int(size.item()), dtype=torch.uint8)
    pg.recv([data], src_rank, 0).wait()
    skeleton = _tensor_to_object(data, int(size.item()))
    _, like = _get_sendable_state_dict(og_state_dict)
    bufs = [torch.empty(t.shape, dtype=t.dtype) for t in like]
    jobs = [pg.recv([b], src_rank, i) for i, b in enumerate(bufs)]
    for j in jobs:
        j.wait()
    return _load_sendable_state_dict(bufs, skeleton)
