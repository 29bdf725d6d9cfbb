"""Cross-cutting helpers: throughput / MFU accounting, state signatures, fake tokenizer, free ports
(reference: src/zeroband/utils/__init__.py:34-196)."""
from __future__ import annotations

import hashlib
import socket
import time
from typing import Any

import torch

__all__ = ["get_peak_flops", "get_num_flop_per_token", "get_num_params", "PerfCounter", "get_module_signature",
           "get_optimizer_signature", "get_tensor_list_signature", "get_tensor_signature", "get_random_available_port",
           "get_random_available_port_list", "FakeTokenizer", "DeviceThroughputMeter"]

# dense bf16 tensor-core peaks (FLOP/s)
_PEAKS = [
    ("B200", 2.25e15), ("GB200", 2.5e15), ("B100", 1.8e15),
    ("H100 NVL", 835e12), ("H100 PCIe", 756e12), ("H100", 989e12), ("H200", 989e12), ("A100", 312e12),
]


def get_peak_flops(device_name: str) -> float:
    """bf16 dense peak of the named GPU. Unknown devices fall back to the A100 figure (as the
    reference does, utils/__init__.py:34-48) — the table here adds the Blackwell rows."""
    for key, val in _PEAKS:
        if key in device_name:
            if key == "H100" and "NVL" in device_name:
                return 835e12
            if key == "H100" and "PCIe" in device_name:
                return 756e12
            return val
    return 312e12


def get_num_flop_per_token(num_params: int, model_config, seq_len: int) -> int:
    l, h, q, t = model_config.n_layers, model_config.n_heads, model_config.dim // model_config.n_heads, seq_len
    return 6 * num_params + 12 * l * h * q * t


def get_num_params(model: torch.nn.Module, exclude_embedding: bool = False) -> int:
    n = sum(p.numel() for p in model.parameters())
    if exclude_embedding:
        n -= model.tok_embeddings.weight.numel()
    return n


class PerfCounter:
    """Rolling tokens/s over the last ``window_size`` steps (wall clock, host side)."""

    def __init__(self, window_size: int = 10):
        self.window_size = window_size
        self.tokens: list[int] = []
        self.times: list[float] = []

    def count_tokens(self, tokens: int):
        self.tokens.append(tokens)
        self.times.append(time.perf_counter())
        if len(self.tokens) > self.window_size:
            self.tokens.pop(0)
            self.times.pop(0)

    def get_tokens_per_second(self) -> float | None:
        if len(self.tokens) < 2:
            return None
        return sum(self.tokens[1:]) / (self.times[-1] - self.times[0])


class DeviceThroughputMeter:
    """tokens/s from CUDA events on the training stream: the device-side counterpart of PerfCounter.
    Events are recorded every step and resolved lazily (no host sync in the hot loop)."""

    def __init__(self, window_size: int = 10):
        self.window = window_size
        self.events: list[tuple[Any, int]] = []

    def step(self, tokens: int):
        if not torch.cuda.is_available():
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.events.append((ev, tokens))
        if len(self.events) > self.window + 1:
            self.events.pop(0)

    def tokens_per_second(self) -> float | None:
        done = [(e, t) for e, t in self.events if e.query()]
        if len(done) < 2:
            return None
        ms = done[0][0].elapsed_time(done[-1][0])
        return sum(t for _, t in done[1:]) / (ms / 1e3) if ms > 0 else None


TENSOR_SIG_SAMPLE_SIZE = 100


def get_tensor_signature(a: torch.Tensor) -> str:
    """md5 of (up to) 100 evenly spaced values plus the shape — cheap equality witness for big tensors."""
    if hasattr(a, "to_local"):
        a = a.to_local()
    flat = a.detach().reshape(-1)
    if flat.is_complex():
        flat = torch.view_as_real(flat).reshape(-1)
    if flat.numel() < TENSOR_SIG_SAMPLE_SIZE:
        sample = flat
    else:
        step = flat.numel() // TENSOR_SIG_SAMPLE_SIZE
        sample = flat[::step][:TENSOR_SIG_SAMPLE_SIZE]
    return hashlib.md5((str(sample.float().cpu().tolist()) + str(tuple(a.shape))).encode("utf-8")).hexdigest()


def get_module_signature(module: torch.nn.Module, compress: bool = True) -> str:
    sd = {k: get_tensor_signature(v) for k, v in module.state_dict().items()}
    s = str(sd)
    return hashlib.md5(s.encode("utf-8")).hexdigest() if compress else s


def get_dict_signature(d: dict, compress: bool = True) -> str:
    def conv(v):
        if isinstance(v, torch.Tensor):
            return get_tensor_signature(v)
        if isinstance(v, dict):
            return {str(k): conv(x) for k, x in v.items()}
        if isinstance(v, (list, tuple)):
            return [conv(x) for x in v]
        return v
    s = str(conv(d))
    return hashlib.md5(s.encode("utf-8")).hexdigest() if compress else s


def get_optimizer_signature(optimizer, compress: bool = True) -> str:
    return get_dict_signature(optimizer.state_dict(), compress)


def get_tensor_list_signature(tensor_list: list[torch.Tensor]) -> str:
    return hashlib.md5(str([get_tensor_signature(t) for t in tensor_list]).encode("utf-8")).hexdigest()


def get_random_available_port_list(num_port: int) -> list[int]:
    ports, socks = [], []
    for _ in range(num_port):
        s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        s.bind(("", 0))
        ports.append(s.getsockname()[1])
        socks.append(s)
    for s in socks:
        s.close()
    return ports


def get_random_available_port() -> int:
    return get_random_available_port_list(1)[0]


class FakeTokenizer:
    """Stand-in tokenizer for fake-data runs: 1000 ids, bos 0, eos 1, pad 2."""

    def __init__(self):
        self.vocab_size = 1000
        self.bos_token_id = 0
        self.eos_token_id = 1
        self.pad_token_id = 2

    def __len__(self):
        return self.vocab_size
