"""uint8 pseudo-gradient quantisers.

Three implementations of the same scheme (6-sigma uniform grid around zero, 256 bins, codebook =
mean of the values that fell into each bin):
  * ``uniform_8bit_quantize`` / ``average_buckets`` / ``quantile_8bit_quantize``: pure torch, the
    readable oracle (reference: src/zeroband/compression.py:17-70);
  * ``host.*``: the multithreaded C++ quantiser of csrc/host/quantize.cpp through ctypes
    (reference: src/zeroband/C/compression.py:6-46, C/csrc/compression.cpp);
  * the CUDA primitives live in :mod:`prime_b200.ops.quant` (csrc/quant.cu).
All return ``(uint8 tensor, fp32[256] codebook)``; ``codebook[q]`` dequantises.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import numpy as np
import torch

from . import native

RANGE_IN_SIGMAS = 6
N_BINS = 256
QUANTIZATION_THREADS = int(os.environ.get("QUANTIZATION_THREADS", "0"))   # 0 = all cores


def average_buckets(tensor: torch.Tensor, quant_weight: torch.Tensor, n_bins: int) -> torch.Tensor:
    """Mean of ``tensor`` per quantisation bin (empty bins give 0)."""
    flat_q = quant_weight.flatten().long()
    sums = torch.zeros(n_bins, dtype=torch.float32).scatter_add_(0, flat_q, tensor.flatten().float())
    counts = torch.bincount(flat_q, minlength=n_bins)
    return sums / counts.clamp_min(1)


def uniform_8bit_quantize(tensor: torch.Tensor, inplace: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    offset = N_BINS // 2
    n = tensor.numel()
    std = (tensor.float().norm() / math.sqrt(max(n - 1, 1))).item()
    scale = RANGE_IN_SIGMAS * std / N_BINS
    if not (scale > 0) or not math.isfinite(scale):
        scale = 1.0
    q = torch.clamp(torch.round(tensor.float() / scale) + offset, 0, N_BINS - 1).to(torch.uint8)
    return q, average_buckets(tensor, q, N_BINS)


def get_chunk_size(num_elements: int, min_chunk_size: int) -> int:
    if num_elements < min_chunk_size:
        return num_elements
    leftover = num_elements % min_chunk_size
    n_chunks = num_elements // min_chunk_size
    return min_chunk_size + (leftover - 1) // n_chunks + 1


def quantile_8bit_quantize(tensor: torch.Tensor, chunk_size: int = 10 ** 5) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantile-of-quantiles bins: borders are the mean of per-chunk quantiles (approximate)."""
    flat = tensor.flatten().float().numpy()
    cs = get_chunk_size(flat.size, chunk_size)
    qs = np.linspace(0.0, 1.0, N_BINS + 1)[1:-1]
    parts = [np.quantile(flat[i:i + cs], qs) for i in range(0, flat.size, cs)]
    borders = torch.as_tensor(np.mean(parts, axis=0), dtype=torch.float32)
    q = torch.bucketize(tensor.float(), borders, right=True).clamp_(0, N_BINS - 1)
    return q.to(torch.uint8), average_buckets(tensor, q, N_BINS)


native.register_host_sigs({})


class _Host:
    """ctypes front-end to the C++ quantiser."""

    def __init__(self):
        self._lib = None

    @property
    def lib(self):
        if self._lib is None:
            lib = native.host()
            vp, i64, i32, f32 = C.c_void_p, C.c_longlong, C.c_int, C.c_float
            lib.pbh_uniform_8bit_quantize.argtypes = [vp, i64, vp, vp, i32]
            lib.pbh_uniform_8bit_quantize.restype = f32
            lib.pbh_quantize_per_tensor_uint8.argtypes = [vp, i64, f32, i32, vp, i32]
            lib.pbh_quantize_per_tensor_uint8.restype = None
            lib.pbh_average_buckets.argtypes = [vp, vp, i64, vp, i32]
            lib.pbh_average_buckets.restype = None
            lib.pbh_dequant_add.argtypes = [vp, vp, vp, i64, i32]
            lib.pbh_dequant_add.restype = None
            lib.pbh_dequant_set.argtypes = [vp, vp, vp, i64, i32]
            lib.pbh_dequant_set.restype = None
            self._lib = lib
        return self._lib

    def uniform_8bit_quantize(self, tensor: torch.Tensor, inplace: bool = True, threads: int = QUANTIZATION_THREADS):
        t = tensor.contiguous().float()
        q = torch.empty(t.shape, dtype=torch.uint8)
        lut = torch.empty(N_BINS, dtype=torch.float32)
        self.lib.pbh_uniform_8bit_quantize(t.data_ptr(), t.numel(), q.data_ptr(), lut.data_ptr(), threads)
        return q, lut

    def quantize_per_tensor_uint8(self, tensor: torch.Tensor, scale: float, zero_point: int, threads: int = QUANTIZATION_THREADS):
        t = tensor.contiguous().float()
        q = torch.empty(t.shape, dtype=torch.uint8)
        self.lib.pbh_quantize_per_tensor_uint8(t.data_ptr(), t.numel(), scale, zero_point, q.data_ptr(), threads)
        return q

    def average_buckets(self, tensor: torch.Tensor, quant_weight: torch.Tensor, n_bins: int = N_BINS,
                        threads: int = QUANTIZATION_THREADS):
        assert n_bins == N_BINS
        t, q = tensor.contiguous().float(), quant_weight.contiguous()
        lut = torch.empty(N_BINS, dtype=torch.float32)
        self.lib.pbh_average_buckets(t.data_ptr(), q.data_ptr(), t.numel(), lut.data_ptr(), threads)
        return lut

    def dequant_add(self, dst: torch.Tensor, q: torch.Tensor, lut: torch.Tensor, threads: int = QUANTIZATION_THREADS):
        self.lib.pbh_dequant_add(dst.data_ptr(), q.data_ptr(), lut.data_ptr(), dst.numel(), threads)

    def dequant_set(self, dst: torch.Tensor, q: torch.Tensor, lut: torch.Tensor, threads: int = QUANTIZATION_THREADS):
        self.lib.pbh_dequant_set(dst.data_ptr(), q.data_ptr(), lut.data_ptr(), dst.numel(), threads)


host = _Host()
