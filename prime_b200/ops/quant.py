"""GPU uint8 quantiser primitives (csrc/diloco_comm.cu), usable on their own.

Same scheme as the host quantiser (:mod:`prime_b200.compression`), applied per 16 Ki-element chunk:
``uniform_8bit_quantize_cuda(x) -> (q uint8 [n], codebooks fp32 [chunks, 256])`` and
``dequantize_cuda(q, codebooks) -> fp32 [n]``. The fused all-reduce uses exactly these kernels for
its stage A; exposing them lets the error of the wire format be measured in isolation."""
from __future__ import annotations

import torch

from .. import native
from ..native import check, ptr, stream_ptr

native.register_cuda_sigs({
    "pb_dl_chunk": [],
    "pb_dl_quantize": [native.vp, native.i64, native.vp, native.vp, native.vp],
})


def uniform_8bit_quantize_cuda(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
    lib = native.cuda()
    chunk = lib.pb_dl_chunk()
    n = x.numel()
    chunks = -(-n // chunk)
    q = torch.empty(n, dtype=torch.uint8, device=x.device)
    lut = torch.empty(chunks, 256, dtype=torch.float32, device=x.device)
    check(lib.pb_dl_quantize(ptr(x), n, ptr(q), ptr(lut), stream_ptr()), "pb_dl_quantize")
    return q, lut


def dequantize_cuda(q: torch.Tensor, lut: torch.Tensor) -> torch.Tensor:
    chunk = native.cuda().pb_dl_chunk()
    idx = torch.arange(q.numel(), device=q.device) // chunk
    return lut[idx, q.long()]
