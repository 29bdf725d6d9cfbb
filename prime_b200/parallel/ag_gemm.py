"""All-gather fused into the consuming GEMM (csrc/gemm2_sm100.cu, ``pb_gemm_bf16_allgather``).

ZeRO-3 keeps a weight ``[N, K]`` row-sharded across the ranks of a worker. ``AllGatherLinear`` owns a
symmetric ``[N, K]`` bf16 buffer in which only this rank's rows are authoritative; ``forward(x)``
launches ONE kernel that pulls the other ranks' rows over NVLink (plain P2P loads issued by the
epilogue warps) while the tensor cores already work on the tiles whose weights have landed
(reference: FSDP2's NCCL all-gather in the pre-forward hook followed by a cuBLAS GEMM,
src/zeroband/train.py:150-168). After the call the buffer holds the full weight, so the dgrad /
wgrad GEMMs of the same step read it locally.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import native
from ..native import check, ptr, stream_ptr
from ..ops.kernels import status_word
from .symm import SymmComm

native.register_cuda_sigs({
    "pb_gemm_bf16_allgather": [native.vp, native.vp, native.vp, native.vp, native.vp, native.i32, native.i32, native.i32, native.i64,
                               native.i64, native.i64, native.i64, native.i32, native.i32, native.i32, native.i32, native.i32,
                               native.vp, native.i32, native.i32, native.vp, native.vp],
})


class AllGatherLinear:
    def __init__(self, comm: SymmComm, out_features: int, in_features: int):
        W = comm.world
        assert out_features % 256 == 0 and (out_features // W) % 32 == 0 and in_features % 8 == 0, \
            "need N % 256 == 0, (N / world) % 32 == 0 and K % 8 == 0"
        self.comm, self.N, self.K = comm, out_features, in_features
        self.rows_per_rank = out_features // W
        self._flat = comm.alloc(out_features * in_features, torch.bfloat16)
        self.weight = self._flat.view(out_features, in_features)
        peers = comm.peer_ptrs(self._flat)
        off = self.rows_per_rank * in_features * 2
        self._shards = (C.c_void_p * W)(*[peers[r] + r * off for r in range(W)])
        self.counters = torch.zeros(out_features // 256, dtype=torch.int32, device=comm.device)
        self.calls = 0

    def local_rows(self) -> torch.Tensor:
        """This rank's authoritative rows (write the shard here, e.g. from the optimizer)."""
        r = self.comm.rank
        return self.weight[r * self.rows_per_rank: (r + 1) * self.rows_per_rank]

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                max_ctas: int = 0) -> torch.Tensor:
        """``x [M, K] @ weight.T`` with the gather of ``weight`` fused in. Collective: every rank calls it."""
        M = x.shape[0]
        if out is None:
            out = torch.empty(M, self.N, dtype=torch.bfloat16, device=x.device)
        self.comm.barrier(slot=4)       # every rank's local rows are in place (and last step's readers are done)
        self.calls += 1
        check(native.cuda().pb_gemm_bf16_allgather(
            ptr(x), self._shards, ptr(self.weight), ptr(out), ptr(residual), M, self.N, self.K, x.stride(0), self.weight.stride(0),
            out.stride(0), residual.stride(0) if residual is not None else 0, 0, int(out.dtype == torch.float32), self.comm.world,
            self.comm.rank, self.rows_per_rank, ptr(self.counters), self.calls, max_ctas, ptr(status_word(x.device)), stream_ptr()),
            "pb_gemm_bf16_allgather")
        return out
