"""ctypes bindings to the package's native libraries.

``cuda()`` returns the sm_100a kernel library, ``host()`` the CPU library. Both are built
in-tree by :mod:`prime_b200._build` on first use if a compiler is present. On a machine with
a GPU a missing kernel library is a hard error: there is no silent PyTorch fallback for CUDA
tensors anywhere in this package.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

import torch

from . import _build

_lock = threading.Lock()
_cuda_lib = None
_host_lib = None

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float

_CUDA_SIGS = {
    # name: argtypes
    "pb_gemm_bf16": [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i32, i32, i32, i32, i32, vp, vp],
    "pb_gemm_bf16_pair": [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i32, i32, i32, i32, vp, vp],
    "pb_gemm_bf16_pair_epi": [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i32, i32, i32, i32, i32, i32, i32, i32, vp, i64,
                              vp, vp, vp],
    "pb_gemm_bf16_pair_splitk": [vp, vp, vp, i32, i32, i32, i64, i64, i32, i32, i32, i32, vp, vp],
    "pb_gemm_splitk_slices": [i32, i32],
    "pb_splitk_reduce": [vp, i32, i64, i32, vp, i64, vp, i64, i32, vp],
    "pb_rmsnorm_fwd": [vp, vp, vp, vp, i32, i32, f32, vp],
    "pb_rmsnorm_bwd_ctas": [],
    "pb_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "pb_rope": [vp, vp, i64, i32, i32, i32, i32, i32, vp],
    "pb_swiglu_fwd": [vp, vp, i64, i32, vp],
    "pb_swiglu_bwd": [vp, vp, vp, i64, i32, vp],
    "pb_embedding_fwd": [vp, vp, vp, i64, i32, vp],
    "pb_embedding_bwd": [vp, vp, vp, i64, i32, i32, vp],
    "pb_count_valid": [vp, i64, i32, vp, vp],
    "pb_cross_entropy": [vp, vp, vp, vp, vp, f32, i64, i32, i64, i32, i32, f32, i32, vp],
    "pb_sum_f32": [vp, i64, vp, vp, f32, vp, i32, vp],
    "pb_sumsq": [vp, i64, i32, vp, vp, i32, vp],
    "pb_adamw": [vp, vp, i32, vp, vp, vp, i64, f32, f32, f32, f32, f32, i32, vp, f32, f32, vp],
    "pb_cast_f32_bf16": [vp, vp, i64, vp],
    "pb_add_bf16": [vp, vp, vp, i64, vp],
}


class NativeError(RuntimeError):
    pass


def _bind(lib, sigs, optional=True):
    for name, args in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if optional:
                continue
            raise
        fn.argtypes = args
        fn.restype = C.c_int
    return lib


def cuda():
    """The CUDA kernel library (raises if it cannot be built / loaded)."""
    global _cuda_lib
    if _cuda_lib is None:
        with _lock:
            if _cuda_lib is None:
                path = _build.OUT / "libpb_cuda.so"
                try:
                    path = _build.build_cuda()
                except Exception as e:  # no nvcc on this machine: use a shipped build if present
                    if not path.exists():
                        raise NativeError(f"prime_b200 CUDA kernels are not built and cannot be built here: {e}") from e
                lib = C.CDLL(str(path))
                _cuda_lib = _bind(lib, _CUDA_SIGS_ALL())
    return _cuda_lib


def host():
    """The host (CPU) native library."""
    global _host_lib
    if _host_lib is None:
        with _lock:
            if _host_lib is None:
                path = _build.build_host()
                lib = C.CDLL(str(path))
                _host_lib = _bind(lib, _HOST_SIGS_ALL())
    return _host_lib


_extra_cuda_sigs: dict = {}
_extra_host_sigs: dict = {}


def register_cuda_sigs(sigs: dict) -> None:
    """Let op modules declare the C signatures of the entry points they use."""
    _extra_cuda_sigs.update(sigs)
    if _cuda_lib is not None:
        _bind(_cuda_lib, sigs)


def register_host_sigs(sigs: dict) -> None:
    _extra_host_sigs.update(sigs)
    if _host_lib is not None:
        _bind(_host_lib, sigs)


def _CUDA_SIGS_ALL():
    d = dict(_CUDA_SIGS)
    d.update(_extra_cuda_sigs)
    return d


def _HOST_SIGS_ALL():
    return dict(_extra_host_sigs)


def ptr(t: torch.Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(stream: torch.cuda.Stream | None = None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


# kernels launched per successful native call (1 unless listed); used for launch accounting
_LAUNCHES = {"pb_rmsnorm_bwd": 2, "pb_attn_bwd": 3, "pb_sum_f32": 2, "pb_sumsq": 2, "pb_zero_reduce_grads": 2}
_launch_count = 0


def check(rc: int, what: str) -> None:
    global _launch_count
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")
    _launch_count += _LAUNCHES.get(what.split("(", 1)[0], 1)


def launch_counter() -> int:
    """Number of kernels of this package launched since the last reset (this process)."""
    return _launch_count


def launch_counter_reset() -> None:
    global _launch_count
    _launch_count = 0


def cuda_loaded_path() -> Path | None:
    return (_build.OUT / "libpb_cuda.so") if _cuda_lib is not None else None
