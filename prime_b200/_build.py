"""In-tree native build of the package's CUDA (sm_100a) and host C++ code.

Two shared objects are produced next to this file:

* ``_C/libpb_cuda.so``  - every ``csrc/*.cu`` translation unit, compiled by nvcc for
  ``compute_100a/sm_100a`` only. Exposes a plain C ABI (``extern "C"``), loaded via ctypes.
* ``_C/libpb_host.so``  - every ``csrc/host/*.cpp`` translation unit (quantizer, TCP ring,
  membership helpers), compiled by g++; has no CUDA dependency so CPU-only ranks can load it.

A content hash of the sources is stored beside each library; a library is rebuilt only when
its hash changes, so a tree built on a machine without a GPU can be shipped to a GPU box and
loaded there without recompiling.
"""
from __future__ import annotations

import concurrent.futures as cf
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "_C"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
GXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-march=x86-64-v3", "-fno-math-errno"]


def _nvcc() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _hash(files: list[Path], extra: list[str]) -> str:
    h = hashlib.sha256()
    for f in sorted(files):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(extra).encode())
    return h.hexdigest()


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"native build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")


def _build_lib(name: str, sources: list[Path], headers: list[Path], compiler: str, flags: list[str],
               link_flags: list[str], force: bool) -> Path:
    OUT.mkdir(exist_ok=True)
    lib = OUT / name
    stamp = OUT / (name + ".hash")
    want = _hash(sources + headers, flags + link_flags)
    def fresh() -> bool:
        return lib.exists() and stamp.exists() and stamp.read_text().strip() == want

    if not force and fresh():
        return lib
    # several ranks of one launcher may get here at once on a new checkout: one of them builds, the others wait for
    # the lock and find the result; the library appears under its name only when it is complete
    with open(OUT / (name + ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and fresh():
                return lib
            objdir = OUT / ("obj_" + name.replace(".", "_"))
            objdir.mkdir(exist_ok=True)
            objs = [objdir / (s.stem + ".o") for s in sources]
            with cf.ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as ex:
                futs = [ex.submit(_run, [compiler, *flags, f"-I{CSRC}", "-c", str(s), "-o", str(o)])
                        for s, o in zip(sources, objs)]
                for f in futs:
                    f.result()
            tmp = OUT / (name + f".tmp{os.getpid()}")
            _run([compiler, "-shared", *[a for a in flags if a not in ("-c",)], *map(str, objs), "-o", str(tmp), *link_flags])
            os.replace(tmp, lib)
            stamp.write_text(want)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


def build_cuda(force: bool = False) -> Path:
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    srcs = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    return _build_lib("libpb_cuda.so", srcs, hdrs, nvcc, NVCC_FLAGS, [], force)


def build_host(force: bool = False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    hdrs = sorted((CSRC / "host").glob("*.h")) + sorted(CSRC.glob("*.h"))
    return _build_lib("libpb_host.so", srcs, hdrs, shutil.which("g++") or "g++", GXX_FLAGS, ["-pthread"], force)


def build_all(force: bool = False) -> dict[str, Path]:
    out = {"host": build_host(force)}
    if _nvcc() is not None:
        out["cuda"] = build_cuda(force)
    return out


if __name__ == "__main__":
    res = build_all(force="--force" in sys.argv)
    for k, v in res.items():
        print(f"{k}: {v}")
