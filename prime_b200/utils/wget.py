"""HTTP directory download used by live recovery: fetch every file a sidecar server lists
(reference: src/zeroband/utils/wget.py:8-20 shells out to ``wget -r``; this is an in-process
client for the JSON listing the sidecar in prime_b200.checkpoint serves)."""
from __future__ import annotations

import json
import os
import shutil
import urllib.request


def wget(source: str, destination: str, timeout: float = 600.0) -> list[str]:
    """Mirror ``source`` (an ``http://host:port/dir/`` URL of a sidecar) into ``destination``."""
    source = source.rstrip("/") + "/"
    with urllib.request.urlopen(source + "?list=1", timeout=timeout) as r:
        files = json.loads(r.read().decode())
    os.makedirs(destination, exist_ok=True)
    root = os.path.realpath(destination)
    for rel in files:
        # the listing comes from a peer: a name may only land inside `destination`
        dst = os.path.realpath(os.path.join(root, rel))
        if not isinstance(rel, str) or os.path.isabs(rel) or os.path.commonpath([root, dst]) != root or dst == root:
            raise ValueError(f"refusing to download {rel!r}: it would be written outside {destination}")
        os.makedirs(os.path.dirname(dst) or destination, exist_ok=True)
        with urllib.request.urlopen(source + rel, timeout=timeout) as r, open(dst, "wb") as f:
            shutil.copyfileobj(r, f, length=8 << 20)
    return files
