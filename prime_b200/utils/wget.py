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
    for rel in files:
        dst = os.path.join(destination, rel)
        os.makedirs(os.path.dirname(dst) or destination, exist_ok=True)
        with urllib.request.urlopen(source + rel, timeout=timeout) as r, open(dst, "wb") as f:
            shutil.copyfileobj(r, f, length=8 << 20)
    return files
