#!/usr/bin/env bash
# One-time setup on a training host (reference: scripts/install/install.sh): system tools the elastic mesh
# shells out to, Python dependencies, and the in-tree native libraries (nvcc, sm_100a).
set -euo pipefail
if command -v apt-get >/dev/null 2>&1; then
    sudo apt-get update && sudo apt-get install -y python3-dev iperf wget
fi
python -m pip install torch numpy pydantic pyarrow transformers pytest
python -c "import __graft_entry__ as g; g.build()"
python -m pytest tests -q -m "not gpu" -x
