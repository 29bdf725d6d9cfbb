#!/usr/bin/env bash
# Migrate the dataloader states of all ranks of one reference checkpoint step
# (reference: scripts/convert_dl_ckpt.sh). Usage:
#   prime_b200/cli/convert_dl_ckpt.sh @configs/10B/B200.toml /ckpt/step_49200/diloco_0 /out/step_49200/diloco_0 [WORLD=8]
set -euo pipefail
CFG="$1"; SRC="$2"; DST="$3"; WORLD="${4:-8}"
mkdir -p "$DST/data"
for ((r = 0; r < WORLD; r++)); do
    python -m prime_b200.cli.convert_dl_state "$CFG" --input-path "$SRC/data/_${r}.pt" --output-path "$DST/data/_${r}.pt" \
        --rank "$r" --world-size "$WORLD"
done
