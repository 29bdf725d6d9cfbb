#!/bin/bash
# Emulate a WAN link on the loopback device for local multi-worker experiments
# (reference: scripts/bandwith/down.sh, up.sh). Needs root and the `tc` tool.
#   bandwidth.sh down [rate, default 500mbit]   throttle lo
#   bandwidth.sh up                             remove the throttle
set -e
case "$1" in
    down) tc qdisc add dev lo root tbf rate "${2:-500mbit}" burst 32kbit latency 400ms ;;
    up)   tc qdisc del dev lo root ;;
    *)    echo "usage: $0 down [rate] | up"; exit 1 ;;
esac
