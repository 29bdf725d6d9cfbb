"""Network helpers (reference: src/zeroband/utils/ip.py:6-35)."""
from __future__ import annotations

import socket
import struct

_UNITS = {"bits/sec": 1, "Kbits/sec": 1e3, "Mbits/sec": 1e6, "Gbits/sec": 1e9, "Tbits/sec": 1e12}


def parse_iperf_output(output: str) -> int:
    """bits/s from the last ``<value> <unit>`` pair of an iperf client report."""
    value, unit = output.strip().split()[-2:]
    if unit not in _UNITS:
        raise ValueError(f"Unknown unit: {unit}")
    return int(float(value) * _UNITS[unit])


def get_ip_address(ifname: str) -> str:
    """IPv4 address of a network interface (SIOCGIFADDR)."""
    import fcntl
    s = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
    try:
        packed = fcntl.ioctl(s.fileno(), 0x8915, struct.pack("256s", ifname.encode("utf-8")[:15]))
        return socket.inet_ntoa(packed[20:24])
    finally:
        s.close()
