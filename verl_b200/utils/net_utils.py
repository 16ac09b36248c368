"""Networking helpers (reference: ``verl/utils/net_utils.py``)."""

from __future__ import annotations

import ipaddress
import socket

__all__ = ["is_ipv4", "is_ipv6", "is_valid_ipv6_address", "get_free_port", "format_host_port"]


def is_ipv4(s: str) -> bool:
    try:
        ipaddress.IPv4Address(s)
        return True
    except ValueError:
        return False


def is_ipv6(s: str) -> bool:
    try:
        ipaddress.IPv6Address(s.strip("[]"))
        return True
    except ValueError:
        return False


is_valid_ipv6_address = is_ipv6


def get_free_port(host: str = "127.0.0.1") -> int:
    fam = socket.AF_INET6 if is_ipv6(host) else socket.AF_INET
    with socket.socket(fam, socket.SOCK_STREAM) as s:
        s.bind((host.strip("[]"), 0))
        return s.getsockname()[1]


def format_host_port(host: str, port: int) -> str:
    return f"[{host.strip('[]')}]:{port}" if is_ipv6(host) else f"{host}:{port}"
