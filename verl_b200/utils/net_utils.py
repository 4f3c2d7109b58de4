"""Address helpers for rendezvous and server start-up.

Parity target: ``verl/utils/net_utils.py`` (``is_ipv4`` :31, ``is_ipv6`` :48, ``is_valid_ipv6_address`` :65,
``get_free_port`` :73).
"""

from __future__ import annotations

import ipaddress
import socket
from typing import Optional

__all__ = ["is_ipv4", "is_ipv6", "is_valid_ipv6_address", "get_free_port"]


def _parse(ip_str: str):
    try:
        return ipaddress.ip_address(ip_str.strip("[]"))
    except (ValueError, AttributeError):
        return None


def is_ipv4(ip_str: str) -> bool:
    return isinstance(_parse(ip_str), ipaddress.IPv4Address)


def is_ipv6(ip_str: str) -> bool:
    return isinstance(_parse(ip_str), ipaddress.IPv6Address)


def is_valid_ipv6_address(address: str) -> bool:
    return is_ipv6(address)


def get_free_port(address: str = "127.0.0.1", with_alive_sock: bool = False) -> tuple[int, Optional[socket.socket]]:
    """A port the OS reports free on ``address``. With ``with_alive_sock`` the bound socket is returned as well, so that
    nobody else can take the port before the caller's server binds it (with SO_REUSEADDR / SO_REUSEPORT)."""
    family = socket.AF_INET6 if is_ipv6(address) else socket.AF_INET
    s = socket.socket(family, socket.SOCK_STREAM)
    s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    if hasattr(socket, "SO_REUSEPORT"):
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEPORT, 1)
    s.bind((address.strip("[]"), 0))
    port = s.getsockname()[1]
    if with_alive_sock:
        return port, s
    s.close()
    return port, None
