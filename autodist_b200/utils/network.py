"""Address helpers (behaviour of the reference's ``autodist/utils/network.py:21-75``).

The reference enumerates NICs through ``netifaces``; that package is not a
dependency here, the local addresses come from the socket layer instead.
"""
import ipaddress
import socket
from functools import lru_cache


def _host_part(address):
    """Strip an optional port / IPv6 brackets: ``1.2.3.4:80``, ``[::1]:80``, ``localhost``."""
    address = address.strip()
    if address.startswith("["):
        return address[1:address.index("]")]
    if address.count(":") == 1:
        return address.split(":")[0]
    return address


def _get_ip_from_address(address):
    host = _host_part(address)
    if host == "localhost":
        return ipaddress.ip_address("127.0.0.1")
    try:
        return ipaddress.ip_address(host)
    except ValueError:
        try:
            return ipaddress.ip_address(socket.gethostbyname(host))
        except OSError:
            return None


def is_loopback_address(address):
    ip = _get_ip_from_address(address)
    return bool(ip is not None and ip.is_loopback)


@lru_cache(maxsize=1)
def _local_ips():
    found = {"127.0.0.1", "::1"}
    names = {socket.gethostname(), "localhost"}
    try:
        names.add(socket.getfqdn())
    except OSError:
        pass
    for name in names:
        try:
            for info in socket.getaddrinfo(name, None):
                found.add(info[4][0])
        except OSError:
            continue
    # The address used for outbound traffic (no packet is sent by connect() on UDP).
    try:
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as s:
            s.connect(("10.255.255.255", 1))
            found.add(s.getsockname()[0])
    except OSError:
        pass
    return frozenset(found)


def is_local_address(address):
    """True if ``address`` names this machine (loopback or one of its interfaces)."""
    ip = _get_ip_from_address(address)
    if ip is None:
        return False
    return ip.is_loopback or str(ip) in _local_ips()
