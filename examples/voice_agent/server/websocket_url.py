"""The websocket address the browser client should dial, given how the server is reached: behind a TLS-terminating proxy the
scheme becomes ``wss``, a forwarded host / prefix replaces the bind address, and a wildcard bind address is never handed out.

(reference: ``examples/voice_agent/server/websocket_url.py``.)"""
from typing import Mapping, Optional


def websocket_url(bind_host: str, port: int, path: str = "/ws", headers: Optional[Mapping[str, str]] = None, public_url: Optional[str] = None) -> str:
    if public_url:
        u = public_url.rstrip("/")
        for http, ws in (("https://", "wss://"), ("http://", "ws://")):
            if u.startswith(http):
                u = ws + u[len(http):]
        if not u.startswith(("ws://", "wss://")):
            u = "ws://" + u
        return u if u.endswith(path) else u + path
    h = {k.lower(): v for k, v in (headers or {}).items()}
    scheme = "wss" if h.get("x-forwarded-proto", "").split(",")[0].strip() == "https" or h.get("x-forwarded-ssl") == "on" else "ws"
    host = h.get("x-forwarded-host", "").split(",")[0].strip() or h.get("host", "")
    if not host:
        host = "localhost" if bind_host in ("0.0.0.0", "::", "") else bind_host
        if ":" in host and not host.startswith("["):
            host = f"[{host}]"
        host = f"{host}:{port}"
    prefix = h.get("x-forwarded-prefix", "").rstrip("/")
    return f"{scheme}://{host}{prefix}{path}"
