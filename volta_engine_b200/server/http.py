"""Binding of the native epoll HTTP/SSE front end (csrc/host/http.cpp)."""
from __future__ import annotations

import ctypes

from .. import _lib


class HttpRequest:
    __slots__ = ("conn", "method", "target", "path", "query", "headers", "body")

    def __init__(self, conn: int, blob: bytes):
        head, _, body = blob.partition(b"\n\n")
        lines = head.decode("latin-1").split("\n")
        self.conn, self.method, self.target = conn, lines[0].upper(), lines[1]
        self.path, _, self.query = self.target.partition("?")
        self.headers = {}
        for ln in lines[2:]:
            k, _, v = ln.partition(":")
            if k:
                self.headers[k.strip().lower()] = v.strip()
        self.body = body


class HttpServer:
    def __init__(self, host: str = "127.0.0.1", port: int = 0, idle_timeout_s: int = 300):
        lib = _lib.host()
        lib.vh_http_start.restype = ctypes.c_void_p
        lib.vh_http_start.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
        lib.vh_http_next.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_uint64),
                                     ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int)]
        lib.vh_http_respond.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_char_p,
                                        ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p]
        lib.vh_http_stream_begin.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_char_p]
        lib.vh_http_stream_send.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_char_p, ctypes.c_int]
        lib.vh_http_stream_end.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
        lib.vh_http_alive.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
        lib.vh_http_stop.argtypes = [ctypes.c_void_p]
        lib.vh_http_port.argtypes = [ctypes.c_void_p]
        lib.vh_free.argtypes = [ctypes.c_void_p]
        self._lib = lib
        self._h = lib.vh_http_start(host.encode(), port, idle_timeout_s)
        if not self._h:
            raise OSError(f"cannot listen on {host}:{port}")
        self.port = lib.vh_http_port(self._h)

    def next_request(self, timeout_ms: int = 200) -> HttpRequest | None:
        conn, buf, ln = ctypes.c_uint64(), ctypes.c_void_p(), ctypes.c_int()
        if not self._lib.vh_http_next(self._h, timeout_ms, ctypes.byref(conn), ctypes.byref(buf), ctypes.byref(ln)):
            return None
        blob = ctypes.string_at(buf, ln.value)
        self._lib.vh_free(buf)
        return HttpRequest(conn.value, blob)

    def respond(self, conn: int, status: int, body: bytes | str, ctype: str = "application/json", headers: str = ""):
        if isinstance(body, str):
            body = body.encode("utf-8")
        return self._lib.vh_http_respond(self._h, conn, status, ctype.encode(), body, len(body), headers.encode())

    def stream_begin(self, conn: int, ctype: str = "text/event-stream", status: int = 200):
        return self._lib.vh_http_stream_begin(self._h, conn, status, ctype.encode())

    def stream_send(self, conn: int, data: bytes | str):
        if isinstance(data, str):
            data = data.encode("utf-8")
        return self._lib.vh_http_stream_send(self._h, conn, data, len(data))

    def stream_end(self, conn: int):
        return self._lib.vh_http_stream_end(self._h, conn)

    def alive(self, conn: int) -> bool:
        return bool(self._lib.vh_http_alive(self._h, conn))

    def stop(self):
        if self._h:
            self._lib.vh_http_stop(self._h)
            self._h = None
