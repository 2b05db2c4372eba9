"""Small asyncio HTTP/1.1 server: routing, JSON bodies, keep-alive, server-sent events.

Stands where the reference uses brpc's HTTP server (xllm/server/xllm_server.cpp:35-91, REST mappings :41-54).  Handlers are
`async def handler(request) -> Response | StreamingResponse`; streaming responses use chunked transfer encoding and are
fed from any thread through `StreamingResponse.put()`.
"""
from __future__ import annotations

import asyncio
import threading
import json
from typing import Any, Awaitable, Callable, Dict, List, Optional, Tuple
from urllib.parse import parse_qs, urlsplit

_REASONS = {200: "OK", 400: "Bad Request", 404: "Not Found", 405: "Method Not Allowed", 413: "Payload Too Large",
            429: "Too Many Requests", 500: "Internal Server Error", 503: "Service Unavailable"}


class Request:
    def __init__(self, method: str, path: str, query: Dict[str, List[str]], headers: Dict[str, str], body: bytes):
        self.method, self.path, self.query, self.headers, self.body = method, path, query, headers, body
        self.disconnected = asyncio.Event()

    def json(self) -> Any:
        return json.loads(self.body.decode("utf-8")) if self.body else {}


class Response:
    def __init__(self, body: Any = b"", status: int = 200, content_type: str = "application/json", headers: Optional[Dict[str, str]] = None):
        if isinstance(body, (dict, list)):
            body = json.dumps(body, ensure_ascii=False).encode()
        elif isinstance(body, str):
            body = body.encode()
        self.body, self.status, self.content_type, self.headers = body, status, content_type, headers or {}


class StreamingResponse:
    """Chunks are queued with `put(bytes)` (thread-safe), the stream ends with `close()`.  A call made on the event
    loop's own thread, which is where handlers produce their chunks, goes straight into the queue; only calls from other
    threads take the loop's wake-up path (a write to its self-pipe, one system call per chunk)."""

    def __init__(self, content_type: str = "text/event-stream", headers: Optional[Dict[str, str]] = None):
        self.content_type, self.headers = content_type, headers or {}
        self.loop = asyncio.get_event_loop()
        self._loop_thread = threading.get_ident()
        self.queue: "asyncio.Queue[Optional[bytes]]" = asyncio.Queue()
        self.closed = False

    def _enqueue(self, item) -> None:
        if threading.get_ident() == self._loop_thread:
            self.queue.put_nowait(item)
        else:
            self.loop.call_soon_threadsafe(self.queue.put_nowait, item)

    def put(self, data) -> None:
        if isinstance(data, str):
            data = data.encode()
        self._enqueue(data)

    def close(self) -> None:
        self._enqueue(None)


Handler = Callable[[Request], Awaitable[Any]]


class HttpServer:
    def __init__(self, max_body: int = 64 << 20):
        self.routes: Dict[Tuple[str, str], Handler] = {}
        self.max_body = max_body
        self.server: Optional[asyncio.AbstractServer] = None

    def route(self, method: str, path: str):
        def deco(fn: Handler):
            self.routes[(method.upper(), path)] = fn
            return fn
        return deco

    def add(self, method: str, path: str, fn: Handler):
        self.routes[(method.upper(), path)] = fn

    async def start(self, host: str, port: int):
        self.server = await asyncio.start_server(self._client, host or "0.0.0.0", port, reuse_address=True)
        return self.server

    async def _client(self, reader: asyncio.StreamReader, writer: asyncio.StreamWriter):
        try:
            while True:
                line = await reader.readline()
                if not line or line in (b"\r\n", b"\n"):
                    if not line:
                        break
                    continue
                try:
                    method, target, _ = line.decode("latin1").split(" ", 2)
                except ValueError:
                    break
                headers: Dict[str, str] = {}
                while True:
                    h = await reader.readline()
                    if h in (b"\r\n", b"\n", b""):
                        break
                    k, _, v = h.decode("latin1").partition(":")
                    headers[k.strip().lower()] = v.strip()
                n = int(headers.get("content-length", "0") or 0)
                if n > self.max_body:
                    await self._send(writer, Response({"error": "payload too large"}, 413), False)
                    break
                body = await reader.readexactly(n) if n else b""
                u = urlsplit(target)
                req = Request(method.upper(), u.path, parse_qs(u.query), headers, body)
                keep = headers.get("connection", "keep-alive").lower() != "close"
                fn = self.routes.get((req.method, req.path))
                if fn is None:
                    known = any(p == req.path for (_, p) in self.routes)
                    resp: Any = Response({"error": {"message": "method not allowed" if known else f"unknown path {req.path}",
                                                    "type": "invalid_request_error"}}, 405 if known else 404)
                else:
                    try:
                        resp = await fn(req)
                    except json.JSONDecodeError as e:
                        resp = Response({"error": {"message": f"invalid JSON body: {e}", "type": "invalid_request_error"}}, 400)
                    except Exception as e:   # a failing handler must not take the connection loop down
                        resp = Response({"error": {"message": f"{type(e).__name__}: {e}", "type": "internal_error"}}, 500)
                if isinstance(resp, StreamingResponse):
                    ok = await self._stream(writer, resp, req)
                    if not ok:
                        break
                else:
                    await self._send(writer, resp, keep)
                if not keep:
                    break
        except (ConnectionError, asyncio.IncompleteReadError):
            pass
        finally:
            try:
                writer.close()
            except Exception:
                pass

    async def _send(self, writer, resp: Response, keep: bool):
        head = [f"HTTP/1.1 {resp.status} {_REASONS.get(resp.status, 'OK')}", f"Content-Type: {resp.content_type}",
                f"Content-Length: {len(resp.body)}", f"Connection: {'keep-alive' if keep else 'close'}"]
        head += [f"{k}: {v}" for k, v in resp.headers.items()]
        writer.write(("\r\n".join(head) + "\r\n\r\n").encode() + resp.body)
        await writer.drain()

    async def _stream(self, writer, resp: StreamingResponse, req: Request) -> bool:
        head = ["HTTP/1.1 200 OK", f"Content-Type: {resp.content_type}", "Cache-Control: no-cache", "Transfer-Encoding: chunked",
                "Connection: keep-alive"] + [f"{k}: {v}" for k, v in resp.headers.items()]
        writer.write(("\r\n".join(head) + "\r\n\r\n").encode())
        try:
            while True:
                chunk = await resp.queue.get()
                parts, end = [], False
                while True:                                # everything that is queued already goes out in one write
                    if chunk is None:
                        end = True
                        break
                    parts.append(f"{len(chunk):X}\r\n".encode() + chunk + b"\r\n")
                    if resp.queue.empty():
                        break
                    chunk = resp.queue.get_nowait()
                if end:
                    parts.append(b"0\r\n\r\n")
                writer.write(b"".join(parts))
                await writer.drain()
                if end:
                    return True
        except (ConnectionError, OSError):
            resp.closed = True
            req.disconnected.set()
            return False
