"""Shared KV-block store: a third tier behind the device cache and the host tier, shared by instances.

Role of the reference's KVCacheStore (xllm/core/framework/kv_cache/kv_cache_store.cpp:89-183: batch_put / batch_get /
batch_exist of host KV blocks in a Mooncake distributed store, keyed by the block's prefix hash; flags
enable_kvcache_store, store_protocol, store_master_server_address, global_flags.cpp:444-466).  Mooncake is not available
here, so the store is a small server of its own (`xllm-kv-store`, or `python -m xllm_wxh_b200.service.kv_store`): blocks
live in its memory under `<prefix key>/<rank>/<world>` with least-recently-used eviction at a byte capacity.

Wire format (one TCP connection per client, requests answered in order):

    request   u32 header length | JSON header {"op": "put"|"get"|"exist"|"stats", "keys": [...], "sizes": [...]} | payload
    response  u32 header length | JSON header {"ok": bool, "found": [...], "sizes": [...]} | payload

Payloads are the raw block records back to back (no encoding), so a block crosses the socket as it lies in pinned memory.
The client never raises into the serving path: an unreachable store reads as a miss, a failed put is dropped.
"""
from __future__ import annotations

import argparse
import json
import logging
import socket
import socketserver
import struct
import threading
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

log = logging.getLogger("xllm.kv_store")


def _recv_exact(sock: socket.socket, n: int) -> Optional[bytearray]:
    buf = bytearray(n)
    view, got = memoryview(buf), 0
    while got < n:
        k = sock.recv_into(view[got:], n - got)
        if k == 0:
            return None
        got += k
    return buf


def _send_msg(sock: socket.socket, header: Dict, payloads: Sequence = ()) -> None:
    h = json.dumps(header).encode()
    sock.sendall(struct.pack("<I", len(h)) + h)
    for p in payloads:
        sock.sendall(p)


# Limits of one message.  They bound what a single peer can make this process allocate: the lengths come from the wire.
MAX_HEADER_BYTES = 1 << 20
MAX_KEYS_PER_MESSAGE = 4096
MAX_PAYLOAD_BYTES = 1 << 30


def _recv_msg(sock: socket.socket, max_payload: int = MAX_PAYLOAD_BYTES) -> Optional[Tuple[Dict, bytearray]]:
    hdr = _recv_exact(sock, 4)
    if hdr is None:
        return None
    n = struct.unpack("<I", hdr)[0]
    if n > MAX_HEADER_BYTES:
        raise ValueError(f"message header of {n} bytes exceeds the limit of {MAX_HEADER_BYTES}")
    raw = _recv_exact(sock, n)
    if raw is None:
        return None
    header = json.loads(bytes(raw))
    if not isinstance(header, dict):
        raise ValueError("message header is not an object")
    sizes = header.get("sizes") or ()
    if len(sizes) > MAX_KEYS_PER_MESSAGE or len(header.get("keys") or ()) > MAX_KEYS_PER_MESSAGE:
        raise ValueError("too many keys in one message")
    if any(int(s) < 0 for s in sizes):
        raise ValueError("negative payload size")
    total = sum(int(s) for s in sizes)
    if total > max_payload:
        raise ValueError(f"payload of {total} bytes exceeds the limit of {max_payload}")
    payload = _recv_exact(sock, total) if total else bytearray()
    if payload is None:
        return None
    return header, payload


class KvStore:
    """The store itself: key -> bytes, least recently used first out."""

    def __init__(self, capacity_bytes: int = 1 << 30):
        self.capacity = int(capacity_bytes)
        self.used = 0
        self.blocks: "OrderedDict[str, bytes]" = OrderedDict()
        self.lock = threading.Lock()
        self.puts = self.gets = self.hits = self.evictions = 0

    def put(self, key: str, data: bytes) -> bool:
        if len(data) > self.capacity:
            return False
        with self.lock:
            old = self.blocks.pop(key, None)
            if old is not None:
                self.used -= len(old)
            while self.used + len(data) > self.capacity and self.blocks:
                _, ev = self.blocks.popitem(last=False)
                self.used -= len(ev)
                self.evictions += 1
            self.blocks[key] = data
            self.used += len(data)
            self.puts += 1
            return True

    def get(self, key: str) -> Optional[bytes]:
        with self.lock:
            self.gets += 1
            data = self.blocks.get(key)
            if data is not None:
                self.blocks.move_to_end(key)
                self.hits += 1
            return data

    def exist(self, key: str) -> bool:
        with self.lock:
            return key in self.blocks

    def stats(self) -> Dict[str, int]:
        with self.lock:
            return {"blocks": len(self.blocks), "bytes": self.used, "capacity": self.capacity, "puts": self.puts,
                    "gets": self.gets, "hits": self.hits, "evictions": self.evictions}


class _Handler(socketserver.BaseRequestHandler):
    def handle(self):
        store: KvStore = self.server.store                     # type: ignore[attr-defined]
        sock = self.request
        sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        while True:
            try:
                # nothing larger than the store itself can be kept: refuse it before it is read
                msg = _recv_msg(sock, min(MAX_PAYLOAD_BYTES, store.capacity))
            except (OSError, ValueError) as e:
                log.warning("kv store: dropping a connection: %s", e)
                return
            if msg is None:
                return
            header, payload = msg
            op, keys = header.get("op"), header.get("keys") or []
            try:
                if op == "put":
                    off, ok = 0, []
                    for k, s in zip(keys, header["sizes"]):
                        ok.append(store.put(str(k), bytes(payload[off:off + int(s)])))
                        off += int(s)
                    _send_msg(sock, {"ok": True, "found": ok})
                elif op == "get":
                    data = [store.get(str(k)) for k in keys]
                    _send_msg(sock, {"ok": True, "found": [d is not None for d in data],
                                     "sizes": [len(d) for d in data if d is not None]}, [d for d in data if d is not None])
                elif op == "exist":
                    _send_msg(sock, {"ok": True, "found": [store.exist(str(k)) for k in keys]})
                elif op == "stats":
                    _send_msg(sock, {"ok": True, "stats": store.stats()})
                else:
                    _send_msg(sock, {"ok": False, "error": f"unknown op {op!r}"})
            except OSError:
                return


class KvStoreServer(socketserver.ThreadingTCPServer):
    allow_reuse_address = True
    daemon_threads = True

    def __init__(self, host: str = "127.0.0.1", port: int = 0, capacity_bytes: int = 1 << 30):
        super().__init__((host, port), _Handler)
        self.store = KvStore(capacity_bytes)
        self.port = self.server_address[1]
        self._thread: Optional[threading.Thread] = None

    def start(self) -> "KvStoreServer":
        self._thread = threading.Thread(target=self.serve_forever, name="xllm-kv-store", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self.shutdown()
        self.server_close()


class KvStoreClient:
    """Client of one store.  Thread-safe (one request at a time on its connection); reconnects after a failure; every
    failure reads as "not found" / "not stored"."""

    def __init__(self, addr: str, timeout_s: float = 2.0):
        host, _, port = addr.rpartition(":")
        self.host, self.port, self.timeout_s = host or "127.0.0.1", int(port), timeout_s
        self._sock: Optional[socket.socket] = None
        self._lock = threading.Lock()
        self.failures = 0

    def _conn(self) -> socket.socket:
        if self._sock is None:
            s = socket.create_connection((self.host, self.port), timeout=self.timeout_s)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            self._sock = s
        return self._sock

    def _call(self, header: Dict, payloads: Sequence = ()) -> Optional[Tuple[Dict, bytearray]]:
        with self._lock:
            try:
                s = self._conn()
                _send_msg(s, header, payloads)
                rep = _recv_msg(s)
                if rep is None:
                    raise OSError("connection closed by the store")
                return rep
            except (OSError, ValueError) as e:
                self.failures += 1
                log.debug("kv store call %s failed: %s", header.get("op"), e)
                if self._sock is not None:
                    try:
                        self._sock.close()
                    except OSError:
                        pass
                    self._sock = None
                return None

    def close(self) -> None:
        with self._lock:
            if self._sock is not None:
                self._sock.close()
                self._sock = None

    def batch_put(self, keys: Sequence[str], blocks: Sequence) -> int:
        """`blocks`: bytes-like objects (memoryviews of pinned records are sent as they are).  Returns how many were stored."""
        if not keys:
            return 0
        rep = self._call({"op": "put", "keys": list(keys), "sizes": [len(b) for b in blocks]}, blocks)
        return sum(1 for f in rep[0].get("found") or () if f) if rep and rep[0].get("ok") else 0

    def batch_exist(self, keys: Sequence[str]) -> List[bool]:
        if not keys:
            return []
        rep = self._call({"op": "exist", "keys": list(keys)})
        return [bool(f) for f in rep[0]["found"]] if rep and rep[0].get("ok") else [False] * len(keys)

    def batch_get(self, keys: Sequence[str]) -> List[Optional[memoryview]]:
        if not keys:
            return []
        rep = self._call({"op": "get", "keys": list(keys)})
        if not rep or not rep[0].get("ok"):
            return [None] * len(keys)
        header, payload = rep
        out: List[Optional[memoryview]] = []
        view, off, sizes = memoryview(payload), 0, iter(header.get("sizes") or ())
        for f in header["found"]:
            if f:
                n = int(next(sizes))
                out.append(view[off:off + n])
                off += n
            else:
                out.append(None)
        return out

    def stats(self) -> Optional[Dict[str, int]]:
        rep = self._call({"op": "stats"})
        return rep[0].get("stats") if rep else None


def block_key(key: Tuple[int, int], rank: int = 0, world: int = 1, namespace: str = "") -> str:
    """Store key of one rank's share of a block: the model's namespace, the 128-bit prefix key in hex, then rank and world
    size (instances with another sharding hold other bytes under the same prefix key)."""
    return f"{namespace}{int(key[1]) & (2**64 - 1):016x}{int(key[0]) & (2**64 - 1):016x}/{rank}/{world}"


def weights_fingerprint(model_dir: Optional[str], random_seed: int = 0) -> str:
    """What tells two sets of weights apart without reading them: for a checkpoint directory the names and sizes of its
    safetensors files (and of the index) plus the first and last 4 KiB of each; for random-initialised presets the seed.
    Two directories with the same base name but different weights, or two presets with different seeds, then keep
    separate keys in a shared store."""
    import hashlib
    import os
    h = hashlib.sha1()
    if not model_dir or not os.path.isdir(model_dir):
        h.update(f"random|{random_seed}".encode())
        return h.hexdigest()[:16]
    for name in sorted(os.listdir(model_dir)):
        if not (name.endswith(".safetensors") or name.endswith(".safetensors.index.json") or name == "config.json"):
            continue
        path = os.path.join(model_dir, name)
        size = os.path.getsize(path)
        h.update(f"{name}|{size}|".encode())
        with open(path, "rb") as f:
            h.update(f.read(4096))
            if size > 8192:
                f.seek(size - 4096)
                h.update(f.read(4096))
    return h.hexdigest()[:16]


def model_namespace(model_name: str, args, block_size: int, record_bytes: int, fingerprint: str = "", kv_dtype: str = "") -> str:
    """Prefix of the keys of one model: equal token prefixes of different models, weights, dtypes or cache geometries must
    not meet."""
    import hashlib
    ident = (f"{model_name}|{args.model_type}|{args.n_layers}|{args.n_kv_heads}|{args.head_dim}|{block_size}|{record_bytes}|"
             f"{getattr(args, 'dtype', '')}|{kv_dtype}|{fingerprint}")
    return hashlib.sha1(ident.encode()).hexdigest()[:12] + ":"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="KV-block store shared by xllm instances")
    ap.add_argument("--host", default="127.0.0.1", help="address to listen on (the store has no authentication: expose it "
                    "only on a network where every peer is trusted)")
    ap.add_argument("--port", type=int, default=50051)
    ap.add_argument("--capacity_gb", type=float, default=16.0)
    ns = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    srv = KvStoreServer(ns.host, ns.port, int(ns.capacity_gb * (1 << 30)))
    log.info("kv store on %s:%d, capacity %.1f GB", ns.host, srv.port, ns.capacity_gb)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        srv.server_close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
