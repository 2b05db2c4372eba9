"""Weights of a waking instance come from an awake instance of the same model instead of the checkpoint.

Role of the reference's MooncakeWeightTransfer (xllm/core/framework/kv_cache/mooncake_weight_transfer.cpp:69-140:
link_d2d / unlink_d2d open and close a session to a remote transfer engine, pull_weights reads weight segments out of the
remote instance's registered memory) and of `WakeupOptions.remote_addrs` (proto/xllm_service.proto:25-34).  There the
transport is Mooncake over RDMA between NPUs.  Here:

* the awake instance runs a `WeightServer` on its `--transfer_listen_port`; it describes its weights (one entry per
  distinct tensor, in the order the sleep code walks the model) and serves them;
* on one host with CUDA devices the server hands out CUDA-IPC handles of the weight allocations of every rank, and each
  rank of the waking instance copies device to device (`xl_copy_d2d`, one copy per tensor: NVLink between GPUs);
* otherwise (CPU engines, another host) the bytes travel over the connection in chunks.

The unit of transfer is the storage range a tensor occupies, so any stride pattern survives; both sides compare their
layouts entry by entry before a byte moves, and a mismatch makes the sleeper read its checkpoint instead.
"""
from __future__ import annotations

import base64
import ctypes
import logging
import socket
import threading
from typing import Any, Dict, List, Optional

import torch

from .disagg_pd import SocketTransport, serve_transport
from .sleep import flat_span, weight_manifest

log = logging.getLogger("xllm.weight_transfer")
CHUNK = 8 << 20            # bytes per message on the TCP path


def runtime_ipc_handle(handle: bytes) -> bytes:
    """The 64-byte CUDA runtime IPC handle inside what torch's storage sharing returns: torch writes the plain handle, or
    the handle behind one or two tag bytes (format version, allocation kind) for memory that came from cudaMalloc.
    Anything longer describes an expandable segment, which the runtime call cannot open."""
    if len(handle) not in (64, 65, 66):
        raise RuntimeError(f"storage is not shareable through a CUDA runtime IPC handle (descriptor of {len(handle)} bytes)")
    return bytes(handle[-64:])


def _export_handles(tensors: List[torch.Tensor]) -> List[Dict[str, Any]]:
    """CUDA-IPC description of every tensor: handle of the allocation it lives in + byte offset inside it."""
    out = []
    for t in tensors:
        _, handle, _, offset, *_ = t.untyped_storage()._share_cuda_()
        handle = runtime_ipc_handle(handle)
        out.append({"handle": base64.b64encode(handle).decode(),
                    "offset": int(offset) + t.storage_offset() * t.element_size()})
    return out


class WeightServer:
    """Serves the weights of `master`'s engine to waking instances."""

    def __init__(self, master):
        self.master = master
        self.engine = master.engine
        self.sessions: List[SocketTransport] = []
        self._srv: Optional[socket.socket] = None
        self.bytes_served = 0
        self._lock = threading.Lock()

    def serve(self, port: int, host: str = "0.0.0.0") -> socket.socket:
        self._srv = serve_transport(port, self._attach, host)
        return self._srv

    def close(self) -> None:
        if self._srv is not None:
            self._srv.close()
        for t in list(self.sessions):
            t.close()

    def _attach(self, t: SocketTransport) -> None:
        t.handler = lambda method, payload, tt=t: self._handle(tt, method, payload)
        t.on_close = lambda tt=t: self.sessions.remove(tt) if tt in self.sessions else None
        self.sessions.append(t)

    def _local(self):
        eng = self.engine
        if eng.sleep_level != 0:
            raise RuntimeError("this instance is asleep and holds no weights")
        return weight_manifest(eng.worker.model, eng.worker.device)

    def _handle(self, t, method: str, p: Dict) -> Dict:
        eng = self.engine
        if method == "describe":
            manifest, _ = self._local()
            return {"model_type": eng.args.model_type, "world_size": eng.world_size, "hostname": socket.gethostname(),
                    "device": eng.device.type, "manifest": manifest}
        if method == "handles":
            if eng.device.type != "cuda":
                return {"error": "no CUDA device"}
            with self.master._step_lock:           # a control operation on every rank: never in the middle of a step
                return {"handles": eng.collect_weight_handles()}
        if method == "bytes":
            if eng.world_size != 1:
                return {"error": "the byte path serves engines of one process"}
            _, tensors = self._local()
            flat = flat_span(tensors[int(p["index"])]).view(torch.uint8)
            lo = int(p["offset"])
            part = flat[lo:lo + min(int(p["size"]), CHUNK)].cpu().contiguous()
            raw = part.numpy().tobytes()
            with self._lock:
                self.bytes_served += len(raw)
            return {"data": base64.b64encode(raw).decode()}
        return {"error": f"unknown method {method}"}


def _same_layout(mine: List[Dict], theirs: List[Dict]) -> Optional[str]:
    if len(mine) != len(theirs):
        return f"{len(mine)} weight tensors here, {len(theirs)} at the source"
    for i, (a, b) in enumerate(zip(mine, theirs)):
        if (a["shape"], a["stride"], a["dtype"]) != (b["shape"], b["stride"], b["dtype"]):
            return f"tensor {i}: {a['dtype']}{a['shape']} here, {b['dtype']}{b['shape']} at the source"
    return None


class WeightPuller:
    """Session of a (sleeping) instance with one weight source (`link_d2d` opens it, `unlink_d2d` closes it)."""

    def __init__(self, addr: str, connect_timeout: float = 3.0):
        host, _, port = addr.rpartition(":")
        self.addr = addr
        self.t = SocketTransport.connect(host or "127.0.0.1", int(port), timeout=connect_timeout)
        self.t.on_close = lambda: None
        self.info: Optional[Dict[str, Any]] = None
        self.bytes_pulled = 0

    def close(self) -> None:
        self.t.close()

    def describe(self) -> Dict[str, Any]:
        info = self.t.call("describe", {}, timeout=30.0)
        if not isinstance(info, dict) or "error" in info:
            raise RuntimeError(f"weight source {self.addr}: {info!r}")
        self.info = info
        return info

    def check(self, engine) -> None:
        """Raises unless the source holds the weights this (deep-sleeping) engine dropped, tensor for tensor."""
        info = self.describe()
        if info["model_type"] != engine.args.model_type or info["world_size"] != engine.world_size:
            raise RuntimeError(f"source serves {info['model_type']} on {info['world_size']} ranks")
        why = _same_layout(engine._sleep_state.manifest, info["manifest"])
        if why:
            raise RuntimeError(f"weight layout differs: {why}")

    def same_host(self) -> bool:
        return bool(self.info) and self.info["hostname"] == socket.gethostname() and self.info["device"] == "cuda"

    def handles(self) -> List[List[Dict[str, Any]]]:
        r = self.t.call("handles", {}, timeout=60.0)
        if not isinstance(r, dict) or "handles" not in r:
            raise RuntimeError(f"weight source {self.addr} gave no IPC handles: {r!r}")
        return r["handles"]

    # TCP path (engines of one process): called by the wake-up code of the rank
    def pull_into(self, manifest: List[Dict], tensors: List[torch.Tensor], rank: int) -> None:
        for i, (m, t) in enumerate(zip(manifest, tensors)):
            flat = flat_span(t).view(torch.uint8)
            lo, n = 0, int(m["nbytes"])
            while lo < n:
                r = self.t.call("bytes", {"index": i, "offset": lo, "size": min(CHUNK, n - lo)}, timeout=120.0)
                if not isinstance(r, dict) or "data" not in r:
                    raise RuntimeError(f"weight source {self.addr} failed on tensor {i}: {r!r}")
                raw = base64.b64decode(r["data"])
                if not raw:
                    raise RuntimeError(f"weight source {self.addr} sent no data for tensor {i}")
                flat[lo:lo + len(raw)].copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
                lo += len(raw)
                self.bytes_pulled += len(raw)


class IpcWeightSource:
    """Runs on every rank of the waking engine: maps the source rank's weight allocations and copies tensor by tensor."""

    def __init__(self, handles_per_rank: List[List[Dict[str, Any]]], device: torch.device):
        self.handles_per_rank, self.device = handles_per_rank, device
        self._opened: Dict[bytes, int] = {}
        self.copy_ms = 0.0                   # device time of the copies of the last pull

    def pull_into(self, manifest: List[Dict], tensors: List[torch.Tensor], rank: int) -> None:
        from ..ops import cuda_ops
        from ..ops.cuda_ops import _check, _stream, c_long, c_void_p, lib
        L = lib()
        L.xl_ipc_open_handle.restype = ctypes.c_void_p
        mine = self.handles_per_rank[rank % len(self.handles_per_rank)]
        if len(mine) != len(tensors):
            raise RuntimeError("the source rank exported a different number of weight tensors")
        # map every allocation first, so that the timed span holds the copies only
        for h in mine:
            raw = base64.b64decode(h["handle"])
            if raw not in self._opened:
                base = L.xl_ipc_open_handle((ctypes.c_char * 64).from_buffer_copy(raw[:64]))
                if not base:
                    raise RuntimeError("cudaIpcOpenMemHandle failed for a weight allocation of the source")
                self._opened[raw] = base
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(torch.cuda.current_stream(self.device))
        for m, t, h in zip(manifest, tensors, mine):
            raw = base64.b64decode(h["handle"])
            base = self._opened.get(raw)
            if base is None:
                base = L.xl_ipc_open_handle((ctypes.c_char * 64).from_buffer_copy(raw[:64]))
                if not base:
                    raise RuntimeError("cudaIpcOpenMemHandle failed for a weight allocation of the source")
                self._opened[raw] = base
            _check(L.xl_copy_d2d(c_void_p(t.data_ptr()), c_void_p(base + h["offset"]), c_long(int(m["nbytes"])), _stream()),
                   "xl_copy_d2d")
            cuda_ops.launch_count += 1
        end.record(torch.cuda.current_stream(self.device))
        torch.cuda.synchronize(self.device)
        self.copy_ms = start.elapsed_time(end)

    def close(self) -> None:
        from ..ops.cuda_ops import c_void_p, lib
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        for base in self._opened.values():
            lib().xl_ipc_close_handle(c_void_p(base))
        self._opened = {}
