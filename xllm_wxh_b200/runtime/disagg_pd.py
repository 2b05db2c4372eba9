"""Prefill / decode disaggregation: control plane between a PREFILL instance and a DECODE instance.

Protocol (the reference's DisaggPDService, xllm/proto/disagg_pd.proto:244-251, scheduler/disagg_pd_scheduler.cpp:316-734,
distributed_runtime/disagg_pd_service_impl.cpp):

  link              P -> D   exchange instance info; D returns the CUDA-IPC descriptions of its KV-cache tensors
  add_new_request   P -> D   request meta (prompt ids, sampling, stop); D reserves KV blocks and replies their ids
  (prefill on P; PUSH mode: the KV blocks of the prompt are pushed into D's reserved blocks chunk by chunk and layer by
   layer under the forward pass.  PULL mode, `--kv_cache_transfer_mode PULL`: P maps nothing and pushes nothing; its
   `link` call hands P's cache descriptions to D, and `first_generation` names P's blocks of the prompt, which D's ranks
   read over NVLink before they activate the request - P waits for that reply before its next scheduling round, so the
   blocks cannot have been given to another request)
  first_generations P -> D   first tokens (+ logprobs) of the requests whose prefill ended in this step: D activates them as
                             running decodes (in PULL mode after one fetch of all their blocks)
  generations       D -> P   tokens decoded on D, forwarded to the client connection that P holds
  cancel            P -> D   client went away

Transports: `InProcTransport` (both instances in one process: tests, single-process deployments) and `SocketTransport`
(length-prefixed JSON over TCP between two `xllm` server processes, `--disagg_pd_port`).  Every call has a time-out; a peer
that stops answering marks the instance unhealthy (utils/health.py) instead of blocking the scheduler.
"""
from __future__ import annotations

import json
import socket
import struct
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

from .. import _core
from ..framework.params import FINISH_REASONS, RequestOutput, RequestParams, SequenceOutput, Status, StatusCode, Usage
from ..utils.health import HEALTH
from ..utils.metrics import METRICS
from .master import LLMMaster


# ----------------------------------------------------------------------------- transports
class InProcTransport:
    """Direct calls between two coordinator objects living in the same process."""

    def __init__(self):
        self.peer: Optional["InProcTransport"] = None
        self.handler: Optional[Callable[[str, Dict], Any]] = None
        self.on_close: Optional[Callable[[], None]] = None
        self.closed = False

    @staticmethod
    def pair() -> Tuple["InProcTransport", "InProcTransport"]:
        a, b = InProcTransport(), InProcTransport()
        a.peer, b.peer = b, a
        return a, b

    def call(self, method: str, payload: Dict, timeout: float = 10.0) -> Any:
        if self.closed:
            raise OSError("peer connection closed")
        return self.peer.handler(method, payload)

    def notify(self, method: str, payload: Dict) -> None:
        if self.closed:
            raise OSError("peer connection closed")
        self.peer.handler(method, payload)

    def close(self):
        """Both ends learn that the link is gone (a vanished peer, in tests)."""
        for end in (self, self.peer):
            if end is not None and not end.closed:
                end.closed = True
                if end.on_close is not None:
                    end.on_close()


class SocketTransport:
    """Length-prefixed JSON messages {id, kind: call|reply|notify, method, payload} over one TCP connection."""

    on_close: Optional[Callable[[], None]] = None

    def __init__(self, sock: socket.socket, start: bool = True):
        self.sock = sock
        self.handler: Optional[Callable[[str, Dict], Any]] = None
        self._lock = threading.Lock()
        self._next = 1
        self._waiting: Dict[int, Tuple[threading.Event, List]] = {}
        self._alive = True
        self._thread = threading.Thread(target=self._recv_loop, name="xllm-pd-recv", daemon=True)
        if start:
            self._thread.start()

    def start(self) -> None:
        """Begin to receive (for a transport made with start=False, once its handler is installed)."""
        if not self._thread.is_alive():
            self._thread.start()

    @classmethod
    def connect(cls, host: str, port: int, timeout: float = 30.0) -> "SocketTransport":
        deadline = time.time() + timeout
        last = None
        while time.time() < deadline:
            try:
                s = socket.create_connection((host, port), timeout=5)
                s.settimeout(None)
                return cls(s)
            except OSError as e:            # the decode instance may still be starting (max_reconnect_count in the reference)
                last = e
                time.sleep(0.25)
        raise ConnectionError(f"cannot reach decode instance at {host}:{port}: {last}")

    def _send(self, obj: Dict):
        data = json.dumps(obj).encode()
        with self._lock:
            self.sock.sendall(struct.pack("<I", len(data)) + data)

    def _recv_exact(self, n: int) -> Optional[bytes]:
        buf = b""
        while len(buf) < n:
            chunk = self.sock.recv(n - len(buf))
            if not chunk:
                return None
            buf += chunk
        return buf

    def _recv_loop(self):
        try:
            while self._alive:
                hdr = self._recv_exact(4)
                if hdr is None:
                    break
                body = self._recv_exact(struct.unpack("<I", hdr)[0])
                if body is None:
                    break
                msg = json.loads(body)
                if msg["kind"] == "reply":
                    w = self._waiting.pop(msg["id"], None)
                    if w:
                        w[1].append(msg.get("payload"))
                        w[0].set()
                elif msg["kind"] == "call":
                    try:
                        res = self.handler(msg["method"], msg["payload"])
                    except Exception as e:      # report instead of dropping the connection
                        res = {"error": f"{type(e).__name__}: {e}"}
                    self._send({"id": msg["id"], "kind": "reply", "payload": res})
                else:
                    self.handler(msg["method"], msg["payload"])
        except OSError:
            pass
        finally:
            self._alive = False
            for ev, _ in list(self._waiting.values()):
                ev.set()
            if self.on_close is not None:
                self.on_close()                       # the coordinator decides what the loss means for this instance
            else:
                HEALTH.set_unhealthy("disaggregated peer connection closed")

    def call(self, method: str, payload: Dict, timeout: float = 10.0) -> Any:
        with self._lock:
            mid = self._next
            self._next += 1
        ev, box = threading.Event(), []
        self._waiting[mid] = (ev, box)
        self._send({"id": mid, "kind": "call", "method": method, "payload": payload})
        if not ev.wait(timeout) or not box:
            self._waiting.pop(mid, None)
            raise TimeoutError(f"disaggregated peer did not answer '{method}' within {timeout}s")
        return box[0]

    def notify(self, method: str, payload: Dict) -> None:
        self._send({"id": 0, "kind": "notify", "method": method, "payload": payload})

    def close(self):
        self._alive = False
        try:
            self.sock.close()
        except OSError:
            pass


def serve_transport(port: int, on_connect: Callable[[SocketTransport], None], host: str = "0.0.0.0") -> socket.socket:
    """Accept loop of the decode instance (one transport per linked prefill instance)."""
    srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    srv.bind((host, port))
    srv.listen(16)

    def loop():
        while True:
            try:
                conn, _ = srv.accept()
            except OSError:
                return
            t = SocketTransport(conn, start=False)   # the peer's first call must not arrive before the handler is installed
            on_connect(t)
            t.start()
    threading.Thread(target=loop, name="xllm-pd-accept", daemon=True).start()
    return srv


# ----------------------------------------------------------------------------- decode side
class DecodeCoordinator:
    def __init__(self, master: LLMMaster):
        self.master = master
        self.engine = master.engine
        self.transports: List[Any] = []
        self._owner: Dict[int, Any] = {}            # D request id -> transport of the prefill instance that owns it
        self._skip_first: Dict[int, bool] = {}       # the first token was delivered to the client by the prefill instance
        self._reserved: Dict[int, List[int]] = {}    # PULL mode: D request id -> the blocks reserved for its prompt
        self._source_of: Dict[int, int] = {}         # id(transport) -> index of that prefill instance's mapped cache
        self._lock = threading.Lock()
        master.extra_step_hooks.append(lambda m: None)
        self._orig_emit = master._emit
        master._emit = self._emit                    # decode-side outputs go back to the prefill instance

    def attach(self, transport) -> None:
        transport.handler = lambda method, payload, t=transport: self._handle(t, method, payload)
        transport.on_close = lambda t=transport: self.unlink(t)
        self.transports.append(transport)

    def unlink(self, transport) -> int:
        """A prefill instance has gone away: release what it reserved here and stop decoding for it
        (unlink_instance and the clean-up of a vanished prefill instance's requests, disagg_pd_scheduler.h:77-90,158-170 of
        the reference).  The decode instance itself stays healthy and keeps serving its other peers."""
        with self._lock:
            mine = [rid for rid, t in self._owner.items() if t is transport]
            for rid in mine:
                self._owner.pop(rid, None)
                self._skip_first.pop(rid, None)
                self._reserved.pop(rid, None)
                self.engine.scheduler.drop_remote(rid)       # reserved, first token never arrived
                self.engine.cancel(rid)                      # already decoding
            if transport in self.transports:
                self.transports.remove(transport)
        self.master._wake.set()
        METRICS.inc("pd_unlinked_prefill_instances_total", 1)
        return len(mine)

    def serve(self, port: int):
        return serve_transport(port, self.attach)

    def _handle(self, transport, method: str, p: Dict):
        if method == "link":
            eng = self.engine
            handles = None
            if p.get("want_handles"):
                with self.master.control_lock():           # a control operation on every rank: never in the middle of a step
                    handles = eng.collect_cache_handles()
            if p.get("mode") == "PULL":
                with self._lock:
                    source = self._source_of.setdefault(id(transport), len(self._source_of))
                if p.get("source_handles"):
                    with self.master.control_lock():
                        eng.link_kv_source(p["source_handles"], source)
            return {"instance_name": self.master.opt.instance_name, "block_size": eng.block_size, "num_blocks": eng.num_blocks,
                    "tp_size": eng.comm.tp_size, "model_type": eng.args.model_type, "handles": handles}
        if method == "add_new_request":
            sp = _core.SamplingParams()
            for k, v in p["sampling"].items():
                setattr(sp, k, v)
            st = _core.StopCriteria()
            for k, v in p["stop"].items():
                setattr(st, k, v)
            with self._lock:
                rid, blocks, dp_rank = self.engine.scheduler.reserve_remote(p["prompt"], sp, st, p.get("ext_id", ""))
                if rid >= 0:
                    self._owner[rid] = transport
                    if id(transport) in self._source_of:
                        self._reserved[rid] = list(blocks)
            return {"ok": rid >= 0, "request_id": rid, "blocks": list(blocks), "dp_rank": dp_rank}
        if method == "first_generations":
            # every request that finished its prefill in one step of the prefill instance: one fetch for all of them
            items = p["items"]
            pairs, ok_items = [], []
            with self._lock:
                source = self._source_of.get(id(transport))
                for it in items:
                    if it.get("src_blocks") is None:
                        ok_items.append(it)
                        continue
                    dst = self._reserved.pop(it["request_id"], None)
                    if dst is None or source is None:
                        continue
                    pairs.extend(zip(it["src_blocks"], dst))
                    ok_items.append(it)
            if pairs:
                with self.master.control_lock():
                    if not self.engine.pull_kv(source, pairs):
                        return {"ok": []}
                METRICS.inc("pd_pulled_blocks_total", len(pairs))
            done = []
            with self._lock:
                for it in ok_items:
                    self._skip_first[it["request_id"]] = True
                    if self.engine.scheduler.activate_remote(it["request_id"], it["token"], it.get("logprob", 0.0)):
                        done.append(it["request_id"])
            self.master._wake.set()
            return {"ok": done}
        if method == "first_generation":
            if p.get("src_blocks") is not None:
                # PULL mode: fetch the prompt's KV out of the prefill instance's cache before the request may run
                with self._lock:
                    dst = self._reserved.pop(p["request_id"], None)
                    source = self._source_of.get(id(transport))
                if dst is None or source is None:
                    return {"ok": False}
                pairs = list(zip(p["src_blocks"], dst))
                with self.master.control_lock():
                    if pairs and not self.engine.pull_kv(source, pairs):
                        return {"ok": False}
                METRICS.inc("pd_pulled_blocks_total", len(pairs))
            with self._lock:
                self._skip_first[p["request_id"]] = True
                ok = self.engine.scheduler.activate_remote(p["request_id"], p["token"], p.get("logprob", 0.0))
            self.master._wake.set()
            return {"ok": bool(ok)}
        if method == "cancel":
            self._reserved.pop(p["request_id"], None)
            self.engine.scheduler.drop_remote(p["request_id"])
            self.engine.cancel(p["request_id"])
            return {"ok": True}
        raise ValueError(f"unknown method {method}")

    def _emit(self, outs) -> None:
        """Forward decode outputs of remote-owned requests to their prefill instance; the rest goes the local way."""
        local = []
        per_t: Dict[int, List[Dict]] = {}
        for o in outs:
            t = self._owner.get(o.request_id)
            if t is None:
                local.append(o)
                continue
            toks, lps = list(o.new_tokens), list(o.new_logprobs)
            if self._skip_first.pop(o.request_id, False) and toks:
                toks, lps = toks[1:], lps[1:]
            if not toks and not o.finished:
                continue
            per_t.setdefault(id(t), []).append({"request_id": o.request_id, "tokens": toks,
                                                "logprobs": lps, "finished": bool(o.finished),
                                                "finish_reason": int(o.finish_reason), "num_generated": o.num_generated})
            if o.finished:
                self._owner.pop(o.request_id, None)
        for t in self.transports:
            msgs = per_t.get(id(t))
            if msgs:
                try:
                    t.notify("generations", {"outputs": msgs})
                except OSError:
                    for m in msgs:
                        self.engine.cancel(m["request_id"])
        if local:
            self._orig_emit(local)


# ----------------------------------------------------------------------------- prefill side
class _RemoteSeqOutput:
    """Shape of `_core.SeqOutput` for tokens that were generated on the decode instance."""

    def __init__(self, request_id, tokens, logprobs, finished, finish_reason, n_prompt, n_gen):
        self.request_id, self.ext_id, self.seq_index = request_id, "", 0
        self.new_tokens, self.new_logprobs = tokens, logprobs
        self.finished, self.finish_reason = finished, finish_reason
        self.num_prompt_tokens, self.num_generated, self.num_cached_tokens = n_prompt, n_gen, 0
        self.request_finished = finished


class PrefillCoordinator:
    """Prefill side of disaggregated serving.  It may be linked to several decode instances: link 0 is made by the
    constructor, further ones by `add_decode_link`.  A request goes to the decode instance its `routing.decode_name` names
    (the service layer chose it), or to the links in turn when it names none.  Destination blocks of link i travel in the
    step message with i in the top byte, so the wire format of a single pair of instances is unchanged."""
    PEER_SHIFT = 24

    def __init__(self, master: LLMMaster, transport=None):
        self.master = master
        self.engine = master.engine
        self.links: List[Dict[str, Any]] = []
        self.remote: Dict[int, Dict] = {}                      # local core id -> {"rid", "blocks", "first", "link"}
        self.by_remote: Dict[Tuple[int, int], int] = {}        # (link, D request id) -> local core id
        self._pending_out: List = []
        self._lock = threading.Lock()
        self._rr = 0
        self.pull = master.opt.kv_cache_transfer_mode == "PULL"
        if transport is not None:                  # None: links are made later (discovery through the service layer)
            self.add_decode_link(transport)
        self.engine.transfer_pairs_provider = self._pairs_for
        self._orig_build = master._build
        master._build = self._build
        self._orig_emit = master._emit
        master._emit = self._emit

    # the first link under its old names (one decode instance is the common case)
    @property
    def t(self):
        return self.links[0]["t"]

    @property
    def peer_info(self):
        return self.links[0]["info"]

    def add_decode_link(self, transport) -> int:
        """Link one more decode instance (link_instance in the reference, disagg_pd_scheduler.h:77-90): exchange cache
        geometry, map its KV cache on every rank of this instance.  Returns the link index."""
        index = len(self.links)
        if index >= 1 << (31 - self.PEER_SHIFT):
            raise ValueError("too many decode links")
        transport.handler = lambda method, payload, i=index: self._handle(method, payload, i)
        transport.on_close = lambda i=index: self.peer_lost(i)
        ipc = self.engine.device.type == "cuda" and not isinstance(transport, InProcTransport)
        req: Dict[str, Any] = {"want_handles": ipc and not self.pull}
        if self.pull:
            req["mode"] = "PULL"
            if ipc:
                with self.master.control_lock():
                    req["source_handles"] = self.engine.collect_cache_handles()
        info = transport.call("link", req, timeout=60.0)
        if not isinstance(info, dict) or "error" in info or "block_size" not in info:
            raise ValueError(f"decode instance refused the link: {info!r}")
        if info["block_size"] != self.engine.block_size:
            raise ValueError("prefill and decode instances must use the same block_size")
        if info["num_blocks"] >= 1 << self.PEER_SHIFT:
            raise ValueError("decode instance has too many KV blocks for the pair encoding")
        self.links.append({"t": transport, "info": info, "alive": True})
        if info.get("handles"):
            with self.master.control_lock():               # links may be made while the instance serves (discovery thread)
                self.engine.link_kv_peer(info["handles"], index)
        return index

    def _alive(self) -> List[int]:
        return [i for i, l in enumerate(self.links) if l["alive"]]

    def _pick_link(self, decode_name: str) -> Tuple[Optional[int], str]:
        alive = self._alive()
        if not alive:
            return None, "no decode instance is linked"
        if decode_name:
            named = [i for i in alive if (self.links[i]["info"].get("instance_name") or "") == decode_name]
            if named:
                return named[0], ""
            known = [self.links[i]["info"].get("instance_name") or "" for i in alive]
            if any(known):
                return None, f"not linked to decode instance {decode_name!r} (linked: {', '.join(repr(k) for k in known)})"
        self._rr += 1
        return alive[self._rr % len(alive)], ""

    def peer_lost(self, link: int = 0) -> int:
        """A decode instance has gone away: every request that was handed over to it (or is about to be) ends with an error
        for its client.  With no decode instance left this instance reports itself unhealthy, since it cannot finish a
        request on its own."""
        with self._lock:
            if link < len(self.links):
                self.links[link]["alive"] = False
            cids = [cid for cid, info in self.remote.items() if info["link"] == link]
            for cid in cids:
                info = self.remote.pop(cid)
                self.by_remote.pop((link, info["rid"]), None)
            self._pending_out = [c for c in self._pending_out if c not in cids]
        for cid in cids:
            st = self.master._states.get(cid)
            if st is None or st.done:
                continue
            self.engine.cancel(cid)
            st.done = True
            try:
                st.callback(RequestOutput(request_id=st.ext_id, finished=True,
                                          status=Status(StatusCode.UNAVAILABLE, "decode instance went away")))
            except Exception:
                pass
            self.master._states.pop(cid, None)
        if not self._alive():
            HEALTH.set_unhealthy("decode instance of the disaggregated pair went away")
        return len(cids)

    # request intake: reserve on the decode instance first (dispatch_requests in the reference)
    def _build(self, prompt, prompt_ids, params: RequestParams, callback):
        if prompt_ids is None:
            prompt_ids = self.master.tokenizer.encode(prompt or "", add_special_tokens=params.add_special_tokens)
        prompt_ids = list(prompt_ids)
        p = RequestParams(**{**params.__dict__})
        link, why = self._pick_link(p.decode_name)
        if link is None:
            # no decode instance, or the service layer routed the request to one this instance holds no KV link to
            callback(RequestOutput(request_id=params.request_id, finished=True, status=Status(StatusCode.UNAVAILABLE, why)))
            return None
        t = self.links[link]["t"]
        max_ctx = self.master.args.max_position_embeddings
        p.max_tokens = max(1, min(p.max_tokens, max_ctx - len(prompt_ids)))
        sp, st = p.to_core(self.master._eos(), list(self.master.args.stop_token_ids), [])
        st.max_context_len = max_ctx
        try:
            rep = t.call("add_new_request", {
                "prompt": prompt_ids, "ext_id": p.request_id,
                "sampling": {k: getattr(sp, k) for k in ("temperature", "top_p", "top_k", "repetition_penalty", "frequency_penalty",
                                                         "presence_penalty", "logprobs", "top_logprobs", "seed")},
                "stop": {"max_tokens": st.max_tokens, "max_context_len": st.max_context_len, "eos_token_id": st.eos_token_id,
                         "ignore_eos": st.ignore_eos, "stop_token_ids": list(st.stop_token_ids)}})
        except (TimeoutError, OSError) as e:
            callback(RequestOutput(request_id=params.request_id, finished=True,
                                   status=Status(StatusCode.UNAVAILABLE, f"decode instance unreachable: {e}")))
            return None
        if not rep.get("ok"):
            callback(RequestOutput(request_id=params.request_id, finished=True,
                                   status=Status(StatusCode.RESOURCE_EXHAUSTED, "decode instance has no free KV blocks")))
            return None
        cid = self._orig_build(prompt, prompt_ids, params, callback)
        if cid is None:
            t.notify("cancel", {"request_id": rep["request_id"]})
            return None
        with self._lock:
            self.remote[cid] = {"rid": rep["request_id"], "blocks": rep["blocks"], "first": None, "link": link}
            self.by_remote[(link, rep["request_id"])] = cid
        return cid

    def _pairs_for(self, batches) -> List[Tuple[int, int]]:
        """(source block, destination block) pairs to push in this step: for every prompt chunk of a handed-over request,
        the blocks that the chunk completes or touches (and, at its first chunk, the blocks its cached prefix already
        held).  A long prompt's KV thus leaves chunk by chunk while later chunks are still being computed; the block a
        chunk leaves partly filled travels again with the next chunk."""
        pairs: List[Tuple[int, int]] = []
        bs = self.engine.block_size
        for b in batches:
            if b.empty:
                continue
            for i, e in enumerate(b.entries()):
                info = self.remote.get(e[1])
                if info is None or info.get("first") is not None:
                    continue
                src = b.seq_blocks(i)
                kv_before, n_tok = e[5], e[5] + e[2]
                if self.pull:                                       # the decode instance fetches them after the last chunk
                    info["src_blocks"] = [int(x) for x in src[:min((n_tok + bs - 1) // bs, len(src), len(info["blocks"]))]]
                    continue
                if kv_before < info.get("pushed", 0) * bs:          # recomputed after a preemption: start over
                    info["pushed"] = 0
                lo = info.get("pushed", 0)
                hi = min((n_tok + bs - 1) // bs, len(src), len(info["blocks"]))
                tag = info["link"] << self.PEER_SHIFT               # which decode instance the blocks belong to
                pairs.extend((src[j], info["blocks"][j] | tag) for j in range(lo, hi))
                info["pushed"] = n_tok // bs                         # whole blocks are done with
        return pairs

    def _emit(self, outs) -> None:
        """Local outputs: the first token is delivered to the client; the hand-off itself is not a finish."""
        keep = []
        for o in outs:
            info = self.remote.get(o.request_id)
            if info is not None and o.finished and o.finish_reason == 5:          # HANDOFF
                info["first"] = (list(o.new_tokens), list(o.new_logprobs))
                keep.append(_RemoteSeqOutput(o.request_id, list(o.new_tokens), list(o.new_logprobs), False, 0, o.num_prompt_tokens,
                                             o.num_generated))
                self._pending_out.append(o.request_id)
            else:
                keep.append(o)
        if keep:
            self._orig_emit(keep)
        self._after_step(self.master)

    def _after_step(self, master) -> None:
        """After a step: make sure the pushed KV has landed everywhere, then tell the decode instance to start."""
        if not self._pending_out:
            return
        self.engine.barrier_sync()
        per_link: Dict[int, List[Dict]] = {}
        for cid in self._pending_out:
            info = self.remote.get(cid)
            if info is None or not info["first"] or not info["first"][0]:
                continue
            toks, lps = info["first"]
            msg = {"request_id": info["rid"], "token": int(toks[0]), "logprob": float(lps[0]) if lps else 0.0}
            if self.pull:
                msg["src_blocks"] = info.get("src_blocks", [])
            per_link.setdefault(info["link"], []).append(msg)
        for link, items in per_link.items():
            try:
                self.links[link]["t"].call("first_generations", {"items": items}, timeout=60.0 if self.pull else 10.0)
            except (TimeoutError, OSError) as e:
                HEALTH.set_unhealthy(f"decode instance did not accept the first generation: {e}")
        self._pending_out = []

    def _handle(self, method: str, p: Dict, link: int = 0):
        if method == "generations":
            outs = []
            for m in p["outputs"]:
                cid = self.by_remote.get((link, m["request_id"]))
                if cid is None:
                    continue
                st = self.master._states.get(cid)
                n_prompt = len(st.prompt_ids) if st else 0
                outs.append(_RemoteSeqOutput(cid, m["tokens"], m["logprobs"], m["finished"], m["finish_reason"], n_prompt,
                                             m["num_generated"]))
                if m["finished"]:
                    self.by_remote.pop((link, m["request_id"]), None)
                    self.remote.pop(cid, None)
            if outs:
                self._orig_emit(outs)
            return None
        raise ValueError(f"unknown method {method}")
