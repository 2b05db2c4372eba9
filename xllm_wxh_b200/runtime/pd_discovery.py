"""Prefill instances find their decode instances through the service layer and follow its membership.

In the reference the xllm-service master tells a prefill instance which decode instances exist and the instance links /
unlinks them (DisaggPDService link_instance / unlink_instance, disagg_pd_scheduler.h:77-90; instance lists from etcd,
xservice_client.cpp:418-463).  Here the prefill instance asks the registry for the DECODE instances, connects to the
control port each of them published (`InstanceInfo.pd_port`), and repeats that whenever the registry changes (long-poll
watch): new decode instances are linked, instances whose registration disappeared (lease ran out, deregistered) are
dropped, which fails only the requests that were handed to them.
"""
from __future__ import annotations

import logging
import threading
from typing import Callable, Dict, Optional

log = logging.getLogger("xllm.pd_discovery")


class DecodeLinker:
    def __init__(self, coordinator, client, connect: Optional[Callable[[str, int], object]] = None,
                 on_link: Optional[Callable[[int, object], None]] = None):
        """`coordinator`: PrefillCoordinator; `client`: XServiceClient; `connect(host, port)` -> transport (default: TCP);
        `on_link(link index, instance info)`: hook run after a link was made (tests install a CPU copy path there)."""
        from .disagg_pd import SocketTransport
        self.pre, self.client = coordinator, client
        self.connect = connect or (lambda host, port: SocketTransport.connect(host, port))
        self.on_link = on_link
        self.by_name: Dict[str, int] = {}            # decode instance name -> link index
        self.revision = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def sync_once(self) -> Dict[str, int]:
        """Bring the links in line with the registry; returns {name: link index} of the live links."""
        names = set(self.client.get_static_decode_list())
        for name in sorted(names - set(self.by_name)):
            info = self.client.get_instance_info(name)
            if info is None or not info.pd_port:
                continue
            host = info.rpc_address.rpartition(":")[0] or "127.0.0.1"
            try:
                t = self.connect(host, int(info.pd_port))
                idx = self.pre.add_decode_link(t)
            except (OSError, TimeoutError, ValueError) as e:
                log.warning("could not link decode instance %s: %s", name, e)
                continue
            self.by_name[name] = idx
            if self.on_link is not None:
                self.on_link(idx, info)
        for name in sorted(set(self.by_name) - names):
            idx = self.by_name.pop(name)
            link = self.pre.links[idx]
            if link["alive"]:
                try:
                    link["t"].close()                  # its on_close callback fails the requests handed to that instance
                except OSError:
                    pass
                if link["alive"]:
                    self.pre.peer_lost(idx)
        # a link that died on its own (connection closed) is forgotten, so that the instance is linked again if it returns
        for name, idx in list(self.by_name.items()):
            if not self.pre.links[idx]["alive"]:
                self.by_name.pop(name)
        return dict(self.by_name)

    def start(self, poll_s: float = 2.0) -> None:
        def loop():
            while not self._stop.is_set():
                try:
                    self.sync_once()
                    rev, _ = self.client.watch(self.revision, timeout_s=poll_s)
                    if rev == self.revision:
                        self._stop.wait(0.05)
                    self.revision = rev
                except Exception as e:               # discovery must not take the serving loop down
                    log.warning("decode discovery failed: %s", e)
                    self._stop.wait(poll_s)
        self._thread = threading.Thread(target=loop, name="pd-discovery", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5.0)
