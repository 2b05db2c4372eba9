"""Expert-parallel load balancing at run time: load aggregation, re-planning, expert weight movement, slot tables.

Role of the reference's EplbManager / EplbExecutor / EplbPolicy trio (xllm/core/framework/eplb/eplb_manager.cpp:52-67
initial placement, eplb_policy.cpp:40-175 policy, eplb_executor.cpp weight loading; docs/en/features/eplb.md):

* every device has `E / ep_size + redundant_experts_num` physical expert slots per MoE layer; a layer's *placement* names
  the logical expert held by every slot; hot experts get replicas, and a token picks one replica by its index;
* workers count how often each logical expert was routed to (`model.expert_load`); every `eplb_update_interval` steps the
  manager (rank 0) compares each layer's load with the load it was last planned for (cosine similarity below
  `eplb_update_threshold` => re-plan, C++ policy `_core.eplb_rebalance`);
* a re-planned layer is installed in two phases, one layer at a time, so that a step never sees half-moved weights:
  **prepare** (every rank copies the weights its new slots need into the spare buffer, on a side stream: from its own
  slots when it already holds the expert, from a peer rank otherwise) and, once every rank has finished, **activate**
  (swap the spare buffer with the layer's weights and switch the routing table).  The reference moves the weights
  through a host shared-memory copy of all experts; here they travel GPU to GPU.

The routing table turns the router's logical expert ids into physical slot ids right before the expert kernels, so the
kernels themselves are unchanged: slot `s` of device `d` is "expert" `d * S + s`.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from .. import _core


def initial_placement(n_experts: int, n_devices: int, slots: int) -> np.ndarray:
    """Contiguous experts per device; the redundant slots duplicate the device's last expert (eplb_manager.cpp:52-67)."""
    per = n_experts // n_devices
    out = np.empty(n_devices * slots, dtype=np.int32)
    for d in range(n_devices):
        for s in range(slots):
            out[d * slots + s] = d * per + min(s, per - 1)
    return out


def build_route_table(placement: Sequence[int], n_experts: int) -> Tuple[np.ndarray, np.ndarray]:
    """(table [E, max_copies] of physical slot ids, padded by repeating; copies [E])."""
    where: List[List[int]] = [[] for _ in range(n_experts)]
    for slot, e in enumerate(placement):
        where[int(e)].append(slot)
    if any(not w for w in where):
        raise ValueError("placement leaves an expert without a slot")
    mc = max(len(w) for w in where)
    table = np.empty((n_experts, mc), dtype=np.int64)
    for e, w in enumerate(where):
        for j in range(mc):
            table[e, j] = w[j % len(w)]
    return table, np.asarray([len(w) for w in where], dtype=np.int64)


class EplbManager:
    """Rank 0: aggregates loads and decides which layers to re-plan (EplbManager + EplbPolicy of the reference)."""

    def __init__(self, n_layers: int, n_experts: int, n_devices: int, slots: int, interval: int, threshold: float):
        self.L, self.E, self.D, self.S = n_layers, n_experts, n_devices, slots
        self.interval, self.threshold = max(1, interval), threshold
        self.load = np.zeros((n_layers, n_experts), dtype=np.float64)          # since the last planning round
        self.planned_load: List[Optional[np.ndarray]] = [None] * n_layers
        self.placement = [initial_placement(n_experts, n_devices, slots) for _ in range(n_layers)]
        self.pending: List[Tuple[int, np.ndarray]] = []                        # (layer, new placement), installed in order
        self.steps = 0
        self.num_replans = 0

    def update_expert_load(self, load: np.ndarray) -> None:
        self.load += load

    def tick(self) -> bool:
        """Called once per step; True when a planning round is due."""
        self.steps += 1
        return self.steps % self.interval == 0

    def plan(self) -> int:
        """Re-plan the layers whose load pattern moved away from the one they were planned for.  Returns how many."""
        n = 0
        for layer in range(self.L):
            cur = self.load[layer]
            if cur.sum() <= 0:
                continue
            old = self.planned_load[layer]
            if old is not None and not _core.eplb_should_update(old.tolist(), cur.tolist(), self.threshold):
                continue
            new = np.asarray(_core.eplb_rebalance([cur.tolist()], self.D, self.S)[0][0], dtype=np.int32)
            self.planned_load[layer] = cur.copy()
            if not np.array_equal(new, self.placement[layer]):
                self.pending.append((layer, new))
                n += 1
        self.load[:] = 0
        self.num_replans += n
        return n

    def next_layer(self) -> Optional[Tuple[int, np.ndarray]]:
        return self.pending.pop(0) if self.pending else None

    def committed(self, layer: int, placement: np.ndarray) -> None:
        self.placement[layer] = placement


class EplbExecutor:
    """Every rank: holds the slot weights, the spare buffer and the routing tables of its model; prepares and activates
    a layer's new placement (EplbExecutor of the reference)."""

    def __init__(self, model, moe_layers: List, n_experts: int, ep_rank: int, ep_size: int, redundant: int, group=None):
        self.model, self.layers = model, moe_layers
        self.E, self.rank, self.D = n_experts, ep_rank, ep_size
        per = n_experts // ep_size
        self.S = per + redundant
        self.group = group
        dev = moe_layers[0].w13.device
        self.device = dev
        # widen every layer's weights to S slots: the redundant ones start as copies of the last local expert
        # per-expert slabs that travel with an expert: the weights and, for block-scaled fp8 checkpoints, their scales
        self.names = [n for n in ("w13", "w2", "w13_scale", "w2_scale") if getattr(moe_layers[0], n, None) is not None]
        for L in moe_layers:
            if L.w13.shape[0] != per:
                raise ValueError("EPLB expects the contiguous initial expert layout")
            idx = torch.tensor([min(s, per - 1) for s in range(self.S)], device=dev)
            for n in self.names:
                setattr(L, n, getattr(L, n).index_select(0, idx).contiguous())
        self.placement = [initial_placement(n_experts, ep_size, self.S) for _ in moe_layers]
        self.tables: List[torch.Tensor] = []
        self.copies: List[torch.Tensor] = []
        for p in self.placement:
            t, c = build_route_table(p, n_experts)
            self.tables.append(torch.from_numpy(t).to(dev))
            self.copies.append(torch.from_numpy(c).to(dev))
        self.spare = {n: torch.empty_like(getattr(moe_layers[0], n)) for n in self.names}     # one layer's worth, reused
        self.stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self.ready_event = None
        self.prepared: Optional[Tuple[int, np.ndarray]] = None
        self.num_activations = 0
        self.rows_moved_remote = 0

    @property
    def expert_offset(self) -> int:
        return self.rank * self.S

    def route(self, layer: int, ids: torch.Tensor) -> torch.Tensor:
        """Logical expert ids [T, k] -> physical slot ids [T, k]; the replicas of an expert take the tokens in turn."""
        t, c = self.tables[layer], self.copies[layer]
        idl = ids.long()
        tok = torch.arange(ids.shape[0], device=ids.device).unsqueeze(1)
        pick = tok % c[idl]
        return t[idl, pick].to(ids.dtype)

    # ------------------------------------------------------------------ phase 1
    def prepare(self, layer: int, new_placement: np.ndarray) -> None:
        """Fill the spare buffer with the weights of this rank's slots under `new_placement`.  Collective: every rank
        calls it with the same arguments (sends and receives are paired)."""
        L = self.layers[layer]
        old = self.placement[layer]
        S, D = self.S, self.D
        new_placement = np.asarray(new_placement, dtype=np.int32)
        holders: Dict[int, List[int]] = {}
        for slot, e in enumerate(old):
            holders.setdefault(int(e), []).append(slot)
        local_copies, recvs, sends = [], [], []            # (dst slot local, src slot local) / (dst local, src rank, src local) / ...
        for d in range(D):
            for s in range(S):
                e = int(new_placement[d * S + s])
                src_slots = holders[e]
                same = [x for x in src_slots if x // S == d]
                if same:
                    if d == self.rank:
                        local_copies.append((s, same[0] % S))
                    continue
                src = src_slots[(d + s) % len(src_slots)]     # spread the senders of a replicated expert
                if d == self.rank:
                    recvs.append((s, src // S, src % S))
                elif src // S == self.rank:
                    sends.append((src % S, d))
        ctx = torch.cuda.stream(self.stream) if self.stream is not None else _null()
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with ctx:
            for dst, src in local_copies:
                for n in self.names:
                    self.spare[n][dst].copy_(getattr(L, n)[src], non_blocking=True)
            ops = []
            for src, d in sends:
                for n in self.names:
                    ops.append(dist.P2POp(dist.isend, getattr(L, n)[src], self._peer(d), group=self.group))
            for dst, r, _src in recvs:
                for n in self.names:
                    ops.append(dist.P2POp(dist.irecv, self.spare[n][dst], self._peer(r), group=self.group))
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
            self.rows_moved_remote += len(recvs)
            if self.stream is not None:
                self.ready_event = torch.cuda.Event()
                self.ready_event.record(self.stream)
        self.prepared = (layer, new_placement)

    def _peer(self, ep_rank: int) -> int:
        return dist.get_global_rank(self.group, ep_rank) if (self.group is not None and dist.is_initialized()) else ep_rank

    # ------------------------------------------------------------------ phase 2
    def activate(self, layer: int) -> None:
        """Swap the prepared weights in and switch the routing table (between steps, on every rank)."""
        if self.prepared is None or self.prepared[0] != layer:
            raise RuntimeError(f"layer {layer} was not prepared")
        if self.ready_event is not None:
            torch.cuda.current_stream(self.device).wait_event(self.ready_event)
        L = self.layers[layer]
        for n in self.names:
            cur = getattr(L, n)
            setattr(L, n, self.spare[n])
            self.spare[n] = cur
        self.placement[layer] = self.prepared[1]
        t, c = build_route_table(self.prepared[1], self.E)
        # same shapes where possible so that captured graphs keep reading valid memory
        if tuple(t.shape) == tuple(self.tables[layer].shape):
            self.tables[layer].copy_(torch.from_numpy(t))
        else:
            self.tables[layer] = torch.from_numpy(t).to(self.device)
            self.graphs_stale = True
        self.copies[layer].copy_(torch.from_numpy(c))
        self.prepared = None
        self.num_activations += 1
        self.graphs_stale = True       # weight tensors were swapped: captured graphs point at the old buffers


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


# ---------------------------------------------------------------------- engine glue
OP_EPLB_PREPARE, OP_EPLB_ACTIVATE, OP_EPLB_SUM_LOAD = 101, 102, 103


def moe_layer_weights(model) -> List:
    return [L.mlp for L in model.layers if getattr(L.mlp, "is_moe", False)] if hasattr(model.layers[0], "mlp") else \
        [L for L in model.layers if getattr(L, "is_moe", False)]


def attach(engine) -> Optional["EplbRuntime"]:
    """Turn EPLB on for an engine whose model has MoE layers (`--enable_eplb`)."""
    o = engine.opt
    model = engine.worker.model
    layers = moe_layer_weights(model)
    if not o.enable_eplb or not layers:
        return None
    # The fused all-to-all addresses physical slots (rank * slots_per_rank + local slot): it was sized for the widened
    # slot count when it was attached, and routes whatever `route` hands it.  Slot moves copy whole weight slabs, whatever
    # their internal row order or scales.
    comm = engine.comm
    ex = EplbExecutor(model, layers, engine.args.n_routed_experts, comm.ep_rank, max(1, comm.ep_size), o.redundant_experts_num,
                      group=comm.ep_group)
    model.eplb = ex
    impl = getattr(model, "moe_impl", None)
    if impl is not None and hasattr(impl, "e0"):
        impl.e0 = ex.expert_offset
    if model.expert_load is None:
        model.expert_load = torch.zeros((len(layers), engine.args.n_routed_experts), dtype=torch.int64, device=engine.device)
    rt = EplbRuntime(engine, ex)
    engine.eplb = rt
    return rt


class EplbRuntime:
    """Drives the manager from the engine's step loop (rank 0) and executes its commands on every rank."""

    def __init__(self, engine, executor: EplbExecutor):
        self.engine, self.ex = engine, executor
        o = engine.opt
        self.manager = EplbManager(len(executor.layers), executor.E, executor.D, executor.S, o.eplb_update_interval,
                                   o.eplb_update_threshold) if engine.rank == 0 else None
        self.in_flight: Optional[Tuple[int, np.ndarray]] = None

    # rank 0, once per step (after the step's results were applied)
    def on_step(self) -> None:
        m = self.manager
        if m is None:
            return
        if self.in_flight is not None:                       # prepared in an earlier step: now make it live
            layer, placement = self.in_flight
            self.engine._control(OP_EPLB_ACTIVATE, layer)
            m.committed(layer, placement)
            self.in_flight = None
        if m.tick():
            load = self._collect_load()
            m.update_expert_load(load)
            m.plan()
        nxt = m.next_layer()
        if nxt is not None:
            layer, placement = nxt
            self.engine._control(OP_EPLB_PREPARE, layer, placement.astype(np.int32).tobytes())
            self.in_flight = (layer, placement)

    def _collect_load(self) -> np.ndarray:
        model = self.engine.worker.model
        if self.engine.world_size > 1 and self.engine.comm.dp_size > 1:
            self.engine._control(OP_EPLB_SUM_LOAD)            # attention-DP ranks saw different tokens: sum on every rank
        out = model.expert_load.cpu().numpy().astype(np.float64)
        model.expert_load.zero_()
        return out

    # every rank (from the engine's control dispatch)
    def do_control(self, op: int, arg: int, payload: bytes) -> None:
        if op == OP_EPLB_PREPARE:
            self.ex.prepare(arg, np.frombuffer(payload, dtype=np.int32).copy())
        elif op == OP_EPLB_SUM_LOAD:
            model = self.engine.worker.model
            dist.all_reduce(model.expert_load)
            if self.engine.rank != 0:
                model.expert_load.zero_()
        elif op == OP_EPLB_ACTIVATE:
            self.ex.activate(arg)
            g = self.engine.worker._graphs
            if g is not None and getattr(self.ex, "graphs_stale", False):
                g.invalidate()
                self.ex.graphs_stale = False
