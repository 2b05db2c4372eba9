"""Sleep and wake-up of an engine: give the device memory back while the instance is idle, keep it registered.

Role of the reference's sleep / wakeup admin calls (xllm/core/distributed_runtime/master.h:38-55,
llm_engine.cpp:1252-1350, runtime/worker_impl.cpp:739-781; there tied to the NPU-only xTensor allocator):

    LIGHT sleep   KV cache and captured graphs are released, the weights move to pinned host memory; wake-up copies
                  them back (seconds for tens of GB over PCIe)
    DEEP sleep    the weights are dropped as well; wake-up loads the checkpoint again (or re-creates the random preset),
                  or, given a weight source (runtime/weight_transfer.py), copies the finished weights from an awake
                  instance of the same model: over NVLink through CUDA-IPC mappings on one host, over TCP otherwise

Both need an idle engine.  The device prefix cache is emptied, since its blocks are gone; with a host tier the host
copies stay valid and prompts that return after the wake-up are served from them.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterator, List, Tuple

import torch

AWAKE, LIGHT_SLEEP, DEEP_SLEEP = 0, 1, 2
STATUS_NAMES = {AWAKE: "WAKEUP", LIGHT_SLEEP: "LIGHT_SLEEP", DEEP_SLEEP: "DEEP_SLEEP"}


def _is_weight_holder(obj: Any) -> bool:
    mod = type(obj).__module__ or ""
    return mod.startswith(__name__.split(".")[0] + ".models") and hasattr(obj, "__dict__")


def iter_weight_slots(model) -> Iterator[Tuple[Callable[[], Any], Callable[[Any], None]]]:
    """(get, set) for every tensor-valued attribute reachable from `model.embed / final_norm / lm_head / layers / ...`
    through the plain weight-holder classes of the models package (lists and tuples of them included).  Communication
    objects, argument structs and anything else that is not a weight holder are not entered."""
    seen = set()

    def walk(obj):
        if id(obj) in seen:
            return
        seen.add(id(obj))
        for name, val in list(vars(obj).items()):
            # not weights: communication state, arguments, and small derived tables (rotary cos / sin) that stay resident
            if name in ("comm", "args", "device", "dtype", "eplb", "moe_impl", "cos_sin") or name.startswith("_"):
                continue
            if isinstance(val, torch.Tensor):
                yield (lambda o=obj, n=name: getattr(o, n)), (lambda v, o=obj, n=name: setattr(o, n, v))
            elif isinstance(val, (list, tuple)):
                for i, item in enumerate(val):
                    if isinstance(item, torch.Tensor) and isinstance(val, list):
                        yield (lambda l=val, j=i: l[j]), (lambda v, l=val, j=i: l.__setitem__(j, v))
                    elif _is_weight_holder(item):
                        yield from walk(item)
            elif _is_weight_holder(val):
                yield from walk(val)
    yield from walk(model)


class SleepState:
    """Per-rank state of one sleep: host copies of the weights (light sleep) and what has to be rebuilt."""

    def __init__(self):
        self.level = AWAKE
        self.bytes_offloaded = 0
        # deep sleep: layout of every distinct weight tensor in walk order, and which slot takes which of them, so that a
        # wake-up from a remote source can rebuild the tensors without reading the checkpoint
        self.manifest: List[Dict[str, Any]] = []
        self.slots: List[Tuple[Callable[[Any], None], int]] = []


def _key(t: torch.Tensor) -> Tuple:
    return (t.untyped_storage().data_ptr(), t.storage_offset(), tuple(t.shape), tuple(t.stride()), t.dtype)


def span_elems(shape, stride) -> int:
    """Elements between the first and the last element of a strided tensor, inclusive (its footprint in the storage)."""
    if any(d == 0 for d in shape):
        return 0
    return 1 + sum((d - 1) * st for d, st in zip(shape, stride))


def flat_span(t: torch.Tensor) -> torch.Tensor:
    """1-D view of the storage range a tensor occupies (any strides): the unit in which weights travel."""
    return t.as_strided((span_elems(t.shape, t.stride()),), (1,))


def weight_manifest(model, dev) -> Tuple[List[Dict[str, Any]], List[torch.Tensor]]:
    """Layout of every distinct weight tensor on `dev` in walk order (tied weights once), and the tensors themselves.
    Two instances of one model with the same parallel layout produce the same list, entry by entry."""
    seen: Dict[Tuple, int] = {}
    out, tensors = [], []
    for get, _ in iter_weight_slots(model):
        t = get()
        if t is None or t.device != dev:
            continue
        k = _key(t)
        if k in seen:
            continue
        seen[k] = len(out)
        out.append({"shape": list(t.shape), "stride": list(t.stride()), "dtype": str(t.dtype).replace("torch.", ""),
                    "nbytes": span_elems(t.shape, t.stride()) * t.element_size()})
        tensors.append(t)
    return out, tensors


def sleep_rank(engine, level: int) -> int:
    """Runs on every rank.  Returns the bytes of device memory given back (weights + KV cache)."""
    w = engine.worker
    st: SleepState = engine._sleep_state
    assert st.level == AWAKE and level in (LIGHT_SLEEP, DEEP_SLEEP)
    dev = w.device
    cuda = dev.type == "cuda"
    if cuda:
        torch.cuda.synchronize(dev)
    if w._graphs is not None:
        w._graphs.invalidate()
        w._graphs = None
    freed = sum(t.numel() * t.element_size() for layer in w.kv_caches for t in layer)
    if engine.host_tier is not None:
        engine.host_tier.drain()
        engine.host_tier.detach()
    w.kv_caches = []
    aliases: Dict[Tuple, Any] = {}                 # tied weights (lm_head = embedding) stay one tensor
    order: Dict[Tuple, int] = {}
    st.manifest, st.slots = [], []
    for get, put in iter_weight_slots(w.model):
        t = get()
        if t is None or t.device != dev:
            continue
        k = _key(t)
        if k not in aliases:
            nbytes = t.numel() * t.element_size()
            freed += nbytes
            order[k] = len(st.manifest)
            st.manifest.append({"shape": list(t.shape), "stride": list(t.stride()), "dtype": str(t.dtype).replace("torch.", ""),
                                "nbytes": span_elems(t.shape, t.stride()) * t.element_size()})
            if level == LIGHT_SLEEP:
                h = torch.empty(t.shape, dtype=t.dtype, pin_memory=cuda)
                h.copy_(t)
                aliases[k] = h
                st.bytes_offloaded += nbytes
            else:
                aliases[k] = None
        st.slots.append((put, order[k]))
        put(aliases[k])
    st.level = level
    if cuda:
        torch.cuda.synchronize(dev)
        torch.cuda.empty_cache()
    return freed


def wakeup_rank(engine, source=None) -> None:
    """`source`: where a deep sleeper takes its weights from instead of the checkpoint; an object with
    `pull_into(manifest, tensors, rank)` (runtime/weight_transfer.py).  A source whose layout differs raises before anything
    was changed here, and the caller may wake up from the checkpoint instead."""
    w = engine.worker
    st: SleepState = engine._sleep_state
    assert st.level != AWAKE
    dev = w.device
    if st.level == DEEP_SLEEP and source is not None and st.manifest:
        tensors = [torch.empty_strided(m["shape"], m["stride"], dtype=getattr(torch, m["dtype"]), device=dev) for m in st.manifest]
        source.pull_into(st.manifest, tensors, engine.rank)
        for put, i in st.slots:
            put(tensors[i])
        engine.weights_pulled_bytes = sum(m["nbytes"] for m in st.manifest)
        engine.weights_pull_ms = float(getattr(source, "copy_ms", 0.0))
    elif st.level == LIGHT_SLEEP:
        back: Dict[Tuple, torch.Tensor] = {}
        for get, put in iter_weight_slots(w.model):
            t = get()
            if t is None or t.device == dev:
                continue
            k = _key(t)
            d = back.get(k)
            if d is None:
                d = t.to(dev, non_blocking=True) if dev.type == "cuda" else t.clone()
                back[k] = d
            put(d)
    else:
        engine._load_model()
    w.allocate_kv_cache(engine.num_blocks, ipc=engine.opt.enable_disagg_pd and engine.opt.instance_role == "DECODE")
    if engine.host_tier is not None:
        engine.host_tier.attach(w.kv_caches)
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    st.level = AWAKE
    st.bytes_offloaded = 0
    st.manifest, st.slots = [], []
