"""Request parameters and outputs of the public API.

Field names and defaults follow the reference's `RequestParams` (xllm/core/framework/request/
request_params.h:40-130) and the pybind surface (xllm/pybind/bind.cpp:203-289, pybind/params.py):
`SamplingParams`, `BeamSearchParams`, `PoolingParams`, `RequestOutput`, `SequenceOutput`, `Usage`,
`Status`, `StatusCode`, `LogProb`.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Any, Dict, List, Optional

from .. import _core


class StatusCode(enum.IntEnum):
    OK = 0
    CANCELLED = 1
    UNKNOWN = 2
    INVALID_ARGUMENT = 3
    DEADLINE_EXCEEDED = 4
    RESOURCE_EXHAUSTED = 8
    UNAVAILABLE = 14


@dataclasses.dataclass
class Status:
    code: StatusCode = StatusCode.OK
    message: str = ""

    @property
    def ok(self) -> bool:
        return self.code == StatusCode.OK


@dataclasses.dataclass
class RequestParams:
    request_id: str = ""
    service_request_id: str = ""
    max_tokens: int = 5120
    n: int = 1
    best_of: Optional[int] = None
    echo: bool = False
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = -1
    logprobs: bool = False
    top_logprobs: int = 0
    skip_special_tokens: bool = True
    ignore_eos: bool = False
    stop: Optional[List[str]] = None
    stop_token_ids: Optional[List[int]] = None
    is_embeddings: bool = False
    beam_width: int = 0
    offline: bool = False
    priority: int = 0               # 0 = default; smaller = more urgent
    ttft_slo_ms: float = 0.0
    tpot_slo_ms: float = 0.0
    ttlt_slo_ms: float = 0.0
    decode_name: str = ""           # routing.decode_name: the decode instance the service layer picked (PD pairs)
    decode_address: str = ""
    ttft_priority_weight: int = 1   # value of meeting the first-token / per-token target (density ordering)
    tpot_priority_weight: int = 1
    seed: int = -1
    add_special_tokens: bool = True
    streaming: bool = False
    include_usage: bool = False
    chat_template_kwargs: Optional[Dict[str, Any]] = None
    tools: Optional[List[Dict[str, Any]]] = None
    tool_choice: Any = "auto"

    def verify(self) -> Status:
        """request_params.cpp `verify_params`."""
        bad = lambda m: Status(StatusCode.INVALID_ARGUMENT, m)
        if self.n < 1:
            return bad("n should be greater than 0")
        if self.best_of is not None and self.best_of < self.n:
            return bad("best_of should be greater than or equal to n")
        if not (-2.0 <= self.frequency_penalty <= 2.0):
            return bad("frequency_penalty must be between -2.0 and 2.0")
        if not (-2.0 <= self.presence_penalty <= 2.0):
            return bad("presence_penalty must be between -2.0 and 2.0")
        if not (0.0 < self.repetition_penalty <= 2.0):
            return bad("repetition_penalty must be between 0.0 and 2.0")
        if not (0.0 <= self.temperature <= 2.0):
            return bad("temperature must be between 0.0 and 2.0")
        if not (0.0 < self.top_p <= 1.0):
            return bad("top_p must be between 0.0 and 1.0")
        if self.max_tokens < 1:
            return bad("max_tokens must be at least 1")
        if self.top_logprobs < 0 or self.top_logprobs > 20:
            return bad("top_logprobs must be between 0 and 20")
        if self.streaming and self.best_of is not None and self.best_of != self.n:
            return bad("best_of must equal n for streaming requests")
        return Status()

    def to_core(self, eos_token_id: int, extra_stop_ids: Optional[List[int]] = None,
                stop_sequences: Optional[List[List[int]]] = None):
        sp = _core.SamplingParams()
        sp.temperature, sp.top_p, sp.top_k = float(self.temperature), float(self.top_p), int(self.top_k)
        sp.repetition_penalty = float(self.repetition_penalty)
        sp.frequency_penalty, sp.presence_penalty = float(self.frequency_penalty), float(self.presence_penalty)
        sp.logprobs = bool(self.logprobs) or self.top_logprobs > 0 or (self.best_of or self.n) > self.n or self.beam_width > 1
        sp.top_logprobs = int(self.top_logprobs)
        sp.seed = int(self.seed)
        st = _core.StopCriteria()
        st.max_tokens = int(self.max_tokens)
        st.eos_token_id = int(eos_token_id)
        st.ignore_eos = bool(self.ignore_eos)
        st.stop_token_ids = sorted(set((self.stop_token_ids or []) + (extra_stop_ids or [])))
        st.stop_sequences = stop_sequences or []
        return sp, st


class _ParamsProxy:
    """Keyword constructor that rejects unknown names, like the reference's `_RequestParamsProxy`."""

    def __init__(self, **kwargs: Any) -> None:
        object.__setattr__(self, "_request_params", RequestParams())
        for k, v in kwargs.items():
            setattr(self, k, v)

    def __getattr__(self, key: str) -> Any:
        return getattr(object.__getattribute__(self, "_request_params"), key)

    def __setattr__(self, key: str, value: Any) -> None:
        rp = object.__getattribute__(self, "_request_params")
        if not hasattr(rp, key):
            raise TypeError(f"Unexpected parameter: {key}")
        setattr(rp, key, value)

    def to_request_params(self) -> RequestParams:
        return dataclasses.replace(object.__getattribute__(self, "_request_params"))


class SamplingParams(_ParamsProxy):
    pass


class BeamSearchParams(SamplingParams):
    def __init__(self, beam_width: int = 1, max_tokens: int = 16, **kwargs: Any) -> None:
        super().__init__(beam_width=beam_width, max_tokens=max_tokens, **kwargs)


class PoolingParams(_ParamsProxy):
    def __init__(self, **kwargs: Any) -> None:
        super().__init__(**kwargs)
        self.is_embeddings = True


def to_request_params(p, default_cls=SamplingParams) -> RequestParams:
    if p is None:
        return default_cls().to_request_params()
    if isinstance(p, RequestParams):
        return dataclasses.replace(p)
    if isinstance(p, _ParamsProxy):
        return p.to_request_params()
    raise TypeError(f"unsupported params object: {type(p)}")


@dataclasses.dataclass
class LogProbData:
    token: str = ""
    token_id: int = -1
    logprob: float = 0.0
    finished_token: bool = False


@dataclasses.dataclass
class LogProb(LogProbData):
    top_logprobs: Optional[List[LogProbData]] = None


@dataclasses.dataclass
class Usage:
    num_prompt_tokens: int = 0
    num_generated_tokens: int = 0
    num_total_tokens: int = 0
    num_cached_tokens: int = 0


@dataclasses.dataclass
class SequenceOutput:
    index: int = 0
    text: str = ""
    token_ids: List[int] = dataclasses.field(default_factory=list)
    finish_reason: Optional[str] = None
    logprobs: Optional[List[LogProb]] = None
    embeddings: Optional[List[float]] = None
    cumulative_logprob: float = 0.0


@dataclasses.dataclass
class RequestOutput:
    request_id: str = ""
    service_request_id: str = ""
    prompt: Optional[str] = None
    prompt_token_ids: Optional[List[int]] = None
    status: Optional[Status] = None
    outputs: List[SequenceOutput] = dataclasses.field(default_factory=list)
    usage: Optional[Usage] = None
    finished: bool = False
    cancelled: bool = False


FINISH_REASONS = {0: None, 1: "stop", 2: "length", 3: "cancelled", 4: "resource_exhausted", 5: "handoff"}
