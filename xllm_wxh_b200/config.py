"""Engine options and the command-line flag set.

One typed dataclass carries what the reference spreads over gflags -> `Options` -> `runtime::Options`
(xllm/core/common/global_flags.cpp:29-659, core/common/options.h, core/runtime/options.h); flag names
and defaults are the reference's so that launch scripts keep working (`--model --devices --port
--block_size --max_memory_utilization --max_tokens_per_batch --max_seqs_per_batch
--enable_chunked_prefill --enable_prefix_cache --enable_schedule_overlap --enable_graph --dp_size
--ep_size --enable_eplb --enable_disagg_pd --instance_role --kv_cache_transfer_mode --draft_model
--num_speculative_tokens ...`).
"""
from __future__ import annotations

import argparse
import dataclasses
from typing import Any, Dict, List, Optional


def _flag(default, help="", group="misc", **kw):
    return dataclasses.field(default=default, metadata={"help": help, "group": group, **kw})


@dataclasses.dataclass
class Options:
    # ---- service (global_flags.cpp:29-52)
    host: str = _flag("", "Host name for brpc server.", "service")
    port: int = _flag(8010, "Port for the HTTP server.", "service")
    num_threads: int = _flag(8, "Number of server threads.", "service")
    max_concurrent_requests: int = _flag(200, "Maximum number of concurrent requests (0 = unlimited).", "service")
    rpc_idle_timeout_s: int = _flag(-1, "Idle connection timeout.", "service")
    rpc_channel_timeout_ms: int = _flag(60000, "Time a step may wait for a worker rank on the step channel before the rank counts as failed.", "service")
    max_reconnect_count: int = _flag(40, "Worker -> master connection retries.", "service")
    # ---- model (56-72)
    model: str = _flag("", "Path of a HF model directory, or a preset name such as 'preset:qwen3-8b'.", "model")
    model_id: str = _flag("", "Model name reported by the API.", "model")
    backend: str = _flag("llm", "llm | vlm | dit | rec (only llm is implemented).", "model")
    task: str = _flag("generate", "generate | embed", "model")
    devices: str = _flag("auto", "Devices, e.g. 'cuda:0,cuda:1' or 'cpu'.", "model")
    dtype: str = _flag("auto", "auto | bfloat16 | float16 | float32", "model")
    random_seed: int = _flag(0, "Seed for random-initialised presets and for sampling.", "model")
    # ---- graph (78-106)
    enable_graph: bool = _flag(True, "Capture decode steps in CUDA graphs per token bucket.", "graph")
    enable_graph_mode_decode_no_padding: bool = _flag(False, "Replay only exact-size decode graphs.", "graph")
    enable_prefill_piecewise_graph: bool = _flag(False, "Also capture prefill / mixed steps (whole step in one graph: attention reads its ranges on the device).", "graph")
    enable_graph_vmm_pool: bool = _flag(True, "Share one memory pool among all captured shapes.", "graph")
    max_tokens_for_graph_mode: int = _flag(2048, "Largest token count captured as a graph.", "graph")
    # ---- threads (116-122)
    num_request_handling_threads: int = _flag(4, "Threads for tokenisation / request building.", "threads")
    num_response_handling_threads: int = _flag(4, "Threads for detokenisation / callbacks.", "threads")
    # ---- kv cache (126-145)
    block_size: int = _flag(128, "Tokens per KV block.", "kv")
    max_cache_size: int = _flag(0, "KV cache bytes (0 = derive from max_memory_utilization).", "kv")
    max_memory_utilization: float = _flag(0.8, "Fraction of device memory the engine may use.", "kv")
    kv_cache_dtype: str = _flag("auto", "auto | fp8", "kv")
    # ---- scheduler (149-213)
    max_tokens_per_batch: int = _flag(10240, "Token budget per step.", "scheduler")
    max_seqs_per_batch: int = _flag(1024, "Sequence budget per step.", "scheduler")
    enable_schedule_overlap: bool = _flag(False, "Schedule step i+1 while step i runs (async scheduling).", "scheduler")
    prefill_scheduling_memory_usage_threshold: float = _flag(0.95, "No new prefill above this KV utilisation.", "scheduler")
    enable_chunked_prefill: bool = _flag(True, "Sarathi-style chunked prefill.", "scheduler")
    enable_prefill_sp: bool = _flag(False, "Prefill sequence parallelism (not implemented; accepted for compatibility).", "scheduler")
    max_tokens_per_chunk_for_prefill: int = _flag(-1, "Prefill chunk size (-1 = token budget).", "scheduler")
    chunked_match_frequency: int = _flag(2, "Re-match the prefix cache every N chunks.", "scheduler")
    use_zero_evict: bool = _flag(False, "Admit prefills only if no eviction can follow.", "scheduler")
    max_decode_token_per_sequence: int = _flag(256, "Decode horizon assumed by the zero-evict policy.", "scheduler")
    priority_strategy: str = _flag("fcfs", "fcfs | priority | deadline; with the mix scheduler also sjf | density | decode_density | "
                                   "decode_deadline | urgency_density | decode_urgency_density | urgency_priority", "scheduler")
    use_mix_scheduler: bool = _flag(False, "One urgency-ordered queue for prefills and decodes (multi-priority SLO scheduling).", "scheduler")
    aggressive_coeff: float = _flag(1.0, "Mix scheduler: a request is urgent when its slack is below this times the queued work.", "scheduler")
    starve_threshold: float = _flag(1.0, "Mix scheduler: a request overdue by this many times its target is starved.", "scheduler")
    enable_starve_prevent: bool = _flag(True, "Mix scheduler: starved prefills go ahead of denser ones.", "scheduler")
    enable_latency_aware_schedule: bool = _flag(False, "Bound each step by predicted latency instead of the token budget.", "scheduler")
    enable_online_preempt_offline: bool = _flag(True, "Online requests may evict offline decodes.", "scheduler")
    request_queue_size: int = _flag(100000, "Bound of the incoming request queue.", "scheduler")
    # ---- parallel (217-226)
    dp_size: int = _flag(1, "Attention data-parallel size.", "parallel")
    ep_size: int = _flag(1, "Expert-parallel size.", "parallel")
    cp_size: int = _flag(1, "Context-parallel size (accepted; must be 1).", "parallel")
    communication_backend: str = _flag("fused", "fused (NVLink kernels) | nccl (baseline).", "parallel")
    enable_numa_binding: bool = _flag(True, "Bind every rank process to the CPUs (and prefer the memory) of its GPU's NUMA node.", "parallel")
    tp_mlp_mode: str = _flag("auto", "Dense MLP under tensor parallelism: tp (weights sharded, two collectives per layer) | rows "
                             "(every rank holds the whole MLP and runs it on its own rows: one reduce-scatter and one all-gather "
                             "per layer instead of two each) | auto (currently tp).", "parallel")
    # ---- EPLB (230-242)
    enable_eplb: bool = _flag(False, "Expert-parallel load balancing.", "eplb")
    redundant_experts_num: int = _flag(1, "Redundant expert slots per device.", "eplb")
    eplb_update_interval: int = _flag(1000, "Steps between rebalancing rounds.", "eplb")
    eplb_update_threshold: float = _flag(0.8, "Cosine-similarity threshold that triggers a re-plan.", "eplb")
    expert_parallel_degree: int = _flag(0, "0/1: gather + all-reduce; 2: all-to-all dispatch/combine.", "eplb")
    # ---- prefix cache (284-293)
    enable_prefix_cache: bool = _flag(True, "Share KV blocks among requests with equal prefixes.", "prefix_cache")
    xxh3_128bits_seed: int = _flag(1024, "Seed of the 128-bit block hash.", "prefix_cache")
    host_blocks_factor: float = _flag(0.0, "Host-memory tier of the prefix cache: host blocks = factor x device blocks (0: off).", "prefix_cache")
    # ---- multi node (297-318)
    master_node_addr: str = _flag("127.0.0.1:19888", "Rendez-vous address.", "multi_node")
    nnodes: int = _flag(1, "Number of nodes.", "multi_node")
    node_rank: int = _flag(0, "Rank of this node.", "multi_node")
    enable_shm: bool = _flag(True, "Step inputs travel over shared memory to local ranks.", "multi_node")
    # ---- PD disaggregation (322-356)
    enable_disagg_pd: bool = _flag(False, "Prefill / decode disaggregation.", "disagg_pd")
    disagg_pd_port: int = _flag(7777, "Port of the PD control service.", "disagg_pd")
    instance_role: str = _flag("DEFAULT", "DEFAULT | PREFILL | DECODE", "disagg_pd")
    instance_name: str = _flag("", "Name of this instance.", "disagg_pd")
    kv_cache_transfer_mode: str = _flag("PUSH", "PUSH | PULL", "disagg_pd")
    transfer_listen_port: int = _flag(26000, "Listen port of the weight service (remote wake-up, with --enable_xtensor).", "disagg_pd")
    # ---- speculative (360-407)
    draft_model: str = _flag("", "Draft (MTP) model directory or preset.", "speculative")
    draft_devices: str = _flag("", "Devices of the draft model (default: same).", "speculative")
    num_speculative_tokens: int = _flag(0, "Draft tokens per step.", "speculative")
    speculative_algorithm: str = _flag("MTP", "MTP | Eagle3 | Suffix", "speculative")
    # ---- service routing (417-425): the registry / router of `python -m xllm_wxh_b200.service.router` stands for etcd +
    # xllm-service
    etcd_addr: str = _flag("", "host:port of the service registry the instance registers with.", "service_routing")
    enable_service_routing: bool = _flag(False, "Register with the service layer and send heartbeats (load, latency, prefix-cache events).", "service_routing")
    heart_beat_interval: float = _flag(0.5, "Seconds between heartbeats to the service layer.", "service_routing")
    # ---- parsers (544-556)
    enable_qwen3_reranker: bool = _flag(False, "/v1/rerank scores a document by P(yes) against P(no) after query + document (Qwen3-Reranker).", "api")
    rerank_no_token_id: int = _flag(2152, "Token id of \"no\" for --enable_qwen3_reranker (Qwen3 vocabulary).", "api")
    rerank_yes_token_id: int = _flag(9693, "Token id of \"yes\" for --enable_qwen3_reranker (Qwen3 vocabulary).", "api")
    reasoning_parser: str = _flag("", "auto | qwen3 | deepseek-r1 | glm45 | ''", "parsers")
    tool_call_parser: str = _flag("", "auto | qwen25 | qwen3_coder | deepseekv3 | kimi_k2 | glm45 | ''", "parsers")
    # ---- profile / SLO (246-280)
    enable_profile_step_time: bool = _flag(False, "Time synthetic prefill / decode steps at start-up and fit step-time predictors.", "profile")
    enable_profile_token_budget: bool = _flag(False, "Derive the per-step token budget from the predictors and the TPOT target.", "profile")
    profile_max_prompt_length: int = _flag(2048, "Longest synthetic prompt used by the start-up profiler.", "profile")
    max_global_ttft_ms: float = _flag(0.0, "Time-to-first-token target of the instance (0: none).", "profile")
    max_global_tpot_ms: float = _flag(0.0, "Time-per-output-token target of the instance (0: none).", "profile")
    # ---- health (653-655)
    health_check_interval_ms: int = _flag(3000, "Worker liveness poll period.", "health")
    # ---- beam
    beam_width: int = _flag(1, "Default beam width.", "beam")
    # ---- remaining flags of the reference's command line (global_flags.cpp).  The first three are wired; the others belong to
    # parts that have no counterpart on this hardware (NPU / MLU kernels, xTensor, Mooncake store, DiT / Rec / VLM pipelines)
    # or describe mechanisms that are always on here; they are accepted with the reference's defaults so that an existing
    # launch line keeps working.
    etcd_ttl: int = _flag(3, "Lease time (s) of the instance's registration with the service layer.", "service_routing")
    speculative_suffix_cache_max_depth: int = _flag(64, "Suffix drafter: longest suffix kept in the tree.", "speculative")
    speculative_suffix_max_cached_requests: int = _flag(-1, "Suffix drafter: sequences kept (-1: 8192).", "speculative")
    speculative_suffix_max_spec_factor: float = _flag(1.0, "Suffix drafter: a match of m tokens proposes at most m * factor + offset tokens.", "speculative")
    speculative_suffix_max_spec_offset: float = _flag(0.0, "Suffix drafter: see --speculative_suffix_max_spec_factor.", "speculative")
    speculative_suffix_min_token_prob: float = _flag(0.1, "Suffix drafter: a token is proposed while the product of branch frequencies on the way to it stays above this.", "speculative")
    speculative_suffix_use_tree_spec: bool = _flag(False, "Accepted.", "compat")
    disable_ttft_profiling: bool = _flag(False, "Accepted.", "compat")
    enable_profile_kv_blocks: bool = _flag(True, "Accepted (the KV block count is always derived from free memory).", "compat")
    enable_dp_balance: bool = _flag(False, "Accepted.", "compat")
    enable_control_h2d_block_num: bool = _flag(False, "Accepted.", "compat")
    enable_forward_interruption: bool = _flag(False, "Accepted.", "compat")
    enable_constrained_decoding: bool = _flag(False, "Accepted.", "compat")
    enable_multi_stream_parallel: bool = _flag(False, "Accepted.", "compat")
    micro_batch_num: int = _flag(1, "Accepted.", "compat")
    max_requests_per_batch: int = _flag(1, "Accepted.", "compat")
    max_decode_rounds: int = _flag(0, "Accepted.", "compat")
    enable_topk_sorted: bool = _flag(True, "Accepted.", "compat")
    enable_opt_validate_probs: bool = _flag(False, "Accepted.", "compat")
    enable_beam_search_kernel: bool = _flag(False, "Accepted.", "compat")
    enable_block_copy_kernel: bool = _flag(True, "Accepted.", "compat")
    enable_intralayer_addnorm: bool = _flag(False, "Accepted (add + norm is always fused).", "compat")
    enable_customize_mla_kernel: bool = _flag(False, "Accepted.", "compat")
    enable_atb_spec_kernel: bool = _flag(False, "Accepted.", "compat")
    enable_xattention_one_stage: bool = _flag(False, "Accepted.", "compat")
    enable_manual_loader: bool = _flag(False, "Accepted.", "compat")
    enable_prefetch_weight: bool = _flag(False, "Accepted.", "compat")
    enable_rolling_load: bool = _flag(False, "Accepted.", "compat")
    rolling_load_num_cached_layers: int = _flag(2, "Accepted.", "compat")
    rolling_load_num_rolling_slots: int = _flag(-1, "Accepted.", "compat")
    enable_xtensor: bool = _flag(False, "Serve this instance's weights on --transfer_listen_port, so that sleeping instances of the same model can wake up from them (/link_d2d, /wakeup with remote_addrs).", "service")
    xtensor_master_node_addr: str = _flag("127.0.0.1:19889", "Accepted.", "compat")
    phy_page_granularity_size: int = _flag(2 * 1024 * 1024, "Accepted.", "compat")
    enable_pd_ooc: bool = _flag(False, "Accepted.", "compat")
    kv_cache_transfer_type: str = _flag("LlmDataDist", "Accepted (KV moves over NVLink peer memory here).", "compat")
    enable_kvcache_store: bool = _flag(False, "Third KV tier: blocks that reach the host tier are also written to the shared store at --store_master_server_address (xllm-kv-store), and prompts are completed from it. Needs --host_blocks_factor.", "prefix_cache")
    enable_cache_upload: bool = _flag(False, "Accepted (prefix-cache events always travel with the heartbeat).", "compat")
    store_protocol: str = _flag("tcp", "Accepted.", "compat")
    store_master_server_address: str = _flag("", "host:port of the shared KV-block store.", "prefix_cache")
    store_metadata_server: str = _flag("", "Accepted.", "compat")
    store_local_hostname: str = _flag("", "Accepted.", "compat")
    prefetch_timeout: int = _flag(0, "Accepted.", "compat")
    prefetch_bacth_size: int = _flag(2, "Accepted.", "compat")
    layers_wise_copy_batchs: int = _flag(4, "Accepted.", "compat")
    input_shm_size: int = _flag(1024, "Accepted (the step channel is sized from the largest message).", "compat")
    output_shm_size: int = _flag(128, "Accepted.", "compat")
    use_contiguous_input_buffer: bool = _flag(True, "Accepted (step inputs are always one packed buffer).", "compat")
    flashinfer_workspace_buffer_size: int = _flag(128 * 1024 * 1024, "Accepted (the attention kernels need no plan workspace).", "compat")
    rank_tablefile: str = _flag("", "Accepted.", "compat")
    npu_kernel_backend: str = _flag("AUTO", "Accepted.", "compat")
    npu_phy_id: int = _flag(-1, "Accepted.", "compat")
    limit_image_per_prompt: int = _flag(4, "Accepted.", "compat")
    use_audio_in_video: bool = _flag(False, "Accepted.", "compat")
    dit_cache_policy: str = _flag("TaylorSeer", "Accepted.", "compat")
    dit_cache_n_derivatives: int = _flag(3, "Accepted.", "compat")
    dit_cache_residual_diff_threshold: float = _flag(0.09, "Accepted.", "compat")
    dit_cache_skip_interval_steps: int = _flag(3, "Accepted.", "compat")
    dit_cache_warmup_steps: int = _flag(0, "Accepted.", "compat")
    enable_rec_fast_sampler: bool = _flag(True, "Accepted.", "compat")
    enable_rec_prefill_only: bool = _flag(False, "Accepted.", "compat")
    output_rec_logprobs: bool = _flag(False, "Accepted.", "compat")
    rec_worker_max_concurrency: int = _flag(1, "Accepted.", "compat")
    # ---- python-side conveniences
    max_model_len: int = _flag(0, "Context limit (0 = model's).", "model")
    num_kv_blocks: int = _flag(0, "Force the number of KV blocks (0 = derive).", "kv")

    def validate(self) -> "Options":
        """The reference's `validate_flags` (xllm/xllm.cpp:59-109) plus range checks."""
        if self.cp_size != 1:
            raise ValueError("cp_size > 1 is not supported")
        if self.instance_role not in ("DEFAULT", "PREFILL", "DECODE", "MIX"):
            raise ValueError(f"bad instance_role {self.instance_role}")
        if self.kv_cache_transfer_mode not in ("PUSH", "PULL"):
            raise ValueError("kv_cache_transfer_mode must be PUSH or PULL")
        if self.enable_disagg_pd and self.instance_role == "PREFILL" and self.enable_schedule_overlap:
            self.enable_schedule_overlap = False      # master.cpp:179-188
        if not (0.0 < self.max_memory_utilization <= 1.0):
            raise ValueError("max_memory_utilization must be in (0, 1]")
        if self.block_size <= 0 or self.max_tokens_per_batch <= 0 or self.max_seqs_per_batch <= 0:
            raise ValueError("block_size, max_tokens_per_batch and max_seqs_per_batch must be positive")
        if self.num_speculative_tokens > 0 and self.enable_schedule_overlap:
            self.enable_schedule_overlap = False
        if self.use_mix_scheduler and not self.enable_chunked_prefill:
            self.enable_chunked_prefill = True        # the mix policy is a chunked-prefill policy (mix_scheduler.h:32)
        ignored = self.ignored_flags()
        if ignored:
            import logging
            logging.getLogger("xllm").warning("flags accepted for command-line compatibility that have no effect in this build: %s",
                                              ", ".join(f"--{k}={v}" for k, v in ignored.items()))
        return self

    def ignored_flags(self) -> Dict[str, Any]:
        """Flags of the compatibility group that were given a value other than their default: they are accepted so that an
        existing launch line keeps working, but nothing reads them."""
        out: Dict[str, Any] = {}
        for f in dataclasses.fields(self):
            if f.metadata.get("group") == "compat" and getattr(self, f.name) != f.default:
                out[f.name] = getattr(self, f.name)
        return out

    def device_list(self) -> List[str]:
        if self.devices in ("auto", ""):
            import torch
            if torch.cuda.is_available():
                return [f"cuda:{i}" for i in range(1)]
            return ["cpu"]
        return [d.strip() for d in self.devices.split(",") if d.strip()]


def add_flags(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    groups: Dict[str, Any] = {}
    for f in dataclasses.fields(Options):
        g = f.metadata.get("group", "misc")
        if g not in groups:
            groups[g] = parser.add_argument_group(g)
        name = "--" + f.name
        if f.type in ("bool", bool):
            groups[g].add_argument(name, type=lambda s: str(s).lower() in ("1", "true", "yes", "on"), nargs="?",
                                   const=True, default=f.default, help=f.metadata.get("help", ""))
        else:
            ty = {"int": int, "float": float, "str": str}.get(f.type if isinstance(f.type, str) else f.type.__name__, str)
            groups[g].add_argument(name, type=ty, default=f.default, help=f.metadata.get("help", ""))
    return parser


def options_from_namespace(ns) -> Options:
    names = {f.name for f in dataclasses.fields(Options)}
    return Options(**{k: v for k, v in vars(ns).items() if k in names}).validate()
