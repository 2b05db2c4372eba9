"""Tensor parallelism: a model sharded over 2 ranks must reproduce the single-rank run.
CPU ranks (gloo) check the sharding / step-broadcast logic; GPU ranks check the NCCL path and the fused NVLink path."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "helpers", "tp_worker.py")


def _run(world, out, device, backend, kind="qwen3", ep=1, port=29611, env_extra=None, timeout=600, dp=1, epd=0):
    env = dict(os.environ)
    env.update(env_extra or {})
    if world == 1:
        env.update(WORLD_SIZE="1", RANK="0", LOCAL_RANK="0")
        cmd = [sys.executable, WORKER, out, device, backend, kind, str(ep), str(dp), str(epd)]
    else:
        for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"):
            env.pop(k, None)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
               "127.0.0.1", "--master-port", str(port), WORKER, out, device, backend, kind, str(ep), str(dp), str(epd)]
    p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)
    assert p.returncode == 0, p.stdout[-4000:]
    return torch.load(out)


def test_tp2_cpu_gloo_matches_single_rank(tmp_path):
    one = _run(1, str(tmp_path / "one.pt"), "cpu", "nccl")
    two = _run(2, str(tmp_path / "two.pt"), "cpu", "nccl", port=29621)
    assert one["tokens"] == two["tokens"]
    for a, b in zip(one["logprobs"], two["logprobs"]):
        assert max(abs(x - y) for x, y in zip(a, b)) < 1e-3


def test_tp2_cpu_gloo_greedy_keeps_logits_sharded(tmp_path):
    """Greedy requests without log-probabilities: each rank takes the maximum of its vocabulary shard and the ranks
    exchange (value, token id) pairs; the tokens are those of one rank holding the whole vocabulary."""
    one = _run(1, str(tmp_path / "one.pt"), "cpu", "nccl", env_extra={"XLLM_TEST_PLAIN_GREEDY": "1"})
    two = _run(2, str(tmp_path / "two.pt"), "cpu", "nccl", port=29691, env_extra={"XLLM_TEST_PLAIN_GREEDY": "1"})
    assert one["sharded_greedy_steps"] == 0 and two["sharded_greedy_steps"] > 0
    assert one["tokens"] == two["tokens"]
    off = _run(2, str(tmp_path / "off.pt"), "cpu", "nccl", port=29695,
               env_extra={"XLLM_TEST_PLAIN_GREEDY": "1", "XLLM_TP_GREEDY_SHARDED": "0"})
    assert off["sharded_greedy_steps"] == 0 and off["tokens"] == two["tokens"]


def test_tp2_cpu_gloo_sampling_keeps_logits_sharded(tmp_path):
    """Seeded top-k / top-p sampling under TP: the ranks exchange per-shard candidates instead of the logits, and the
    tokens are those of the single-rank run (same seeds, draw in vocabulary order)."""
    env = {"XLLM_TEST_SAMPLED": "1", "XLLM_TEST_PLAIN_GREEDY": "1", "XLLM_TP_SAMPLE_SHARDED": "1"}
    one = _run(1, str(tmp_path / "one.pt"), "cpu", "nccl", env_extra=env)
    two = _run(2, str(tmp_path / "two.pt"), "cpu", "nccl", port=29699, env_extra=env)
    assert two["sharded_sampling_steps"] > 0 and two["shard_sampling_overflows"] == 0
    assert one["tokens"] == two["tokens"]


def test_tp2_cpu_gloo_host_kv_tier(tmp_path):
    """Two ranks, a device cache too small to keep the prompts, host tier on: every rank offloads and reloads its own
    shard of the blocks from the copy lists in the step message, and the second pass equals a run without the tier."""
    off = _run(2, str(tmp_path / "off.pt"), "cpu", "nccl", port=29671, env_extra={"XLLM_TEST_HOST_TIER": "0"})
    on = _run(2, str(tmp_path / "on.pt"), "cpu", "nccl", port=29681, env_extra={"XLLM_TEST_HOST_TIER": "1"})
    assert off["host_loaded_blocks"] == 0 and on["host_offloaded_blocks"] > 0 and on["host_loaded_blocks"] > 0
    assert on["tokens"] == off["tokens"]
    for a, b in zip(on["logprobs"], off["logprobs"]):
        assert max(abs(x - y) for x, y in zip(a, b)) < 1e-3


def test_tp2_cpu_gloo_shared_kv_store(tmp_path):
    """Two tensor-parallel ranks and a shared block store: the first instance writes every rank's share of its blocks
    through; a second instance (new processes, empty caches) fetches them rank by rank inside a control operation and
    loads them instead of computing the prompts again."""
    from xllm_wxh_b200.service.kv_store import KvStoreServer
    srv = KvStoreServer("127.0.0.1", 0, 256 << 20).start()
    try:
        env = {"XLLM_TEST_KV_STORE": f"127.0.0.1:{srv.port}"}
        plain = _run(2, str(tmp_path / "plain.pt"), "cpu", "nccl", port=29711)
        first = _run(2, str(tmp_path / "first.pt"), "cpu", "nccl", port=29715, env_extra=env)
        st = srv.store.stats()
        # prompts of 9, 33, 70 and 4 tokens with 6 generated: 0 + 2 + 4 + 0 full blocks, one record per rank
        assert first["store_prefetched_blocks"] == 0 and st["blocks"] == 2 * 6 and first["tokens"] == plain["tokens"]
        assert all(k.endswith("/0/2") or k.endswith("/1/2") for k in srv.store.blocks)
        second = _run(2, str(tmp_path / "second.pt"), "cpu", "nccl", port=29719, env_extra=env)
        # whole blocks before the last prompt token: 2 of the 33-token prompt, 4 of the 70-token prompt
        assert second["store_prefetched_blocks"] == 6 and second["host_loaded_blocks"] == 6
        assert second["cached_tokens"] == [0, 32, 64, 0]
        assert second["tokens"] == plain["tokens"]
        assert srv.store.stats()["puts"] == st["puts"]                # nothing is written twice
    finally:
        srv.stop()


def test_dp2_cpu_gloo_shared_kv_store(tmp_path):
    """Two attention-DP ranks (one process each, a cache each) behind one scheduler: either rank writes the blocks of its
    own requests through; in a second instance the fetch runs on the DP rank that takes the request."""
    from xllm_wxh_b200.service.kv_store import KvStoreServer
    srv = KvStoreServer("127.0.0.1", 0, 256 << 20).start()
    try:
        env = {"XLLM_TEST_KV_STORE": f"127.0.0.1:{srv.port}"}
        plain = _run(2, str(tmp_path / "plain.pt"), "cpu", "nccl", dp=2, port=29731)
        first = _run(2, str(tmp_path / "first.pt"), "cpu", "nccl", dp=2, port=29735, env_extra=env)
        assert first["tokens"] == plain["tokens"] and first["store_prefetched_blocks"] == 0
        assert srv.store.stats()["blocks"] == 6 and all(k.endswith("/0/1") for k in srv.store.blocks)
        second = _run(2, str(tmp_path / "second.pt"), "cpu", "nccl", dp=2, port=29739, env_extra=env)
        assert second["store_prefetched_blocks"] == 6 and second["host_loaded_blocks"] == 6
        assert second["cached_tokens"] == [0, 32, 64, 0] and second["tokens"] == plain["tokens"]
    finally:
        srv.stop()


def test_ep2_cpu_gloo_moe_matches_single_rank(tmp_path):
    one = _run(1, str(tmp_path / "one.pt"), "cpu", "nccl", kind="qwen3_moe")
    two = _run(2, str(tmp_path / "two.pt"), "cpu", "nccl", kind="qwen3_moe", ep=2, port=29631)
    assert one["tokens"] == two["tokens"]


def test_ep2_cpu_gloo_eplb_moves_experts_between_ranks(tmp_path):
    """Expert-parallel load balancing over two ranks: layers are re-planned every other step, expert weights travel
    between the ranks, and the generated tokens stay those of the single-rank run."""
    one = _run(1, str(tmp_path / "one.pt"), "cpu", "nccl", kind="qwen3_moe", env_extra={"XLLM_TEST_EPLB": "0"})
    two = _run(2, str(tmp_path / "two.pt"), "cpu", "nccl", kind="qwen3_moe", ep=2, port=29641, env_extra={"XLLM_TEST_EPLB": "1"})
    assert two["eplb_activations"] > 0 and two["eplb_rows_moved_remote"] > 0
    assert one["tokens"] == two["tokens"]


def test_dp2_ep2_cpu_gloo_moe_matches_single_rank(tmp_path):
    """Attention data parallel x expert parallel: two ranks with their own batches, experts split between them."""
    one = _run(1, str(tmp_path / "one.pt"), "cpu", "nccl", kind="qwen3_moe")
    two = _run(2, str(tmp_path / "two.pt"), "cpu", "nccl", kind="qwen3_moe", ep=2, dp=2, port=29651)
    assert one["tokens"] == two["tokens"]


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("epd,graph", [(0, "0"), (2, "0"), (0, "1"), (2, "1")])
def test_dp2_ep2_gpu_moe_matches_single_gpu(tmp_path, epd, graph):
    """epd=0: NCCL gather + all-reduce baseline; epd=2: fused NVLink dispatch / combine kernels.  With CUDA graphs the two
    DP ranks see different step shapes and capture at different times, yet each must run every exchange once per step."""
    one = _run(1, str(tmp_path / "one.pt"), "cuda", "nccl", kind="qwen3_moe")
    two = _run(2, str(tmp_path / "two.pt"), "cuda", "fused", kind="qwen3_moe", ep=2, dp=2, epd=epd, port=29661,
               env_extra={"NCCL_NVLS_ENABLE": "0", "XLLM_TEST_GRAPH": graph})
    assert two["status"] == 0, "a bounded wait in a fused kernel expired"
    for a, b in zip(one["logprobs"], two["logprobs"]):
        assert max(abs(x - y) for x, y in zip(a, b)) < 0.08
    same = sum(x == y for a, b in zip(one["tokens"], two["tokens"]) for x, y in zip(a, b))
    assert same >= sum(len(a) for a in one["tokens"]) - 2


@pytest.mark.gpu
@pytest.mark.multigpu
def test_tp2_gpu_greedy_keeps_logits_sharded(tmp_path):
    one = _run(1, str(tmp_path / "one.pt"), "cuda", "nccl", env_extra={"XLLM_TEST_PLAIN_GREEDY": "1"})
    two = _run(2, str(tmp_path / "two.pt"), "cuda", "fused", port=29697,
               env_extra={"NCCL_NVLS_ENABLE": "0", "XLLM_TEST_PLAIN_GREEDY": "1"})
    assert two["status"] == 0 and two["sharded_greedy_steps"] > 0
    same = sum(x == y for a, b in zip(one["tokens"], two["tokens"]) for x, y in zip(a, b))
    assert same >= sum(len(a) for a in one["tokens"]) - 2        # bf16 sums are associated differently across ranks


@pytest.mark.gpu
@pytest.mark.multigpu
def test_tp2_gpu_sampling_keeps_logits_sharded(tmp_path):
    """As the CPU test above, through the candidates kernel: tokens equal the single-GPU run's except where bf16 sums
    associated differently across ranks move a draw over a boundary."""
    env = {"XLLM_TEST_SAMPLED": "1", "XLLM_TEST_PLAIN_GREEDY": "1", "NCCL_NVLS_ENABLE": "0", "XLLM_TP_SAMPLE_SHARDED": "1"}
    one = _run(1, str(tmp_path / "one.pt"), "cuda", "nccl", env_extra=env)
    two = _run(2, str(tmp_path / "two.pt"), "cuda", "fused", port=29701, env_extra=env)
    assert two["status"] == 0 and two["sharded_sampling_steps"] > 0 and two["shard_sampling_overflows"] == 0
    same = sum(x == y for a, b in zip(one["tokens"], two["tokens"]) for x, y in zip(a, b))
    assert same >= sum(len(a) for a in one["tokens"]) - 6


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("backend", ["nccl", "fused", "fused_nvls", "fused_nvls_mlp_rows"])
def test_tp2_gpu_matches_single_gpu(tmp_path, backend):
    """`fused`: reduce-scatter / all-gather by peer loads and stores; `fused_nvls`: the same step with the reduction and
    the broadcast done by the NVSwitch (`multimem.ld_reduce` / `multimem.st` on a multicast-bound buffer);
    `fused_nvls_mlp_rows`: tensor-parallel attention around an MLP that every rank holds whole and runs on its own rows."""
    one = _run(1, str(tmp_path / "one.pt"), "cuda", "nccl")
    env = {"NCCL_NVLS_ENABLE": "0"}
    if backend == "fused_nvls":
        env = {"XLLM_TP_FUSED_MODE": "nvls", "XLLM_TEST_GRAPH": "1"}
    if backend == "fused_nvls_mlp_rows":    # the prompt step runs the replicated MLP by rows, the decode steps its TP slices
        env = {"XLLM_TP_FUSED_MODE": "nvls", "XLLM_TEST_GRAPH": "1", "XLLM_TEST_TP_MLP": "rows", "XLLM_TP_MLP_ROWS_MIN_TOKENS": "8"}
    two = _run(2, str(tmp_path / "two.pt"), "cuda", "fused" if backend.startswith("fused") else backend, port=29641, env_extra=env)
    assert two["status"] == 0, "a bounded wait in a fused kernel expired"
    # bf16 sums are associated differently across ranks: compare log-probabilities, and tokens where they are decisive
    for a, b in zip(one["logprobs"], two["logprobs"]):
        assert max(abs(x - y) for x, y in zip(a, b)) < 0.08
    same = sum(x == y for a, b in zip(one["tokens"], two["tokens"]) for x, y in zip(a, b))
    total = sum(len(a) for a in one["tokens"])
    assert same >= total - 2


@pytest.mark.parametrize("kind", ["deepseek_v3", "deepseek_v32"])
def test_tp2_cpu_gloo_deepseek_matches_single_rank(tmp_path, kind):
    """`deepseek_v32`: the lightning indexer is replicated, so both ranks keep the same keys for their halves of the heads."""
    one = _run(1, str(tmp_path / "one.pt"), "cpu", "nccl", kind=kind)
    two = _run(2, str(tmp_path / "two.pt"), "cpu", "nccl", kind=kind, port=29653 if kind == "deepseek_v3" else 29663)
    assert one["tokens"] == two["tokens"]
    for a, b in zip(one["logprobs"], two["logprobs"]):
        assert max(abs(x - y) for x, y in zip(a, b)) < 1e-3


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("mode", ["nccl", "pull", "nvls"])
def test_tp2_gpu_deepseek_takes_the_fused_path(tmp_path, mode):
    """MLA + MoE model under TP 2: o_proj, the dense MLP and the routed + shared experts' partial sums all go through the
    fused reduce + residual + RMSNorm + all-gather kernels (`nccl`: the same sharding with NCCL all-reduces, as the
    yardstick for what two-rank bf16 summation alone changes); log-probabilities must agree with the single-GPU run.
    Sigmoid routing over bf16 scores lets a near-tie pick another expert, hence the wider tolerance than for Qwen."""
    one = _run(1, str(tmp_path / "one.pt"), "cuda", "nccl", kind="deepseek_v3")
    env = {"XLLM_TP_FUSED_MODE": mode}
    if mode != "nvls":
        env["NCCL_NVLS_ENABLE"] = "0"
    else:
        env["XLLM_TEST_GRAPH"] = "1"          # the NVLS run also replays its steps from CUDA graphs
    two = _run(2, str(tmp_path / "two.pt"), "cuda", "nccl" if mode == "nccl" else "fused", kind="deepseek_v3", port=29657,
               env_extra=env)
    assert two["status"] == 0 and (mode == "nccl" or two["fused_tp_launches"] > 0)
    worst = max(max(abs(x - y) for x, y in zip(a, b)) for a, b in zip(one["logprobs"], two["logprobs"]))
    assert worst < 0.2, worst
    same = sum(x == y for a, b in zip(one["tokens"], two["tokens"]) for x, y in zip(a, b))
    assert same >= sum(len(a) for a in one["tokens"]) - 3


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fused_expert_parallel_exchange(tmp_path):
    """Dispatch (count exchange, expert-major placement, optional e4m3 quantisation), grouped GEMMs, return and combine on
    every GPU of the box (2, 4 or 8), against the layer computed with all experts in PyTorch."""
    import json
    n = min(8, torch.cuda.device_count())
    n = 8 if n >= 8 else (4 if n >= 4 else 2)
    out = str(tmp_path / "ep.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"):
        env.pop(k, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29675", os.path.join(HERE, "helpers", "ep_worker.py"), out]
    p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-4000:]
    with open(out) as f:
        reports = json.load(f)
    assert len(reports) == n
    for r in reports:
        assert r["status"] == 0, r
        for c in r["cases"]:
            tol = (0.06 if c["fp8"] else 0.03) * c["scale"] + 1e-3
            assert c["err"] <= (1e-6 if c["layer"] == "graph" else tol), (r["rank"], c)
    # every (token, slot) pair arrived somewhere: the rows received over all ranks add up to the pairs sent
    for fp8 in (False, True):
        for layer, tokens in ((0, sum(200 - 37 * r for r in range(n))), (2, 300 * n)):
            rows = sum(c["rows"] for r in reports for c in r["cases"] if c["fp8"] == fp8 and c["layer"] == layer)
            assert rows == tokens * 4
