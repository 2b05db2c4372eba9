"""CUDA graphs of several step shapes share one memory pool: what they hold together is close to what the largest
shape needs, not the sum over shapes (the reference checks the same for its VMM-backed pool,
xllm/core/runtime/cuda_graph_executor_test.cpp)."""
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _capture_all(shared_pool: bool, sizes, width=4096) -> int:
    """Capture one small MLP-like graph per row count, replay each once, and return the bytes that the captures made the
    allocator reserve.  Inputs, weights and graphs live only inside this function: nothing is replayed after its
    tensors are gone."""
    torch.cuda.synchronize()
    gc.collect()
    torch.cuda.empty_cache()
    w1 = torch.randn(width, width, device="cuda", dtype=torch.bfloat16) * 0.02
    w2 = torch.randn(width, width, device="cuda", dtype=torch.bfloat16) * 0.02
    xs = {n: torch.randn(n, width, device="cuda", dtype=torch.bfloat16) for n in sizes}
    stream = torch.cuda.Stream()
    pool = torch.cuda.graph_pool_handle() if shared_pool else None
    with torch.cuda.stream(stream):     # library handles and workspaces are created outside any capture
        warm = torch.nn.functional.silu(xs[sizes[-1]] @ w1) @ w2
    torch.cuda.synchronize()
    del warm
    before = torch.cuda.memory_reserved()
    graphs = []
    for n in sizes:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=pool, stream=stream):
            h = xs[n] @ w1
            h = torch.nn.functional.silu(h) * h
            h = h @ w2
            y = (h * 2).sum(-1)
        graphs.append((g, y))
    torch.cuda.synchronize()
    held = torch.cuda.memory_reserved() - before
    for g, y in graphs:                 # every graph still works next to the others (their outputs do not overlap)
        g.replay()
    torch.cuda.synchronize()
    assert all(bool(torch.isfinite(y.float()).all()) for _, y in graphs)
    del graphs, xs, w1, w2
    gc.collect()
    torch.cuda.synchronize()
    return held


def test_shared_pool_holds_the_maximum_over_shapes_not_the_sum():
    sizes = [16384, 12288, 8192, 4096, 2048]           # rows; one activation of 128, 96, 64, 32, 16 MiB each
    alone = _capture_all(False, sizes)
    shared = _capture_all(True, sizes)
    # a capture keeps at most three activations alive at once (h, silu(h), their product), so the largest shape needs
    # three times its 128 MiB; the five shapes together need (128 + 96 + 64 + 32 + 16) x 3 when every graph has its own pool
    largest_peak = 3 * sizes[0] * 4096 * 2
    assert shared <= 1.25 * largest_peak + (32 << 20), (alone, shared, largest_peak)
    assert shared <= 0.6 * alone, (alone, shared, largest_peak)


def test_engine_graph_executor_uses_one_pool():
    """The serving engine's executor captures every bucket into the same pool (`enable_graph_vmm_pool`, default on)."""
    from xllm_wxh_b200.config import Options
    from xllm_wxh_b200.models.args import ModelArgs
    from xllm_wxh_b200 import LLM, SamplingParams
    from xllm_wxh_b200.runtime.engine import LLMEngine
    args = ModelArgs(model_type="qwen3", vocab_size=2048, hidden_size=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128,
                     intermediate_size=1024, qk_norm=True, max_position_embeddings=1024)
    eng = LLMEngine(Options(model="preset:t", devices="cuda:0", block_size=16, num_kv_blocks=128, max_tokens_per_batch=512,
                            max_seqs_per_batch=16, enable_graph=True), model_args=args)
    llm = LLM(model="preset:t", devices="cuda:0", engine=eng)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    llm.generate([[1, 2, 3]], sp)                       # decode bucket 1
    llm.generate([[5, 6, 7], [8, 9], [3, 3, 3]], sp)    # decode bucket 4
    ex = eng.worker._graph_executor()
    assert ex.pool is not None and ex.num_captures >= 2 and ex.num_replays > 0
