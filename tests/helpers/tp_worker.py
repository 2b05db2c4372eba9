"""Rank program of the multi-process tensor-parallel tests (launched with torch.distributed.run).

Every rank builds the same small model sharded over the world, runs one prefill step and a few decode steps on
fixed prompts, and rank 0 writes the logits / tokens to a file for the parent test to compare with a single-rank run.
    argv: <out.pt> <device: cpu|cuda> <backend: fused|nccl> [model_type]
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from xllm_wxh_b200 import LLM, SamplingParams  # noqa: E402
from xllm_wxh_b200.config import Options  # noqa: E402
from xllm_wxh_b200.models.args import ModelArgs  # noqa: E402
from xllm_wxh_b200.runtime.engine import LLMEngine  # noqa: E402


def model_args(kind: str, device: str) -> ModelArgs:
    dt = "bfloat16" if device == "cuda" else "float32"
    if kind == "qwen3_moe":
        return ModelArgs(model_type="qwen3_moe", dtype=dt, vocab_size=512, hidden_size=256, n_layers=2, n_heads=8, n_kv_heads=2,
                         head_dim=64 if device == "cpu" else 128, intermediate_size=512, qk_norm=True, n_routed_experts=8,
                         num_experts_per_tok=2, moe_intermediate_size=128, max_position_embeddings=1024)
    if kind in ("deepseek_v3", "deepseek_v32"):
        # the GPU kernels serve the production head shape (latent 512 + rope 64, nope 128) and 16 heads per rank
        gpu = device == "cuda"
        # V3.2: a lightning indexer that keeps 12 keys per query, fewer than the prompts are long
        extra = dict(index_topk=12, index_n_heads=16, index_head_dim=128 if gpu else 32) if kind == "deepseek_v32" else {}
        return ModelArgs(model_type=kind, dtype=dt, **extra, vocab_size=512, hidden_size=256, n_layers=3, n_heads=32 if gpu else 4,
                         n_kv_heads=32 if gpu else 4, head_dim=192 if gpu else 48, intermediate_size=512, n_routed_experts=8,
                         num_experts_per_tok=2, moe_intermediate_size=128, n_shared_experts=1, first_k_dense_replace=1,
                         scoring_func="sigmoid", topk_method="noaux_tc", n_group=2, topk_group=1, routed_scaling_factor=1.5,
                         q_lora_rank=128, kv_lora_rank=512 if gpu else 32, qk_nope_head_dim=128 if gpu else 32,
                         qk_rope_head_dim=64 if gpu else 16, v_head_dim=128 if gpu else 32, rope_theta=1e4,
                         max_position_embeddings=1024)
    return ModelArgs(model_type="qwen3", dtype=dt, vocab_size=1024, hidden_size=512, n_layers=3, n_heads=8, n_kv_heads=2,
                     head_dim=64 if device == "cpu" else 128, intermediate_size=1024, qk_norm=True, max_position_embeddings=1024)


def main():
    out, device, backend = sys.argv[1], sys.argv[2], sys.argv[3]
    kind = sys.argv[4] if len(sys.argv) > 4 else "qwen3"
    ep = int(sys.argv[5]) if len(sys.argv) > 5 else 1
    dp = int(sys.argv[6]) if len(sys.argv) > 6 else 1
    epd = int(sys.argv[7]) if len(sys.argv) > 7 else 0
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    devs = ",".join(f"cuda:{i}" for i in range(world)) if device == "cuda" else "cpu"
    opts = Options(model="preset:test", devices=devs, block_size=16, num_kv_blocks=128, max_tokens_per_batch=512,
                   max_seqs_per_batch=16, communication_backend=backend, ep_size=ep, dp_size=dp,
                   enable_graph=os.environ.get("XLLM_TEST_GRAPH") == "1",
                   enable_prefill_piecewise_graph=os.environ.get("XLLM_TEST_GRAPH") == "1",
                   expert_parallel_degree=epd,
                   dtype="float32" if device == "cpu" else "auto")
    if os.environ.get("XLLM_TEST_TP_MLP"):             # "rows": every rank holds the whole MLP and runs it on its own rows
        opts.tp_mlp_mode = os.environ["XLLM_TEST_TP_MLP"]
    eplb = os.environ.get("XLLM_TEST_EPLB")            # "0": weights from the engine's own seed; "1": the same + EPLB on
    if eplb is not None:
        opts.random_seed = 5
        if eplb == "1":
            opts.enable_eplb, opts.redundant_experts_num, opts.eplb_update_interval, opts.eplb_update_threshold = True, 1, 2, 1.1
    tier = os.environ.get("XLLM_TEST_HOST_TIER")       # "1": small device cache + host tier, the prompts run twice
    if tier is not None:
        opts.num_kv_blocks = 7
        opts.max_seqs_per_batch = 1
        if tier == "1":
            opts.host_blocks_factor = 6.0
    store = os.environ.get("XLLM_TEST_KV_STORE")       # host:port of a shared block store: host tier on, written through
    if store:
        opts.host_blocks_factor = 2.0
        opts.enable_kvcache_store, opts.store_master_server_address = True, store
    eng = LLMEngine(opts, model_args=model_args(kind, device))
    if eplb is None:
        m = eng.worker.model.init_random(seed=5, std=0.05)
        if hasattr(m, "finalize_weights"):
            m.finalize_weights()
    if rank != 0:
        eng.worker_loop()
        return 0
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, eng.args.vocab_size, (n,), generator=g).tolist() for n in (9, 33, 70, 4)]
    llm = LLM(model="preset:test", devices=devs, engine=eng)
    plain = os.environ.get("XLLM_TEST_PLAIN_GREEDY") == "1"    # no log-probabilities: tensor-parallel ranks keep the logits sharded
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=not plain)
    if os.environ.get("XLLM_TEST_SAMPLED") == "1":     # seeded sampling with top-k / top-p, no log-probabilities
        sp = [SamplingParams(temperature=0.9, top_k=k, top_p=p, seed=11 + i, max_tokens=6, ignore_eos=True)
              for i, (k, p) in enumerate([(20, 0.9), (5, 1.0), (64, 0.5), (1, 1.0)])]
    outs = llm.generate(prompts, sp)
    if tier is not None:
        outs = llm.generate(prompts, sp)               # second pass: prefixes come back from the host tier (when on)
    status = 0
    if device == "cuda":
        from xllm_wxh_b200.ops import cuda_ops
        status = cuda_ops.read_status()
    ex = getattr(eng.worker.model, "eplb", None)
    st = eng.scheduler.stats()
    torch.save({"host_loaded_blocks": st["host_loaded_blocks"], "host_offloaded_blocks": st["host_offloaded_blocks"],
                "eplb_activations": ex.num_activations if ex is not None else 0,
                "eplb_rows_moved_remote": ex.rows_moved_remote if ex is not None else 0,
                "tokens": [o.outputs[0].token_ids for o in outs],
                "logprobs": [[l.logprob for l in (o.outputs[0].logprobs or [])] for o in outs], "status": status,
                "sharded_greedy_steps": eng.worker.sharded_greedy_steps,
                "sharded_sampling_steps": eng.worker.sharded_sampling_steps,
                "shard_sampling_overflows": eng.worker.shard_sampling_overflows,
                "fused_tp_launches": getattr(getattr(eng.comm, "fused_tp", None), "launches", 0),
                "store_prefetched_blocks": getattr(eng, "store_prefetched_blocks", 0),
                "cached_tokens": [o.usage.num_cached_tokens for o in outs]}, out)
    llm.finish()
    return 0


if __name__ == "__main__":
    sys.exit(main())
