"""One instance of a disaggregated pair, run as its own process (GPU test).
    argv: <role: prefill|decode|colocated> <gpu index> <port> <out.pt> [PUSH|PULL]
The decode instance serves until the prefill instance has finished its prompts and tells it to stop."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from xllm_wxh_b200 import LLM, SamplingParams  # noqa: E402
from xllm_wxh_b200.config import Options  # noqa: E402
from xllm_wxh_b200.models.args import ModelArgs  # noqa: E402
from xllm_wxh_b200.runtime.disagg_pd import DecodeCoordinator, PrefillCoordinator, SocketTransport  # noqa: E402
from xllm_wxh_b200.runtime.engine import LLMEngine  # noqa: E402
from xllm_wxh_b200.runtime.master import LLMMaster  # noqa: E402


def main():
    role, gpu, port, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    mode = sys.argv[5] if len(sys.argv) > 5 else "PUSH"
    args = ModelArgs(model_type="qwen3", vocab_size=1024, hidden_size=512, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=128,
                     intermediate_size=1024, qk_norm=True, max_position_embeddings=1024)
    opts = Options(model="preset:test", devices=f"cuda:{gpu}", block_size=16, num_kv_blocks=128, max_tokens_per_batch=512,
                   max_seqs_per_batch=16, enable_disagg_pd=role != "colocated",
                   instance_role={"prefill": "PREFILL", "decode": "DECODE", "colocated": "DEFAULT"}[role], enable_graph=False,
                   kv_cache_transfer_mode=mode)
    os.environ["LOCAL_RANK"] = str(gpu)
    eng = LLMEngine(opts, model_args=args, rank=0, world_size=1)
    eng.worker.model.init_random(seed=5, std=0.05).finalize_weights()
    master = LLMMaster(opts, eng)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (9, 33, 70, 4, 50)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    if role == "decode":
        dec = DecodeCoordinator(master)
        dec.serve(port)
        master.run()
        deadline = time.time() + 200
        while not os.path.exists(out + ".stop") and time.time() < deadline:
            time.sleep(0.05)
        from xllm_wxh_b200.ops import cuda_ops
        torch.save({"status": cuda_ops.read_status(), "generated": eng.scheduler.stats()["generated_tokens"],
                    "pulled": sum(t.bytes_moved for t in eng.kv_sources.values())}, out)
        return 0
    llm = LLM(model="preset:test", devices=f"cuda:{gpu}", engine=eng)
    llm.master = master
    if role == "prefill":
        PrefillCoordinator(master, SocketTransport.connect("127.0.0.1", port))
    llm.generate_timeout_s = 120.0
    outs = llm.generate(prompts, sp)
    from xllm_wxh_b200.ops import cuda_ops
    torch.save({"tokens": [o.outputs[0].token_ids for o in outs], "status": cuda_ops.read_status(),
                "moved": getattr(eng.kv_transfer, "bytes_moved", 0) if eng.kv_transfer else 0}, out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
