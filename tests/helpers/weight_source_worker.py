"""An awake instance that serves its weights (GPU test of the remote wake-up).
    argv: <gpu index> <port> <out.pt>
Writes its greedy continuation of the test prompt to <out.pt>, then serves until <out.pt>.stop exists."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from xllm_wxh_b200 import LLM, SamplingParams  # noqa: E402
from xllm_wxh_b200.config import Options  # noqa: E402
from xllm_wxh_b200.models.args import ModelArgs  # noqa: E402
from xllm_wxh_b200.runtime.engine import LLMEngine  # noqa: E402
from xllm_wxh_b200.runtime.master import LLMMaster  # noqa: E402
from xllm_wxh_b200.runtime.weight_transfer import WeightServer  # noqa: E402

# XLLM_TEST_WEIGHT_SCALE=8 makes the layers as wide as an 8B model's (about 3 GB of weights) for a bandwidth reading
_S = int(os.environ.get("XLLM_TEST_WEIGHT_SCALE", "1"))
ARGS = dict(model_type="qwen3", vocab_size=2048, hidden_size=512 * _S, n_layers=3 if _S == 1 else 8, n_heads=8 * _S // (2 if _S > 1 else 1),
            n_kv_heads=2 if _S == 1 else 8, head_dim=128, intermediate_size=1536 * _S, qk_norm=True, rope_theta=1e6, max_position_embeddings=4096, dtype="bfloat16")
PROMPT = list(range(11, 75))


def make(gpu: int, seed: int):
    opts = Options(model="preset:x", devices=f"cuda:{gpu}", block_size=16, num_kv_blocks=128, max_tokens_per_batch=512,
                   max_seqs_per_batch=16, enable_graph=False)
    eng = LLMEngine(opts, model_args=ModelArgs(**ARGS))
    eng.worker.model.init_random(seed=seed, std=0.05).finalize_weights()
    return LLMMaster(opts, eng)


def tokens(master):
    llm = LLM(model="preset:x", devices=str(master.engine.device), engine=master.engine)
    llm.master = master
    llm.generate_timeout_s = 60.0
    return llm.generate([PROMPT], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0].outputs[0].token_ids


def main():
    gpu, port, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    master = make(gpu, seed=5)
    toks = tokens(master)
    srv = WeightServer(master)
    srv.serve(port, "127.0.0.1")
    torch.save({"tokens": toks}, out)
    deadline = time.time() + 150
    while not os.path.exists(out + ".stop") and time.time() < deadline:
        time.sleep(0.05)
    srv.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
