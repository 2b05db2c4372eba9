"""Rank program of the failure-detection test (gloo, CPU): rank 1 leaves between two steps; rank 0 must notice on the
step channel within the configured time, fail the requests in flight and report the instance unhealthy.
    argv: <out.pt>
"""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from xllm_wxh_b200 import _core  # noqa: E402
from xllm_wxh_b200.config import Options  # noqa: E402
from xllm_wxh_b200.models.args import ModelArgs  # noqa: E402
from xllm_wxh_b200.runtime import engine as E  # noqa: E402
from xllm_wxh_b200.runtime.engine import LLMEngine  # noqa: E402


def main():
    out = sys.argv[1]
    rank = int(os.environ.get("RANK", "0"))
    args = ModelArgs(model_type="qwen3", dtype="float32", vocab_size=512, hidden_size=128, n_layers=2, n_heads=4, n_kv_heads=2,
                     head_dim=32, intermediate_size=256, qk_norm=True, max_position_embeddings=512)
    opts = Options(model="preset:test", devices="cpu", block_size=16, num_kv_blocks=64, max_tokens_per_batch=256, max_seqs_per_batch=8,
                   communication_backend="nccl", enable_graph=False, dtype="float32", rpc_channel_timeout_ms=1500)
    eng = LLMEngine(opts, model_args=args)
    if rank != 0:
        # serve exactly two steps, then leave between steps (no collective in flight)
        served = 0
        reader = eng.rank - 1
        msg = eng._ensure_msg(eng._max_message_words())
        while served < 2:
            rc = eng._chan.read_into(reader, msg.data_ptr(), msg.numel() * 4, 60.0)
            assert rc == 0
            ctrl = msg[:E.CTRL_WORDS].numpy()
            if int(ctrl[0]) == E.CMD_STEP:
                eng._run_local(msg, bool(ctrl[1]), bool(ctrl[2]))
                served += 1
        os._exit(0)
    st = _core.StopCriteria()
    st.max_tokens, st.ignore_eos = 50, True
    eng.add_request(list(range(1, 20)), _core.SamplingParams(), st)
    steps_ok, err, t_detect = 0, "", 0.0
    try:
        for _ in range(10):
            t0 = time.perf_counter()
            eng.step()
            steps_ok += 1
    except RuntimeError as e:
        err, t_detect = str(e), time.perf_counter() - t0
    torch.save({"steps_ok": steps_ok, "error": err, "detect_s": t_detect}, out)
    os._exit(0)


if __name__ == "__main__":
    main()
