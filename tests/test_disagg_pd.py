"""Prefill / decode disaggregation: a PREFILL engine and a DECODE engine in one process (in-process transport, tensor
copies for the KV blocks).  Tokens must equal those of a single colocated engine."""
import pytest
import torch

from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import preset
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.parallel.kv_transfer import LocalCopyTransfer
from xllm_wxh_b200.runtime.disagg_pd import DecodeCoordinator, InProcTransport, PrefillCoordinator
from xllm_wxh_b200.runtime.engine import LLMEngine
from xllm_wxh_b200.runtime.master import LLMMaster


def _opts(**kw):
    o = dict(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32")
    o.update(kw)
    return Options(**o)


def test_pd_pair_matches_colocated_engine():
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (20, 45, 7, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in
            LLM(model="preset:tiny-qwen2", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)]

    p_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="PREFILL"), model_args=args, model=model)
    d_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="DECODE"), model_args=args, model=model)
    p_master, d_master = LLMMaster(p_eng.opt, p_eng), LLMMaster(d_eng.opt, d_eng)
    tp, td = InProcTransport.pair()
    dec = DecodeCoordinator(d_master)
    dec.attach(td)
    pre = PrefillCoordinator(p_master, tp)
    p_eng.kv_transfer = LocalCopyTransfer(p_eng.worker.kv_caches, d_eng.worker.kv_caches)
    p_master.idle_wait = lambda: d_master.step()

    llm = LLM(model="preset:tiny-qwen2", devices="cpu", engine=p_eng)
    llm.master = p_master
    outs = llm.generate(prompts, sp)
    got = [o.outputs[0].token_ids for o in outs]
    assert got == want
    assert all(o.outputs[0].finish_reason == "length" for o in outs)
    assert p_eng.kv_transfer.bytes_moved > 0
    # the prefill instance never decoded: every request left it after one token
    assert p_eng.scheduler.stats()["generated_tokens"] == len(prompts)
    # all blocks returned on both sides
    assert d_eng.scheduler.block_manager(0).num_used_blocks == 0 and p_eng.scheduler.block_manager(0).num_used_blocks == 0


def test_pd_decode_refuses_when_out_of_blocks():
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    p_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="PREFILL"), model_args=args, model=model)
    d_eng = LLMEngine(_opts(enable_disagg_pd=True, instance_role="DECODE", num_kv_blocks=3), model_args=args, model=model)
    p_master, d_master = LLMMaster(p_eng.opt, p_eng), LLMMaster(d_eng.opt, d_eng)
    tp, td = InProcTransport.pair()
    DecodeCoordinator(d_master).attach(td)
    PrefillCoordinator(p_master, tp)
    llm = LLM(model="preset:tiny-qwen2", devices="cpu", engine=p_eng)
    llm.master = p_master
    outs = llm.generate([list(range(100))], SamplingParams(max_tokens=4))
    assert outs[0].status.code.name == "RESOURCE_EXHAUSTED"


@pytest.mark.gpu
@pytest.mark.multigpu
def test_pd_two_processes_nvlink_push(tmp_path):
    """PREFILL on GPU 0 and DECODE on GPU 1 as separate processes: TCP control plane, CUDA-IPC mapped decode cache,
    KV blocks written by the push kernel over NVLink."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    worker = os.path.join(here, "helpers", "pd_worker.py")
    port = 27811
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    co = str(tmp_path / "co.pt")
    logs = {k: open(str(tmp_path / f"{k}.log"), "w") for k in ("co", "d", "p")}

    def tail(k):
        logs[k].flush()
        return open(str(tmp_path / f"{k}.log")).read()[-3000:]
    r = subprocess.run([sys.executable, worker, "colocated", "0", str(port), co], env=env, timeout=180, stdout=logs["co"], stderr=subprocess.STDOUT)
    assert r.returncode == 0, tail("co")
    d_out, p_out = str(tmp_path / "d.pt"), str(tmp_path / "p.pt")
    d = subprocess.Popen([sys.executable, worker, "decode", "1", str(port), d_out], env=env, stdout=logs["d"], stderr=subprocess.STDOUT)
    try:
        try:
            p = subprocess.run([sys.executable, worker, "prefill", "0", str(port), p_out], env=env, timeout=180, stdout=logs["p"],
                               stderr=subprocess.STDOUT)
        except subprocess.TimeoutExpired:
            raise AssertionError("prefill instance timed out\n--- prefill\n" + tail("p") + "\n--- decode\n" + tail("d"))
        assert p.returncode == 0, "--- prefill\n" + tail("p") + "\n--- decode\n" + tail("d")
    finally:
        open(d_out + ".stop", "w").close()
        try:
            d.wait(timeout=60)
        except subprocess.TimeoutExpired:
            d.kill()
    want, got, dec = torch.load(co), torch.load(p_out), torch.load(d_out)
    assert got["status"] == 0 and dec["status"] == 0
    assert got["moved"] > 0
    assert got["tokens"] == want["tokens"]
    assert dec["generated"] > 0
