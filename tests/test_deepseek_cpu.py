"""DeepSeek-V3-style model (MLA absorbed form, sigmoid group-limited routing, shared expert, YaRN) on CPU in fp32,
through the engine, against the plain non-absorbed oracle."""
import pytest
import torch

from oracle import deepseek_greedy
from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import ModelArgs
from xllm_wxh_b200.models.deepseek_impl import DeepseekForCausalLM
from xllm_wxh_b200.ops import reference as ref
from xllm_wxh_b200.runtime.engine import LLMEngine


def tiny_ds(**kw):
    base = dict(model_type="deepseek_v3", dtype="float32", vocab_size=512, hidden_size=128, n_layers=3, n_heads=4, n_kv_heads=4,
                head_dim=48, intermediate_size=256, n_routed_experts=16, num_experts_per_tok=4, moe_intermediate_size=64,
                n_shared_experts=1, first_k_dense_replace=1, scoring_func="sigmoid", topk_method="noaux_tc", n_group=4, topk_group=2,
                routed_scaling_factor=2.5, q_lora_rank=64, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                rope_theta=1e4, rope_scaling_type="yarn", rope_scaling_factor=4.0, rope_original_max_position=64, rope_mscale=1.0,
                rope_mscale_all_dim=1.0, max_position_embeddings=512)
    base.update(kw)
    return ModelArgs(**base)


def _yarn(args):
    inv = ref.yarn_inv_freq(args.qk_rope_head_dim, args.rope_theta, args.rope_scaling_factor, args.rope_original_max_position,
                            args.rope_beta_fast, args.rope_beta_slow)
    m_all = ref.yarn_mscale(args.rope_scaling_factor, args.rope_mscale_all_dim)
    mscale = ref.yarn_mscale(args.rope_scaling_factor, args.rope_mscale) / m_all
    return inv, mscale, (args.qk_nope_head_dim + args.qk_rope_head_dim) ** -0.5 * m_all * m_all


@pytest.mark.parametrize("q_lora", [64, 0])
def test_deepseek_greedy_matches_oracle(q_lora):
    args = tiny_ds(q_lora_rank=q_lora)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    sd = {k: v.float() for k, v in model.state_dict().items()}
    inv, mscale, sscale = _yarn(args)
    eng = LLMEngine(Options(model="preset:x", devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32",
                            max_tokens_per_chunk_for_prefill=24), model_args=args, model=model)
    llm = LLM(model="preset:x", devices="cpu", engine=eng)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (20, 37, 5)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == deepseek_greedy(sd, args, p, 10, inv, mscale, sscale)


def test_deepseek_checkpoint_roundtrip_fp8_block_scaled(tmp_path):
    """Write a bf16 checkpoint and an fp8 128x128 block-scaled one (HF `weight_scale_inv` layout); load both."""
    import json
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader, save_safetensors
    args = tiny_ds(hidden_size=256, q_lora_rank=128, kv_lora_rank=128, moe_intermediate_size=128, intermediate_size=256,
                   qk_nope_head_dim=32, v_head_dim=32, n_heads=4)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=1, std=0.05)
    sd = model.state_dict()
    d = tmp_path / "bf16"
    d.mkdir()
    save_safetensors(str(d / "model.safetensors"), sd)
    loaded = DeepseekForCausalLM(args, device="cpu").load_weights(CheckpointReader(str(d)))
    for (k, a), (_, b) in zip(sorted(sd.items()), sorted(loaded.state_dict().items())):
        assert torch.equal(a, b), k
    # fp8 variant of the 2-D projection weights
    q = tmp_path / "fp8"
    q.mkdir()
    sdq = {}
    for k, v in sd.items():
        if v.dim() == 2 and "proj" in k and v.shape[0] % 128 == 0 and v.shape[1] % 128 == 0:
            w8, s = ref.quant_weight_128x128(v)
            sdq[k], sdq[k.replace(".weight", ".weight_scale_inv")] = w8, s
        else:
            sdq[k] = v
    save_safetensors(str(q / "model.safetensors"), sdq)
    deq = DeepseekForCausalLM(args, device="cpu").load_weights(CheckpointReader(str(q)))
    a, b = sd["model.layers.0.mlp.down_proj.weight"], deq.state_dict()["model.layers.0.mlp.down_proj.weight"]
    assert (a - b).abs().max() < 0.07 * a.abs().max()
