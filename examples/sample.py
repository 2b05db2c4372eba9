# python examples/sample.py --model=/path/to/Qwen3-8B --devices=cuda:0
"""Next-token distributions at the positions of a selector token (reference: examples/sample.py, `/v1/sample`)."""
from xllm import ArgumentParser, LLM, RequestParams

parser = ArgumentParser()
args = parser.parse_args()
llm = LLM(**vars(args))

if str(args.model).startswith("preset:"):
    selector = "7"                               # token id 7 of the id "tokenizer" of random-weight presets
    prompts = ["1 2 7 3 4 7", "5 7"]
else:
    selector = "<|fim_middle|>"                  # must encode to exactly one token of the model's tokenizer
    prompts = [f"candidate_a={selector}, candidate_b={selector}", f"user_feature={selector}"]

request_params_list = []
for _ in prompts:
    rp = RequestParams()
    rp.temperature, rp.top_p = 0.0, 1.0
    request_params_list.append(rp)

outputs = llm.sample(prompts, selector=selector, request_params=request_params_list, logprobs=5, wait_schedule_done=True)
for i, output in enumerate(outputs):
    print(f"[prompt-{i}] {output.prompt!r}")
    for s in output.outputs:
        print(f"  sample_id={s.index}, token={s.text!r}, token_ids={s.token_ids}, finish_reason={s.finish_reason}")

llm.finish()
