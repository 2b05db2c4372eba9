# python examples/generate_beam_search.py --model=/path/to/Qwen3-8B --devices=cuda:0
"""Beam search through the Python API (reference: examples/generate_beam_search.py)."""
from xllm import ArgumentParser, BeamSearchParams, LLM

parser = ArgumentParser()
args = parser.parse_args()
llm = LLM(**vars(args))

params = BeamSearchParams(beam_width=4, max_tokens=20)
prompts = ["1 2 3 4 5"] if str(args.model).startswith("preset:") else ["The capital of France is"]
for output in llm.beam_search(prompts, params):
    for seq in output.outputs:
        print(f"Prompt: {output.prompt!r}, beam {seq.index}: {seq.text!r} (cumulative logprob {seq.cumulative_logprob:.3f})")

llm.finish()
