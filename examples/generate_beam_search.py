# python examples/generate_beam_search.py --model=/path/to/Qwen3-8B --devices=cuda:0
"""Beam search through the Python API (the call sequence of the reference's examples/generate_beam_search.py)."""
from xllm import ArgumentParser, BeamSearchParams, LLM

parser = ArgumentParser()
llm = LLM(**vars(parser.parse_args()))

params = BeamSearchParams(beam_width=2, max_tokens=20)
outputs = llm.beam_search([{"prompt": "Hello, my name is "}, {"prompt": "The capital of France is "}], params=params)
for output in outputs:
    best = output.sequences[0]
    print(f"Prompt: {output.prompt!r}, best beam: {best.text!r} (cumulative logprob {best.cumulative_logprob:.3f})")

llm.finish()
