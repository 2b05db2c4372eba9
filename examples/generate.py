# python examples/generate.py --model=/path/to/Qwen3-8B --devices=cuda:0
# python examples/generate.py --model=/path/to/Qwen3-8B --devices=cuda:0,cuda:1      (tensor parallel over two GPUs)
# python examples/generate.py --model=preset:tiny-qwen2 --devices=cpu                  (random weights; prompts are token ids)
"""Offline generation through the Python API (same call sequence as the reference's examples/generate.py)."""
from xllm import ArgumentParser, LLM, SamplingParams

parser = ArgumentParser()
args = parser.parse_args()
llm = LLM(**vars(args))

sampling_params = SamplingParams(temperature=0.8, top_p=0.95, max_tokens=10)

if str(args.model).startswith("preset:"):       # no tokenizer files: the "text" is a list of token ids
    prompts = ["1 2 3 4 5", "100 200 300", "7 7 7 7", "42"]
else:
    prompts = ["Hello, my name is", "The president of the United States is", "The capital of France is", "The future of AI is"]

outputs = llm.generate(prompts, sampling_params=sampling_params)
for output in outputs:
    print(f"Prompt: {output.prompt!r}, Generated text: {output.outputs[0].text!r}")

llm.finish()
