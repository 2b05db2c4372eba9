# python examples/generate_embedding.py --model=/path/to/Qwen3-Embedding-0.6B --devices=cuda:0 --runner pooling
"""Sentence embeddings (last-token pooling + L2 normalisation) through the Python API (the call sequence of the
reference's examples/generate_embedding.py)."""
from xllm import ArgumentParser, LLM, PoolingParams

parser = ArgumentParser()
llm = LLM(**vars(parser.parse_args()))

inputs = ["Hello, my name is", "The capital of France is"]
for output in llm.embed(inputs, pooling_params=PoolingParams()):
    vec = output.outputs.embedding
    print(f"Prompt: {output.prompt!r}, dim {len(vec)}, head {vec[:4]}")

llm.finish()
