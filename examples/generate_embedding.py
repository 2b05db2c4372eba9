# python examples/generate_embedding.py --model=/path/to/Qwen3-Embedding-0.6B --devices=cuda:0
"""Sentence embeddings (last-token pooling + L2 normalisation) through the Python API
(reference: examples/generate_embedding.py)."""
from xllm import ArgumentParser, Embedding

parser = ArgumentParser()
args = parser.parse_args()
emb = Embedding(**vars(args))

inputs = ["1 2 3 4 5", "9 8 7"] if str(args.model).startswith("preset:") else ["Hello, my name is", "The capital of France is"]
for output in emb.embedding(inputs):
    vec = output.outputs[0].embeddings
    print(f"Prompt: {output.prompt!r}, dim {len(vec)}, head {vec[:4]}")

emb.finish()
