"""The example scripts run as a user would run them, on the tiny random-initialised preset (CPU).

With `XLLM_REFERENCE_EXAMPLES` naming the `examples` directory of an xLLM source tree, that tree's own
`generate_beam_search.py` and `generate_embedding.py` are executed unmodified against this package's `xllm` module: they
rely on `{"prompt": ...}` inputs, `output.sequences[i].text` and `output.outputs.embedding`."""
import os
import runpy
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ARGS = ["--model", "preset:tiny-qwen2", "--devices", "cpu", "--block_size", "16", "--max_tokens_per_batch", "512"]


def _run(path, extra, capsys, monkeypatch):
    monkeypatch.setattr(sys, "argv", [path] + ARGS + extra)
    monkeypatch.syspath_prepend(ROOT)
    runpy.run_path(path, run_name="__main__")
    return capsys.readouterr().out


def _dirs():
    out = [os.path.join(ROOT, "examples")]
    ref = os.environ.get("XLLM_REFERENCE_EXAMPLES")
    if ref and os.path.isdir(ref):
        out.append(ref)
    return out


@pytest.mark.parametrize("where", _dirs())
def test_beam_search_example(where, capsys, monkeypatch):
    out = _run(os.path.join(where, "generate_beam_search.py"), [], capsys, monkeypatch)
    assert out.count("\n") >= 2 and ("Generated text" in out or "best beam" in out)


@pytest.mark.parametrize("where", _dirs())
def test_embedding_example(where, capsys, monkeypatch):
    out = _run(os.path.join(where, "generate_embedding.py"), ["--runner", "pooling"], capsys, monkeypatch)
    assert out.count("\n") >= 2 and ("embedding" in out or "dim 256" in out)


def test_generate_example(capsys, monkeypatch):
    out = _run(os.path.join(ROOT, "examples", "generate.py"), [], capsys, monkeypatch)
    assert "Prompt" in out or "Generated" in out
