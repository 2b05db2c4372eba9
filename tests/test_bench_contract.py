"""The parts of `bench.py`'s contract that need no GPU: the reference arm's one line, and refusals that name their reason."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    e = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        e.pop(k, None)
    e.update(env or {})
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                       text=True, timeout=120)
    return p.returncode, p.stdout.strip().splitlines()


def test_reference_arm_prints_one_unavailable_line():
    rc, lines = _run("--impl", "reference", "--gpus", "4", "--steps", "2", "--warmup", "1")
    assert rc == 0 and len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unavailable"].startswith("refused by a safety check") and d["n_gpus"] == 4
    # launched as several ranks, only rank 0 speaks
    rc, lines = _run("--impl", "reference", "--gpus", "4", env={"RANK": "2", "WORLD_SIZE": "4"})
    assert rc == 0 and lines == []


def test_pd_mode_names_what_it_supports():
    rc, lines = _run("--pd", "4+4")
    assert rc == 0 and "1+1" in json.loads(lines[-1])["unavailable"]


def test_host_overhead_benchmark_runs():
    """The CPU-only benchmark of the host path (own process: it replaces the attention op by a copy)."""
    import json
    import subprocess
    import sys
    out = subprocess.run([sys.executable, "-m", "xllm_wxh_b200.runtime.bench_host_overhead", "--concurrency", "8", "--tokens", "4", "--watchdog", "200"],
                         capture_output=True, text=True, timeout=300, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.returncode == 0, out.stderr[-2000:]
    row = json.loads(out.stdout.strip().splitlines()[-1])
    assert row["offline_generate"]["steps"] >= 4 and row["offline_generate"]["ms_per_step"] > 0
    assert row["http_streaming"]["chunks"] == 8 * 4 and row["http_streaming"]["streamed_tokens_per_second"] > 0
