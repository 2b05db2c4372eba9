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
