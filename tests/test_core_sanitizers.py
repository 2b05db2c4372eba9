"""The host-only C++ tests again, against an AddressSanitizer + UBSan build of the core (no sanitizer exists for the
device side here; the host runtime is where the pointer-heavy code lives: scheduler queues, block tables, the packed
step message, the tokenizer, the shared-memory channel)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST_TESTS = ["tests/test_core_scheduler.py", "tests/test_mix_scheduler.py", "tests/test_core_blocks_batch.py",
              "tests/test_core_misc.py", "tests/test_host_kv_tier.py", "tests/test_kv_store.py"]


def test_host_tests_pass_under_asan_and_ubsan():
    from xllm_wxh_b200 import build_ext
    so = build_ext.build_core_sanitized()
    rt = build_ext.sanitizer_runtime()
    if not rt or not all(os.path.exists(x) for x in rt.split()):
        pytest.skip("libasan not found")
    env = dict(os.environ, XLLM_CORE_SO=so, LD_PRELOAD=rt, PYTHONPATH=ROOT,
               # the interpreter and torch leak by design at exit; container overflow checks need an instrumented libstdc++
               ASAN_OPTIONS="detect_leaks=0:detect_container_overflow=0:abort_on_error=1:halt_on_error=1",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    p = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "not gpu", "-p", "no:cacheprovider"] + HOST_TESTS,
                       cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1500)
    tail = p.stdout[-4000:]
    assert p.returncode == 0, tail
    assert "AddressSanitizer" not in p.stdout and "runtime error" not in p.stdout, tail
