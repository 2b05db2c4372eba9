"""The command-line programs together, as a user starts them (CPU, preset model): `xllm-kv-store`, `xllm-service` and two
`xllm` instances that register with the service, share the block store and serve their weights for remote wake-up.  The
reference's counterpart is the `xllm` binary with --enable_service_routing / --enable_kvcache_store / --enable_xtensor
(xllm/xllm.cpp) next to the xllm-service processes."""
import os
import socket
import subprocess
import sys
import time

import pytest
import requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _wait_http(url, timeout=90.0, proc=None):
    deadline = time.time() + timeout
    while time.time() < deadline:
        if proc is not None and proc.poll() is not None:
            raise AssertionError(f"process exited with {proc.returncode}")
        try:
            if requests.get(url, timeout=1).status_code == 200:
                return
        except requests.RequestException:
            pass
        time.sleep(0.2)
    raise AssertionError(f"{url} did not come up")


def _wait_port(port, timeout=30.0):
    deadline = time.time() + timeout
    while time.time() < deadline:
        try:
            socket.create_connection(("127.0.0.1", port), timeout=0.5).close()
            return
        except OSError:
            time.sleep(0.1)
    raise AssertionError(f"port {port} did not open")


@pytest.fixture
def procs():
    started = []
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))

    def start(*argv):
        p = subprocess.Popen([sys.executable, "-m", *argv], env=env, cwd=ROOT, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        started.append(p)
        return p
    yield start
    for p in started:
        if p.poll() is None:
            p.terminate()
    for p in started:
        try:
            p.wait(timeout=15)
        except subprocess.TimeoutExpired:
            p.kill()


def test_store_service_and_two_instances_from_the_command_line(procs):
    store_port, svc_port = _free_port(), _free_port()
    procs("xllm_wxh_b200.service.kv_store", "--host", "127.0.0.1", "--port", str(store_port), "--capacity_gb", "0.25")
    procs("xllm_wxh_b200.service.router", "--host", "127.0.0.1", "--port", str(svc_port), "--load_balance_policy", "RR")
    _wait_port(store_port)
    _wait_http(f"http://127.0.0.1:{svc_port}/health")
    inst = []
    for i in range(2):
        port, wport = _free_port(), _free_port()
        p = procs("xllm_wxh_b200.cli", "--model", "preset:tiny-qwen2", "--devices", "cpu", "--host", "127.0.0.1", "--port", str(port),
                  "--model_id", "tiny", "--block_size", "16", "--num_kv_blocks", "64", "--host_blocks_factor", "2",
                  "--enable_kvcache_store", "--store_master_server_address", f"127.0.0.1:{store_port}",
                  "--enable_service_routing", "--etcd_addr", f"127.0.0.1:{svc_port}", "--instance_name", f"i{i}",
                  "--heart_beat_interval", "0.1", "--enable_xtensor", "--transfer_listen_port", str(wport))
        inst.append((p, port, wport))
    for p, port, _ in inst:
        _wait_http(f"http://127.0.0.1:{port}/health", proc=p)
    svc = f"http://127.0.0.1:{svc_port}"
    deadline = time.time() + 20
    while time.time() < deadline:
        names = sorted(i["name"] for i in requests.get(svc + "/xservice/instances").json()["instances"])
        if names == ["i0", "i1"]:
            break
        time.sleep(0.2)
    assert names == ["i0", "i1"]
    prompt = list(range(10, 110))                                           # 6 full blocks
    body = {"model": "tiny", "prompt": prompt, "max_tokens": 5, "temperature": 0}
    # instance 0 serves the prompt and writes its blocks through to the store
    a = requests.post(f"http://127.0.0.1:{inst[0][1]}/v1/completions", json=body).json()
    assert a["usage"]["prompt_tokens"] == 100 and a["usage"]["prompt_tokens_details"]["cached_tokens"] == 0
    from xllm_wxh_b200.service.kv_store import KvStoreClient
    c = KvStoreClient(f"127.0.0.1:{store_port}")
    deadline = time.time() + 10
    while time.time() < deadline and c.stats()["blocks"] < 6:
        time.sleep(0.1)
    assert c.stats()["blocks"] >= 6
    # instance 1 has never seen the prompt: its blocks come out of the store
    b = requests.post(f"http://127.0.0.1:{inst[1][1]}/v1/completions", json=body).json()
    assert b["choices"][0]["text"] == a["choices"][0]["text"]
    assert b["usage"]["prompt_tokens_details"]["cached_tokens"] == 96
    # through the service: both instances take requests in turn
    for _ in range(2):
        r = requests.post(svc + "/v1/completions", json=body)
        assert r.status_code == 200 and r.json()["choices"][0]["text"] == a["choices"][0]["text"]
    # instance 1 sleeps deeply and wakes up from instance 0's weight service
    u1 = f"http://127.0.0.1:{inst[1][1]}"
    assert requests.post(u1 + "/sleep", json={"master_status": 2}).status_code == 200
    assert requests.post(u1 + "/v1/completions", json=body).status_code == 503
    r = requests.post(u1 + "/wakeup", json={"remote_addrs": [f"127.0.0.1:{inst[0][2]}"]})
    assert r.status_code == 200 and r.json()["weights_pulled_bytes"] > 0
    assert requests.post(u1 + "/v1/completions", json=body).json()["choices"][0]["text"] == a["choices"][0]["text"]
