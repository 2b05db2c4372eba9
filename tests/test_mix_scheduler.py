"""Urgency-ordered single-queue ("mix") policy of the C++ scheduler, host only, with a hand-driven clock.

Behaviour under test is that of the reference's MixScheduler (mix_scheduler.cpp:41-114 ranking, :232-480 admission) and
its orderings (priority_comparator.cpp).
"""
import numpy as np
import pytest

from xllm_wxh_b200 import _core
from test_core_scheduler import answer, entries, make, run_to_completion, stop


def model(a0=0.0, a1=0.0, a2=0.0, b0=0.0, b1=0.0, b2=0.0):
    m = _core.StepTimeModel()
    m.a0, m.a1, m.a2, m.b0, m.b1, m.b2 = a0, a1, a2, b0, b1, b2
    return m


def test_step_time_model_max_chunk():
    m = model(a1=0.1, a2=0.0)                       # 0.1 ms per prefill token
    assert m.prefill_ms(100, 0) == pytest.approx(10.0)
    assert m.max_chunk(1000, 0, 25.0) == 250
    assert m.max_chunk(1000, 400, 25.0) == 650
    assert m.max_chunk(100, 0, 25.0) == 100        # everything fits
    assert m.max_chunk(100, 0, 0.0) == 0           # nothing fits: stays at the cached length
    q = model(a1=0.01, a2=1e-4)                     # attention term: later chunks cost more
    assert q.max_chunk(4000, 0, 50.0) > q.max_chunk(4000, 2000, 50.0) - 2000


def test_without_targets_it_is_first_come_first_served_and_complete():
    s = make(use_mix_scheduler=True, max_tokens_per_batch=64)
    ids = [s.add_request(list(range(i * 50, i * 50 + 40)), stop=stop(3)) for i in range(3)]
    bs = s.schedule()
    es = entries(bs[0])
    assert [e["req"] for e in es] == ids[:2] and [e["n"] for e in es] == [40, 24]      # strict order, chunked to the budget
    answer(s, bs)
    bs = s.schedule()
    es = entries(bs[0])
    # the first request decodes; the second finishes its prompt; the third starts with what is left
    assert {e["req"]: e["n"] for e in es} == {ids[0]: 1, ids[1]: 16, ids[2]: 40}
    answer(s, bs)
    outs, _ = run_to_completion(s)
    fin = {o.request_id: o.num_generated for o in outs if o.request_finished}
    assert fin == {i: 3 for i in ids}
    assert s.block_manager(0).num_used_blocks == 0


def test_tighter_first_token_target_goes_first():
    s = make(use_mix_scheduler=True, max_tokens_per_batch=64, max_seqs_per_batch=1)
    s.set_clock_override(100.0)
    relaxed = s.add_request([1] * 30, stop=stop(2), ttft_slo_ms=10_000)
    tight = s.add_request([2] * 30, stop=stop(2), ttft_slo_ms=200)
    none = s.add_request([3] * 30, stop=stop(2))
    assert s.mix_order() == [tight, relaxed, none]
    bs = s.schedule()
    assert [e["req"] for e in entries(bs[0])] == [tight]


def test_decode_deadline_accumulates_per_generated_token():
    s = make(use_mix_scheduler=True, max_seqs_per_batch=8)
    s.set_clock_override(10.0)
    a = s.add_request([1] * 8, stop=stop(50), tpot_slo_ms=100)
    b = s.add_request([2] * 8, stop=stop(50), tpot_slo_ms=20)
    answer(s, s.schedule())                                   # both prefilled at t = 10 s (first token at once)
    for step in range(1, 4):
        s.set_clock_override(10.0 + 0.03 * step)               # 30 ms per step: b (20 ms target) falls behind, a does not
        bs = s.schedule()
        assert [e["req"] for e in entries(bs[0])][0] == b      # the decode with the smaller slack is served first
        answer(s, bs)
    s.set_clock_override(-1.0)


def test_urgent_requests_are_served_by_density_and_starved_prefills_first():
    s = make(use_mix_scheduler=True, max_tokens_per_batch=4096, max_seqs_per_batch=1)
    s.set_step_time_model(model(a1=1.0))                       # 1 ms per prompt token
    s.set_clock_override(50.0)
    long_ = s.add_request([1] * 400, stop=stop(1), ttft_slo_ms=300)      # cost 400 ms
    short = s.add_request([2] * 50, stop=stop(1), ttft_slo_ms=300)       # cost 50 ms: 8x the value density
    heavy = s.add_request([3] * 100, stop=stop(1), ttft_slo_ms=300, ttft_weight=4)   # cost 100 ms, weight 4
    # queued work (550 ms) exceeds every slack (300 ms): all are urgent, served by weight / cost
    assert s.mix_order() == [heavy, short, long_]
    # 0.7 s later everybody is overdue by more than its target -> starved -> earliest deadline first; equal deadlines
    # fall back to arrival order
    s.set_clock_override(50.7)
    assert s.mix_order() == [long_, short, heavy]
    s2 = make(use_mix_scheduler=True, enable_starve_prevent=False, max_tokens_per_batch=4096)
    s2.set_step_time_model(model(a1=1.0))
    s2.set_clock_override(50.0)
    l2 = s2.add_request([1] * 400, stop=stop(1), ttft_slo_ms=300)
    h2 = s2.add_request([3] * 100, stop=stop(1), ttft_slo_ms=300, ttft_weight=4)
    s2.set_clock_override(50.7)
    assert s2.mix_order() == [h2, l2]                          # without the guard density keeps deciding


def test_aggressive_coeff_moves_the_urgency_boundary():
    def order(coeff):
        s = make(use_mix_scheduler=True, aggressive_coeff=coeff, max_tokens_per_batch=4096)
        s.set_step_time_model(model(a1=1.0))
        s.set_clock_override(5.0)
        a = s.add_request([1] * 300, stop=stop(1), ttft_slo_ms=1000)     # slack 1000 ms, cost 300
        b = s.add_request([2] * 100, stop=stop(1), ttft_slo_ms=2000)     # slack 2000 ms, cost 100
        return s.mix_order(), a, b
    o, a, b = order(1.0)          # queued work 400 ms < both slacks: nobody urgent -> earliest deadline
    assert o == [a, b]
    o, a, b = order(6.0)          # 2400 ms > both slacks: both urgent -> the denser (cheaper) one first
    assert o == [b, a]


def test_latency_budget_bounds_the_prefill_chunk_next_to_decodes():
    s = make(num_blocks=512, use_mix_scheduler=True, enable_latency_aware_schedule=True, max_global_tpot_ms=100.0,
             max_tokens_per_batch=4096, max_seqs_per_batch=64)
    s.set_step_time_model(model(a1=0.125, b0=5.0, b1=0.5))      # 1/8 ms / prompt token, 0.5 ms / decode row, 5 ms fixed
    s.set_clock_override(20.0)
    dec = [s.add_request([i] * 8, stop=stop(64)) for i in range(10)]
    answer(s, s.schedule())
    s.set_clock_override(20.0078125)
    big = s.add_request([99] * 3000, stop=stop(1))
    # the decodes have produced one token 7.8125 ms ago: 100 ms target - 7.8125 ms of slack bounds the step
    assert s.mix_latency_budget() == pytest.approx(92.1875)
    bs = s.schedule()
    es = entries(bs[0])
    chunk = [e for e in es if e["req"] == big]
    assert len([e for e in es if e["req"] in dec]) == 10 and len(chunk) == 1
    # 92.1875 ms - 5 ms fixed - 10 x 0.5 ms of decodes = 82.1875 ms -> 657 prompt tokens
    assert chunk[0]["n"] == 657
    answer(s, bs)
    # 0.2 s later the decodes are (one token's worth) late: late requests no longer shrink the budget, which falls
    # back to 0.65 x the tightest per-token target
    s.set_clock_override(20.25)
    assert s.mix_latency_budget() == pytest.approx(65.0)
    bs = s.schedule()
    chunk = [e for e in entries(bs[0]) if e["req"] == big]
    assert chunk[0]["kv"] == 657 and chunk[0]["n"] == 440
    # without the latency bound the whole prompt would have gone into one step
    s2 = make(num_blocks=512, use_mix_scheduler=True, max_tokens_per_batch=4096)
    r = s2.add_request([99] * 3000, stop=stop(1))
    assert entries(s2.schedule()[0])[0]["n"] == 3000


def test_sliver_chunks_are_postponed():
    s = make(num_blocks=512, use_mix_scheduler=True, enable_latency_aware_schedule=True, max_global_tpot_ms=20.0,
             max_tokens_per_batch=4096, max_seqs_per_batch=64)
    s.set_step_time_model(model(a1=0.1, b1=1.0))
    s.set_clock_override(1.0)
    dec = [s.add_request([i] * 8, stop=stop(64)) for i in range(10)]
    answer(s, s.schedule())
    big = s.add_request([99] * 3000, stop=stop(1))
    s.set_clock_override(1.0078125)
    bs = s.schedule()                    # budget 13 ms, decodes use 10 ms, 3 ms = 30 tokens < 50: not worth a chunk
    assert big not in [e["req"] for e in entries(bs[0])]
    assert len(entries(bs[0])) == 10


def test_blocks_run_out_least_important_request_is_recomputed():
    s = make(use_mix_scheduler=True, num_blocks=9, block_size=4, max_tokens_per_batch=64,
             prefill_scheduling_memory_usage_threshold=1.0)
    s.set_clock_override(3.0)
    relaxed = s.add_request(list(range(12)), stop=stop(12), ttft_slo_ms=60_000, tpot_slo_ms=60_000)
    tight = s.add_request(list(range(50, 62)), stop=stop(12), ttft_slo_ms=100, tpot_slo_ms=50)
    outs, _ = run_to_completion(s)
    assert s.stats()["num_preemptions"] >= 1
    fin = {o.request_id: o.num_generated for o in outs if o.finished}
    assert fin == {relaxed: 12, tight: 12}
    assert s.block_manager(0).num_used_blocks == 0


def test_request_that_can_never_fit_is_failed():
    s = make(use_mix_scheduler=True, num_blocks=5, block_size=4, max_tokens_per_batch=256)
    rid = s.add_request(list(range(64)), stop=stop(2))
    s.schedule()
    outs = s.take_outputs()
    assert [(o.request_id, o.finish_reason) for o in outs] == [(rid, 4)]


@pytest.mark.parametrize("strategy", ["priority", "deadline", "sjf", "density", "decode_density", "decode_deadline",
                                      "urgency_priority", "decode_urgency_density", "urgency_density"])
def test_every_ordering_serves_all_requests(strategy):
    s = make(use_mix_scheduler=True, priority_strategy=strategy, max_tokens_per_batch=48, max_seqs_per_batch=3)
    s.set_step_time_model(model(a1=0.2, b1=0.3, b2=0.001, a0=1.0))
    rng = np.random.default_rng(0)
    ids = []
    for i in range(8):
        ids.append(s.add_request(rng.integers(0, 100, int(rng.integers(5, 70))).tolist(), stop=stop(int(rng.integers(1, 6))),
                                 priority=int(rng.integers(1, 4)), ttft_slo_ms=float(rng.choice([0, 50, 500])),
                                 tpot_slo_ms=float(rng.choice([0, 20, 200])), ttft_weight=int(rng.integers(1, 4))))
    outs, steps = run_to_completion(s)
    assert {o.request_id for o in outs if o.request_finished} == set(ids)
    assert s.block_manager(0).num_used_blocks == 0


def test_sjf_and_priority_orderings():
    s = make(use_mix_scheduler=True, priority_strategy="sjf")
    s.set_step_time_model(model(a1=1.0))
    a = s.add_request([1] * 90, stop=stop(1))
    b = s.add_request([2] * 10, stop=stop(1))
    c = s.add_request([3] * 40, stop=stop(1))
    assert s.mix_order() == [b, c, a]
    s = make(use_mix_scheduler=True, priority_strategy="priority")
    a = s.add_request([1] * 9, stop=stop(1), priority=2)
    b = s.add_request([2] * 9, stop=stop(1), priority=1)
    assert s.mix_order() == [b, a]


def test_speculative_steps_are_all_prefill_or_all_decode():
    """With speculative decoding every sampling row of a decode step owns k + 1 rows, so the mix policy must not put a
    prefill chunk (no draft rows) beside decode entries (k draft rows): a step is one kind or the other."""
    k = 2
    s = make(use_mix_scheduler=True, enable_chunked_prefill=True, prefill_only_batches=True, num_speculative_tokens=k,
             max_tokens_per_batch=64, max_seqs_per_batch=8, num_blocks=128)
    first = s.add_request(list(range(40)), stop=stop(6))
    answer(s, s.schedule())                                   # the first request is prefilled and now decodes
    late = [s.add_request(list(range(100 + 50 * i, 140 + 50 * i)), stop=stop(6)) for i in range(2)]
    kinds = []
    for _ in range(200):
        if not s.has_unfinished():
            break
        bs = s.schedule()
        es = entries(bs[0])
        if es:
            decode = [e["spec"] == k and e["n"] == k + 1 for e in es]
            prefill = [e["spec"] == 0 for e in es]
            assert all(decode) or all(prefill), es
            kinds.append("d" if all(decode) else "p")
        for b in bs:                                          # the fake engine accepts one token per row
            if b.empty:
                continue
            rows = [e for e in b.entries() if e[4]]
            toks = np.full((len(rows), k + 1), -1, dtype=np.int32)
            toks[:, 0] = 7
            s.process_output(b.id, toks)
        s.take_outputs()
    assert not s.has_unfinished()
    assert "d" in kinds and "p" in kinds
