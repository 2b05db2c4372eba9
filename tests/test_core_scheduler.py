"""Host-only tests of the C++ scheduler (no model, no device): a fake engine answers every step with made-up tokens.

Same tier as the reference's continuous_scheduler_test.cpp / chunked_prefill_scheduler_test.cpp (a FakeEngine with a
real block manager; the tests inspect the batches and the preemptions), plus the urgency-ordered mix policy.
"""
import numpy as np
import pytest

from xllm_wxh_b200 import _core

DECODE, PREFILL, CHUNKED, MIXED = 2, 0, 1, 3


def make(num_blocks=64, block_size=16, prefix=False, **kw):
    so = _core.SchedulerOptions()
    so.max_tokens_per_batch = 256
    so.max_seqs_per_batch = 16
    for k, v in kw.items():
        assert hasattr(so, k), k
        setattr(so, k, v)
    return _core.Scheduler(so, num_blocks, block_size, prefix)


def stop(max_tokens, eos=-1, ignore_eos=True):
    st = _core.StopCriteria()
    st.max_tokens, st.eos_token_id, st.ignore_eos = max_tokens, eos, ignore_eos
    return st


def answer(s, batches, token=7):
    """The fake engine: every sampling row of every batch gets `token` (or token(request_id))."""
    for b in batches:
        if b.empty:
            continue
        rows = [e for e in b.entries() if e[4]]
        toks = np.array([[token(e[1]) if callable(token) else token] for e in rows], dtype=np.int32).reshape(len(rows), 1)
        s.process_output(b.id, toks)


def run_to_completion(s, token=7, limit=10000):
    outs, steps = [], 0
    while s.has_unfinished() and steps < limit:
        bs = s.schedule()
        answer(s, bs, token)
        outs += s.take_outputs()
        steps += 1
    assert steps < limit
    return outs, steps


def entries(b):
    return [dict(seq=e[0], req=e[1], n=e[2], spec=e[3], sample=e[4], kv=e[5], slot=e[6], idx=e[7]) for e in b.entries()]


# ------------------------------------------------------------------ continuous (prefill-first) policy
def test_prefill_first_then_decode():
    s = make(enable_chunked_prefill=False)
    a = s.add_request(list(range(40)), stop=stop(3))
    b = s.add_request(list(range(100, 130)), stop=stop(3))
    bs = s.schedule()
    assert bs[0].forward_type == PREFILL and bs[0].num_tokens == 70 and bs[0].num_prefill_seqs == 2
    assert [e["n"] for e in entries(bs[0])] == [40, 30] and all(e["sample"] for e in entries(bs[0]))
    answer(s, bs)
    bs = s.schedule()
    assert bs[0].forward_type == DECODE and bs[0].num_tokens == 2 and bs[0].num_decode_seqs == 2
    assert [e["kv"] for e in entries(bs[0])] == [40, 30]
    # a request that arrives while others decode is prefilled alone first (prefill priority)
    answer(s, bs)
    c = s.add_request(list(range(200, 210)), stop=stop(2))
    bs = s.schedule()
    assert bs[0].forward_type == PREFILL and [e["req"] for e in entries(bs[0])] == [c]
    answer(s, bs)
    outs, _ = run_to_completion(s)
    done = {o.request_id: o for o in outs if o.request_finished}
    assert set(done) == {a, b, c} and all(o.finish_reason == 2 for o in done.values())       # LENGTH


def test_prompt_longer_than_budget_without_chunking_is_rejected():
    s = make(enable_chunked_prefill=False, max_tokens_per_batch=64)
    rid = s.add_request(list(range(100)), stop=stop(4))
    bs = s.schedule()
    assert bs[0].empty
    outs = s.take_outputs()
    assert len(outs) == 1 and outs[0].request_id == rid and outs[0].finished and outs[0].finish_reason == 4
    assert not s.has_unfinished() or s.schedule()[0].empty


def test_token_and_sequence_budgets_bound_a_step():
    s = make(enable_chunked_prefill=False, max_tokens_per_batch=64, max_seqs_per_batch=3)
    for i in range(5):
        s.add_request(list(range(i * 100, i * 100 + 20)), stop=stop(2))
    bs = s.schedule()
    assert bs[0].num_prefill_seqs == 3 and bs[0].num_tokens == 60          # 4 x 20 > 64 and at most 3 sequences
    answer(s, bs)
    bs = s.schedule()
    assert bs[0].forward_type == PREFILL and bs[0].num_prefill_seqs == 2   # the rest before any decode


# ------------------------------------------------------------------ chunked prefill
def test_chunked_prefill_splits_long_prompt_and_mixes_with_decode():
    s = make(max_tokens_per_batch=64)
    a = s.add_request(list(range(30)), stop=stop(8))
    bs = s.schedule()
    assert bs[0].forward_type == PREFILL
    answer(s, bs)
    b = s.add_request(list(range(1000, 1150)), stop=stop(2))
    seen = []
    for _ in range(3):
        bs = s.schedule()
        es = entries(bs[0])
        assert bs[0].forward_type == MIXED and es[0]["req"] == a and es[0]["n"] == 1       # decode rows come first
        assert es[1]["req"] == b and es[1]["kv"] == sum(seen)
        seen.append(es[1]["n"])
        # only the last chunk samples
        assert es[1]["sample"] == (sum(seen) == 150)
        assert bs[0].num_sample == (2 if es[1]["sample"] else 1)
        answer(s, bs)
    assert seen == [63, 63, 24]


def test_chunk_size_cap():
    s = make(max_tokens_per_batch=256, max_tokens_per_chunk_for_prefill=32)
    s.add_request(list(range(100)), stop=stop(1))
    sizes = []
    while s.has_unfinished():
        bs = s.schedule()
        if bs[0].empty:
            break
        sizes.append(bs[0].num_tokens)
        answer(s, bs)
        s.take_outputs()
    assert sizes == [32, 32, 32, 4]


def test_stop_on_eos_and_stop_sequences():
    s = make()
    st = stop(10, eos=9, ignore_eos=False)
    a = s.add_request([1, 2, 3], stop=st)
    st2 = stop(10)
    st2.stop_sequences = [[5, 5, 5]]
    b = s.add_request([4, 5, 6], stop=st2)
    outs, _ = run_to_completion(s, token=lambda rid: 9 if rid == a else 5)
    fin = {o.request_id: o for o in outs if o.finished}
    assert fin[a].finish_reason == 1 and fin[a].num_generated == 1
    assert fin[b].finish_reason == 1 and fin[b].num_generated == 3


def test_cancel_frees_blocks():
    s = make()
    a = s.add_request(list(range(50)), stop=stop(100))
    answer(s, s.schedule())
    bm = s.block_manager(0)
    assert bm.num_used_blocks > 0
    s.cancel(a)
    s.schedule()
    outs = s.take_outputs()
    assert any(o.request_id == a and o.finished and o.finish_reason == 3 for o in outs)
    assert bm.num_used_blocks == 0 and not s.has_unfinished()


# ------------------------------------------------------------------ preemption
def test_decode_preempts_latest_request_when_blocks_run_out():
    # 6 usable blocks of 4 tokens; two requests of 8 prompt tokens grow until one has to yield
    s = make(num_blocks=7, block_size=4, max_tokens_per_batch=64, prefill_scheduling_memory_usage_threshold=1.0)
    a = s.add_request(list(range(8)), stop=stop(12))
    b = s.add_request(list(range(50, 58)), stop=stop(12))
    outs, _ = run_to_completion(s)
    st = s.stats()
    assert st["num_preemptions"] >= 1
    fin = {o.request_id: o for o in outs if o.finished}
    assert fin[a].num_generated == 12 and fin[b].num_generated == 12       # the victim is recomputed, nothing is lost
    assert s.block_manager(0).num_used_blocks == 0


def test_online_request_evicts_offline_decode():
    s = make(num_blocks=9, block_size=4, max_tokens_per_batch=64, prefill_scheduling_memory_usage_threshold=1.0)
    off = s.add_request(list(range(16)), stop=stop(30), offline=True)
    answer(s, s.schedule())
    on = s.add_request(list(range(100, 120)), stop=stop(2))
    bs = s.schedule()
    assert on in [e["req"] for e in entries(bs[0])]
    assert s.stats()["num_offline_evictions"] == 1
    answer(s, bs)
    outs, _ = run_to_completion(s)
    assert {o.request_id for o in outs if o.request_finished} == {on, off}


def test_zero_evict_admits_only_what_can_finish():
    # each request may grow to 8 + 16 tokens = 6 blocks of 4; 13 usable blocks hold two of them, not three
    s = make(num_blocks=14, block_size=4, use_zero_evict=True, max_decode_token_per_sequence=16)
    ids = [s.add_request(list(range(i * 10, i * 10 + 8)), stop=stop(16)) for i in range(3)]
    bs = s.schedule()
    first = [e["req"] for e in entries(bs[0])]
    answer(s, bs)
    bs = s.schedule()
    second = [e["req"] for e in entries(bs[0])]
    assert ids[2] not in first + second and s.num_waiting == 1
    outs, _ = run_to_completion(s)
    assert s.stats()["num_preemptions"] == 0
    assert {o.request_id for o in outs if o.request_finished} == set(ids)


# ------------------------------------------------------------------ priorities
def test_priority_strategy_orders_the_waiting_queue():
    s = make(priority_strategy="priority", max_seqs_per_batch=1)
    lo = s.add_request([1] * 8, stop=stop(1), priority=3)
    hi = s.add_request([2] * 8, stop=stop(1), priority=1)
    mid = s.add_request([3] * 8, stop=stop(1), priority=2)
    order = []
    while s.has_unfinished():
        bs = s.schedule()
        order += [e["req"] for e in entries(bs[0]) if e["kv"] == 0]
        answer(s, bs)
    assert order == [hi, mid, lo]


def test_deadline_strategy_orders_by_ttft_target():
    s = make(priority_strategy="deadline", max_seqs_per_batch=1)
    slow = s.add_request([1] * 8, stop=stop(1), ttft_slo_ms=5000)
    fast = s.add_request([2] * 8, stop=stop(1), ttft_slo_ms=50)
    bs = s.schedule()
    assert [e["req"] for e in entries(bs[0])] == [fast]


# ------------------------------------------------------------------ best_of / n
def test_best_of_expands_after_first_token_and_shares_prompt_blocks():
    s = make(prefix=True, block_size=4)
    rid = s.add_request(list(range(16)), stop=stop(3), n=2, best_of=3)
    bs = s.schedule()
    assert bs[0].num_prefill_seqs == 1
    answer(s, bs)
    bs = s.schedule()
    es = entries(bs[0])
    assert sorted(e["idx"] for e in es) == [0, 1, 2]
    sib = [e for e in es if e["idx"] > 0]
    assert all(e["kv"] == 12 and e["n"] == 4 for e in sib)                 # 3 of 4 prompt blocks come from the cache
    answer(s, bs)
    outs, _ = run_to_completion(s)
    assert sum(1 for o in outs if o.finished and o.request_id == rid) == 3


# ------------------------------------------------------------------ schedule overlap (placeholders)
def test_placeholder_tokens_are_patched_one_step_later():
    s = make()
    rid = s.add_request(list(range(10)), stop=stop(4))
    b0 = s.schedule()[0]
    s.process_placeholder_output(b0.id)                 # step 1 is scheduled before step 0 has answered
    b1 = s.schedule()[0]
    assert b1.forward_type == DECODE and entries(b1)[0]["kv"] == 10
    assert s.request_tokens(rid, 0)[-1] < 0             # a placeholder sits where the first token will go
    s.update_output(b0.id, np.array([41], dtype=np.int32))
    assert s.request_tokens(rid, 0)[-1] == 41
    s.process_placeholder_output(b1.id)
    s.update_output(b1.id, np.array([42], dtype=np.int32))
    outs = s.take_outputs()
    toks = [t for o in outs for t in o.new_tokens]
    assert toks == [41, 42]


# ------------------------------------------------------------------ speculative slots
def test_speculative_slots_and_rejection():
    s = make(num_speculative_tokens=2, prefill_only_batches=True)
    rid = s.add_request(list(range(10)), stop=stop(20))
    b = s.schedule()[0]
    s.process_output(b.id, np.array([[5, -1, -1]], dtype=np.int32))         # prefill: one token
    b = s.schedule()[0]
    e = entries(b)[0]
    assert e["n"] == 3 and e["spec"] == 2 and b.num_sample_rows == 3
    s.process_output(b.id, np.array([[6, 7, -1]], dtype=np.int32))          # one draft accepted + bonus, one rejected
    assert s.request_tokens(rid, 0)[10:] == [5, 6, 7]
    b = s.schedule()[0]
    assert entries(b)[0]["kv"] == 12


# ------------------------------------------------------------------ data parallel
def test_dp_ranks_get_separate_batches():
    s = make(dp_size=2)
    ids = [s.add_request(list(range(i * 10, i * 10 + 6)), stop=stop(2)) for i in range(4)]
    bs = s.schedule()
    assert len(bs) == 2 and all(b.num_prefill_seqs == 2 for b in bs)
    assert sorted(e["req"] for b in bs for e in entries(b)) == ids
    answer(s, bs)
    outs, _ = run_to_completion(s)
    assert {o.request_id for o in outs if o.request_finished} == set(ids)


def test_dp_rank_choice_follows_the_cached_prefix():
    """A new request goes to the attention-DP rank that caches the beginning of its prompt, even when the other rank has
    more free blocks; without a cached prefix (or without room on that rank) the rank with the most free blocks is taken."""
    s = make(num_blocks=33, block_size=4, prefix=True, dp_size=2, max_tokens_per_batch=256)
    shared = list(range(500, 532))                                   # 8 full blocks
    first = s.add_request(shared + [1, 2, 3], stop=stop(2))
    bs = s.schedule()
    home = [b.dp_rank for b in bs if not b.empty][0]
    answer(s, bs)
    run_to_completion(s)
    other = 1 - home
    # unrelated, still running traffic until `home` is the fuller rank (requests nobody caches go to the emptier one)
    sizes = [30, 10, 30, 10, 30, 10]
    for i, n in enumerate(sizes):
        before = [s.block_manager(r).num_available_blocks for r in range(2)]
        rid = s.add_request(list(range(900 + 100 * i, 900 + 100 * i + n)), stop=stop(60))
        bs = s.schedule()
        landed = [b.dp_rank for b in bs if not b.empty for e in entries(b) if e["req"] == rid]
        assert landed and before[landed[0]] == max(before)            # nothing cached for it: most free blocks
        answer(s, bs)
        free = [s.block_manager(r).num_available_blocks for r in range(2)]
        if free[home] < free[other]:
            break
    assert free[home] < free[other] and free[home] >= 4
    # a request that shares the prefix is placed on `home` although `other` is emptier, and reuses the 8 blocks
    again = s.add_request(shared + [9, 9, 9, 9, 9], stop=stop(2))
    bs = s.schedule()
    placed = [(b.dp_rank, e) for b in bs if not b.empty for e in entries(b) if e["req"] == again]
    assert placed and placed[0][0] == home and placed[0][1]["kv"] == 32
    # a prompt whose prefix is cached on a rank that has no room for the rest goes elsewhere
    s2 = make(num_blocks=13, block_size=4, prefix=True, dp_size=2, max_tokens_per_batch=256)
    a = s2.add_request(shared[:16] + [1], stop=stop(2))
    bs = s2.schedule()
    home2 = [b.dp_rank for b in bs if not b.empty][0]
    answer(s2, bs)
    run_to_completion(s2)
    hog = s2.add_request(list(range(3000, 3030)), stop=stop(30))     # lands on the emptier rank: 1 - home2 ... or home2
    bs = s2.schedule()
    hog_rank = [b.dp_rank for b in bs if not b.empty][0]
    answer(s2, bs)
    big = s2.add_request(shared[:16] + list(range(4000, 4028)), stop=stop(2))     # 44 tokens: 12 blocks in all
    bs = s2.schedule()
    ranks = [b.dp_rank for b in bs if not b.empty for e in entries(b) if e["req"] == big]
    if ranks:                                                        # admitted now: only on a rank with room for it
        need = 12 - (4 if ranks[0] == home2 else 0)
        assert s2.block_manager(ranks[0]).num_blocks - 1 >= need


# ------------------------------------------------------------------ token budget from the profiler
def test_set_token_budget_clamps():
    s = make(max_tokens_per_batch=128)
    s.set_token_budget(64)
    assert s.token_budget == 64
    s.set_token_budget(4096)
    assert s.token_budget == 128
    s.set_token_budget(1)
    assert s.token_budget == 16


# ------------------------------------------------------------------ threads
def test_requests_and_cancels_from_many_threads_while_scheduling():
    """API threads add and cancel requests (the binding releases the GIL around `add_request`) while one thread drives the
    scheduler, as the serving loop does.  Every request must end exactly once and all blocks must return."""
    import random
    import threading
    s = make(num_blocks=96, block_size=4, prefix=True, max_tokens_per_batch=64, max_seqs_per_batch=8,
             prefill_scheduling_memory_usage_threshold=1.0)
    n_threads, per_thread = 6, 40
    ids, lock = [], threading.Lock()
    stop_flag = threading.Event()

    def producer(seed):
        rng = random.Random(seed)
        for i in range(per_thread):
            prompt = [rng.randrange(50) for _ in range(rng.randrange(1, 40))]
            rid = s.add_request(prompt, stop=stop(rng.randrange(1, 6)), priority=rng.randrange(3), offline=rng.random() < 0.2)
            with lock:
                ids.append(rid)
            if rng.random() < 0.25:
                s.cancel(rid)
            if rng.random() < 0.1:
                s.cancel(10 ** 9 + i)                # unknown ids are ignored

    finished = {}

    def driver():
        while not stop_flag.is_set() or s.has_unfinished():
            bs = s.schedule()
            answer(s, bs)
            for o in s.take_outputs():
                if o.request_finished:
                    finished[o.request_id] = finished.get(o.request_id, 0) + 1

    d = threading.Thread(target=driver)
    d.start()
    ps = [threading.Thread(target=producer, args=(k,)) for k in range(n_threads)]
    [p.start() for p in ps]
    [p.join() for p in ps]
    stop_flag.set()
    d.join(60)
    assert not d.is_alive()
    assert len(ids) == n_threads * per_thread and len(set(ids)) == len(ids)
    assert set(finished) == set(ids) and all(v == 1 for v in finished.values())
    assert s.block_manager(0).num_used_blocks == 0 and not s.has_unfinished()
