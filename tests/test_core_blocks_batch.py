"""Host-only tests of the C++ block manager, prefix cache and batch builder (no model, no device).

Same tier as the reference's block_manager_test.cpp, prefix_cache_test.cpp and batch_test.cpp (hand-made sequences,
every field of the step input checked).
"""
import numpy as np
import pytest

from xllm_wxh_b200 import _core
from test_core_scheduler import answer, entries, make, stop


# ------------------------------------------------------------------ block manager
def test_block_ids_zero_is_padding_and_smallest_first():
    bm = _core.BlockManager(8, 4, False)
    assert bm.num_free_blocks == 7 and bm.num_used_blocks == 0
    a = bm.allocate(3)
    assert a == [1, 2, 3]
    b = bm.allocate(4)
    assert b == [4, 5, 6, 7]
    assert bm.allocate(1) == [] and bm.utilization == pytest.approx(1.0)
    bm.release([2, 5])
    assert bm.num_free_blocks == 2 and sorted(bm.allocate(2)) == [2, 5]
    with pytest.raises(IndexError):
        bm.release([0])                                   # the padding block is never owned
    with pytest.raises(Exception):
        bm.release([7, 7])                                # double release


def test_reference_counts_and_shared_blocks():
    bm = _core.BlockManager(8, 4, True)
    toks = list(range(12))
    blocks = bm.allocate(3)
    assert bm.insert(toks, blocks) == 3
    assert all(bm.ref_count(b) == 2 for b in blocks)      # the owner + the cache
    hit = bm.match(toks + [99])
    assert hit == blocks and all(bm.ref_count(b) == 3 for b in blocks)
    bm.release(blocks)
    bm.release(hit)
    # only the cache holds them now: they count as available, not as used
    assert bm.num_used_blocks == 0 and bm.num_available_blocks == 7 and bm.num_blocks_in_prefix_cache == 3


# ------------------------------------------------------------------ prefix cache
def test_match_is_chained_whole_blocks_only():
    bm = _core.BlockManager(16, 4, True)
    toks = list(range(100, 110))                           # 2 full blocks + 2 tokens
    blocks = bm.allocate(3)
    assert bm.insert(toks, blocks) == 2                    # the partial block is not cached
    assert bm.match(toks) == blocks[:2]
    # same second block after a different first block: the chain differs, nothing matches past the divergence
    other = [7, 7, 7, 7] + toks[4:8]
    assert bm.match(other) == []
    # shorter query: one block
    assert bm.match(toks[:5]) == blocks[:1]
    # max_blocks bounds the match
    assert bm.match(toks, 1) == blocks[:1]
    assert bm.match_hits == 4 and bm.match_queries >= 5


def test_duplicate_content_keeps_first_block():
    bm = _core.BlockManager(16, 4, True)
    toks = [5, 6, 7, 8]
    a = bm.allocate(1)
    b = bm.allocate(1)
    assert bm.insert(toks, a) == 1
    assert bm.insert(toks, b) == 0                         # the content is already cached under `a`
    assert bm.match(toks) == a
    assert bm.ref_count(b[0]) == 1


def test_lru_eviction_order_and_pinned_blocks_survive():
    bm = _core.BlockManager(6, 2, True)                    # 5 usable blocks
    seqs = [[i, i] for i in range(1, 6)]
    owned = []
    for t in seqs:
        blk = bm.allocate(1)
        bm.insert(t, blk)
        owned.append(blk)
    for blk in owned[1:]:
        bm.release(blk)                                    # blocks 2..5 are cache-only; block 1 stays pinned by its owner
    assert bm.num_free_blocks == 0 and bm.num_available_blocks == 4
    assert bm.match(seqs[1]) == owned[1]                   # touch: most recently used, and pinned again by the match
    got = bm.allocate(2)                                   # needs two evictions: least recently used, unpinned first
    assert sorted(got) == sorted(owned[2] + owned[3])
    assert bm.match(seqs[2]) == [] and bm.match(seqs[3]) == []
    assert bm.match(seqs[0]) == owned[0]                   # never evicted while its owner holds it
    assert bm.match(seqs[4]) == owned[4]
    assert bm.evict(10) == 0                               # everything left is pinned


def test_hash_is_seeded_and_stable():
    a = _core.hash128(b"hello world", 1024)
    assert a == _core.hash128(b"hello world", 1024)
    assert a != _core.hash128(b"hello world", 1025) and a != _core.hash128(b"hello worle", 1024)
    # managers with different seeds do not share keys, equal seeds do
    t = list(range(8))
    m1, m2 = _core.BlockManager(8, 4, True, 1), _core.BlockManager(8, 4, True, 1)
    b1 = m1.allocate(2)
    m1.insert(t, b1)
    assert m2.match(t) == []


# ------------------------------------------------------------------ batch builder
def _build(s, b, T=64, B=8, MB=8, S=8, P=64, block_size=4):
    L = _core.BatchLayout(T, B, MB, S, P)
    buf = np.full(L.total_words, -12345, dtype=np.int32)
    rc = b.build(L, buf.ctypes.data, buf.size, block_size)
    return L, buf, rc


def _f(buf, off, n):
    return buf[off:off + n].view(np.float32)


def test_step_input_of_a_mixed_batch():
    s = make(num_blocks=32, block_size=4, max_tokens_per_batch=64)
    sp = _core.SamplingParams()
    sp.temperature, sp.top_p, sp.top_k, sp.seed = 0.7, 0.9, 40, 11
    a = s.add_request([10, 11, 12, 13, 14], sampling=sp, stop=stop(8))
    answer(s, s.schedule(), token=20)
    b_ = s.add_request(list(range(100, 107)), stop=stop(8))
    batch = s.schedule()[0]
    assert batch.forward_type == 3 and batch.num_decode_seqs == 1 and batch.num_prefill_seqs == 1
    L, buf, rc = _build(s, batch)
    assert rc == 0
    H = buf[L.header:L.header + 32]
    assert H[0] == 8 and H[1] == 2 and H[2] == 2 and H[3] == 1 and H[4] == 1          # tokens, seqs, samples, decode, prefill
    assert H[5] == 7 and H[6] == 7 and H[7] == 3 and H[8] == 0 and H[17] == 4 and H[21] == 7
    assert H[15] == 0                                                                 # not all greedy
    blocks_a, blocks_b = batch.seq_blocks(0), batch.seq_blocks(1)
    assert blocks_a == [1, 2] and blocks_b == [3, 4]
    # decode row first: the token sampled last step at position 5, then the 7 prompt tokens
    assert buf[L.tokens:L.tokens + 8].tolist() == [20] + list(range(100, 107))
    assert buf[L.positions:L.positions + 8].tolist() == [5, 0, 1, 2, 3, 4, 5, 6]
    assert buf[L.slots:L.slots + 8].tolist() == [2 * 4 + 1] + [3 * 4 + i for i in range(4)] + [4 * 4 + i for i in range(3)]
    assert buf[L.token_seq:L.token_seq + 8].tolist() == [0] + [1] * 7
    assert buf[L.next_tokens:L.next_tokens + 8].tolist() == [-1] + list(range(101, 107)) + [-1]
    assert buf[L.q_cu:L.q_cu + 3].tolist() == [0, 1, 8]
    assert buf[L.kv_lens:L.kv_lens + 2].tolist() == [6, 7]
    bt = buf[L.block_tables:L.block_tables + 2 * 8].reshape(2, 8)
    assert bt[0].tolist() == [1, 2, 0, 0, 0, 0, 0, 0] and bt[1].tolist() == [3, 4, 0, 0, 0, 0, 0, 0]
    assert buf[L.sample_idx:L.sample_idx + 2].tolist() == [0, 7]
    assert _f(buf, L.temperature, 2).tolist() == pytest.approx([0.7, 0.0])
    assert _f(buf, L.top_p, 2).tolist() == pytest.approx([0.9, 1.0])
    assert buf[L.top_k:L.top_k + 2].tolist() == [40, -1]
    # padding: rows beyond the batch point at the reserved block 0 and belong to no sequence
    assert buf[L.token_seq + 8:L.token_seq + 64].tolist() == [-1] * 56
    assert all(0 <= x < 4 for x in buf[L.slots + 8:L.slots + 64])
    assert buf[L.q_cu + 3:L.q_cu + 9].tolist() == [8] * 6 and buf[L.kv_lens + 2:L.kv_lens + 8].tolist() == [0] * 6
    assert buf[L.top_k + 2:L.top_k + 8].tolist() == [-1] * 6
    # no word of the message is left unwritten in the sections the kernels read (block-table rows of padding sequences
    # are never read: their kv length is 0)
    for off, n in ((L.tokens, 64), (L.positions, 64), (L.slots, 64), (L.q_cu, 9), (L.kv_lens, 8), (L.block_tables, 16),
                   (L.sample_idx, 8), (L.temperature, 8), (L.seed_lo, 8), (L.seed_hi, 8), (L.want_logprobs, 8)):
        assert not (buf[off:off + n] == -12345).any(), off


def test_seeds_differ_per_position_and_repeat_per_seed():
    def seeds(seed):
        s = make(num_blocks=32, block_size=4)
        sp = _core.SamplingParams()
        sp.temperature, sp.seed = 1.0, seed
        s.add_request([1, 2, 3], sampling=sp, stop=stop(4))
        out = []
        for _ in range(3):
            batch = s.schedule()[0]
            L, buf, rc = _build(s, batch)
            out.append((int(buf[L.seed_lo]), int(buf[L.seed_hi])))
            answer(s, [batch], token=9)
        return out
    a, b, c = seeds(5), seeds(5), seeds(6)
    assert a == b and a != c and len(set(a)) == 3


def test_penalty_section_counts_prompt_and_generated_tokens():
    s = make(num_blocks=32, block_size=4)
    sp = _core.SamplingParams()
    sp.repetition_penalty, sp.frequency_penalty = 1.2, 0.5
    s.add_request([4, 4, 9], sampling=sp, stop=stop(8))
    answer(s, s.schedule(), token=9)
    answer(s, s.schedule(), token=4)
    batch = s.schedule()[0]                                # sequence is now 4 4 9 | 9 4
    L, buf, rc = _build(s, batch)
    assert rc == 0 and buf[L.header + 14] == 1 and buf[L.header + 18] == 2
    assert buf[L.pen_cu:L.pen_cu + 2].tolist() == [0, 2]
    ids = buf[L.pen_ids:L.pen_ids + 2].tolist()
    cnt = buf[L.pen_counts:L.pen_counts + 2].tolist()
    got = {i: (c & 0xffff, c >> 16) for i, c in zip(ids, cnt)}
    assert got == {4: (3, 1), 9: (2, 1)}                   # (all occurrences, generated occurrences)
    # a penalty section that is too small is reported with the size that would fit
    L2, buf2, rc2 = _build(s, batch, P=1)
    assert rc2 == -(2) - 16


def test_capacity_overflow_is_reported():
    s = make(num_blocks=32, block_size=4, max_tokens_per_batch=64)
    s.add_request(list(range(20)), stop=stop(2))
    batch = s.schedule()[0]
    assert _build(s, batch, T=16)[2] == -1                 # tokens
    assert _build(s, batch, MB=4)[2] == -1                 # blocks per sequence
    assert _build(s, batch, T=32, MB=5)[2] == 0
    L = _core.BatchLayout(32, 8, 8, 8, 16)
    small = np.zeros(L.total_words - 1, dtype=np.int32)
    with pytest.raises(RuntimeError):
        batch.build(L, small.ctypes.data, small.size, 4)


def test_speculative_rows_in_step_input():
    s = make(num_blocks=32, block_size=4, num_speculative_tokens=2, prefill_only_batches=True)
    s.add_request([1, 2, 3, 4, 5], stop=stop(16))
    b0 = s.schedule()[0]
    s.process_output(b0.id, np.array([[6, -1, -1]], dtype=np.int32))
    b1 = s.schedule()[0]
    L, buf, rc = _build(s, b1)
    assert rc == 0 and buf[L.header + 8] == 2 and buf[L.header + 2] == 3      # two draft slots, three sampling rows
    assert buf[L.tokens:L.tokens + 3].tolist() == [6, 0, 0]                   # draft slots are filled by the worker
    assert buf[L.positions:L.positions + 3].tolist() == [5, 6, 7]
    assert buf[L.sample_idx:L.sample_idx + 3].tolist() == [0, 1, 2]
    assert buf[L.kv_lens] == 8
