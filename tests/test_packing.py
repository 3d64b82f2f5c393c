"""Oracle of the reference's batch packing (core/src/queue.rs:118-200,
backends/candle/tests/common.rs:327-356) against hand-derived expectations."""
import json
import os

import numpy as np

from oracle.packing import Request, batch_from_encodings, next_batch, split_batch

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "packing_cases.json")


def _req(n, pooling=True, offset=0, start=0):
    return Request(input_ids=list(range(start, start + n)), pooling=pooling, position_offset=offset)


def test_token_budget_is_a_hard_limit_and_fifo():
    # 5 + 7 = 12 <= 12 fits, the third (1 token) would make 13 > 12 and stays queued.
    q = [_req(5), _req(7), _req(1), _req(2)]
    b, rest = next_batch(q, max_batch_tokens=12)
    assert b.cumulative_seq_lengths.tolist() == [0, 5, 12]
    assert b.max_length == 7
    assert len(rest) == 2 and len(rest[0].input_ids) == 1
    assert b.cumulative_seq_lengths.dtype == np.uint32


def test_oversized_head_of_queue_blocks_the_batch():
    # queue.rs:157-160: the entry is pushed back and the loop breaks, nothing behind it is taken.
    q = [_req(20), _req(1)]
    b, rest = next_batch(q, max_batch_tokens=12)
    assert b is None and len(rest) == 2


def test_max_batch_requests():
    q = [_req(1), _req(1), _req(1)]
    b, rest = next_batch(q, max_batch_tokens=100, max_batch_requests=2)
    assert len(b) == 2 and len(rest) == 1


def test_pooled_and_raw_indices_are_batch_positions():
    q = [_req(3, True), _req(2, False), _req(4, True), _req(1, False)]
    b, _ = next_batch(q, max_batch_tokens=100)
    assert b.pooled_indices.tolist() == [0, 2]
    assert b.raw_indices.tolist() == [1, 3]
    assert b.cumulative_seq_lengths.tolist() == [0, 3, 5, 9, 10]


def test_positions_restart_per_sequence_with_offset():
    # tokenization.rs:406-411 with the RoBERTa offset of router/src/lib.rs:185-192.
    q = [_req(3, offset=2), _req(2, offset=2)]
    b, _ = next_batch(q, max_batch_tokens=100)
    assert b.position_ids.tolist() == [2, 3, 4, 2, 3]
    b2 = batch_from_encodings([[7, 8, 9], [1, 2]], [0, 1], [], position_offset=0)
    assert b2.position_ids.tolist() == [0, 1, 2, 0, 1]
    assert b2.token_type_ids.tolist() == [0] * 5


def test_padded_rule():
    # queue.rs:150-152: a padded model counts max_length * batch size.
    q = [_req(10), _req(2), _req(2)]
    b, rest = next_batch(q, max_batch_tokens=25, padded_model=True)
    assert len(b) == 2 and len(rest) == 1  # 10*3 = 30 > 25


def test_golden_packing_cases():
    cases = json.load(open(GOLDEN))
    assert len(cases) >= 5
    for c in cases:
        q = [Request(input_ids=r["ids"], token_type_ids=r.get("types"), pooling=r["pooling"],
                     position_offset=r["offset"]) for r in c["requests"]]
        b, rest = next_batch(q, c["max_batch_tokens"], c.get("max_batch_requests"))
        e = c["expect"]
        assert b.input_ids.tolist() == e["input_ids"]
        assert b.token_type_ids.tolist() == e["token_type_ids"]
        assert b.position_ids.tolist() == e["position_ids"]
        assert b.cumulative_seq_lengths.tolist() == e["cu"]
        assert b.max_length == e["max_length"]
        assert b.pooled_indices.tolist() == e["pooled"]
        assert b.raw_indices.tolist() == e["raw"]
        assert len(rest) == e["left"]


def test_split_batch_round_trip():
    rng = np.random.default_rng(0)
    lens = rng.integers(1, 40, size=11)
    encs = [rng.integers(0, 100, size=int(n)) for n in lens]
    b = batch_from_encodings(encs, [0, 2, 3, 7, 10], [1, 4, 5, 6, 8, 9])
    shard_of = [int(x) for x in rng.integers(0, 3, size=11)]
    parts = split_batch(b, shard_of, 3)
    seen = []
    for sb, members in parts:
        cu = sb.cumulative_seq_lengths
        for j, s in enumerate(members):
            a, e = int(cu[j]), int(cu[j + 1])
            assert sb.input_ids[a:e].tolist() == encs[s].tolist()
            assert sb.position_ids[a:e].tolist() == list(range(len(encs[s])))
            seen.append(s)
        pooled_members = [members[i] for i in sb.pooled_indices]
        raw_members = [members[i] for i in sb.raw_indices]
        assert all(s in b.pooled_indices for s in pooled_members)
        assert all(s in b.raw_indices for s in raw_members)
    assert sorted(seen) == list(range(11))
