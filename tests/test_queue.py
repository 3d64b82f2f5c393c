"""The library's batching queue (include/tei_b200_queue.h, csrc/queue.cpp) against the oracle of
the reference's NextBatch rule (oracle/packing.py, core/src/queue.rs:118-200): bit-exact batches
on the golden cases and on seeded random request streams.  Host-only: runs without a GPU."""
import json
import os
import sys
import threading

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "text-embeddings-inference_b200"))

from oracle.packing import Request, next_batch  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "packing_cases.json")


@pytest.fixture(scope="module")
def tq():
    import tei_b200.queue as q
    return q


def _same(batch, oracle_batch):
    assert batch.input_ids.dtype == np.uint32 and batch.cumulative_seq_lengths.dtype == np.uint32
    assert np.array_equal(batch.input_ids, oracle_batch.input_ids)
    assert np.array_equal(batch.token_type_ids, oracle_batch.token_type_ids)
    assert np.array_equal(batch.position_ids, oracle_batch.position_ids)
    assert np.array_equal(batch.cumulative_seq_lengths, oracle_batch.cumulative_seq_lengths)
    assert batch.max_length == oracle_batch.max_length
    assert np.array_equal(batch.pooled_indices, oracle_batch.pooled_indices)
    assert np.array_equal(batch.raw_indices, oracle_batch.raw_indices)


def test_golden_packing_cases(tq):
    cases = json.load(open(GOLDEN))
    for c in cases:
        q = tq.BatchQueue(c["max_batch_tokens"], c.get("max_batch_requests"))
        for i, r in enumerate(c["requests"]):
            q.append(r["ids"], r.get("types"), pooling=r["pooling"], tag=i, position_offset=r["offset"])
        got = q.next_batch()
        e = c["expect"]
        assert got is not None
        b, tags = got
        assert b.input_ids.tolist() == e["input_ids"]
        assert b.token_type_ids.tolist() == e["token_type_ids"]
        assert b.position_ids.tolist() == e["position_ids"]
        assert b.cumulative_seq_lengths.tolist() == e["cu"]
        assert b.max_length == e["max_length"]
        assert b.pooled_indices.tolist() == e["pooled"]
        assert b.raw_indices.tolist() == e["raw"]
        assert len(q) == e["left"]
        assert tags == list(range(len(b)))
        q.close()


@pytest.mark.parametrize("padded", [False, True])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_streams_match_the_oracle(tq, seed, padded):
    rng = np.random.default_rng(seed)
    budget = int(rng.integers(64, 4096))
    max_req = None if seed == 0 else int(rng.integers(2, 40))
    reqs = []
    for i in range(300):
        n = int(rng.integers(1, 600))
        reqs.append(Request(input_ids=rng.integers(0, 30000, size=n).tolist(),
                            token_type_ids=rng.integers(0, 2, size=n).tolist() if i % 3 else None,
                            pooling=bool(rng.integers(0, 2)), position_offset=int(rng.integers(0, 3))))
    q = tq.BatchQueue(budget, max_req, padded_model=padded)
    for i, r in enumerate(reqs):
        q.append(r.input_ids, r.token_type_ids, pooling=r.pooling, tag=1000 + i, position_offset=r.position_offset)
    rest = list(reqs)
    next_tag = 1000
    while True:
        want, rest_after = next_batch(rest, budget, max_req, padded_model=padded)
        got = q.next_batch()
        if want is None:
            # the head of the queue is larger than the budget: it blocks everything behind it
            assert got is None
            assert len(q) == len(rest)
            break
        b, tags = got
        _same(b, want)
        assert tags == list(range(next_tag, next_tag + len(want)))
        next_tag += len(want)
        rest = rest_after
        assert len(q) == len(rest)
        if not rest:
            assert q.next_batch() is None
            break
    q.close()


def test_explicit_positions_and_cancel(tq):
    q = tq.BatchQueue(100)
    q.append([5, 6, 7], position_ids=[9, 8, 7], tag=1)
    q.append([1, 2], tag=2, pooling=False, position_offset=2)
    q.append([3], tag=3)
    q.append([4, 4], tag=2)
    assert q.cancel(2) == 2  # dropped clients are skipped (queue.rs:142-146)
    b, tags = q.next_batch()
    assert tags == [1, 3]
    assert b.input_ids.tolist() == [5, 6, 7, 3]
    assert b.position_ids.tolist() == [9, 8, 7, 0]
    assert b.cumulative_seq_lengths.tolist() == [0, 3, 4]
    assert b.pooled_indices.tolist() == [0, 1] and b.raw_indices.tolist() == []
    assert len(q) == 0 and q.next_batch() is None
    q.close()


def test_caller_buffers_limit_the_batch_and_refusals(tq):
    q = tq.BatchQueue(100)
    for i in range(4):
        q.append([i] * 10, tag=i)
    b, tags = q.next_batch(token_cap=25)  # room for two requests only
    assert tags == [0, 1] and len(q) == 2
    b, tags = q.next_batch(seq_cap=1)
    assert tags == [2] and len(q) == 1
    with pytest.raises(tq.BackendError):
        q.append([])
    with pytest.raises(tq.BackendError):
        q.append([1, 2], token_type_ids=[0])
    with pytest.raises(tq.BackendError):
        tq.BatchQueue(0)
    q.close()


def test_producers_and_consumers_in_parallel(tq):
    """Four producer threads and two consumers: every request comes out exactly once, and within
    one producer in the order it went in."""
    q = tq.BatchQueue(512, 16)
    n_prod, per = 4, 400
    done = threading.Event()
    out, lock = [], threading.Lock()

    def produce(p):
        rng = np.random.default_rng(p)
        for i in range(per):
            q.append(rng.integers(0, 100, size=int(rng.integers(1, 64))).tolist(), tag=p * 100000 + i)

    def consume():
        while True:
            got = q.next_batch()
            if got is None:
                if done.is_set() and len(q) == 0:
                    return
                continue
            b, tags = got
            assert int(b.cumulative_seq_lengths[-1]) <= 512 and len(b) <= 16
            assert int(b.cumulative_seq_lengths[-1]) == b.input_ids.size
            with lock:
                out.append(tags)

    cons = [threading.Thread(target=consume) for _ in range(2)]
    prods = [threading.Thread(target=produce, args=(p,)) for p in range(n_prod)]
    for t in cons + prods:
        t.start()
    for t in prods:
        t.join()
    done.set()
    for t in cons:
        t.join()
    flat = [t for tags in out for t in tags]
    assert sorted(flat) == sorted(p * 100000 + i for p in range(n_prod) for i in range(per))
    for tags in out:  # inside one batch a producer's requests keep their order
        for p in range(n_prod):
            mine = [t for t in tags if t // 100000 == p]
            assert mine == sorted(mine)
    q.close()
