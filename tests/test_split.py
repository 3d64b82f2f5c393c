"""The split of one packed batch over several replicas and the scatter of the rows back, as the
library does them inside embed / predict on a multi-device handle (csrc/split.cpp), through the
host-only entry point tei_b200_split_echo: no GPU, a stand-in for the forward that echoes each
shard's own sub-batch.  Every expectation is computed here from the UNSPLIT batch, so a token
that went to the wrong shard, a cumulative length that was not rebased, a pooled / raw index
that was not renumbered or a row that came back to the wrong place all show.

Reference contract: pooled row i belongs to pooled_indices[i], raw rows follow raw_indices order,
scores go by batch position (backends/candle/src/lib.rs:694-706,718-722)."""
import ctypes

import numpy as np
import pytest


def _p(a, ct):
    return a.ctypes.data_as(ctypes.POINTER(ct)) if a is not None and a.size else None


def _echo(lib, ids, types, pos, cu, pooled, raw, predict, n_shards, width, lin=1.0, quad=0.01):
    n_seqs = len(cu) - 1
    lens = np.diff(cu.astype(np.int64))
    raw_rows = int(sum(lens[i] for i in raw)) if not predict else 0
    pooled_out = np.full((len(pooled), width), -1.0, np.float32)
    raw_out = np.full((raw_rows, width), -1.0, np.float32)
    scores = np.full((n_seqs, width), -1.0, np.float32)
    shard_tokens = np.zeros(n_shards, np.int32)
    u32, f32 = ctypes.c_uint32, ctypes.c_float
    rc = lib.tei_b200_split_echo(_p(ids, u32), _p(types, u32), _p(pos, u32), ids.size, _p(cu, u32), n_seqs,
                                 _p(pooled, u32), pooled.size, _p(raw, u32), raw.size, int(predict), n_shards,
                                 lin, quad, width, _p(pooled_out, f32), _p(raw_out, f32), _p(scores, f32),
                                 shard_tokens.ctypes.data_as(ctypes.POINTER(ctypes.c_int)))
    return rc, pooled_out, raw_out, scores, shard_tokens


def _expect(ids, types, pos, cu, pooled, raw, width):
    col = np.arange(width, dtype=np.float32)
    seq_val = np.array([int(ids[cu[s]:cu[s + 1]].astype(np.uint64).sum() % 65521) for s in range(len(cu) - 1)],
                       dtype=np.float32)
    exp_pooled = seq_val[pooled.astype(np.int64)][:, None] + col[None] if pooled.size else np.zeros((0, width), np.float32)
    rows = []
    for s in raw:
        t = np.arange(cu[s], cu[s + 1])
        rows.append((ids[t] % 4096 + 7 * types[t] + 13 * (pos[t] % 4096)).astype(np.float32)[:, None] + col[None])
    exp_raw = np.concatenate(rows) if rows else np.zeros((0, width), np.float32)
    return exp_pooled, exp_raw, seq_val[:, None] + col[None]


def _batch(seed, lens, vocab=30000):
    rng = np.random.default_rng(seed)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    T = int(cu[-1])
    ids = rng.integers(0, vocab, T).astype(np.uint32)
    types = rng.integers(0, 2, T).astype(np.uint32)
    pos = np.concatenate([np.arange(n) for n in lens]).astype(np.uint32)
    return ids, types, pos, cu


@pytest.mark.parametrize("n_shards", [1, 2, 3, 8])
def test_embed_rows_come_back_to_their_places(lib, n_shards):
    lens = [7, 33, 150, 2, 64, 129, 300, 1, 512, 18, 77]
    ids, types, pos, cu = _batch(3, lens)
    # pooled and raw requests interleaved and out of order, as the queue may produce them
    pooled = np.array([9, 0, 2, 3, 10, 6], np.uint32)
    raw = np.array([8, 1, 5, 4, 7], np.uint32)
    rc, p, r, _, tok = _echo(lib, ids, types, pos, cu, pooled, raw, False, n_shards, 5)
    assert rc == 0
    ep, er, _ = _expect(ids, types, pos, cu, pooled, raw, 5)
    assert np.array_equal(p, ep)
    assert np.array_equal(r, er)
    assert int(tok.sum()) == int(cu[-1])
    if n_shards > 1:
        assert tok.max() < int(cu[-1])  # really split


@pytest.mark.parametrize("n_shards", [2, 5])
def test_predict_scores_go_by_batch_position(lib, n_shards):
    lens = [40, 3, 511, 90, 90, 90, 17]
    ids, types, pos, cu = _batch(4, lens)
    none = np.zeros(0, np.uint32)
    rc, _, _, sc, tok = _echo(lib, ids, types, pos, cu, none, none, True, n_shards, 3)
    assert rc == 0
    assert np.array_equal(sc, _expect(ids, types, pos, cu, none, none, 3)[2])
    assert int(tok.sum()) == int(cu[-1])


def test_more_shards_than_sequences_and_a_single_sequence(lib):
    ids, types, pos, cu = _batch(5, [12, 900])
    pooled = np.array([1, 0], np.uint32)
    none = np.zeros(0, np.uint32)
    rc, p, _, _, tok = _echo(lib, ids, types, pos, cu, pooled, none, False, 8, 4)
    assert rc == 0 and np.array_equal(p, _expect(ids, types, pos, cu, pooled, none, 4)[0])
    assert sorted(tok.tolist()) == [0] * 6 + [12, 900]
    ids, types, pos, cu = _batch(6, [77])
    rc, p, _, _, _ = _echo(lib, ids, types, pos, cu, np.array([0], np.uint32), none, False, 4, 4)
    assert rc == 0 and np.array_equal(p, _expect(ids, types, pos, cu, np.array([0], np.uint32), none, 4)[0])


def test_the_benchmark_batch_split_eight_ways(lib):
    from oracle import generators as G
    b = G.batch_cfg2()
    n = len(b)
    pooled = np.arange(n, dtype=np.uint32)
    none = np.zeros(0, np.uint32)
    rc, p, _, _, tok = _echo(lib, b.input_ids, b.token_type_ids, b.position_ids, b.cumulative_seq_lengths, pooled,
                             none, False, 8, 8, lin=169.87e6, quad=4 * 768.0)
    assert rc == 0
    assert np.array_equal(p, _expect(b.input_ids, b.token_type_ids, b.position_ids, b.cumulative_seq_lengths,
                                     pooled, none, 8)[0])
    assert int(tok.sum()) == 68576 and tok.max() - tok.min() < 0.03 * tok.mean()  # balanced


def test_malformed_batches_are_refused_before_anything_is_split(lib):
    ids, types, pos, cu = _batch(7, [5, 6])
    none = np.zeros(0, np.uint32)
    bad_cu = cu.copy()
    bad_cu[1] = 0  # not strictly increasing
    assert _echo(lib, ids, types, pos, bad_cu, none, none, True, 2, 2)[0] == 2
    assert _echo(lib, ids, types, pos, cu, np.array([2], np.uint32), none, False, 2, 2)[0] == 2  # pooled index out of range
    assert _echo(lib, ids, types, pos, cu, none, none, True, 0, 2)[0] == 2
