"""One handle, several replicas: the packed batch is split at sequence boundaries across the
replicas inside a single embed / predict call and the rows come back in their original places.
No collective runs: each replica computes its sequences independently.  The tests over several
GPUs need at least two (skipped otherwise); the same split, gather and scatter also run with
several replicas of ONE GPU (each with its own stream, workspace and pinned buffers), which is
how a single-GPU box exercises them."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from oracle import generators as G  # noqa: E402

pytestmark = pytest.mark.gpu


def _n_gpus():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


needs_two = pytest.mark.skipif(_n_gpus() < 2, reason="needs two GPUs")


@needs_two
def test_sharded_embed_matches_single_replica(lib, model_dirs):
    import tei_b200
    n = min(_n_gpus(), 4)
    one = tei_b200.B200Backend(model_dirs["bert"], "float16", "embedding", "mean", devices=[0])
    many = tei_b200.B200Backend(model_dirs["bert"], "float16", "embedding", "mean", devices=list(range(n)))
    lens = [7, 300, 33, 150, 2, 64, 129, 511, 90]
    b = G.random_batch(5, lens, 0, 1000, pooled=[0, 2, 3, 6, 8], raw=[1, 4, 5, 7], type_vocab=2)
    a, m = one.embed(b), many.embed(b)
    assert sorted(a) == sorted(m) == list(range(len(lens)))
    for i in range(len(lens)):
        assert a[i].kind == m[i].kind and a[i].values.shape == m[i].values.shape
        # same kernels, same per-sequence inputs: the rows agree to rounding of the GEMM tiling
        assert np.abs(a[i].values - m[i].values).max() <= 4e-3
    # a single-sequence batch stays on the first replica
    solo = G.random_batch(6, [40], 0, 1000, type_vocab=2)
    assert np.array_equal(one.embed(solo)[0].values, many.embed(solo)[0].values)
    st = many.stats()
    assert st["tokens"] > 0
    one.close()
    many.close()


@needs_two
def test_sharded_predict_and_errors(lib, model_dirs):
    import tei_b200
    one = tei_b200.B200Backend(model_dirs["xlmr"], "float16", "classifier", devices=[0])
    two = tei_b200.B200Backend(model_dirs["xlmr"], "float16", "classifier", devices=[0, 1])
    b = G.random_batch(7, [12, 200, 31, 77, 5], 5, 1000, position_offset=2)
    a, m = one.predict(b), two.predict(b)
    for i in range(5):
        assert abs(a[i][0] - m[i][0]) <= 2e-3
    bad = G.random_batch(7, [12, 200], 5, 1000, position_offset=2)
    bad.input_ids = np.full(212, 5000, dtype=np.uint32)
    with pytest.raises(tei_b200.BackendError):
        two.predict(bad)
    two.health()
    again = two.predict(b)
    for i in range(5):
        assert again[i] == m[i]
    one.close()
    two.close()


@needs_two
def test_sharded_embed_with_dense_modules(lib, model_dirs, tmp_path):
    # Dense modules change the width of the pooled rows but not of the raw rows; both kinds are
    # scattered back from the replicas with their own widths.
    import shutil
    import tei_b200
    d = tmp_path / "bert_dense"
    shutil.copytree(model_dirs["bert"], d)
    G.write_dense_dir(d, "2_Dense", 128, 72, seed=31, bias=True, activation="tanh")
    one = tei_b200.B200Backend(d, "float16", "embedding", "mean", dense_paths=["2_Dense"], devices=[0])
    two = tei_b200.B200Backend(d, "float16", "embedding", "mean", dense_paths=["2_Dense"], devices=[0, 1])
    assert two.output_dim == 72 and two.hidden_size == 128
    lens = [7, 300, 33, 150, 2, 64, 129]
    b = G.random_batch(8, lens, 0, 1000, pooled=[0, 2, 3, 6], raw=[1, 4, 5], type_vocab=2)
    a, m = one.embed(b, normalize=True), two.embed(b, normalize=True)
    for i in range(len(lens)):
        assert a[i].kind == m[i].kind and a[i].values.shape == m[i].values.shape
        assert np.abs(a[i].values - m[i].values).max() <= 4e-3
    assert m[0].values.shape == (72,) and m[1].values.shape == (300, 128)
    one.close()
    two.close()


@pytest.mark.parametrize("n_replicas", [2, 3])
def test_split_over_replicas_of_one_gpu(lib, model_dirs, n_replicas):
    """embed / predict on a handle with n replicas of device 0 against a single replica: pooled
    and raw requests interleaved, every row back at its place; a malformed batch is an error for
    the whole call and the handle recovers."""
    import tei_b200
    one = tei_b200.B200Backend(model_dirs["bert"], "float16", "embedding", "mean", devices=[0])
    many = tei_b200.B200Backend(model_dirs["bert"], "float16", "embedding", "mean", devices=[0] * n_replicas)
    assert many.num_replicas == n_replicas
    lens = [7, 300, 33, 150, 2, 64, 129, 511, 90, 18, 1]
    b = G.random_batch(15, lens, 0, 1000, pooled=[9, 0, 2, 3, 6, 8], raw=[10, 1, 4, 5, 7], type_vocab=2)
    a = one.embed(b, normalize=True)
    for _ in range(3):  # the per-replica threads and buffers are reused from call to call
        m = many.embed(b, normalize=True)
        assert sorted(a) == sorted(m) == list(range(len(lens)))
        for i in range(len(lens)):
            assert a[i].kind == m[i].kind and a[i].values.shape == m[i].values.shape
            assert np.abs(a[i].values - m[i].values).max() <= 4e-3
    assert many.stats()["tokens"] == sum(lens)
    bad = G.random_batch(15, lens, 0, 1000, type_vocab=2)
    bad.input_ids = bad.input_ids.copy()
    bad.input_ids[400] = 5000  # beyond the vocabulary, inside one shard only
    with pytest.raises(tei_b200.BackendError):
        many.embed(bad)
    many.health()
    m = many.embed(b, normalize=True)
    for i in range(len(lens)):
        assert np.abs(a[i].values - m[i].values).max() <= 4e-3
    # the phases of a call one by one
    many.stage(b, normalize=True)
    many.run_staged()
    many.sync()
    pooled, raw, _ = many.fetch(n_pooled=6, raw_rows=1 + 300 + 2 + 64 + 511)
    for row, i in enumerate([9, 0, 2, 3, 6, 8]):
        assert np.array_equal(pooled[row], m[i].values)
    assert np.array_equal(raw[0], m[10].values[0]) and np.array_equal(raw[1:301], m[1].values)
    one.close()
    many.close()


def test_split_predict_over_replicas_of_one_gpu(lib, model_dirs):
    import tei_b200
    one = tei_b200.B200Backend(model_dirs["xlmr"], "float16", "classifier", devices=[0])
    three = tei_b200.B200Backend(model_dirs["xlmr"], "float16", "classifier", devices=[0, 0, 0])
    b = G.random_batch(17, [12, 200, 31, 77, 5, 300, 64], 5, 1000, position_offset=2)
    a, m = one.predict(b), three.predict(b)
    for i in range(7):
        assert abs(a[i][0] - m[i][0]) <= 2e-3
    one.close()
    three.close()
