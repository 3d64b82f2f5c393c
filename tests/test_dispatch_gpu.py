"""Several batches in flight: one caller thread per replica (`tei_b200_embed_on` /
`tei_b200_predict_on`), the counterpart of running N of the reference's backend threads
(backends/src/lib.rs:612-647) instead of one.  Two replicas on ONE GPU are enough to exercise it:
each has its own stream, workspace and pinned buffers."""
import os
import sys
import threading

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from oracle import generators as G  # noqa: E402

pytestmark = pytest.mark.gpu


def _batches(seed0, n, type_vocab=2, position_offset=0, pad=0):
    out = []
    rng = np.random.default_rng(seed0)
    for i in range(n):
        lens = [int(x) for x in rng.integers(1, 300, size=int(rng.integers(1, 9)))]
        out.append(G.random_batch(seed0 + i, lens, pad, 1000, type_vocab=type_vocab,
                                  position_offset=position_offset))
    return out


def test_two_threads_two_replicas_embed(lib, model_dirs):
    import tei_b200
    be = tei_b200.B200Backend(model_dirs["bert"], "float16", "embedding", "mean", devices=[0, 0])
    assert be.num_replicas == 2
    work = [_batches(100, 12), _batches(200, 12)]
    # every batch alone, one after the other, on the replica that will run it again
    want = [[be.embed(b, replica=r) for b in work[r]] for r in range(2)]
    got = [[None] * 12, [None] * 12]
    errors = []

    def worker(r):
        try:
            for rep in range(3):  # three passes: the threads stay interleaved for a while
                for i, b in enumerate(work[r]):
                    got[r][i] = be.embed(b, replica=r)
        except Exception as exc:  # surfaced below: an exception in a thread is otherwise lost
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for r in range(2):
        for w, g in zip(want[r], got[r]):
            assert sorted(w) == sorted(g)
            for i in w:
                # same kernels on the same inputs on the same replica: bit-exact
                assert np.array_equal(w[i].values, g[i].values)
    # the two replicas hold the same weights
    a = be.embed(work[0][0], replica=0)
    b = be.embed(work[0][0], replica=1)
    for i in a:
        assert np.array_equal(a[i].values, b[i].values)
    # the whole-handle call still works afterwards (splits the batch over both replicas)
    c = be.embed(work[0][0])
    for i in a:
        assert np.abs(a[i].values - c[i].values).max() <= 4e-3
    be.close()


def test_same_replica_from_two_threads_is_serialised(lib, model_dirs):
    import tei_b200
    be = tei_b200.B200Backend(model_dirs["bert"], "float16", "embedding", "cls", devices=[0])
    work = _batches(300, 8)
    want = [be.embed(b, replica=0) for b in work]
    got = [[None] * 8, [None] * 8]
    errors = []

    def worker(k):
        try:
            for i, b in enumerate(work):
                got[k][i] = be.embed(b, replica=0)
        except Exception as exc:
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for k in range(2):
        for w, g in zip(want, got[k]):
            for i in w:
                assert np.array_equal(w[i].values, g[i].values)
    be.close()


def test_predict_on_and_refusals(lib, model_dirs):
    import tei_b200
    be = tei_b200.B200Backend(model_dirs["xlmr"], "float16", "classifier", devices=[0, 0])
    b = G.random_batch(7, [12, 200, 31, 77, 5], 5, 1000, position_offset=2)
    a, c = be.predict(b, replica=0), be.predict(b, replica=1)
    assert a == c
    with pytest.raises(tei_b200.BackendError, match="replica index"):
        be.predict(b, replica=2)
    with pytest.raises(tei_b200.BackendError, match="replica index"):
        be.predict(b, replica=-1)
    with pytest.raises(tei_b200.BackendError, match="not implemented"):
        be.embed(b, replica=0)
    # a refused batch on one replica leaves the other usable, and the first one too
    bad = G.random_batch(7, [12, 200], 5, 1000, position_offset=2)
    bad.input_ids = np.full(212, 5000, dtype=np.uint32)
    with pytest.raises(tei_b200.BackendError):
        be.predict(bad, replica=1)
    assert be.predict(b, replica=1) == a
    assert be.predict(b, replica=0) == a
    be.close()


def test_queue_feeds_two_replicas(lib, model_dirs):
    """The whole caller side: requests go into the library's queue, two consumer threads (one per
    replica) take batches and run them; every request's embedding equals the one it gets alone."""
    import tei_b200
    be = tei_b200.B200Backend(model_dirs["bert"], "float16", "embedding", "cls", devices=[0, 0])
    rng = np.random.default_rng(11)
    reqs = {tag: rng.integers(0, 1000, size=int(rng.integers(2, 120))).astype(np.uint32) for tag in range(60)}
    alone = {}
    for tag, ids in reqs.items():
        b = G.random_batch(0, [len(ids)], 0, 1000)
        b.input_ids = ids
        alone[tag] = be.embed(b, replica=0)[0].values
    q = tei_b200.BatchQueue(max_batch_tokens=400, max_batch_requests=8)
    for tag, ids in reqs.items():
        q.append(ids, tag=tag)
    got, errors, lock = {}, [], threading.Lock()

    def consume(r):
        try:
            while True:
                nb = q.next_batch()
                if nb is None:
                    return
                batch, tags = nb
                out = be.embed(batch, replica=r)
                with lock:
                    for i, tag in enumerate(tags):
                        got[tag] = out[i].values
        except Exception as exc:
            errors.append(exc)

    threads = [threading.Thread(target=consume, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert sorted(got) == sorted(reqs)
    for tag in reqs:
        # batched with neighbours against alone: same kernels, other tile positions
        assert np.abs(got[tag] - alone[tag]).max() <= 4e-3
    q.close()
    be.close()


def test_n_backend_threads_in_c_over_the_queue(lib, model_dirs, tmp_path):
    """tests/c/router_threads.c: the reference's backend-thread loop (backends/src/lib.rs:612-647)
    run N times over one handle, in C over the C ABI, fed by the library's queue."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib_dir = os.path.join(root, "text-embeddings-inference_b200", "lib")
    exe = tmp_path / "router_threads"
    subprocess.run(["gcc", "-std=c99", "-D_POSIX_C_SOURCE=200809L", "-Wall", "-Werror", "-I", os.path.join(root, "include"),
                    os.path.join(root, "tests", "c", "router_threads.c"), "-o", str(exe), "-L", lib_dir, "-ltei_b200",
                    f"-Wl,-rpath,{lib_dir}", "-lpthread", "-lm"], check=True)
    for n_replicas in (1, 3):
        out = subprocess.run([str(exe), str(model_dirs["bert"]), str(n_replicas), "200", "1000", "2048"],
                             capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, (out.returncode, out.stdout, out.stderr)
        assert out.stdout.startswith("ok batches=")
        n_batches = int(out.stdout.split("batches=")[1].split()[0])
        assert n_batches >= 200 * 150 // 2048  # the requests did not all fit one batch
