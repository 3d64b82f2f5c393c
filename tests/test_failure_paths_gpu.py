"""What happens when a kernel's bounded wait runs out, exercised without making one run out in
a real forward: every device-side wait is limited, a wait that gives up writes a code to the status
word and the kernel returns; the host turns the code into TIMEOUT (-> BackendError::Inference,
backends/candle/src/lib.rs:728-740), marks the handle unhealthy (backends/src/lib.rs:621-642) and
the next health() runs a one-token probe (backends/src/lib.rs:393-409).

Nothing here hangs, traps or faults a GPU: the status word is written by a kernel that only
writes it, and the one real wait is on a barrier of the test's own, limited to a few hundred
probes."""
import ctypes
import threading

import numpy as np
import pytest
import torch

from oracle import generators as G

pytestmark = pytest.mark.gpu


def _backend(model_dirs, key, model_type="embedding", pool="mean", devices=None):
    import tei_b200
    return tei_b200.B200Backend(model_dirs[key], "float16", model_type, pool, devices=devices)


def test_a_wait_that_gives_up_reports_and_returns(lib):
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gave_up = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for limit in (1, 300, 4096):
        status.zero_()
        rc = lib.tei_b200_op_bounded_wait_probe(status.data_ptr(), limit, gave_up.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert status.item() == 101 and gave_up.item() == 1  # DEV_TIMEOUT_PRODUCER
    # the limit is capped and the status word is mandatory: refused before any launch
    assert lib.tei_b200_op_bounded_wait_probe(status.data_ptr(), 1 << 20, None, stream) != 0
    assert lib.tei_b200_op_bounded_wait_probe(None, 10, None, stream) != 0
    # the context is as usable as before
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_timeout_code_turns_into_an_inference_error_and_health_recovers(lib, model_dirs):
    from tei_b200.backend import BackendError
    be = _backend(model_dirs, "bert")
    b = G.random_batch(5, [9, 140, 33], 0, 1000, type_vocab=2)
    good = be.embed(b)
    be.health()
    be.selftest_report_timeout(0, 104)  # DEV_TIMEOUT_ATTN
    with pytest.raises(BackendError) as e:
        be.embed(b)
    assert e.value.code == 5 and e.value.kind == "Inference" and "104" in str(e.value)
    # unhealthy now: health() runs the one-token probe, which passes, and the handle is back
    be.health()
    again = be.embed(b)
    for i in good:
        assert np.array_equal(good[i].values, again[i].values)
    # one shot: nothing is reported a second time
    be.embed(b)
    be.close()


def test_timeout_on_a_classifier_and_through_the_split_api(lib, model_dirs):
    from tei_b200.backend import BackendError
    be = _backend(model_dirs, "xlmr", "classifier", "cls")
    b = G.random_batch(6, [20, 77], 5, 1000, type_vocab=1, position_offset=2)
    want = be.predict(b)
    be.selftest_report_timeout(0, 102)
    with pytest.raises(BackendError) as e:
        be.predict(b)
    assert e.value.code == 5
    be.health()
    assert be.predict(b) == want
    # stage / run / sync: the code surfaces at the sync
    be.stage(b, predict=True)
    be.selftest_report_timeout(0, 103)
    be.run_staged()
    with pytest.raises(BackendError) as e:
        be.sync()
    assert e.value.code == 5
    be.health()
    be.close()


def test_health_probe_next_to_per_replica_callers(lib, model_dirs):
    """Two replicas of one GPU, one caller thread each; replica 0 reports a timeout, its caller
    sees the error, and health() probes while the other thread keeps calling embed_on: the probe
    takes replica 0's lock and leaves replica 1 and the handle's staged state alone."""
    from tei_b200.backend import BackendError
    be = _backend(model_dirs, "bert", devices=[0, 0])
    batches = [G.random_batch(50 + i, [30, 200, 7, 64], 0, 1000, type_vocab=2) for i in range(6)]
    want = [be.embed(b, replica=1) for b in batches]
    stop = threading.Event()
    errors, rounds = [], [0]

    def steady():  # replica 1 never fails
        try:
            while not stop.is_set():
                for b, w in zip(batches, want):
                    g = be.embed(b, replica=1)
                    for i in w:
                        assert np.array_equal(w[i].values, g[i].values)
                rounds[0] += 1
        except Exception as exc:
            errors.append(exc)

    t = threading.Thread(target=steady)
    t.start()
    try:
        for k in range(5):
            be.selftest_report_timeout(0, 104)
            with pytest.raises(BackendError):
                be.embed(batches[k], replica=0)
            be.health()  # probe on replica 0 while replica 1 is busy
            g = be.embed(batches[k], replica=0)
            assert sorted(g) == sorted(want[k])
    finally:
        stop.set()
        t.join()
    assert not errors, errors
    assert rounds[0] >= 1
    be.close()
