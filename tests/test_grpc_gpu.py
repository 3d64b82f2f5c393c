"""The gRPC adapter in front of the real backend, started the way the TEI router starts its
Python backend (backends/python/src/management.rs:43-75): a child process with the model path,
dtype, socket path and pool on its command line; the socket file appearing means ready."""
import os
import signal
import subprocess
import sys
import time

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from oracle import generators as G  # noqa: E402

pytestmark = pytest.mark.gpu
grpc = pytest.importorskip("grpc")
PKG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "text-embeddings-inference_b200")


def _spawn(model_dir, uds, pool, dtype="float16"):
    env = dict(os.environ, PYTHONPATH=PKG + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.Popen(
        [sys.executable, "-m", "tei_b200.grpc_server", str(model_dir), "--dtype", dtype, "--uds-path", uds,
         "--logger-level", "INFO", "--json-output", "--pool", pool, "--otlp-service-name", "test"],
        env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    t0 = time.time()
    while not os.path.exists(uds):
        if p.poll() is not None:
            raise RuntimeError("server exited: " + p.stdout.read().decode(errors="replace")[-2000:])
        if time.time() - t0 > 240:
            p.kill()
            raise RuntimeError("server did not become ready")
        time.sleep(0.05)
    return p


def _stop(p):
    p.send_signal(signal.SIGTERM)
    try:
        p.wait(timeout=30)
    except subprocess.TimeoutExpired:
        p.kill()
        p.wait()


def _request(m, batch):
    return m["EmbedRequest"](input_ids=batch.input_ids.tolist(), token_type_ids=batch.token_type_ids.tolist(),
                             position_ids=batch.position_ids.tolist(),
                             cu_seq_lengths=batch.cumulative_seq_lengths.tolist(), max_length=int(batch.max_length))


def _call(ch, m, method, req, resp_name):
    from tei_b200 import grpc_server as GS
    fn = ch.unary_unary(f"/{GS.SERVICE}/{method}", request_serializer=lambda x: x.SerializeToString(),
                        response_deserializer=m[resp_name].FromString)
    return fn(req, timeout=120)


def test_embed_and_predict_through_the_socket(lib, model_dirs, tmp_path):
    import tei_b200
    from tei_b200 import grpc_server as GS
    m = GS.message_classes()
    # embedding model, mean pooling ("lasttoken" etc. are spelled as the router spells them)
    uds = str(tmp_path / "embed.sock")
    p = _spawn(model_dirs["bert"], uds, "mean")
    try:
        b = G.random_batch(71, [7, 300, 33, 129], 0, 1000, type_vocab=2)
        with grpc.insecure_channel(f"unix://{uds}") as ch:
            _call(ch, m, "Health", m["HealthRequest"](), "HealthResponse")
            resp = _call(ch, m, "Embed", _request(m, b), "EmbedResponse")
            got = np.array([list(e.values) for e in resp.embeddings], dtype=np.float32)
            # an id beyond the vocabulary comes back as an error value, and the server lives on
            bad = _request(m, b)
            bad.input_ids[0] = 50000
            with pytest.raises(grpc.RpcError):
                _call(ch, m, "Embed", bad, "EmbedResponse")
            again = _call(ch, m, "Embed", _request(m, b), "EmbedResponse")
            assert np.array_equal(got, np.array([list(e.values) for e in again.embeddings], dtype=np.float32))
    finally:
        _stop(p)
    be = tei_b200.B200Backend(model_dirs["bert"], "float16", "embedding", "mean")
    want = be.embed(b)
    be.close()
    assert got.shape == (4, 128)
    for i in range(4):
        assert np.array_equal(got[i], want[i].values)  # same library, same kernels: bit-identical

    # classifier: the server picks `predict` from config.json's architectures
    uds = str(tmp_path / "predict.sock")
    p = _spawn(model_dirs["xlmr"], uds, "cls")
    try:
        b = G.random_batch(72, [12, 200, 31], 5, 1000, position_offset=2)
        with grpc.insecure_channel(f"unix://{uds}") as ch:
            resp = _call(ch, m, "Predict", _request(m, b), "PredictResponse")
            scores = [list(s.values) for s in resp.scores]
    finally:
        _stop(p)
    be = tei_b200.B200Backend(model_dirs["xlmr"], "float16", "classifier")
    want = be.predict(b)
    be.close()
    assert len(scores) == 3 and all(len(s) == 1 for s in scores)
    for i in range(3):
        assert scores[i][0] == pytest.approx(want[i][0], abs=0.0)
