"""The `embedding.v1.EmbeddingService` adapter (tei_b200/grpc_server.py) on CPU: message classes
match backends/proto/embed.proto field by field, and a client speaking that protocol over a Unix
socket gets one row per sequence in batch order from whatever implements the Backend-trait
methods - here a stand-in, so no GPU is needed."""
import os
import sys
import types

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "text-embeddings-inference_b200"))

grpc = pytest.importorskip("grpc")
from tei_b200 import grpc_server as GS  # noqa: E402


def test_messages_follow_the_proto_file():
    m = GS.message_classes()
    # backends/proto/embed.proto:17-24: field numbers 1..5 of EmbedRequest
    fields = {f.name: (f.number, f.type) for f in m["EmbedRequest"].DESCRIPTOR.fields}
    U32 = 13  # FieldDescriptor.TYPE_UINT32
    assert fields == {"input_ids": (1, U32), "token_type_ids": (2, U32), "position_ids": (3, U32),
                      "cu_seq_lengths": (4, U32), "max_length": (5, U32)}
    assert [f.name for f in m["EmbedResponse"].DESCRIPTOR.fields] == ["embeddings"]
    assert [f.name for f in m["PredictResponse"].DESCRIPTOR.fields] == ["scores"]
    assert m["Embedding"].DESCRIPTOR.fields[0].type == 2  # TYPE_FLOAT
    # known wire bytes: packed repeated uint32 [1, 300] in field 1, max_length 7 in field 5
    req = m["EmbedRequest"](input_ids=[1, 300], max_length=7)
    assert req.SerializeToString() == bytes([0x0A, 0x03, 0x01, 0xAC, 0x02, 0x28, 0x07])
    assert m["HealthRequest"]().SerializeToString() == b""


class _StandIn:
    """Pooled row of sequence i = [i, length_i, sum of its ids]; scores = [length_i]."""

    def __init__(self):
        self.healthy = True

    def embed(self, batch):
        cu = batch.cumulative_seq_lengths.astype(np.int64)
        assert list(batch.pooled_indices) == list(range(len(cu) - 1)) and len(batch.raw_indices) == 0
        out = {}
        for i in range(len(cu) - 1):
            ids = batch.input_ids[cu[i]:cu[i + 1]]
            out[i] = types.SimpleNamespace(kind="pooled", values=np.array([i, len(ids), ids.sum()], dtype=np.float32))
        return out

    def predict(self, batch):
        cu = batch.cumulative_seq_lengths.astype(np.int64)
        return {i: [float(cu[i + 1] - cu[i])] for i in range(len(cu) - 1)}

    def health(self):
        if not self.healthy:
            raise RuntimeError("unhealthy")


def _call(channel, m, method, req, resp_name):
    fn = channel.unary_unary(f"/{GS.SERVICE}/{method}", request_serializer=lambda x: x.SerializeToString(),
                             response_deserializer=m[resp_name].FromString)
    return fn(req, timeout=20)


@pytest.mark.parametrize("classifier", [False, True])
def test_round_trip_over_a_unix_socket(tmp_path, classifier):
    uds = str(tmp_path / "sock")
    backend = _StandIn()
    server = GS.serve(GS.EmbeddingService(backend, classifier), uds)
    try:
        assert os.path.exists(uds)  # the readiness signal (backends/python/src/management.rs:136-138)
        m = GS.message_classes()
        with grpc.insecure_channel(f"unix://{uds}") as ch:
            req = m["EmbedRequest"](input_ids=[5, 6, 7, 100, 200], token_type_ids=[0] * 5, position_ids=[0, 1, 2, 0, 1],
                                    cu_seq_lengths=[0, 3, 5], max_length=3)
            _call(ch, m, "Health", m["HealthRequest"](), "HealthResponse")
            if classifier:
                resp = _call(ch, m, "Predict", req, "PredictResponse")
                assert [list(s.values) for s in resp.scores] == [[3.0], [2.0]]
                with pytest.raises(grpc.RpcError) as e:
                    _call(ch, m, "Embed", req, "EmbedResponse")
                assert "not implemented" in e.value.details()
            else:
                resp = _call(ch, m, "Embed", req, "EmbedResponse")
                assert [list(e.values) for e in resp.embeddings] == [[0.0, 3.0, 18.0], [1.0, 2.0, 300.0]]
                with pytest.raises(grpc.RpcError):
                    _call(ch, m, "Predict", req, "PredictResponse")
            backend.healthy = False
            with pytest.raises(grpc.RpcError):
                _call(ch, m, "Health", m["HealthRequest"](), "HealthResponse")
    finally:
        server.stop(grace=None)


def test_classifier_detection(tmp_path):
    (tmp_path / "config.json").write_text('{"architectures": ["XLMRobertaForSequenceClassification"]}')
    assert GS.is_classifier(tmp_path)
    (tmp_path / "config.json").write_text('{"architectures": ["BertModel"]}')
    assert not GS.is_classifier(tmp_path)


class _TwoReplicas(_StandIn):
    """Stand-in with two replicas: records which replica served each call and how many calls
    were inside `embed` at once."""

    num_replicas = 2

    def __init__(self):
        super().__init__()
        import threading
        self.lock = threading.Lock()
        self.inside = 0
        self.peak = 0
        self.busy = set()
        self.served = []

    def embed(self, batch, replica=None):
        import time
        with self.lock:
            assert replica in (0, 1) and replica not in self.busy  # a replica serves one call at a time
            self.busy.add(replica)
            self.inside += 1
            self.peak = max(self.peak, self.inside)
            self.served.append(replica)
        time.sleep(0.05)
        out = _StandIn.embed(self, batch)
        with self.lock:
            self.busy.discard(replica)
            self.inside -= 1
        return out


def test_per_replica_dispatch_runs_calls_concurrently(tmp_path):
    from concurrent.futures import ThreadPoolExecutor
    uds = str(tmp_path / "sock2")
    backend = _TwoReplicas()
    server = GS.serve(GS.EmbeddingService(backend, False, per_replica=True), uds)
    try:
        m = GS.message_classes()
        with grpc.insecure_channel(f"unix://{uds}") as ch:
            def one(k):
                req = m["EmbedRequest"](input_ids=[k, k + 1], token_type_ids=[0, 0], position_ids=[0, 1],
                                        cu_seq_lengths=[0, 2], max_length=2)
                resp = _call(ch, m, "Embed", req, "EmbedResponse")
                return list(resp.embeddings[0].values)
            with ThreadPoolExecutor(max_workers=6) as ex:
                rows = list(ex.map(one, range(12)))
        assert rows == [[0.0, 2.0, float(2 * k + 1)] for k in range(12)]
        assert backend.peak == 2               # both replicas were busy at once, never more
        assert set(backend.served) == {0, 1}
    finally:
        server.stop(grace=None)
