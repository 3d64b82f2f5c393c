"""`embedding.v1.EmbeddingService` over a Unix socket, in front of libtei_b200.so.

The unmodified TEI router, built with its `python` backend feature, spawns an executable called
`python-text-embeddings-server` with

    <model_path> --dtype <dtype> --uds-path <path> --logger-level INFO --json-output
                 --pool <cls|mean|lasttoken|splade> [--otlp-endpoint <url>] --otlp-service-name <name>

(backends/python/src/management.rs:19-75), treats the appearance of the socket file as "ready"
(`:136-138`) and then talks the protocol of backends/proto/embed.proto:5-40 through
backends/grpc-client/src/client.rs:26-87: `Embed` and `Predict` take the packed batch
(`input_ids`, `token_type_ids`, `position_ids`, `cu_seq_lengths`, `max_length`) and return one
pooled row / one score row per sequence, in batch order; `Health` takes and returns nothing.
Raw (per-token) embeddings do not exist on this protocol (backends/python/src/lib.rs:76-80).

This module is that executable's body: `python -m tei_b200.grpc_server ...` (or a two-line
wrapper script named `python-text-embeddings-server` on PATH) serves a model directory with the
CUDA backend.  The message classes are built at run time from the .proto's definition, so no
generated stubs are needed.  Like the reference's Python server it decides between embedding and
classifier from `architectures[0]` of config.json
(backends/python/server/text_embeddings_server/models/__init__.py:112-113,132-133).
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import sys
import threading
from concurrent import futures
from pathlib import Path
from typing import Optional

import numpy as np

SERVICE = "embedding.v1.EmbeddingService"
POOLS = {"cls": "cls", "mean": "mean", "lasttoken": "last_token", "last_token": "last_token", "splade": "splade"}


def message_classes():
    """Message classes of backends/proto/embed.proto, built from a descriptor written here."""
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

    f = descriptor_pb2.FileDescriptorProto()
    f.name = "tei_b200/embed.proto"
    f.package = "embedding.v1"
    f.syntax = "proto3"
    T = descriptor_pb2.FieldDescriptorProto

    def msg(name, fields):
        m = f.message_type.add()
        m.name = name
        for number, (fname, ftype, label, type_name) in enumerate(fields, start=1):
            fd = m.field.add()
            fd.name, fd.number, fd.type, fd.label = fname, number, ftype, label
            if type_name:
                fd.type_name = type_name

    rep, opt = T.LABEL_REPEATED, T.LABEL_OPTIONAL
    msg("HealthRequest", [])
    msg("HealthResponse", [])
    msg("EmbedRequest", [("input_ids", T.TYPE_UINT32, rep, None), ("token_type_ids", T.TYPE_UINT32, rep, None),
                         ("position_ids", T.TYPE_UINT32, rep, None), ("cu_seq_lengths", T.TYPE_UINT32, rep, None),
                         ("max_length", T.TYPE_UINT32, opt, None)])
    msg("Embedding", [("values", T.TYPE_FLOAT, rep, None)])
    msg("EmbedResponse", [("embeddings", T.TYPE_MESSAGE, rep, ".embedding.v1.Embedding")])
    msg("Score", [("values", T.TYPE_FLOAT, rep, None)])
    msg("PredictResponse", [("scores", T.TYPE_MESSAGE, rep, ".embedding.v1.Score")])
    pool = descriptor_pool.DescriptorPool()
    pool.Add(f)
    names = ["HealthRequest", "HealthResponse", "EmbedRequest", "Embedding", "EmbedResponse", "Score",
             "PredictResponse"]
    return {n: message_factory.GetMessageClass(pool.FindMessageTypeByName("embedding.v1." + n)) for n in names}


class _Batch:
    """The fields of `Batch` (backends/core/src/lib.rs:9-27) the backend reads; every sequence is
    pooled, none is raw (the protocol carries neither index list)."""

    def __init__(self, req):
        self.input_ids = np.asarray(req.input_ids, dtype=np.uint32)
        self.token_type_ids = np.asarray(req.token_type_ids, dtype=np.uint32)
        self.position_ids = np.asarray(req.position_ids, dtype=np.uint32)
        self.cumulative_seq_lengths = np.asarray(req.cu_seq_lengths, dtype=np.uint32)
        self.max_length = int(req.max_length)
        n = max(len(self.cumulative_seq_lengths) - 1, 0)
        self.pooled_indices = np.arange(n, dtype=np.uint32)
        self.raw_indices = np.zeros(0, dtype=np.uint32)

    def __len__(self):
        return len(self.pooled_indices)


class EmbeddingService:
    """The three RPCs on top of any object with the Backend-trait methods `embed`, `predict`
    and `health` (tei_b200.B200Backend, or a stand-in in the protocol tests).  The backend is
    single-caller (backends/src/lib.rs:618-644), so calls are serialised here; with
    `per_replica=True` every call instead takes one free replica of the handle and runs its
    whole batch there, so as many calls as replicas run at once."""

    def __init__(self, backend, classifier: bool, per_replica: bool = False):
        self.backend = backend
        self.classifier = classifier
        self.msgs = message_classes()
        self._lock = threading.Lock()
        self.workers = 1
        self._free = None
        if per_replica:
            import queue
            self.workers = int(backend.num_replicas)
            self._free = queue.SimpleQueue()
            for r in range(self.workers):
                self._free.put(r)

    def _run(self, method, batch):
        if self._free is None:
            with self._lock:
                return method(batch)
        r = self._free.get()
        try:
            return method(batch, replica=r)
        finally:
            self._free.put(r)

    def _abort(self, context, exc):
        import grpc
        context.abort(grpc.StatusCode.INTERNAL, str(exc))

    def embed(self, request, context):
        m = self.msgs
        try:
            if self.classifier:
                raise RuntimeError("`embed` is not implemented for classifier models")
            batch = _Batch(request)
            rows = self._run(self.backend.embed, batch)
            resp = m["EmbedResponse"]()
            for i in range(len(batch)):
                resp.embeddings.add().values.extend(np.asarray(rows[i].values, dtype=np.float32).tolist())
            return resp
        except Exception as exc:  # errors are values on this boundary (BackendError::Inference)
            self._abort(context, exc)

    def predict(self, request, context):
        m = self.msgs
        try:
            if not self.classifier:
                raise RuntimeError("`predict` is not implemented for this model")
            batch = _Batch(request)
            scores = self._run(self.backend.predict, batch)
            resp = m["PredictResponse"]()
            for i in range(len(batch)):
                resp.scores.add().values.extend([float(v) for v in scores[i]])
            return resp
        except Exception as exc:
            self._abort(context, exc)

    def health(self, request, context):
        try:
            with self._lock:
                self.backend.health()
            return self.msgs["HealthResponse"]()
        except Exception as exc:
            self._abort(context, exc)

    def handler(self):
        import grpc
        m = self.msgs

        def unary(fn, req, resp):
            return grpc.unary_unary_rpc_method_handler(
                fn, request_deserializer=m[req].FromString, response_serializer=m[resp].SerializeToString)

        return grpc.method_handlers_generic_handler(SERVICE, {
            "Embed": unary(self.embed, "EmbedRequest", "EmbedResponse"),
            "Predict": unary(self.predict, "EmbedRequest", "PredictResponse"),
            "Health": unary(self.health, "HealthRequest", "HealthResponse"),
        })


def serve(service: EmbeddingService, uds_path: str):
    """Starts the server on `unix://<uds_path>`; the socket file appearing is the readiness
    signal the router waits for.  Returns the grpc server (call .stop() / .wait_for_termination())."""
    import grpc
    if os.path.exists(uds_path):
        os.remove(uds_path)
    # one worker per batch the backend can take at a time; no message size limit (a packed batch
    # of 16k tokens is small, but the router's budget is configurable)
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=service.workers),
                         options=[("grpc.max_receive_message_length", -1), ("grpc.max_send_message_length", -1)])
    server.add_generic_rpc_handlers((service.handler(),))
    server.add_insecure_port(f"unix://{uds_path}")
    server.start()
    return server


def is_classifier(model_path) -> bool:
    cfg = json.loads((Path(model_path) / "config.json").read_text())
    arch = (cfg.get("architectures") or [""])[0]
    return arch.endswith("Classification")


def main(argv: Optional[list] = None) -> int:
    ap = argparse.ArgumentParser(prog="python-text-embeddings-server")
    ap.add_argument("model_path")
    ap.add_argument("--dtype", default="float16")
    ap.add_argument("--uds-path", default="/tmp/text-embeddings-server")
    ap.add_argument("--logger-level", default="INFO")
    ap.add_argument("--json-output", action="store_true")
    ap.add_argument("--pool", default="cls")
    ap.add_argument("--otlp-endpoint", default=None)
    ap.add_argument("--otlp-service-name", default="text-embeddings-inference.server")
    ap.add_argument("--devices", default=os.environ.get("TEI_B200_DEVICES", "0"),
                    help="comma-separated CUDA indices: one replica each (an index may repeat)")
    ap.add_argument("--dispatch", default=os.environ.get("TEI_B200_DISPATCH", "split"), choices=["split", "per-replica"],
                    help="split: every batch is split across the replicas (one call at a time, what the "
                         "unmodified router sends); per-replica: concurrent calls each take one free replica")
    args = ap.parse_args(argv)

    def log(level, message):
        line = json.dumps({"level": level, "message": message}) if args.json_output else f"{level} {message}"
        print(line, flush=True)

    import tei_b200
    classifier = is_classifier(args.model_path)
    dtype = {"float16": "float16", "bfloat16": "bfloat16"}.get(args.dtype)
    if dtype is None:
        log("ERROR", f"DType {args.dtype} is not supported (float16 or bfloat16)")
        return 1
    pool = POOLS.get(args.pool)
    if pool is None:
        log("ERROR", f"unknown pool {args.pool}")
        return 1
    devices = [int(d) for d in args.devices.split(",") if d.strip()]
    try:
        backend = tei_b200.B200Backend(args.model_path, dtype, "classifier" if classifier else "embedding", pool,
                                       devices=devices)
    except tei_b200.BackendError as exc:
        log("ERROR", f"Could not start backend: {exc}")
        return 1
    server = serve(EmbeddingService(backend, classifier, per_replica=args.dispatch == "per-replica"), args.uds_path)
    log("INFO", f"Server started at unix://{args.uds_path}")
    stop = threading.Event()
    for sig in (signal.SIGTERM, signal.SIGINT):
        signal.signal(sig, lambda *_: stop.set())
    stop.wait()
    server.stop(grace=1.0)
    backend.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
