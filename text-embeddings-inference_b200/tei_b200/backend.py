"""Python mirror of the reference's backend interface on top of libtei_b200.so.

`B200Backend` has the constructor shape of `CandleBackend::new(model_path, dtype, model_type,
dense_paths)` (backends/candle/src/lib.rs:163-168) and the methods of the `Backend` trait
(backends/core/src/lib.rs:37-48): `health`, `max_batch_size`, `is_padded`, `embed`, `predict`.
`embed` returns `{batch position: Embedding}` and `predict` `{batch position: [scores]}` exactly
like the reference's `Embeddings` / `Predictions` IntMaps (lib.rs:694-706, 718-722).

All compute happens in the shared library; there is no fallback path.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import numpy as np

from . import _lib

POOLS = {"cls": 0, "mean": 1, "splade": 2, "last_token": 3}


class BackendError(Exception):
    """Mirror of text_embeddings_backend_core::BackendError (backends/core/src/lib.rs:84-95)."""

    KINDS = {1: "Start", 2: "Inference", 3: "Unhealthy", 4: "WeightsNotFound", 5: "Inference"}

    def __init__(self, code: int, message: str):
        self.code = code
        self.kind = self.KINDS.get(code, "Inference")
        super().__init__(f"{self.kind}: {message}" if message else self.kind)


@dataclass
class Batch:
    """Mirror of text_embeddings_backend_core::Batch (backends/core/src/lib.rs:9-17)."""

    input_ids: np.ndarray
    token_type_ids: np.ndarray
    position_ids: np.ndarray
    cumulative_seq_lengths: np.ndarray
    max_length: int
    pooled_indices: np.ndarray
    raw_indices: np.ndarray

    def __len__(self) -> int:
        return len(self.cumulative_seq_lengths) - 1


@dataclass
class Embedding:
    """`Embedding::Pooled(Vec<f32>)` or `Embedding::All(Vec<Vec<f32>>)`."""

    kind: str  # "pooled" | "all"
    values: np.ndarray


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint32))


def _ptr(a: Optional[np.ndarray], ctype):
    if a is None or a.size == 0:
        return None
    return a.ctypes.data_as(ctypes.POINTER(ctype))


class B200Backend:
    def __init__(self, model_path, dtype: str = "float16", model_type: Union[str, tuple] = "embedding",
                 pool: str = "cls", dense_paths: Optional[Sequence[str]] = None,
                 devices: Optional[Sequence[int]] = None):
        self._lib = _lib.load()
        self._h = ctypes.c_void_p()
        mt = 0 if model_type == "classifier" else 1
        devs = list(devices) if devices else [0]
        arr = (ctypes.c_int * len(devs))(*devs)
        err = ctypes.create_string_buffer(1024)
        rc = self._lib.tei_b200_create(str(model_path).encode(), dtype.encode(), mt, POOLS[pool], arr,
                                       len(devs), ctypes.byref(self._h), err, len(err))
        if rc != 0:
            self._h = ctypes.c_void_p()
            raise BackendError(rc, err.value.decode(errors="replace"))
        self.warnings = []
        for dense_path in dense_paths or []:
            err = ctypes.create_string_buffer(1024)
            rc = self._lib.tei_b200_add_dense(self._h, str(dense_path).encode(), err, len(err))
            if rc != 0:
                msg = err.value.decode(errors="replace")
                self.close()
                raise BackendError(rc, msg)
            if err.value:
                self.warnings.append(err.value.decode(errors="replace"))
        self.output_dim = self._lib.tei_b200_output_dim(self._h)
        self.hidden_size = self._lib.tei_b200_hidden_size(self._h)
        self.num_classes = self._lib.tei_b200_num_classes(self._h)
        # first position id of every sequence (router/src/lib.rs:184-192)
        self.position_offset = int(self._lib.tei_b200_position_offset(self._h))
        self._keep = None

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            self._lib.tei_b200_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ Backend trait
    def health(self) -> None:
        rc = self._lib.tei_b200_health(self._h)
        if rc != 0:
            raise BackendError(rc, "")

    def max_batch_size(self) -> Optional[int]:
        v = self._lib.tei_b200_max_batch_size(self._h)
        return None if v < 0 else v

    def is_padded(self) -> bool:
        return bool(self._lib.tei_b200_is_padded(self._h))

    def _arrays(self, batch):
        ids = _u32(batch.input_ids)
        types = _u32(batch.token_type_ids)
        pos = _u32(batch.position_ids)
        cu = _u32(batch.cumulative_seq_lengths)
        pooled = _u32(batch.pooled_indices)
        raw = _u32(batch.raw_indices)
        return ids, types, pos, cu, pooled, raw

    @property
    def num_replicas(self) -> int:
        return int(self._lib.tei_b200_num_replicas(self._h))

    def embed(self, batch, normalize: bool = False, replica: Optional[int] = None) -> Dict[int, Embedding]:
        """`replica=None`: the batch is split over every replica of the handle (one caller at a
        time).  `replica=i`: the whole batch runs on replica i; callers with different indices may
        run at the same time from different threads (one backend thread per replica instead of the
        single one of backends/src/lib.rs:612-647)."""
        ids, types, pos, cu, pooled, raw = self._arrays(batch)
        n_seqs = len(cu) - 1
        lengths = (cu[1:].astype(np.int64) - cu[:-1].astype(np.int64))
        raw_rows = int(sum(int(lengths[i]) for i in raw)) if raw.size and raw.max(initial=0) < n_seqs else 0
        pooled_out = np.empty((len(pooled), self.output_dim), dtype=np.float32)
        raw_out = np.empty((raw_rows, self.hidden_size), dtype=np.float32)
        err = ctypes.create_string_buffer(1024)
        c_u32, c_f = ctypes.c_uint32, ctypes.c_float
        tail = (_ptr(ids, c_u32), _ptr(types, c_u32), _ptr(pos, c_u32), ids.size, _ptr(cu, c_u32),
                n_seqs, int(batch.max_length), _ptr(pooled, c_u32), pooled.size, _ptr(raw, c_u32), raw.size,
                int(normalize), _ptr(pooled_out, c_f), _ptr(raw_out, c_f), err, len(err))
        if replica is None:
            rc = self._lib.tei_b200_embed(self._h, *tail)
        else:
            rc = self._lib.tei_b200_embed_on(self._h, int(replica), *tail)
        if rc != 0:
            raise BackendError(rc, err.value.decode(errors="replace"))
        out: Dict[int, Embedding] = {}
        for i, idx in enumerate(pooled):
            out[int(idx)] = Embedding("pooled", pooled_out[i])
        row = 0
        for idx in raw:
            n = int(lengths[idx])
            out[int(idx)] = Embedding("all", raw_out[row:row + n])
            row += n
        return out

    def predict(self, batch, replica: Optional[int] = None) -> Dict[int, List[float]]:
        ids, types, pos, cu, _, _ = self._arrays(batch)
        n_seqs = len(cu) - 1
        scores = np.empty((max(n_seqs, 0), max(self.num_classes, 1)), dtype=np.float32)
        err = ctypes.create_string_buffer(1024)
        c_u32, c_f = ctypes.c_uint32, ctypes.c_float
        tail = (_ptr(ids, c_u32), _ptr(types, c_u32), _ptr(pos, c_u32), ids.size, _ptr(cu, c_u32),
                n_seqs, int(batch.max_length), _ptr(scores, c_f), err, len(err))
        if replica is None:
            rc = self._lib.tei_b200_predict(self._h, *tail)
        else:
            rc = self._lib.tei_b200_predict_on(self._h, int(replica), *tail)
        if rc != 0:
            raise BackendError(rc, err.value.decode(errors="replace"))
        return {i: scores[i].tolist() for i in range(n_seqs)}

    # ------------------------------------------------------------------ resident-batch phases
    def stage(self, batch, normalize: bool = False, predict: bool = False) -> None:
        ids, types, pos, cu, pooled, raw = self._arrays(batch)
        self._keep = (ids, types, pos, cu, pooled, raw)
        err = ctypes.create_string_buffer(1024)
        c_u32 = ctypes.c_uint32
        rc = self._lib.tei_b200_stage(
            self._h, _ptr(ids, c_u32), _ptr(types, c_u32), _ptr(pos, c_u32), ids.size, _ptr(cu, c_u32),
            len(cu) - 1, int(batch.max_length), _ptr(pooled, c_u32), pooled.size, _ptr(raw, c_u32),
            raw.size, int(normalize), int(predict), err, len(err))
        if rc != 0:
            raise BackendError(rc, err.value.decode(errors="replace"))

    def run_staged(self) -> None:
        err = ctypes.create_string_buffer(1024)
        rc = self._lib.tei_b200_run_staged(self._h, err, len(err))
        if rc != 0:
            raise BackendError(rc, err.value.decode(errors="replace"))

    def sync(self) -> None:
        err = ctypes.create_string_buffer(1024)
        rc = self._lib.tei_b200_sync(self._h, err, len(err))
        if rc != 0:
            raise BackendError(rc, err.value.decode(errors="replace"))

    def run_staged_timed(self, steps: int) -> float:
        """Device milliseconds of `steps` back-to-back forwards of the staged batch."""
        err = ctypes.create_string_buffer(1024)
        ms = ctypes.c_double(0.0)
        rc = self._lib.tei_b200_run_staged_timed(self._h, int(steps), ctypes.byref(ms), err, len(err))
        if rc != 0:
            raise BackendError(rc, err.value.decode(errors="replace"))
        return ms.value

    def fetch(self, n_pooled: int = 0, raw_rows: int = 0, n_scores_rows: int = 0):
        pooled = np.empty((n_pooled, self.output_dim), dtype=np.float32)
        raw = np.empty((raw_rows, self.hidden_size), dtype=np.float32)
        scores = np.empty((n_scores_rows, max(self.num_classes, 1)), dtype=np.float32)
        err = ctypes.create_string_buffer(1024)
        c_f = ctypes.c_float
        rc = self._lib.tei_b200_fetch(self._h, _ptr(pooled, c_f), _ptr(raw, c_f), _ptr(scores, c_f), err, len(err))
        if rc != 0:
            raise BackendError(rc, err.value.decode(errors="replace"))
        return pooled, raw, scores

    KERNEL_CLASSES = ["embedding", "gemm", "attention", "norm", "rotary", "pool_heads"]

    def set_profiling(self, on: bool) -> None:
        self._lib.tei_b200_set_profiling(self._h, int(on))

    def kernel_times(self) -> dict:
        ms = (ctypes.c_double * 6)()
        ln = (ctypes.c_double * 6)()
        n = self._lib.tei_b200_kernel_times(self._h, ms, ln, 6)
        return {self.KERNEL_CLASSES[i]: {"ms": ms[i], "launches": ln[i]} for i in range(n)}

    def set_last_layer_shortcut(self, on: bool) -> None:
        """Off: every call computes every row of the last layer, as the reference does."""
        self._lib.tei_b200_set_last_layer_shortcut(self._h, int(on))

    def set_fused_rope(self, on) -> None:
        """True: RoPE / q-k RMSNorm in the epilogue of the q/k/v projection; False: a kernel of
        their own behind it; None: whichever is faster for the model (the default)."""
        self._lib.tei_b200_set_fused_rope(self._h, -1 if on is None else int(bool(on)))

    def set_fused_residual(self, on: bool) -> None:
        """On: the feed-forward residual of the post-LN models is added in the output projection's
        epilogue; off (the default): by the LayerNorm kernel behind it, as in the reference."""
        self._lib.tei_b200_set_fused_residual(self._h, int(bool(on)))

    def selftest_report_timeout(self, replica: int = 0, device_code: int = 104) -> None:
        """The next forward on `replica` reports `device_code` through the status word, like a
        kernel whose bounded wait ran out (self-test of the TIMEOUT path; nothing hangs)."""
        rc = self._lib.tei_b200_selftest_report_timeout(self._h, int(replica), int(device_code))
        if rc != 0:
            raise BackendError(rc, "selftest_report_timeout")

    def stats(self) -> dict:
        buf = (ctypes.c_double * 8)()
        n = self._lib.tei_b200_stats(self._h, buf, 8)
        keys = ["gpu_ms", "h2d_bytes", "d2h_bytes", "launches", "tokens", "calls", "total_gpu_ms",
                "total_tokens"]
        return {k: buf[i] for i, k in enumerate(keys[:n])}


def plan_shards(cumulative_seq_lengths, n_shards: int, linear_cost: float, quadratic_cost: float) -> np.ndarray:
    """Replica of every sequence for a handle with n_shards devices (host-only helper)."""
    lib = _lib.load()
    cu = _u32(cumulative_seq_lengths)
    out = np.zeros(len(cu) - 1, dtype=np.int32)
    rc = lib.tei_b200_plan_shards(_ptr(cu, ctypes.c_uint32), len(cu) - 1, int(n_shards), float(linear_cost),
                                  float(quadratic_cost), out.ctypes.data_as(ctypes.POINTER(ctypes.c_int)))
    if rc != 0:
        raise BackendError(rc, "plan_shards")
    return out
