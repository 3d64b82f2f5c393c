"""The batching queue of libtei_b200.so from Python.

`BatchQueue` has the shape of `Queue` (core/src/queue.rs:40-96): `append` one encoded request,
`next_batch` packs the longest FIFO prefix that fits `max_batch_tokens` / `max_batch_requests`
into a `Batch` (backends/core/src/lib.rs:9-27) and returns it with the requests' tags (the
reference returns their `Metadata`).  The packing itself happens in the shared library
(`csrc/queue.cpp`); several threads may append and ask for batches at once, which is what a
host with one consumer per replica needs.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from .backend import BackendError, Batch


class BatchQueue:
    def __init__(self, max_batch_tokens: int, max_batch_requests: Optional[int] = None,
                 padded_model: bool = False):
        self._lib = _lib.load()
        self._q = ctypes.c_void_p()
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_batch_requests = None if max_batch_requests is None else int(max_batch_requests)
        rc = self._lib.tei_b200_queue_create(int(padded_model), self.max_batch_tokens,
                                             self.max_batch_requests or 0, ctypes.byref(self._q))
        if rc != 0:
            raise BackendError(rc, "could not create the queue (max_batch_tokens must be positive)")

    def close(self):
        if self._q:
            self._lib.tei_b200_queue_destroy(self._q)
            self._q = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __len__(self) -> int:
        return int(self._lib.tei_b200_queue_len(self._q))

    def append(self, input_ids: Sequence[int], token_type_ids: Optional[Sequence[int]] = None,
               position_ids: Optional[Sequence[int]] = None, pooling: bool = True, tag: int = 0,
               position_offset: int = 0) -> None:
        u32 = ctypes.POINTER(ctypes.c_uint32)
        ids = np.ascontiguousarray(np.asarray(input_ids, dtype=np.uint32))
        types = None if token_type_ids is None else np.ascontiguousarray(np.asarray(token_type_ids, dtype=np.uint32))
        pos = None if position_ids is None else np.ascontiguousarray(np.asarray(position_ids, dtype=np.uint32))
        for other in (types, pos):
            if other is not None and other.size != ids.size:
                raise BackendError(2, "token_type_ids / position_ids must be as long as input_ids")
        rc = self._lib.tei_b200_queue_append(
            self._q, ids.ctypes.data_as(u32), None if types is None else types.ctypes.data_as(u32),
            None if pos is None else pos.ctypes.data_as(u32), ids.size, int(position_offset), int(bool(pooling)),
            int(tag))
        if rc != 0:
            raise BackendError(rc, "the queue refused the request (empty encoding?)")

    def cancel(self, tag: int) -> int:
        n = ctypes.c_size_t(0)
        self._lib.tei_b200_queue_cancel(self._q, int(tag), ctypes.byref(n))
        return int(n.value)

    def next_batch(self, token_cap: Optional[int] = None,
                   seq_cap: Optional[int] = None) -> Optional[Tuple[Batch, List[int]]]:
        """`(batch, tags)` or None.  The buffer sizes default to the queue's own limits (with no
        `max_batch_requests`, one request per token is the worst case)."""
        tcap = self.max_batch_tokens if token_cap is None else int(token_cap)
        scap = (self.max_batch_requests or min(tcap, max(len(self), 1))) if seq_cap is None else int(seq_cap)
        u32 = ctypes.POINTER(ctypes.c_uint32)
        ids, types, pos = (np.empty(tcap, dtype=np.uint32) for _ in range(3))
        cu = np.empty(scap + 1, dtype=np.uint32)
        pooled, raw = np.empty(scap, dtype=np.uint32), np.empty(scap, dtype=np.uint32)
        tags = np.empty(scap, dtype=np.uint64)
        n_tok, n_seq, n_p, n_r = (ctypes.c_size_t(0) for _ in range(4))
        mx = ctypes.c_uint32(0)
        rc = self._lib.tei_b200_queue_next_batch(
            self._q, ids.ctypes.data_as(u32), types.ctypes.data_as(u32), pos.ctypes.data_as(u32), tcap,
            cu.ctypes.data_as(u32), pooled.ctypes.data_as(u32), raw.ctypes.data_as(u32),
            tags.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)), scap, ctypes.byref(n_tok), ctypes.byref(n_seq),
            ctypes.byref(n_p), ctypes.byref(n_r), ctypes.byref(mx))
        if rc != 0:
            raise BackendError(rc, "next_batch failed")
        if n_seq.value == 0:
            return None
        t, s = n_tok.value, n_seq.value
        batch = Batch(ids[:t].copy(), types[:t].copy(), pos[:t].copy(), cu[:s + 1].copy(), int(mx.value),
                      pooled[:n_p.value].copy(), raw[:n_r.value].copy())
        return batch, [int(x) for x in tags[:s]]
