"""TEST INFRASTRUCTURE - CPU restatement of how the reference packs requests into a `Batch`.

Only tests/, `__graft_entry__.smoke()` and bench.py's cpu_baseline / reference legs may import
this package; the product path (libtei_b200.so and the `tei_b200` host package) never does.

Follows, in plain Python integers (bit-exact by construction):
  * `struct Batch`                      backends/core/src/lib.rs:9-27
  * `queue_blocking_task` NextBatch arm core/src/queue.rs:118-200 (unpadded rule :150-155,
                                        max_batch_requests :179, pooled / raw split :162-165)
  * test helper `batch(...)`            backends/candle/tests/common.rs:327-356
  * `position_ids = offset..len+offset` core/src/tokenization.rs:406-411, with the offset of
                                        router/src/lib.rs:185-192 (pad_token_id + 1 for the
                                        RoBERTa family, else 0)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np


@dataclass
class Batch:
    """Mirror of text_embeddings_backend_core::Batch; every array is uint32."""

    input_ids: np.ndarray
    token_type_ids: np.ndarray
    position_ids: np.ndarray
    cumulative_seq_lengths: np.ndarray
    max_length: int
    pooled_indices: np.ndarray
    raw_indices: np.ndarray

    def __len__(self) -> int:
        return len(self.cumulative_seq_lengths) - 1

    def lengths(self) -> np.ndarray:
        cu = self.cumulative_seq_lengths.astype(np.int64)
        return cu[1:] - cu[:-1]


@dataclass
class Request:
    """One queue entry: the tokenizer's output plus the `pooling` flag of its metadata."""

    input_ids: Sequence[int]
    token_type_ids: Optional[Sequence[int]] = None
    pooling: bool = True
    position_offset: int = 0
    position_ids: Optional[Sequence[int]] = field(default=None)

    def resolved(self) -> Tuple[List[int], List[int], List[int]]:
        ids = [int(x) for x in self.input_ids]
        types = [0] * len(ids) if self.token_type_ids is None else [int(x) for x in self.token_type_ids]
        if self.position_ids is None:
            pos = list(range(self.position_offset, len(ids) + self.position_offset))
        else:
            pos = [int(x) for x in self.position_ids]
        assert len(types) == len(ids) and len(pos) == len(ids)
        return ids, types, pos


def _u32(xs) -> np.ndarray:
    return np.asarray(xs, dtype=np.uint32)


def next_batch(
    queue: List[Request],
    max_batch_tokens: int,
    max_batch_requests: Optional[int] = None,
    padded_model: bool = False,
) -> Tuple[Optional[Batch], List[Request]]:
    """One NextBatch command: pops requests FIFO from `queue` and returns (batch, rest).

    Restates core/src/queue.rs:124-200.  Dropped-client filtering (:142-146) has no counterpart
    here because a Request has no response channel.
    """
    input_ids: List[int] = []
    token_type_ids: List[int] = []
    position_ids: List[int] = []
    pooled_indices: List[int] = []
    raw_indices: List[int] = []
    cu = [0]
    current_tokens = 0
    max_length = 0
    entry_index = 0
    taken = 0
    rest = list(queue)
    while rest:
        entry = rest[0]
        ids, types, pos = entry.resolved()
        entry_tokens = len(ids)
        if padded_model:
            total_tokens = max(max_length, entry_tokens) * (taken + 1)
        else:
            total_tokens = current_tokens + entry_tokens
        if total_tokens > max_batch_tokens:
            break
        rest.pop(0)
        (pooled_indices if entry.pooling else raw_indices).append(entry_index)
        max_length = max(max_length, entry_tokens)
        input_ids.extend(ids)
        token_type_ids.extend(types)
        position_ids.extend(pos)
        current_tokens += entry_tokens
        taken += 1
        cu.append(current_tokens)
        entry_index += 1
        if max_batch_requests is not None and taken == max_batch_requests:
            break
    if taken == 0:
        return None, rest
    return (
        Batch(_u32(input_ids), _u32(token_type_ids), _u32(position_ids), _u32(cu), max_length,
              _u32(pooled_indices), _u32(raw_indices)),
        rest,
    )


def batch_from_encodings(
    encodings: Sequence[Sequence[int]],
    pooled_indices: Sequence[int],
    raw_indices: Sequence[int],
    type_ids: Optional[Sequence[Sequence[int]]] = None,
    position_offset: int = 0,
) -> Batch:
    """The reference tests' `batch(encodings, pooled_indices, raw_indices)` helper
    (backends/candle/tests/common.rs:327-356): positions restart at 0 for every sequence
    (plus `position_offset`, which the router adds for the RoBERTa family)."""
    input_ids: List[int] = []
    token_type_ids: List[int] = []
    position_ids: List[int] = []
    cu = [0]
    max_length = 0
    total = 0
    for i, enc in enumerate(encodings):
        n = len(enc)
        input_ids.extend(int(x) for x in enc)
        token_type_ids.extend([0] * n if type_ids is None else [int(x) for x in type_ids[i]])
        position_ids.extend(range(position_offset, n + position_offset))
        total += n
        cu.append(total)
        max_length = max(max_length, n)
    return Batch(_u32(input_ids), _u32(token_type_ids), _u32(position_ids), _u32(cu), max_length,
                 _u32(pooled_indices), _u32(raw_indices))


def split_batch(batch: Batch, shard_of_seq: Sequence[int], n_shards: int):
    """Splits a packed batch at sequence boundaries into per-replica batches.

    Returns [(Batch, original batch positions)] per shard; sequences keep their relative order.
    The reference has no counterpart (it is single-GPU, backends/candle/src/lib.rs:241); this is
    the oracle of the replica sharding the library performs inside one embed call.
    """
    cu = batch.cumulative_seq_lengths.astype(np.int64)
    pooled = set(int(i) for i in batch.pooled_indices)
    out = []
    for d in range(n_shards):
        members = [s for s in range(len(batch)) if shard_of_seq[s] == d]
        ids, types, pos, cu_d = [], [], [], [0]
        p_idx, r_idx = [], []
        mx = 0
        for j, s in enumerate(members):
            a, b = int(cu[s]), int(cu[s + 1])
            ids.extend(batch.input_ids[a:b].tolist())
            types.extend(batch.token_type_ids[a:b].tolist())
            pos.extend(batch.position_ids[a:b].tolist())
            cu_d.append(cu_d[-1] + (b - a))
            mx = max(mx, b - a)
            (p_idx if s in pooled else r_idx).append(j)
        out.append((Batch(_u32(ids), _u32(types), _u32(pos), _u32(cu_d), mx, _u32(p_idx), _u32(r_idx)),
                    members))
    return out
