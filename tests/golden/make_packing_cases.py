"""Writes tests/golden/packing_cases.json: packing cases whose expected `Batch` was derived by
hand from the rules of core/src/queue.rs:118-200 (FIFO, `current_tokens + len >
max_batch_tokens` stops the batch, `max_batch_requests`, pooled / raw split by the request's
`pooling` flag, cumulative lengths starting at 0) and core/src/tokenization.rs:406-411
(`position_ids = offset .. len + offset`).  The expectations are literals in this file, not the
output of the oracle, so the oracle is checked against them rather than against itself.

Usage: python tests/golden/make_packing_cases.py
"""
import json
import os

CASES = [
    {   # everything fits
        "requests": [
            {"ids": [101, 7, 102], "pooling": True, "offset": 0},
            {"ids": [101, 8, 9, 102], "pooling": True, "offset": 0},
        ],
        "max_batch_tokens": 16,
        "expect": {"input_ids": [101, 7, 102, 101, 8, 9, 102], "token_type_ids": [0] * 7,
                   "position_ids": [0, 1, 2, 0, 1, 2, 3], "cu": [0, 3, 7], "max_length": 4,
                   "pooled": [0, 1], "raw": [], "left": 0},
    },
    {   # budget cuts after two, exact fit allowed (3 + 4 = 7 <= 7)
        "requests": [
            {"ids": [1, 2, 3], "pooling": True, "offset": 0},
            {"ids": [4, 5, 6, 7], "pooling": False, "offset": 0},
            {"ids": [8], "pooling": True, "offset": 0},
        ],
        "max_batch_tokens": 7,
        "expect": {"input_ids": [1, 2, 3, 4, 5, 6, 7], "token_type_ids": [0] * 7,
                   "position_ids": [0, 1, 2, 0, 1, 2, 3], "cu": [0, 3, 7], "max_length": 4,
                   "pooled": [0], "raw": [1], "left": 1},
    },
    {   # RoBERTa-family offset 2, mixed pooled / raw, token types carried through
        "requests": [
            {"ids": [0, 11, 2], "types": [0, 0, 0], "pooling": False, "offset": 2},
            {"ids": [0, 12, 13, 2], "types": [0, 0, 0, 0], "pooling": True, "offset": 2},
            {"ids": [0, 2], "types": [0, 0], "pooling": False, "offset": 2},
        ],
        "max_batch_tokens": 100,
        "expect": {"input_ids": [0, 11, 2, 0, 12, 13, 2, 0, 2], "token_type_ids": [0] * 9,
                   "position_ids": [2, 3, 4, 2, 3, 4, 5, 2, 3], "cu": [0, 3, 7, 9], "max_length": 4,
                   "pooled": [1], "raw": [0, 2], "left": 0},
    },
    {   # max_batch_requests stops the batch before the token budget does
        "requests": [
            {"ids": [5], "pooling": True, "offset": 0},
            {"ids": [6, 7], "pooling": True, "offset": 0},
            {"ids": [8, 9, 10], "pooling": True, "offset": 0},
        ],
        "max_batch_tokens": 100, "max_batch_requests": 2,
        "expect": {"input_ids": [5, 6, 7], "token_type_ids": [0, 0, 0], "position_ids": [0, 0, 1],
                   "cu": [0, 1, 3], "max_length": 2, "pooled": [0, 1], "raw": [], "left": 1},
    },
    {   # pair input with token types 0 / 1 (BERT reranker style)
        "requests": [
            {"ids": [101, 5, 102, 6, 7, 102], "types": [0, 0, 0, 1, 1, 1], "pooling": True, "offset": 0},
            {"ids": [101, 9, 102, 4, 102], "types": [0, 0, 0, 1, 1], "pooling": True, "offset": 0},
        ],
        "max_batch_tokens": 11,
        "expect": {"input_ids": [101, 5, 102, 6, 7, 102, 101, 9, 102, 4, 102],
                   "token_type_ids": [0, 0, 0, 1, 1, 1, 0, 0, 0, 1, 1],
                   "position_ids": [0, 1, 2, 3, 4, 5, 0, 1, 2, 3, 4], "cu": [0, 6, 11], "max_length": 6,
                   "pooled": [0, 1], "raw": [], "left": 0},
    },
    {   # second entry does not fit: it blocks the ones behind it even if they would fit
        "requests": [
            {"ids": [1, 2], "pooling": False, "offset": 0},
            {"ids": [3, 4, 5, 6, 7], "pooling": True, "offset": 0},
            {"ids": [8], "pooling": True, "offset": 0},
        ],
        "max_batch_tokens": 6,
        "expect": {"input_ids": [1, 2], "token_type_ids": [0, 0], "position_ids": [0, 1], "cu": [0, 2],
                   "max_length": 2, "pooled": [], "raw": [0], "left": 2},
    },
]

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "packing_cases.json")
    with open(out, "w") as f:
        json.dump(CASES, f, indent=1)
    print("wrote", out, len(CASES), "cases")
