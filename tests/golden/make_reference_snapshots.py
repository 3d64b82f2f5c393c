"""Writes tests/golden/reference_snapshots.npz: the golden vectors the reference's own backend
tests hold for the model families this backend serves, read as text from
backends/candle/tests/snapshots/*.snap (insta YAML: a list of float lists behind a three-line
header).  Nothing of the reference runs; the numbers are its committed expectations.

Keys are the snapshot file names without `.snap` (`test_flash_bert__mini_batch`, ...).  The
`test_flash_*` files are the reference's fp16 CUDA outputs, the others its fp32 CPU outputs.
tests/reference_cases.py says which model, pooling and sentences each belongs to.

Usage: python tests/golden/make_reference_snapshots.py <path to a text-embeddings-inference checkout>
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import reference_cases  # noqa: E402


def parse_snap(path):
    """insta YAML snapshot -> float32 [rows, width]."""
    rows = []
    with open(path) as f:
        text = f.read()
    body = text.split("---\n", 2)[2]
    for line in body.splitlines():
        line = line.rstrip()
        if not line:
            continue
        if line.startswith("- - "):
            rows.append([float(line[4:])])
        elif line.startswith("  - "):
            rows[-1].append(float(line[4:]))
        else:
            raise ValueError(f"{path}: unexpected line {line!r}")
    width = {len(r) for r in rows}
    if len(width) != 1:
        raise ValueError(f"{path}: ragged rows {sorted(width)}")
    return np.asarray(rows, dtype=np.float32)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    ref = sys.argv[1]
    snap_dir = os.path.join(ref, "backends", "candle", "tests", "snapshots")
    out = {}
    for key in reference_cases.all_snapshot_keys():
        out[key] = parse_snap(os.path.join(snap_dir, key + ".snap"))
        print(key, out[key].shape)
    np.savez_compressed(os.path.join(HERE, "reference_snapshots.npz"), **out)
