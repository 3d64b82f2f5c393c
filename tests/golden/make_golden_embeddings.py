"""Writes tests/golden/embeddings.npz: outputs of the fp32 CPU oracle (oracle/models.py) for the
small seeded model directories and batches of tests/small_models.py.

The oracle itself is pinned by tests/test_oracle_vs_hf.py (Hugging Face transformers, fp32 CPU);
this file freezes its outputs so that the GPU parity tests also compare against committed
numbers.  Pooled rows are stored un-normalised, scores as raw logits.

Usage: python tests/golden/make_golden_embeddings.py
"""
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import small_models  # noqa: E402
from oracle import models as M  # noqa: E402

if __name__ == "__main__":
    dirs = small_models.write_all(Path(tempfile.mkdtemp()))
    out = {}
    for name, (key, model_type, pool, kw) in small_models.GOLDEN_CASES.items():
        o = M.build_oracle(dirs[key], model_type, pool)
        b = small_models.golden_batch(kw)
        if model_type == "classifier":
            out[name] = o.predict(b).numpy().astype(np.float32)
        else:
            pooled, _ = o.embed(b)
            out[name] = pooled.numpy().astype(np.float32)
        print(name, out[name].shape)
    np.savez_compressed(os.path.join(HERE, "embeddings.npz"), **out)
