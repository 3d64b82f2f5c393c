"""The oracle reproduces the committed golden outputs (CPU; guards against silent drift of the
generators, the oracle or numpy's PCG64 stream)."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import small_models  # noqa: E402
from oracle import models as M  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "embeddings.npz")


def test_oracle_reproduces_golden(model_dirs):
    gold = np.load(GOLDEN)
    assert sorted(gold.files) == sorted(small_models.GOLDEN_CASES)
    for name, (key, model_type, pool, kw) in small_models.GOLDEN_CASES.items():
        o = M.build_oracle(model_dirs[key], model_type, pool)
        b = small_models.golden_batch(kw)
        got = o.predict(b).numpy() if model_type == "classifier" else o.embed(b)[0].numpy()
        assert got.shape == gold[name].shape
        assert np.abs(got - gold[name]).max() < 1e-5, name
