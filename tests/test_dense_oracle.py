"""CPU checks of the Dense-module restatement (backends/candle/src/models/dense.rs:26-75 and the
loader loop of backends/candle/src/lib.rs:579-629): the layout written by the generator is the
one the reference reads, modules apply in order, Identity is the default activation, and a path
without a weight file is skipped."""
import json

import numpy as np
import torch

from oracle import generators as G
from oracle import models as M


def _read(d):
    from safetensors.numpy import load_file
    return json.loads((d / "config.json").read_text()), load_file(str(d / "model.safetensors"))


def test_dense_chain_matches_the_formula(tmp_path):
    d1 = G.write_dense_dir(tmp_path, "2_Dense", 16, 8, seed=1, bias=True, activation="tanh")
    d2 = G.write_dense_dir(tmp_path, "3_Dense", 8, 12, seed=2, bias=False, activation=None)
    c1, t1 = _read(d1)
    c2, t2 = _read(d2)
    # field names and activation strings of DenseConfig / DenseActivation (dense.rs:6-32)
    assert c1 == {"in_features": 16, "out_features": 8, "bias": True,
                  "activation_function": "torch.nn.modules.activation.Tanh"}
    assert c2 == {"in_features": 8, "out_features": 12, "bias": False}
    assert t1["linear.weight"].shape == (8, 16) and t1["linear.bias"].shape == (8,)
    assert sorted(t2) == ["linear.weight"]
    x = np.random.default_rng(0).standard_normal((5, 16)).astype(np.float32)
    want = np.tanh(x.astype(np.float64) @ t1["linear.weight"].T.astype(np.float64) + t1["linear.bias"])
    want = want @ t2["linear.weight"].T.astype(np.float64)
    got = M.apply_dense(torch.from_numpy(x), tmp_path, ["2_Dense", "7_Missing", "3_Dense"]).numpy()
    assert got.shape == (5, 12)
    assert np.abs(got - want).max() < 1e-5
    # no modules: unchanged
    assert torch.equal(M.apply_dense(torch.from_numpy(x), tmp_path, None), torch.from_numpy(x))
