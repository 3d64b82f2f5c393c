"""The C-ABI library loads and exports every symbol that include/*.h declares (no compute calls,
so this runs without a GPU), and the product path fails loudly when no GPU is there."""
import ctypes
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for hdr in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(hdr).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(tei_b200_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_headers_declare_the_backend_and_the_kernels():
    names = declared_symbols()
    for must in ("tei_b200_create", "tei_b200_embed", "tei_b200_predict", "tei_b200_health",
                 "tei_b200_is_padded", "tei_b200_max_batch_size", "tei_b200_op_linear",
                 "tei_b200_op_attention", "tei_b200_op_add_norm", "tei_b200_op_pool"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_python_prototypes_cover_every_declared_symbol(lib):
    from tei_b200 import _lib
    protos = _lib.prototypes()
    assert sorted(protos) == declared_symbols()


def test_trait_constants(lib):
    # is_padded is always false and max_batch_size is None on this path
    # (flash_bert.rs:530-532, backends/core/src/lib.rs:39-41); both ignore the handle.
    assert lib.tei_b200_is_padded(None) == 0
    assert lib.tei_b200_max_batch_size(None) == -1
    assert lib.tei_b200_health(None) == 3  # UNHEALTHY for a null handle


def test_create_reports_start_errors(lib, tmp_path):
    import tei_b200
    with pytest.raises(tei_b200.BackendError) as e:
        tei_b200.B200Backend(tmp_path / "missing")
    assert e.value.kind == "Start"
    (tmp_path / "config.json").write_text('{"model_type": "bert", "vocab_size": 10}')
    with pytest.raises(tei_b200.BackendError) as e:
        tei_b200.B200Backend(tmp_path)
    assert e.value.kind == "Start" and "missing field" in str(e.value)
    (tmp_path / "config.json").write_text('{"model_type": "gpt2"}')
    with pytest.raises(tei_b200.BackendError) as e:
        tei_b200.B200Backend(tmp_path)
    assert "not served" in str(e.value)
    with pytest.raises(tei_b200.BackendError) as e:
        tei_b200.B200Backend(tmp_path, dtype="float32")
    assert "float32" in str(e.value)


def test_weights_not_found_and_no_cpu_fallback(lib, tmp_path, model_dirs):
    import json
    import shutil
    import torch
    import tei_b200
    cfg = json.load(open(model_dirs["bert"] / "config.json"))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(tei_b200.BackendError) as e:
        tei_b200.B200Backend(tmp_path)
    assert e.value.kind == "WeightsNotFound"
    if not torch.cuda.is_available():
        # With weights present but no GPU the constructor must refuse, not fall back.
        shutil.copy(model_dirs["bert"] / "model.safetensors", tmp_path / "model.safetensors")
        with pytest.raises(tei_b200.BackendError) as e:
            tei_b200.B200Backend(tmp_path)
        assert e.value.kind == "Start" and "no CUDA device" in str(e.value)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "text-embeddings-inference_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cpp", ".cu", ".h", ".cuh", ".rs")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "import oracle" not in text and "from oracle" not in text, os.path.join(dirpath, f)
