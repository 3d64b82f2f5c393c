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


def _start_error(tmp_path, cfg, **kw):
    import json
    import tei_b200
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(tei_b200.BackendError) as e:
        tei_b200.B200Backend(tmp_path, **kw)
    return e.value


def test_config_dispatch_refusals_follow_the_reference(lib, tmp_path):
    """The architecture dispatch and its refusals happen on the host, before any device is
    touched, so they are checked here without a GPU: every case must end as the error the
    reference gives, or as 'weights not found' once the config itself was accepted."""
    from oracle import generators as G
    # accepted configs of every family get as far as looking for the weights
    for cfg, kw in [
        (G.bert_config(), {}),
        (G.jina_config(alibi=True), dict(pool="mean")),
        (G.jina_code_config(alibi=True), dict(pool="mean")),
        (G.nomic_config(), dict(pool="mean")),
        (G.nomic_config(moe_every=2), dict(pool="mean")),
        (G.qwen3_config(), dict(pool="last_token")),
        (G.qwen2_config(), dict(pool="last_token")),
        (G.mistral_config(), dict(pool="last_token")),
        (G.mistral_config(model_type="llama"), dict(pool="mean")),
        (G.modernbert_config(), dict(pool="mean")),
        (G.modernbert_config(num_labels=2), dict(model_type="classifier")),
        (G.distilbert_config(), dict(pool="mean")),
        (G.gte_config(), dict(pool="cls")),
    ]:
        err = _start_error(tmp_path, cfg, **kw)
        assert err.kind == "WeightsNotFound", (cfg["model_type"], str(err))
    # refusals (file:line of the reference's bail! in each message's origin)
    e = _start_error(tmp_path, dict(G.jina_code_config(), id2label={"0": "a"}), model_type="classifier")  # flash_jina_code.rs:305-307
    assert e.kind == "Start" and "not supported for Jina Code" in str(e)
    e = _start_error(tmp_path, G.jina_code_config(), pool="splade")     # flash_jina_code.rs:309-311
    assert "`splade` is not supported for Jina Code" in str(e)
    e = _start_error(tmp_path, dict(G.qwen3_config(), model_type="bidirectional_pplx_qwen3"), pool="mean")  # lib.rs:537-542
    assert e.kind == "Start" and "Pplx1 is only supported in fp32 precision" in str(e)
    e = _start_error(tmp_path, G.jina_config(), pool="splade")          # flash_jina.rs:262-264
    assert "`splade` is not supported for Jina" in str(e)
    e = _start_error(tmp_path, dict(G.bert_config(), position_embedding_type="relative_key"))  # flash_bert.rs:241-243
    assert "absolute position embeddings" in str(e)
    e = _start_error(tmp_path, G.qwen3_config(), model_type="classifier")  # flash_qwen3.rs:312-316
    assert "`classifier` model type is not supported for Qwen3" in str(e)
    e = _start_error(tmp_path, dict(G.qwen2_config(), use_sliding_window=True), pool="mean")  # flash_qwen2.rs:26-29
    assert "Sliding window is not supported for Qwen2" in str(e)
    e = _start_error(tmp_path, dict(G.mistral_config(model_type="llama"), rope_scaling={"rope_type": "llama3", "factor": 8.0}),
                     pool="mean")                                         # backends/candle/src/lib.rs:549-553
    assert "Rope scaling is not supported for FlashLlama yet" in str(e)
    e = _start_error(tmp_path, G.modernbert_config(), pool="splade")     # flash_modernbert.rs:270-272
    assert "`splade` is not supported for ModernBert" in str(e)
    e = _start_error(tmp_path, dict(G.gte_config(), logn_attention_scale=True))  # flash_gte.rs:180-182
    assert "`logn_attention_scale` is not supported" in str(e)
    e = _start_error(tmp_path, dict(G.gte_config(), position_embedding_type="absolute"))  # flash_gte.rs:184-186
    assert "Only `PositionEmbeddingType::Rope` is supported" in str(e)
    e = _start_error(tmp_path, G.distilbert_config(), model_type="classifier")  # flash_distilbert.rs:199-201
    assert "`classifier` model type is not supported for DistilBert" in str(e)
    e = _start_error(tmp_path, dict(G.nomic_config(), prenorm=True), pool="mean")  # nomic.rs:49-54
    assert "config is not supported" in str(e)
    e = _start_error(tmp_path, dict(G.nomic_config(moe_every=2), num_experts=128), pool="mean")
    assert "mixture of experts" in str(e)
    cfg = G.qwen3_config()
    del cfg["rope_theta"]                                                 # flash_qwen3.rs:360-366
    e = _start_error(tmp_path, cfg, pool="last_token")
    assert "Neither `rope_theta` nor `rope_parameters.rope_theta`" in str(e)
    e = _start_error(tmp_path, G.bert_config(id2label=None), model_type="classifier")  # bert.rs:376-379
    assert "`id2label` must be set" in str(e)


def test_headers_are_plain_c(tmp_path):
    """The boundary is a C ABI: every header compiles as C99 on its own and together, and a C
    program that uses a few entry points links against the library."""
    import subprocess
    hdrs = sorted(glob.glob(os.path.join(ROOT, "include", "*.h")))
    assert len(hdrs) >= 3
    for h in hdrs:
        subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", h], check=True)
    src = tmp_path / "use.c"
    src.write_text(
        "".join(f'#include "{os.path.basename(h)}"\n' for h in hdrs) +
        "#include <stdio.h>\n"
        "int main(void) {\n"
        "  tei_b200_queue_t* q = NULL;\n"
        "  if (tei_b200_queue_create(0, 16, 0, &q) != TEI_B200_OK) return 1;\n"
        "  uint32_t ids[3] = {7, 8, 9};\n"
        "  if (tei_b200_queue_append(q, ids, NULL, NULL, 3, 2, 1, 42) != TEI_B200_OK) return 2;\n"
        "  uint32_t a[16], b[16], c[16], cu[5], p[4], r[4], mx; uint64_t tags[4]; size_t nt, ns, np, nr;\n"
        "  if (tei_b200_queue_next_batch(q, a, b, c, 16, cu, p, r, tags, 4, &nt, &ns, &np, &nr, &mx)) return 3;\n"
        "  if (nt != 3 || ns != 1 || np != 1 || nr != 0 || mx != 3 || tags[0] != 42 || c[0] != 2 || c[2] != 4) return 4;\n"
        "  tei_b200_queue_destroy(q);\n"
        "  tei_b200_t* h = NULL; char err[256];\n"
        "  int rc = tei_b200_create(\"/nonexistent\", \"float16\", TEI_B200_EMBEDDING, TEI_B200_POOL_CLS, NULL, 0, &h, err, sizeof err);\n"
        "  if (rc != TEI_B200_ERR_START || h != NULL) return 5;\n"
        "  puts(err);\n"
        "  return 0;\n"
        "}\n")
    lib_dir = os.path.join(ROOT, "text-embeddings-inference_b200", "lib")
    exe = tmp_path / "use"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", lib_dir, "-ltei_b200", f"-Wl,-rpath,{lib_dir}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, (out.returncode, out.stdout, out.stderr)
    assert "config.json" in out.stdout


def test_the_c_backend_thread_program_compiles_and_links(tmp_path):
    """tests/c/router_threads.c (run by the GPU tests) builds as C99 against include/*.h."""
    import subprocess
    lib_dir = os.path.join(ROOT, "text-embeddings-inference_b200", "lib")
    exe = tmp_path / "router_threads"
    subprocess.run(["gcc", "-std=c99", "-D_POSIX_C_SOURCE=200809L", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "c", "router_threads.c"), "-o", str(exe), "-L", lib_dir, "-ltei_b200",
                    f"-Wl,-rpath,{lib_dir}", "-lpthread", "-lm"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 64 and "usage" in out.stderr


def test_kernel_entry_points_refuse_a_null_status_word(lib):
    """The GEMM and attention kernels report a wait that ran out through *status; without it the
    report would be a write to address 0.  Refused on the host, before any CUDA call."""
    assert lib.tei_b200_op_linear(None, None, None, None, None, 128, 256, 64, 64, 256, 0, 0, 0, None, None) == 1
    assert lib.tei_b200_op_attention(None, None, None, None, None, 1, 128, 1, 1, 64, 64, 64, 64, 64, 0, 0.125,
                                     None, 0, None, None) == 1
    assert lib.tei_b200_op_bounded_wait_probe(None, 10, None, None) == 1
