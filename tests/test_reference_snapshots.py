"""Replays the reference's own backend tests against its committed golden vectors.

The vectors (tests/golden/reference_snapshots.npz, extracted from
backends/candle/tests/snapshots/*.snap by tests/golden/make_reference_snapshots.py) belong to hub
checkpoints: all-MiniLM-L6-v2, roberta-base-go_emotions, re2g-reranker-nq,
nomic-embed-text-v1.5 / v2-moe, Qwen3-Embedding-0.6B and the others listed in
tests/reference_cases.py.  A test runs when its checkpoint is found under the directory named by
TEI_B200_MODEL_ROOT (or HUGGINGFACE_HUB_CACHE, the variable the reference's tests read,
common.rs:140-142) and is skipped otherwise; the checks that need no checkpoint always run.

Layouts accepted under the root: `<org>/<name>/`, `<name>/`, `<org>--<name>/` and the hub cache
form `models--<org>--<name>/snapshots/<revision>/`; the directory must hold config.json,
tokenizer.json and the safetensors weights.

Matchers are the reference's (tests/common.rs:17-30,57-73): cosine similarity > 0.999 per
embedding row, absolute difference <= 5e-3 per score.  Batches are built like its `batch()`
helper (common.rs:327-356): positions restart at 0 for every sequence, with no offset.

  * fp32 CPU snapshots (test_bert__*, test_nomic__*, test_qwen3__qwen3_cpu_*, ...) pin the
    ORACLE (CPU, not marked gpu);
  * fp16 CUDA snapshots (test_flash_*, *_flash) pin the BACKEND through the C ABI (marked gpu).
"""
import glob
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import reference_cases as R  # noqa: E402
from oracle import models as M  # noqa: E402
from oracle import packing as P  # noqa: E402

SNAP = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_snapshots.npz")


def _find_model(hub_id):
    org, name = hub_id.split("/")
    roots = [os.environ.get(v) for v in ("TEI_B200_MODEL_ROOT", "HUGGINGFACE_HUB_CACHE")]
    for root in [r for r in roots if r]:
        cands = [os.path.join(root, org, name), os.path.join(root, name), os.path.join(root, f"{org}--{name}")]
        cands += sorted(glob.glob(os.path.join(root, f"models--{org}--{name}", "snapshots", "*")))
        for c in cands:
            has_weights = os.path.exists(os.path.join(c, "model.safetensors")) or \
                os.path.exists(os.path.join(c, "model.safetensors.index.json"))
            if os.path.exists(os.path.join(c, "config.json")) and os.path.exists(os.path.join(c, "tokenizer.json")) \
                    and has_weights:
                return c
    return None


def _load_tokenizer(model_dir, hub_id):
    """common.rs:278-325: no padding; a Metaspace pre-tokenizer prepends only at the start."""
    import tokenizers
    tok = tokenizers.Tokenizer.from_file(os.path.join(model_dir, "tokenizer.json"))
    tok.no_padding()
    pre = tok.pre_tokenizer
    if pre is not None and type(pre).__name__ == "Metaspace":
        pre.prepend_scheme = "first"
        tok.pre_tokenizer = pre
    if hub_id == "Alibaba-NLP/gte-Qwen2-1.5B-instruct":  # test_flash_qwen2.rs:20-41
        from tokenizers.processors import Sequence, TemplateProcessing
        tpl = TemplateProcessing(single="$A:0 <|endoftext|>:0", pair="$A:0 <|endoftext|>:0 $B:1 <|endoftext|>:1",
                                 special_tokens=[("<|endoftext|>", 151643)])
        tok.post_processor = tpl if tok.post_processor is None else Sequence([tok.post_processor, tpl])
    return tok


def _batch(tok, sentences, pooled, raw):
    encs = [tok.encode(*s, add_special_tokens=True) if isinstance(s, tuple) else tok.encode(s, add_special_tokens=True)
            for s in sentences]
    return P.batch_from_encodings([e.ids for e in encs], pooled, raw, type_ids=[e.type_ids for e in encs])


def _check_rows(got, want, key):
    assert got.shape == want.shape, (key, got.shape, want.shape)
    for i in range(len(want)):
        assert R.embedding_matches(got[i], want[i]), f"{key} row {i}"


def _check_scores(got, want, key):
    assert got.shape == want.shape, (key, got.shape, want.shape)
    for g, w in zip(got.ravel(), want.ravel()):
        assert R.score_matches(g, w), f"{key}: {g} vs {w}"


# ----------------------------------------------------------------- always on: the fixture itself
def test_fixture_holds_every_snapshot_with_the_tests_own_shapes():
    snaps = np.load(SNAP)
    assert sorted(snaps.files) == R.all_snapshot_keys()
    # test_flash_bert.rs:79,118-119,146: 8 / 22 / 7 raw rows; all-MiniLM-L6-v2 is 384 wide
    assert snaps["test_flash_bert__mini_batch"].shape == (3, 384)
    assert snaps["test_flash_bert__mini_batch_raw"].shape == (22, 384)
    assert snaps["test_flash_bert__mini_single_raw"].shape == (7, 384)
    assert snaps["test_flash_bert__emotions_batch"].shape == (3, 28)
    assert snaps["test_flash_qwen3__qwen3_batch"].shape == (3, 1024)
    assert snaps["test_flash_nomic__nomic_batch"].shape == (3, 768)


def test_matchers_on_the_invariants_the_reference_asserts_between_snapshots():
    s = np.load(SNAP)
    # test_flash_bert.rs:54-55: a sentence embeds the same alone and in a batch
    for stem in ("test_flash_bert__mini", "test_flash_nomic__nomic", "test_flash_qwen3__qwen3", "test_bert__bert",
                 "test_nomic__nomic", "test_qwen3__qwen3_cpu"):
        b, one = s[stem + "_batch"], s[stem + "_single"]
        assert R.embedding_matches(b[0], one[0]) and R.embedding_matches(b[2], one[0])
        assert not R.embedding_matches(b[1], one[0])
    # test_flash_bert.rs:115-119,144-145: CLS pooled rows equal the first raw row of their sequence
    p, r = s["test_flash_bert__mini_batch_pooled"], s["test_flash_bert__mini_batch_raw"]
    assert R.embedding_matches(p[0], r[0]) and R.embedding_matches(p[1], r[7]) and R.embedding_matches(p[2], r[15])
    assert R.embedding_matches(r[0], s["test_flash_bert__mini_single_raw"][0])
    # the reference's CUDA and CPU paths agree within its own matchers
    assert all(R.embedding_matches(a, b) for a, b in zip(s["test_flash_bert__mini_batch"], s["test_bert__bert_batch"]))
    assert all(R.score_matches(a, b) or abs(a - b) <= 2e-2
               for a, b in zip(s["test_flash_bert__emotions_batch"].ravel(), s["test_bert__emotions_batch"].ravel()))
    assert R.score_matches(1.0, 1.004) and not R.score_matches(1.0, 1.006)


# ----------------------------------------------------------------- the oracle against the fp32 CPU snapshots
@pytest.mark.parametrize("case", R.CPU_CASES, ids=[c[0] for c in R.CPU_CASES])
def test_oracle_reproduces_the_reference_cpu_snapshots(case):
    name, hub_id, _rev, model_type, pool, steps = case
    model_dir = _find_model(hub_id)
    if model_dir is None:
        pytest.skip(f"checkpoint {hub_id} is not mounted (set TEI_B200_MODEL_ROOT)")
    snaps = np.load(SNAP)
    tok = _load_tokenizer(model_dir, hub_id)
    o = M.build_oracle(model_dir, model_type, pool)
    for sentences, pooled, raw, pooled_key, raw_key in steps:
        b = _batch(tok, sentences, pooled, raw)
        if model_type == "classifier":
            _check_scores(o.predict(b).numpy(), snaps[pooled_key], pooled_key)
            continue
        got_pooled, got_raw = o.embed(b)
        if pooled_key:
            _check_rows(got_pooled.numpy(), snaps[pooled_key], pooled_key)
        if raw_key:
            _check_rows(got_raw.numpy(), snaps[raw_key], raw_key)


# ----------------------------------------------------------------- the backend against the fp16 CUDA snapshots
@pytest.mark.gpu
@pytest.mark.parametrize("case", R.FLASH_CASES, ids=[c[0] for c in R.FLASH_CASES])
def test_backend_reproduces_the_reference_cuda_snapshots(lib, case):
    name, hub_id, _rev, model_type, pool, steps = case
    model_dir = _find_model(hub_id)
    if model_dir is None:
        pytest.skip(f"checkpoint {hub_id} is not mounted (set TEI_B200_MODEL_ROOT)")
    import tei_b200
    snaps = np.load(SNAP)
    tok = _load_tokenizer(model_dir, hub_id)
    be = tei_b200.B200Backend(model_dir, "float16", model_type, pool)
    try:
        first = {}
        for sentences, pooled, raw, pooled_key, raw_key in steps:
            b = _batch(tok, sentences, pooled, raw)
            if model_type == "classifier":
                got = be.predict(b)
                _check_scores(np.array([got[i] for i in range(len(b))], dtype=np.float32), snaps[pooled_key], pooled_key)
                continue
            got = be.embed(b, normalize=False)  # the trait returns un-normalised rows
            # sort_embeddings (common.rs:94-106): pooled rows, then all raw rows, in batch order
            rows_p = [got[i].values for i in sorted(got) if got[i].kind == "pooled"]
            rows_r = [got[i].values for i in sorted(got) if got[i].kind == "all"]
            if pooled_key:
                g = np.stack(rows_p)
                _check_rows(g, snaps[pooled_key], pooled_key)
                first.setdefault("pooled", g[0])
                assert R.embedding_matches(g[0], first["pooled"])  # batch == single (test_flash_bert.rs:54-55)
            if raw_key:
                _check_rows(np.concatenate(rows_r), snaps[raw_key], raw_key)
    finally:
        be.close()


# ----------------------------------------------------------------- the harness is live, not vacuous
def test_harness_runs_on_a_mounted_checkpoint_and_rejects_wrong_weights(tmp_path, monkeypatch):
    """A random-weight model of the MiniLM shape (384 wide, 12 heads of 32) mounted under the
    MiniLM name with a small word-level tokenizer: the lookup, the tokenizer handling, the batch
    helper and the oracle all run, and the reference's matcher refuses the result."""
    import tokenizers
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    from tokenizers.processors import TemplateProcessing
    from oracle import generators as G
    d = tmp_path / "sentence-transformers" / "all-MiniLM-L6-v2"
    G.write_model_dir(d, G.bert_config(hidden=384, layers=1, heads=12, inter=512, vocab=64, max_pos=64), seed=3)
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "What", "is", "Deep", "Learning", "?", ".", "..."]
    tok = tokenizers.Tokenizer(WordLevel({w: i for i, w in enumerate(words)}, unk_token="[UNK]"))
    tok.pre_tokenizer = Whitespace()
    tok.post_processor = TemplateProcessing(single="[CLS] $A [SEP]", pair="[CLS] $A [SEP] $B:1 [SEP]:1",
                                            special_tokens=[("[CLS]", 2), ("[SEP]", 3)])
    tok.save(str(d / "tokenizer.json"))
    monkeypatch.setenv("TEI_B200_MODEL_ROOT", str(tmp_path))
    assert _find_model("sentence-transformers/all-MiniLM-L6-v2") == str(d)
    assert _find_model("Qwen/Qwen3-Embedding-0.6B") is None
    t = _load_tokenizer(str(d), "sentence-transformers/all-MiniLM-L6-v2")
    b = _batch(t, [R.WHAT, R.DEEP, R.WHAT], [0, 1, 2], [])
    assert b.cumulative_seq_lengths.tolist() == [0, 7, 13, 20] and b.position_ids[:8].tolist() == [0, 1, 2, 3, 4, 5, 6, 0]
    with pytest.raises(AssertionError):
        test_oracle_reproduces_the_reference_cpu_snapshots(R.CPU_CASES[0])
