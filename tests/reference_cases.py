"""The reference's own backend tests for the families served here, as data: which hub model,
dtype, pooling and sentences produce which committed snapshot
(backends/candle/tests/test_flash_bert.rs, test_flash_nomic.rs, test_flash_qwen3.rs,
test_flash_jina.rs, test_flash_jina_code.rs, test_flash_gte.rs, test_flash_mistral.rs,
test_flash_qwen2.rs, test_modernbert.rs for the CUDA path; test_bert.rs, test_nomic.rs,
test_qwen3.rs, test_jina.rs, test_jina_code.rs, test_gte.rs for the fp32 CPU path).

A step is (sentences, pooled_indices, raw_indices, snapshot of the pooled rows or scores,
snapshot of the raw rows); a sentence is a string or a (query, passage) pair.
"""
WHAT = "What is Deep Learning?"
DEEP = "Deep Learning is..."

# test_flash_bert.rs:30-53 and the same shape in every embedding test
BATCH_THEN_SINGLE = lambda stem: [  # noqa: E731
    ([WHAT, DEEP, WHAT], [0, 1, 2], [], stem + "_batch", None),
    ([WHAT], [0], [], stem + "_single", None),
]
# test_flash_bert.rs:93-142 (CLS pooling, pooled [0, 2, 3], raw [1, 4, 5])
POOLED_RAW = lambda stem, sfx="": [  # noqa: E731
    ([WHAT, WHAT, DEEP, WHAT, DEEP, WHAT], [0, 2, 3], [1, 4, 5], stem + "_batch_pooled" + sfx, stem + "_batch_raw" + sfx),
    ([WHAT], [0], [], stem + "_single_pooled" + sfx, None),
    ([WHAT], [], [0], None, stem + "_single_raw" + sfx),
]

# (name, hub id, revision, model_type, pool, steps); the flash (fp16 CUDA) tests.
FLASH_CASES = [
    ("flash_mini", "sentence-transformers/all-MiniLM-L6-v2", None, "embedding", "mean", BATCH_THEN_SINGLE("test_flash_bert__mini")),
    ("flash_mini_pooled_raw", "sentence-transformers/all-MiniLM-L6-v2", None, "embedding", "cls", POOLED_RAW("test_flash_bert__mini")),
    ("flash_emotions", "SamLowe/roberta-base-go_emotions", None, "classifier", "cls", [
        (["I like you.", "I am not having a great day.", "I like you."], [0, 1, 2], [], "test_flash_bert__emotions_batch", None),
        (["I like you."], [0], [], "test_flash_bert__emotions_single", None)]),
    ("flash_bert_classification", "ibm-research/re2g-reranker-nq", "refs/pr/3", "classifier", "cls", [
        ([("PrimeTime is a timing signoff tool", "PrimeTime can perform most accurate timing analysis")], [0], [],
         "test_flash_bert__bert_classification_single", None)]),
    ("flash_nomic", "nomic-ai/nomic-embed-text-v1.5", None, "embedding", "mean", BATCH_THEN_SINGLE("test_flash_nomic__nomic")),
    ("flash_nomic_moe", "nomic-ai/nomic-embed-text-v2-moe", None, "embedding", "mean", BATCH_THEN_SINGLE("test_flash_nomic__nomic_moe")),
    ("flash_qwen3", "Qwen/Qwen3-Embedding-0.6B", None, "embedding", "last_token", BATCH_THEN_SINGLE("test_flash_qwen3__qwen3")),
    ("flash_jina", "jinaai/jina-embeddings-v2-small-en", None, "embedding", "mean", BATCH_THEN_SINGLE("test_flash_jina__jina")),
    ("flash_jina_code", "jinaai/jina-embeddings-v2-base-code", None, "embedding", "mean", BATCH_THEN_SINGLE("test_flash_jina_code__jina_code")),
    ("flash_gte", "Alibaba-NLP/gte-base-en-v1.5", None, "embedding", "cls", BATCH_THEN_SINGLE("test_flash_gte__gte")),
    ("flash_gte_classification", "Alibaba-NLP/gte-multilingual-reranker-base", None, "classifier", "cls", [
        ([(WHAT, "Deep Learning is not...")], [0], [], "test_flash_gte__gte_classification_single", None)]),
    ("flash_mistral", "Salesforce/SFR-Embedding-2_R", None, "embedding", "mean", BATCH_THEN_SINGLE("test_flash_mistral__mistral")),
    ("flash_qwen2", "Alibaba-NLP/gte-Qwen2-1.5B-instruct", None, "embedding", "last_token", BATCH_THEN_SINGLE("test_flash_qwen2__qwen2")),
    ("flash_modernbert", "answerdotai/ModernBERT-base", None, "embedding", "mean", [
        ([WHAT, DEEP, WHAT], [0, 1, 2], [], "test_modernbert__modernbert_batch_flash", None),
        ([WHAT], [0], [], "test_modernbert__modernbert_single_flash", None)]),
    ("flash_modernbert_pooled_raw", "answerdotai/ModernBERT-base", None, "embedding", "cls", POOLED_RAW("test_modernbert__modernbert", "_flash")),
]

# The fp32 CPU tests of the same families: what the oracle (an fp32 CPU restatement) must match.
CPU_CASES = [
    ("cpu_mini", "sentence-transformers/all-MiniLM-L6-v2", None, "embedding", "mean", BATCH_THEN_SINGLE("test_bert__bert")),
    ("cpu_mini_pooled_raw", "sentence-transformers/all-MiniLM-L6-v2", None, "embedding", "cls", POOLED_RAW("test_bert__bert")),
    ("cpu_emotions", "SamLowe/roberta-base-go_emotions", None, "classifier", "cls", [
        (["I like you.", "I am not having a great day.", "I like you."], [0, 1, 2], [], "test_bert__emotions_batch", None),
        (["I like you."], [0], [], "test_bert__emotions_single", None)]),
    ("cpu_bert_classification", "ibm-research/re2g-reranker-nq", "refs/pr/3", "classifier", "cls", [
        ([("PrimeTime is a timing signoff tool", "PrimeTime can perform most accurate timing analysis")], [0], [],
         "test_bert__bert_classification_single", None)]),
    ("cpu_nomic", "nomic-ai/nomic-embed-text-v1.5", None, "embedding", "mean", BATCH_THEN_SINGLE("test_nomic__nomic")),
    ("cpu_nomic_moe", "nomic-ai/nomic-embed-text-v2-moe", None, "embedding", "mean", BATCH_THEN_SINGLE("test_nomic__nomic_moe")),
    ("cpu_qwen3", "Qwen/Qwen3-Embedding-0.6B", None, "embedding", "last_token", BATCH_THEN_SINGLE("test_qwen3__qwen3_cpu")),
    ("cpu_jina", "jinaai/jina-embeddings-v2-small-en", None, "embedding", "mean", BATCH_THEN_SINGLE("test_jina__jina")),
    ("cpu_jina_code", "jinaai/jina-embeddings-v2-base-code", None, "embedding", "mean", BATCH_THEN_SINGLE("test_jina_code__jina_code")),
    ("cpu_modernbert", "answerdotai/ModernBERT-base", None, "embedding", "mean", BATCH_THEN_SINGLE("test_modernbert__modernbert")),
    ("cpu_modernbert_pooled_raw", "answerdotai/ModernBERT-base", None, "embedding", "cls", POOLED_RAW("test_modernbert__modernbert")),
]


def all_snapshot_keys():
    keys = []
    for _, _, _, _, _, steps in FLASH_CASES + CPU_CASES:
        for _, _, _, pooled_key, raw_key in steps:
            keys += [k for k in (pooled_key, raw_key) if k]
    return sorted(set(keys))


# The matchers of backends/candle/tests/common.rs.
def embedding_matches(a, b):
    """SnapEmbedding::eq (common.rs:57-73): cosine similarity above 0.999, summed in f32."""
    import numpy as np
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    assert a.shape == b.shape
    return float((a * b).sum() / np.sqrt((a * a).sum() * (b * b).sum())) > 0.999


def score_matches(a, b):
    """Score::eq (common.rs:17-30): absolute tolerance 5e-3."""
    return abs(float(a) - float(b)) <= 5e-3
