"""Small seeded model directories and batches shared by the tests and the golden-fixture script."""
from oracle import generators as G


def write_all(base):
    dirs = {}
    dirs["bert"] = G.write_model_dir(
        base / "bert", G.bert_config(hidden=128, layers=2, heads=2, inter=256, vocab=1000, max_pos=512),
        seed=1, norm_jitter=0.1, std=0.05)
    dirs["bert_prefixed"] = G.write_model_dir(
        base / "bert_prefixed", G.bert_config(hidden=128, layers=2, heads=2, inter=256, vocab=1000, max_pos=512),
        seed=1, norm_jitter=0.1, std=0.05, prefix="bert.")
    dirs["bert_cls3"] = G.write_model_dir(
        base / "bert_cls3",
        G.bert_config(hidden=128, layers=2, heads=2, inter=256, vocab=1000, max_pos=512,
                      id2label={"0": "a", "1": "b", "2": "c"}),
        seed=6, classifier="bert", norm_jitter=0.1, std=0.05, prefix="bert.")
    dirs["xlmr"] = G.write_model_dir(
        base / "xlmr",
        G.bert_config(hidden=128, layers=2, heads=2, inter=256, vocab=1000, max_pos=514, type_vocab=1,
                      model_type="xlm-roberta", pad_token_id=1, id2label={"0": "LABEL_0"}),
        seed=3, classifier="roberta", norm_jitter=0.1, std=0.05)
    dirs["splade"] = G.write_model_dir(
        base / "splade", G.bert_config(hidden=128, layers=2, heads=2, inter=256, vocab=1003, max_pos=512),
        seed=7, splade=True, norm_jitter=0.1, std=0.05)
    dirs["jina"] = G.write_model_dir(
        base / "jina", G.jina_config(alibi=True, hidden=128, layers=2, heads=2, inter=256, vocab=1000, max_pos=512),
        seed=8, norm_jitter=0.1, std=0.05)
    dirs["jina_alibi6"] = G.write_model_dir(
        base / "jina_alibi6", G.jina_config(alibi=True, hidden=384, layers=2, heads=6, inter=512, vocab=1000, max_pos=512),
        seed=10, norm_jitter=0.1, std=0.05)
    dirs["jina_abs_cls"] = G.write_model_dir(
        base / "jina_abs_cls",
        G.jina_config(alibi=False, hidden=384, layers=2, heads=6, inter=512, vocab=1000, max_pos=512,
                      id2label={"0": "a", "1": "b"}),
        seed=9, classifier="bert", norm_jitter=0.1, std=0.05, prefix="bert.")
    dirs["jina_code"] = G.write_model_dir(
        base / "jina_code",
        G.jina_code_config(alibi=True, hidden=128, layers=2, heads=2, inter=256, vocab=1000, max_pos=512),
        seed=21, norm_jitter=0.1, std=0.05)
    dirs["jina_code_abs"] = G.write_model_dir(
        base / "jina_code_abs",
        G.jina_code_config(alibi=False, hidden=384, layers=2, heads=6, inter=512, vocab=1000, max_pos=512),
        seed=22, norm_jitter=0.1, std=0.05, prefix="bert.")
    dirs["nomic"] = G.write_model_dir(
        base / "nomic", G.nomic_config(hidden=128, layers=2, heads=2, inter=256, vocab=1000, n_positions=2048),
        seed=4, norm_jitter=0.1, std=0.05)
    dirs["qwen3"] = G.write_model_dir(
        base / "qwen3",
        G.qwen3_config(hidden=256, layers=3, heads=4, kv_heads=2, head_dim=128, inter=512, vocab=1000, max_pos=2048),
        seed=5, norm_jitter=0.1, std=0.05)
    dirs["qwen2"] = G.write_model_dir(
        base / "qwen2",
        G.qwen2_config(hidden=256, layers=2, heads=4, kv_heads=2, inter=512, vocab=1000, max_pos=2048),
        seed=11, norm_jitter=0.1, std=0.05)
    dirs["qwen2_bidir"] = G.write_model_dir(
        base / "qwen2_bidir",
        G.qwen2_config(hidden=256, layers=2, heads=4, kv_heads=4, inter=512, vocab=1000, max_pos=2048, is_causal=False),
        seed=12, norm_jitter=0.1, std=0.05)
    dirs["mistral"] = G.write_model_dir(
        base / "mistral",
        G.mistral_config(hidden=512, layers=2, heads=4, kv_heads=2, inter=512, vocab=1000, max_pos=2048,
                         sliding_window=100),
        seed=13, norm_jitter=0.1, std=0.05)
    # rope scaling: the Llama3 rule (original context 64, so that low, middle and high bands all
    # occur at head_dim 128) and the NTK rule
    dirs["mistral_rope_l3"] = G.write_model_dir(
        base / "mistral_rope_l3",
        dict(G.mistral_config(hidden=512, layers=2, heads=4, kv_heads=2, inter=512, vocab=1000, max_pos=2048,
                              sliding_window=None),
             rope_scaling={"rope_type": "llama3", "factor": 8.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                           "original_max_position_embeddings": 64}),
        seed=23, norm_jitter=0.1, std=0.05)
    dirs["mistral_rope_ntk"] = G.write_model_dir(
        base / "mistral_rope_ntk",
        dict(G.mistral_config(hidden=256, layers=2, heads=4, kv_heads=4, inter=512, vocab=1000, max_pos=2048,
                              sliding_window=None),
             rope_scaling={"type": "ntk", "factor": 4.0}),
        seed=24, norm_jitter=0.1, std=0.05)
    dirs["llama"] = G.write_model_dir(
        base / "llama",
        G.mistral_config(hidden=256, layers=2, heads=4, kv_heads=4, inter=512, vocab=1000, max_pos=2048,
                         model_type="llama"),
        seed=14, norm_jitter=0.1, std=0.05)
    dirs["distilbert"] = G.write_model_dir(
        base / "distilbert", G.distilbert_config(hidden=128, layers=2, heads=2, inter=256, vocab=1000, max_pos=512),
        seed=18, norm_jitter=0.1, std=0.05)
    dirs["gte"] = G.write_model_dir(
        base / "gte", G.gte_config(hidden=128, layers=2, heads=2, inter=256, vocab=1000, max_pos=2048, ntk_factor=2.0),
        seed=19, norm_jitter=0.1, std=0.05)
    dirs["gte_cls"] = G.write_model_dir(
        base / "gte_cls",
        G.gte_config(hidden=256, layers=2, heads=2, inter=256, vocab=1000, max_pos=2048, type_vocab=2, ntk_factor=None,
                     id2label={"0": "a", "1": "b"}),
        seed=20, norm_jitter=0.1, std=0.05)
    # head_dim 32: the shape of all-MiniLM-L6-v2 (384 wide, 12 heads), the model of the reference's
    # own flash-BERT test (backends/candle/tests/test_flash_bert.rs:18), and the same head size
    # behind RoPE and behind q/k RMSNorm + GQA
    dirs["minilm"] = G.write_model_dir(
        base / "minilm", G.bert_config(hidden=384, layers=2, heads=12, inter=1536, vocab=1000, max_pos=512),
        seed=26, norm_jitter=0.1, std=0.05)
    dirs["nomic_d32"] = G.write_model_dir(
        base / "nomic_d32", G.nomic_config(hidden=128, layers=2, heads=4, inter=256, vocab=1000, n_positions=2048),
        seed=27, norm_jitter=0.1, std=0.05)
    dirs["qwen3_d32"] = G.write_model_dir(
        base / "qwen3_d32",
        G.qwen3_config(hidden=128, layers=2, heads=4, kv_heads=2, head_dim=32, inter=256, vocab=1000, max_pos=2048),
        seed=28, norm_jitter=0.1, std=0.05)
    dirs["nomic_moe"] = G.write_model_dir(
        base / "nomic_moe",
        G.nomic_config(hidden=128, layers=4, heads=2, inter=256, vocab=1000, n_positions=2048, moe_every=2,
                       num_experts=8, moe_top_k=2),
        seed=17, norm_jitter=0.1, std=0.05)
    # three layers: the last one is a local-attention layer (index 2 with a global layer every 3)
    dirs["modernbert_local_last"] = G.write_model_dir(
        base / "modernbert_local_last",
        G.modernbert_config(hidden=128, layers=3, heads=2, inter=256, vocab=1000, max_pos=1024, local_attention=64,
                            global_every=3),
        seed=25, norm_jitter=0.1, std=0.05)
    dirs["modernbert"] = G.write_model_dir(
        base / "modernbert",
        G.modernbert_config(hidden=128, layers=4, heads=2, inter=256, vocab=1000, max_pos=1024, local_attention=64,
                            global_every=3),
        seed=15, norm_jitter=0.1, std=0.05)
    dirs["modernbert_cls"] = G.write_model_dir(
        base / "modernbert_cls",
        G.modernbert_config(hidden=256, layers=3, heads=2, inter=384, vocab=1000, max_pos=1024, local_attention=32,
                            global_every=2, num_labels=3, classifier_pooling="mean"),
        seed=16, norm_jitter=0.1, std=0.05)
    return dirs


LENS = [5, 1, 300, 77, 128, 129, 200]

# name -> (model dir key, model_type, pool, batch kwargs)
GOLDEN_CASES = {
    "bert_mean": ("bert", "embedding", "mean", dict(seed=101, lens=LENS, lo=0, hi=1000, type_vocab=2, offset=0)),
    "bert_cls": ("bert", "embedding", "cls", dict(seed=102, lens=LENS, lo=0, hi=1000, type_vocab=2, offset=0)),
    "xlmr_scores": ("xlmr", "classifier", "cls", dict(seed=103, lens=LENS, lo=5, hi=1000, type_vocab=1, offset=2)),
    "bert_cls3_scores": ("bert_cls3", "classifier", "cls", dict(seed=104, lens=LENS, lo=0, hi=1000, type_vocab=2, offset=0)),
    "nomic_mean": ("nomic", "embedding", "mean", dict(seed=105, lens=LENS + [700], lo=0, hi=1000, type_vocab=2, offset=0)),
    "qwen3_last": ("qwen3", "embedding", "last_token", dict(seed=106, lens=LENS + [700], lo=0, hi=1000, type_vocab=1, offset=0)),
    "jina_mean": ("jina", "embedding", "mean", dict(seed=108, lens=LENS + [511], lo=0, hi=1000, type_vocab=2, offset=0)),
    "jina_alibi6_cls": ("jina_alibi6", "embedding", "cls", dict(seed=109, lens=LENS, lo=0, hi=1000, type_vocab=2, offset=0)),
    "jina_abs_scores": ("jina_abs_cls", "classifier", "cls", dict(seed=110, lens=LENS, lo=0, hi=1000, type_vocab=2, offset=0)),
    "qwen2_last": ("qwen2", "embedding", "last_token", dict(seed=111, lens=LENS + [700], lo=0, hi=1000, type_vocab=1, offset=0)),
    "qwen2_bidir_mean": ("qwen2_bidir", "embedding", "mean", dict(seed=112, lens=LENS, lo=0, hi=1000, type_vocab=1, offset=0)),
    "mistral_window_last": ("mistral", "embedding", "last_token", dict(seed=113, lens=LENS + [700], lo=0, hi=1000, type_vocab=1, offset=0)),
    "mistral_window_mean": ("mistral", "embedding", "mean", dict(seed=114, lens=[400, 101, 100, 99], lo=0, hi=1000, type_vocab=1, offset=0)),
    "mistral_rope_l3_last": ("mistral_rope_l3", "embedding", "last_token", dict(seed=125, lens=LENS + [700], lo=0, hi=1000, type_vocab=1, offset=0)),
    "mistral_rope_ntk_mean": ("mistral_rope_ntk", "embedding", "mean", dict(seed=126, lens=LENS, lo=0, hi=1000, type_vocab=1, offset=0)),
    "llama_cls": ("llama", "embedding", "cls", dict(seed=115, lens=LENS, lo=0, hi=1000, type_vocab=1, offset=0)),
    "modernbert_mean": ("modernbert", "embedding", "mean", dict(seed=116, lens=LENS + [700], lo=0, hi=1000, type_vocab=1, offset=0)),
    "modernbert_cls": ("modernbert", "embedding", "cls", dict(seed=117, lens=[33, 64, 65, 400], lo=0, hi=1000, type_vocab=1, offset=0)),
    "modernbert_scores": ("modernbert_cls", "classifier", "cls", dict(seed=118, lens=LENS, lo=0, hi=1000, type_vocab=1, offset=0)),
    "nomic_moe_mean": ("nomic_moe", "embedding", "mean", dict(seed=119, lens=LENS + [700], lo=0, hi=1000, type_vocab=2, offset=0)),
    "distilbert_mean": ("distilbert", "embedding", "mean", dict(seed=120, lens=LENS, lo=0, hi=1000, type_vocab=1, offset=0)),
    "gte_cls_pool": ("gte", "embedding", "cls", dict(seed=121, lens=LENS + [700], lo=0, hi=1000, type_vocab=1, offset=0)),
    "gte_scores": ("gte_cls", "classifier", "cls", dict(seed=122, lens=LENS, lo=0, hi=1000, type_vocab=2, offset=0)),
    "jina_code_mean": ("jina_code", "embedding", "mean", dict(seed=123, lens=LENS + [511], lo=0, hi=1000, type_vocab=2, offset=0)),
    "jina_code_abs_cls": ("jina_code_abs", "embedding", "cls", dict(seed=124, lens=LENS, lo=0, hi=1000, type_vocab=2, offset=0)),
    "minilm_mean": ("minilm", "embedding", "mean", dict(seed=127, lens=LENS + [511], lo=0, hi=1000, type_vocab=2, offset=0)),
    "minilm_cls": ("minilm", "embedding", "cls", dict(seed=128, lens=LENS, lo=0, hi=1000, type_vocab=2, offset=0)),
    "nomic_d32_mean": ("nomic_d32", "embedding", "mean", dict(seed=129, lens=LENS + [700], lo=0, hi=1000, type_vocab=2, offset=0)),
    "qwen3_d32_last": ("qwen3_d32", "embedding", "last_token", dict(seed=130, lens=LENS + [700], lo=0, hi=1000, type_vocab=1, offset=0)),
    "splade": ("splade", "embedding", "splade", dict(seed=107, lens=[5, 1, 130, 40], lo=0, hi=1003, type_vocab=2, offset=0)),
}


def golden_batch(kw):
    return G.random_batch(kw["seed"], kw["lens"], kw["lo"], kw["hi"], type_vocab=kw["type_vocab"],
                          position_offset=kw["offset"])
