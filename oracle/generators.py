"""TEST INFRASTRUCTURE - seeded synthetic model directories and packed batches.

Only tests/, `__graft_entry__.smoke()` and bench.py may import this package.

No checkpoint, tokenizer or dataset is available offline, so every workload is synthetic:
random-init weights of the named architecture (N(0, 0.02), LayerNorm/RMSNorm gamma = 1,
beta = 0) written as `config.json` + `model.safetensors` under the tensor names the reference's
loaders read (flash_bert.rs:30-60,130-158,264-356; nomic.rs:70-79,109-139; flash_nomic.rs:207-270;
flash_qwen3.rs:43-89,190-204,322-357), and token batches drawn with numpy's PCG64
`default_rng(seed)`.  The `config.json` fields are the ones the reference deserialises
(bert.rs:11-30, nomic.rs:11-45, qwen3.rs:13-37), so the same directories load in the real server.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import numpy as np

from .packing import Batch, batch_from_encodings


# --------------------------------------------------------------------------- configs
def bert_config(hidden=768, layers=12, heads=12, inter=3072, vocab=30522, max_pos=512,
                type_vocab=2, model_type="bert", act="gelu", eps=1e-12, pad_token_id=0,
                id2label=None) -> dict:
    arch = {"bert": "BertModel", "roberta": "RobertaModel", "xlm-roberta": "XLMRobertaModel",
            "camembert": "CamembertModel"}[model_type]
    if id2label is not None:
        arch = arch.replace("Model", "ForSequenceClassification")
    c = {
        "architectures": [arch], "model_type": model_type, "vocab_size": vocab, "hidden_size": hidden,
        "num_hidden_layers": layers, "num_attention_heads": heads, "intermediate_size": inter,
        "hidden_act": act, "hidden_dropout_prob": 0.1, "max_position_embeddings": max_pos,
        "type_vocab_size": type_vocab, "initializer_range": 0.02, "layer_norm_eps": eps,
        "pad_token_id": pad_token_id, "position_embedding_type": "absolute",
    }
    if id2label is not None:
        c["id2label"] = id2label
        c["label2id"] = {v: int(k) for k, v in id2label.items()}
    return c


def distilbert_config(hidden=768, layers=6, heads=12, inter=3072, vocab=30522, max_pos=512, act="gelu") -> dict:
    """Fields of DistilBertConfig (models/distilbert.rs:9-21)."""
    return {
        "architectures": ["DistilBertModel"], "model_type": "distilbert", "vocab_size": vocab, "dim": hidden,
        "n_layers": layers, "n_heads": heads, "hidden_dim": inter, "activation": act,
        "max_position_embeddings": max_pos, "pad_token_id": 0, "dropout": 0.1, "attention_dropout": 0.1,
        "sinusoidal_pos_embds": False,
    }


def _distilbert_shapes(c: dict) -> Dict[str, Tuple[tuple, str]]:
    """Names under `distilbert.` as a checkpoint of DistilBertForMaskedLM carries them
    (flash_distilbert.rs:211-214, models/distilbert.rs:27-56,103-140)."""
    H, I, V = c["dim"], c["hidden_dim"], c["vocab_size"]
    e = "distilbert.embeddings."
    t: Dict[str, Tuple[tuple, str]] = {e + "word_embeddings.weight": ((V, H), "normal"),
                                       e + "position_embeddings.weight": ((c["max_position_embeddings"], H), "normal"),
                                       e + "LayerNorm.weight": ((H,), "ones"), e + "LayerNorm.bias": ((H,), "zeros")}
    for i in range(c["n_layers"]):
        p = f"distilbert.transformer.layer.{i}."
        for n in ("q_lin", "k_lin", "v_lin", "out_lin"):
            t[p + f"attention.{n}.weight"] = ((H, H), "normal")
            t[p + f"attention.{n}.bias"] = ((H,), "normal")
        t[p + "sa_layer_norm.weight"] = ((H,), "ones")
        t[p + "sa_layer_norm.bias"] = ((H,), "zeros")
        t[p + "ffn.lin1.weight"] = ((I, H), "normal")
        t[p + "ffn.lin1.bias"] = ((I,), "normal")
        t[p + "ffn.lin2.weight"] = ((H, I), "normal")
        t[p + "ffn.lin2.bias"] = ((H,), "normal")
        t[p + "output_layer_norm.weight"] = ((H,), "ones")
        t[p + "output_layer_norm.bias"] = ((H,), "zeros")
    return t


def gte_config(hidden=768, layers=12, heads=12, inter=3072, vocab=30528, max_pos=8192, type_vocab=0,
               theta=500000.0, ntk_factor: Optional[float] = 2.0, eps=1e-12, id2label=None) -> dict:
    """Fields of GTEConfig (models/gte.rs:14-36); model_type "new" as the Alibaba-NLP checkpoints
    spell it (backends/candle/src/lib.rs:134-135)."""
    c = {
        "architectures": ["NewModel" if id2label is None else "NewForSequenceClassification"], "model_type": "new",
        "vocab_size": vocab, "hidden_size": hidden, "num_hidden_layers": layers, "num_attention_heads": heads,
        "intermediate_size": inter, "hidden_act": "gelu", "max_position_embeddings": max_pos,
        "type_vocab_size": type_vocab, "layer_norm_type": "layer_norm", "layer_norm_eps": eps,
        "position_embedding_type": "rope", "rope_theta": theta,
        "rope_scaling": None if ntk_factor is None else {"type": "ntk", "factor": ntk_factor},
        "logn_attention_scale": False, "logn_attention_clip1": False,
    }
    if id2label is not None:
        c["id2label"] = id2label
    return c


def _gte_shapes(c: dict) -> Dict[str, Tuple[tuple, str]]:
    """Names as flash_gte.rs:243-268 and models/gte.rs:52-66,196-205,290-312 read them, under `new.`."""
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    t: Dict[str, Tuple[tuple, str]] = {"new.embeddings.word_embeddings.weight": ((V, H), "normal"),
                                       "new.embeddings.LayerNorm.weight": ((H,), "ones"),
                                       "new.embeddings.LayerNorm.bias": ((H,), "zeros")}
    if c["type_vocab_size"] > 0:
        t["new.embeddings.token_type_embeddings.weight"] = ((c["type_vocab_size"], H), "normal")
    for i in range(c["num_hidden_layers"]):
        p = f"new.encoder.layer.{i}."
        t[p + "attention.qkv_proj.weight"] = ((3 * H, H), "normal")
        t[p + "attention.qkv_proj.bias"] = ((3 * H,), "normal")
        t[p + "attention.o_proj.weight"] = ((H, H), "normal")
        t[p + "attention.o_proj.bias"] = ((H,), "normal")
        t[p + "mlp.up_gate_proj.weight"] = ((2 * I, H), "normal")
        t[p + "mlp.down_proj.weight"] = ((H, I), "normal")
        t[p + "mlp.down_proj.bias"] = ((H,), "normal")
        for n in ("attn_ln", "mlp_ln"):
            t[p + n + ".weight"] = ((H,), "ones")
            t[p + n + ".bias"] = ((H,), "zeros")
    if c.get("id2label") is not None:
        n_cls = len(c["id2label"])
        t["new.pooler.dense.weight"] = ((H, H), "normal")
        t["new.pooler.dense.bias"] = ((H,), "normal")
        t["classifier.weight"] = ((n_cls, H), "normal")
        t["classifier.bias"] = ((n_cls,), "normal")
    return t


def jina_config(alibi: bool = True, **kw) -> dict:
    """A JinaBERT config: model_type "bert" plus the markers the reference dispatches on
    (backends/candle/src/lib.rs:83-121) and `position_embedding_type`."""
    c = bert_config(**kw)
    c["_name_or_path"] = "jinaai/jina-bert-implementation"
    c["auto_map"] = {"AutoConfig": "jinaai/jina-bert-implementation--configuration_bert.JinaBertConfig"}
    c["position_embedding_type"] = "alibi" if alibi else "absolute"
    c["feed_forward_type"] = "geglu"
    return c


def nomic_config(hidden=768, layers=12, heads=12, inter=3072, vocab=30528, n_positions=2048,
                 rotary_base=1000.0, eps=1e-12, moe_every: int = 0, num_experts: int = 8, moe_top_k: int = 2) -> dict:
    """moe_every > 0: the mixture-of-experts variant (nomic-embed-text-v2-moe style: GELU
    feed-forwards, every moe_every-th layer (index % moe_every == 1) routed; nomic.rs:402-414)."""
    c = _nomic_dense_config(hidden, layers, heads, inter, vocab, n_positions, rotary_base, eps)
    if moe_every > 0:
        c.update({"activation_function": "gelu", "mlp_fc1_bias": True, "mlp_fc2_bias": True, "qkv_proj_bias": True,
                  "moe_every_n_layers": moe_every, "num_experts": num_experts, "moe_top_k": moe_top_k,
                  "moe_normalize_expert_weights": False})
    return c


def _nomic_dense_config(hidden, layers, heads, inter, vocab, n_positions, rotary_base, eps) -> dict:
    return {
        "architectures": ["NomicBertModel"], "model_type": "nomic_bert", "prenorm": False,
        "rotary_emb_fraction": 1.0, "qkv_proj_bias": False, "rotary_emb_base": rotary_base,
        "rotary_emb_interleaved": False, "mlp_fc1_bias": False, "mlp_fc2_bias": False,
        "n_embd": hidden, "n_head": heads, "n_inner": inter, "n_layer": layers,
        "n_positions": n_positions, "max_trained_positions": n_positions,
        "activation_function": "swiglu", "vocab_size": vocab, "type_vocab_size": 2,
        "layer_norm_epsilon": eps,
    }


def qwen3_config(hidden=1024, layers=28, heads=16, kv_heads=8, head_dim=128, inter=3072,
                 vocab=151669, max_pos=8192, theta=1e6, eps=1e-6) -> dict:
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "attention_bias": False,
        "vocab_size": vocab, "hidden_size": hidden, "intermediate_size": inter,
        "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
        "head_dim": head_dim, "hidden_act": "silu", "max_position_embeddings": max_pos,
        "rms_norm_eps": eps, "rope_theta": theta, "use_sliding_window": False, "eos_token_id": 151643,
    }


def qwen2_config(hidden=1536, layers=28, heads=12, kv_heads=2, inter=8960, vocab=151646, max_pos=32768,
                 theta=1e6, eps=1e-6, is_causal: Optional[bool] = None) -> dict:
    """Fields of Qwen2Config (models/qwen2.rs:9-28); `is_causal` absent means causal."""
    c = {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": vocab,
        "hidden_size": hidden, "intermediate_size": inter, "num_hidden_layers": layers,
        "num_attention_heads": heads, "num_key_value_heads": kv_heads, "hidden_act": "silu",
        "max_position_embeddings": max_pos, "rms_norm_eps": eps, "rope_theta": theta,
        "sliding_window": None, "use_sliding_window": False,
    }
    if is_causal is not None:
        c["is_causal"] = is_causal
    return c


def mistral_config(hidden=4096, layers=32, heads=32, kv_heads=8, inter=14336, vocab=32000, max_pos=32768,
                   theta=10000.0, eps=1e-5, sliding_window: Optional[int] = 4096, model_type="mistral") -> dict:
    """Fields of MistralConfig (models/mistral.rs:5-24); model_type "llama" is run through the
    same model (backends/candle/src/lib.rs:549-575)."""
    c = {
        "architectures": ["MistralModel" if model_type == "mistral" else "LlamaModel"], "model_type": model_type,
        "vocab_size": vocab, "hidden_size": hidden, "intermediate_size": inter,
        "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
        "hidden_act": "silu", "max_position_embeddings": max_pos, "initializer_range": 0.02,
        "rms_norm_eps": eps, "rope_theta": theta, "rope_scaling": None,
    }
    if model_type == "mistral":
        c["sliding_window"] = sliding_window
    return c


def modernbert_config(hidden=768, layers=22, heads=12, inter=1152, vocab=50368, max_pos=8192, local_attention=128,
                      global_every=3, global_theta=160000.0, local_theta=10000.0, eps=1e-5,
                      num_labels: Optional[int] = None, classifier_pooling: str = "mean") -> dict:
    """Fields of ModernBertConfig (models/modernbert.rs:12-49)."""
    c = {
        "architectures": ["ModernBertModel" if num_labels is None else "ModernBertForSequenceClassification"],
        "model_type": "modernbert", "vocab_size": vocab, "hidden_size": hidden, "intermediate_size": inter,
        "num_hidden_layers": layers, "num_attention_heads": heads, "hidden_activation": "gelu",
        "max_position_embeddings": max_pos, "initializer_range": 0.02, "initializer_cutoff_factor": 2.0,
        "norm_eps": eps, "norm_bias": False, "pad_token_id": 50283, "eos_token_id": 50282, "bos_token_id": 50281,
        "cls_token_id": 50281, "sep_token_id": 50282, "global_rope_theta": global_theta, "attention_bias": False,
        "attention_dropout": 0.0, "global_attn_every_n_layers": global_every, "local_attention": local_attention,
        "local_rope_theta": local_theta, "mlp_bias": False, "classifier_pooling": classifier_pooling,
        "classifier_activation": "gelu", "classifier_bias": False,
    }
    if num_labels is not None:
        c["num_labels"] = num_labels
        c["id2label"] = {str(i): f"LABEL_{i}" for i in range(num_labels)}
    return c


def _modernbert_shapes(c: dict) -> Dict[str, Tuple[tuple, str]]:
    """Names as flash_modernbert.rs:279-293 and modernbert.rs:58-70,88-101,408-432 read them."""
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    t: Dict[str, Tuple[tuple, str]] = {"model.embeddings.tok_embeddings.weight": ((V, H), "normal"),
                                       "model.embeddings.norm.weight": ((H,), "ones"),
                                       "model.final_norm.weight": ((H,), "ones")}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        if i != 0:
            t[p + "attn_norm.weight"] = ((H,), "ones")
        t[p + "attn.Wqkv.weight"] = ((3 * H, H), "normal")
        t[p + "attn.Wo.weight"] = ((H, H), "normal")
        t[p + "mlp_norm.weight"] = ((H,), "ones")
        t[p + "mlp.Wi.weight"] = ((2 * I, H), "normal")
        t[p + "mlp.Wo.weight"] = ((H, I), "normal")
    if c.get("num_labels") is not None:
        t["head.dense.weight"] = ((H, H), "normal")
        t["head.norm.weight"] = ((H,), "ones")
        t["classifier.weight"] = ((c["num_labels"], H), "normal")
        t["classifier.bias"] = ((c["num_labels"],), "normal")
    return t


def jina_code_config(alibi: bool = True, **kw) -> dict:
    """A JinaCodeBert config: model_type "bert" plus the `jina-bert-v2-qk-post-norm` markers
    (backends/candle/src/lib.rs:83-121)."""
    c = bert_config(**kw)
    c["_name_or_path"] = "jinaai/jina-bert-v2-qk-post-norm"
    c["auto_map"] = {"AutoConfig": "jinaai/jina-bert-v2-qk-post-norm--configuration_bert.JinaBertConfig"}
    c["position_embedding_type"] = "alibi" if alibi else "absolute"
    c["feed_forward_type"] = "geglu"
    return c


# --------------------------------------------------------------------------- tensor lists
def _bert_shapes(c: dict, prefix: str, classifier: Optional[str], splade: bool) -> Dict[str, Tuple[tuple, str]]:
    """name -> (shape, kind) with kind in {normal, ones, zeros}."""
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    t: Dict[str, Tuple[tuple, str]] = {}
    e = prefix + "embeddings."
    jina = c.get("_name_or_path") == "jinaai/jina-bert-implementation"
    t[e + "word_embeddings.weight"] = ((V, H), "normal")
    if c.get("position_embedding_type", "absolute") == "absolute":
        t[e + "position_embeddings.weight"] = ((c["max_position_embeddings"], H), "normal")
    t[e + "token_type_embeddings.weight"] = ((c["type_vocab_size"], H), "normal")
    t[e + "LayerNorm.weight"] = ((H,), "ones")
    t[e + "LayerNorm.bias"] = ((H,), "zeros")
    for i in range(c["num_hidden_layers"]):
        p = f"{prefix}encoder.layer.{i}."
        for n in ("query", "key", "value"):
            t[p + f"attention.self.{n}.weight"] = ((H, H), "normal")
            t[p + f"attention.self.{n}.bias"] = ((H,), "normal")
        t[p + "attention.output.dense.weight"] = ((H, H), "normal")
        t[p + "attention.output.dense.bias"] = ((H,), "normal")
        t[p + "attention.output.LayerNorm.weight"] = ((H,), "ones")
        t[p + "attention.output.LayerNorm.bias"] = ((H,), "zeros")
        if c.get("_name_or_path") == "jinaai/jina-bert-v2-qk-post-norm":  # flash_jina_code.rs:27-212
            for n in ("layer_norm_q", "layer_norm_k"):
                t[p + f"attention.self.{n}.weight"] = ((H,), "ones")
                t[p + f"attention.self.{n}.bias"] = ((H,), "zeros")
            t[p + "mlp.up_gated_layer.weight"] = ((2 * I, H), "normal")
            t[p + "mlp.down_layer.weight"] = ((H, I), "normal")
            t[p + "mlp.down_layer.bias"] = ((H,), "normal")
            for n in ("layer_norm_1", "layer_norm_2"):
                t[p + f"{n}.weight"] = ((H,), "ones")
                t[p + f"{n}.bias"] = ((H,), "zeros")
            continue
        if jina:  # flash_jina.rs:133-155
            t[p + "mlp.gated_layers.weight"] = ((2 * I, H), "normal")
            t[p + "mlp.wo.weight"] = ((H, I), "normal")
            t[p + "mlp.wo.bias"] = ((H,), "normal")
            t[p + "mlp.layernorm.weight"] = ((H,), "ones")
            t[p + "mlp.layernorm.bias"] = ((H,), "zeros")
            continue
        t[p + "intermediate.dense.weight"] = ((I, H), "normal")
        t[p + "intermediate.dense.bias"] = ((I,), "normal")
        t[p + "output.dense.weight"] = ((H, I), "normal")
        t[p + "output.dense.bias"] = ((H,), "normal")
        t[p + "output.LayerNorm.weight"] = ((H,), "ones")
        t[p + "output.LayerNorm.bias"] = ((H,), "zeros")
    if classifier == "roberta":
        n_cls = len(c["id2label"])
        t["classifier.dense.weight"] = ((H, H), "normal")
        t["classifier.dense.bias"] = ((H,), "normal")
        t["classifier.out_proj.weight"] = ((n_cls, H), "normal")
        t["classifier.out_proj.bias"] = ((n_cls,), "normal")
    elif classifier == "bert":
        n_cls = len(c["id2label"])
        t["bert.pooler.dense.weight"] = ((H, H), "normal")
        t["bert.pooler.dense.bias"] = ((H,), "normal")
        t["classifier.weight"] = ((n_cls, H), "normal")
        t["classifier.bias"] = ((n_cls,), "normal")
    if splade:
        t["cls.predictions.transform.dense.weight"] = ((H, H), "normal")
        t["cls.predictions.transform.dense.bias"] = ((H,), "normal")
        t["cls.predictions.transform.LayerNorm.weight"] = ((H,), "ones")
        t["cls.predictions.transform.LayerNorm.bias"] = ((H,), "zeros")
        t["cls.predictions.decoder.weight"] = ((V, H), "normal")
        t["cls.predictions.bias"] = ((V,), "normal")
    return t


def _nomic_shapes(c: dict) -> Dict[str, Tuple[tuple, str]]:
    H, I, V = c["n_embd"], c["n_inner"], c["vocab_size"]
    t: Dict[str, Tuple[tuple, str]] = {
        "embeddings.word_embeddings.weight": ((V, H), "normal"),
        "embeddings.token_type_embeddings.weight": ((c["type_vocab_size"], H), "normal"),
        "emb_ln.weight": ((H,), "ones"), "emb_ln.bias": ((H,), "zeros"),
    }
    for i in range(c["n_layer"]):
        p = f"encoder.layers.{i}."
        t[p + "attn.Wqkv.weight"] = ((3 * H, H), "normal")
        t[p + "attn.out_proj.weight"] = ((H, H), "normal")
        if c["qkv_proj_bias"]:
            t[p + "attn.Wqkv.bias"] = ((3 * H,), "normal")
            t[p + "attn.out_proj.bias"] = ((H,), "normal")
        moe_every = c.get("moe_every_n_layers") or 0
        if moe_every > 0 and i % moe_every == 1:  # nomic.rs:213-219,255-262,289-294
            E = c["num_experts"]
            t[p + "mlp.router.layer.weight"] = ((E, H), "normal")
            t[p + "mlp.experts.mlp.w1"] = ((E * I, H), "normal")
            t[p + "mlp.experts.mlp.w2"] = ((E * I, H), "normal")
            t[p + "mlp.experts.bias"] = ((H,), "normal")
        elif c["activation_function"] == "swiglu":
            t[p + "mlp.fc11.weight"] = ((I, H), "normal")
            t[p + "mlp.fc12.weight"] = ((I, H), "normal")
            t[p + "mlp.fc2.weight"] = ((H, I), "normal")
        else:
            t[p + "mlp.fc1.weight"] = ((I, H), "normal")
            t[p + "mlp.fc2.weight"] = ((H, I), "normal")
            if c["mlp_fc1_bias"]:
                t[p + "mlp.fc1.bias"] = ((I,), "normal")
            if c["mlp_fc2_bias"]:
                t[p + "mlp.fc2.bias"] = ((H,), "normal")
        for n in ("norm1", "norm2"):
            t[p + n + ".weight"] = ((H,), "ones")
            t[p + n + ".bias"] = ((H,), "zeros")
    return t


def _qwen3_shapes(c: dict) -> Dict[str, Tuple[tuple, str]]:
    """Qwen3, and with fewer tensors Qwen2 (q/k/v biases, no q/k norm; `model.` prefix as in
    flash_qwen2.rs:266-275) and Mistral / Llama (neither; bare names as flash_mistral.rs:257-267
    reads them)."""
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    mt = c["model_type"]
    nh, nkv = c["num_attention_heads"], c["num_key_value_heads"]
    dh = c["head_dim"] if mt == "qwen3" else H // nh
    root = "" if mt in ("mistral", "llama") else "model."
    t: Dict[str, Tuple[tuple, str]] = {root + "embed_tokens.weight": ((V, H), "normal"),
                                       root + "norm.weight": ((H,), "ones")}
    for i in range(c["num_hidden_layers"]):
        p = f"{root}layers.{i}."
        t[p + "self_attn.q_proj.weight"] = ((nh * dh, H), "normal")
        t[p + "self_attn.k_proj.weight"] = ((nkv * dh, H), "normal")
        t[p + "self_attn.v_proj.weight"] = ((nkv * dh, H), "normal")
        t[p + "self_attn.o_proj.weight"] = ((H, nh * dh), "normal")
        if mt == "qwen3":
            t[p + "self_attn.q_norm.weight"] = ((dh,), "ones")
            t[p + "self_attn.k_norm.weight"] = ((dh,), "ones")
        if mt == "qwen2":
            t[p + "self_attn.q_proj.bias"] = ((nh * dh,), "normal")
            t[p + "self_attn.k_proj.bias"] = ((nkv * dh,), "normal")
            t[p + "self_attn.v_proj.bias"] = ((nkv * dh,), "normal")
        t[p + "mlp.gate_proj.weight"] = ((I, H), "normal")
        t[p + "mlp.up_proj.weight"] = ((I, H), "normal")
        t[p + "mlp.down_proj.weight"] = ((H, I), "normal")
        t[p + "input_layernorm.weight"] = ((H,), "ones")
        t[p + "post_attention_layernorm.weight"] = ((H,), "ones")
    return t


def tensor_shapes(config: dict, classifier: Optional[str] = None, splade: bool = False,
                  prefix: Optional[str] = None):
    mt = config["model_type"]
    if mt in ("bert", "roberta", "xlm-roberta", "camembert"):
        if prefix is None:
            prefix = "" if mt == "bert" else "roberta."
        return _bert_shapes(config, prefix, classifier, splade)
    if mt == "nomic_bert":
        return _nomic_shapes(config)
    if mt in ("qwen3", "qwen2", "mistral", "llama"):
        return _qwen3_shapes(config)
    if mt == "modernbert":
        return _modernbert_shapes(config)
    if mt == "distilbert":
        return _distilbert_shapes(config)
    if mt in ("gte", "new"):
        return _gte_shapes(config)
    raise ValueError(mt)


def write_model_dir(path, config: dict, seed: int, classifier: Optional[str] = None,
                    splade: bool = False, prefix: Optional[str] = None, std: float = 0.02,
                    norm_jitter: float = 0.0, store_dtype: str = "float32") -> Path:
    """Draws every tensor (sorted by name) from default_rng(seed) and writes the model dir.

    norm_jitter > 0 perturbs norm weights / biases away from (1, 0) so that tests exercise gamma
    and beta; the benchmark configs keep the stated gamma = 1, beta = 0.
    """
    from safetensors.numpy import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    shapes = tensor_shapes(config, classifier, splade, prefix)
    np_dtype = {"float32": np.float32, "float16": np.float16}[store_dtype]
    tensors = {}
    for name in sorted(shapes):
        shape, kind = shapes[name]
        if kind == "normal":
            arr = rng.standard_normal(size=shape, dtype=np.float32) * np.float32(std)
        elif kind == "ones":
            arr = np.ones(shape, dtype=np.float32)
            if norm_jitter:
                arr = arr + rng.standard_normal(size=shape, dtype=np.float32) * np.float32(norm_jitter)
        else:
            arr = np.zeros(shape, dtype=np.float32)
            if norm_jitter:
                arr = arr + rng.standard_normal(size=shape, dtype=np.float32) * np.float32(norm_jitter)
        tensors[name] = arr.astype(np_dtype)
    save_file(tensors, str(path / "model.safetensors"))
    (path / "config.json").write_text(json.dumps(config, indent=1))
    return path


DENSE_ACTIVATIONS = {"tanh": "torch.nn.modules.activation.Tanh", "identity": "torch.nn.modules.linear.Identity"}


def write_dense_dir(model_dir, dense_path: str, in_features: int, out_features: int, seed: int,
                    bias: bool = True, activation: Optional[str] = "tanh", std: float = 0.05) -> Path:
    """A Sentence-Transformers Dense module under `<model_dir>/<dense_path>/` in the layout the
    reference loads (backends/candle/src/lib.rs:579-629, models/dense.rs:26-62): config.json with
    in_features / out_features / bias / activation_function, model.safetensors with
    `linear.weight` [out, in] and `linear.bias` [out]."""
    from safetensors.numpy import save_file

    path = Path(model_dir) / dense_path
    path.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    tensors = {"linear.weight": rng.standard_normal(size=(out_features, in_features), dtype=np.float32) * np.float32(std)}
    if bias:
        tensors["linear.bias"] = rng.standard_normal(size=(out_features,), dtype=np.float32) * np.float32(std)
    save_file(tensors, str(path / "model.safetensors"))
    cfg = {"in_features": in_features, "out_features": out_features, "bias": bias}
    if activation is not None:
        cfg["activation_function"] = DENSE_ACTIVATIONS[activation]
    (path / "config.json").write_text(json.dumps(cfg, indent=1))
    return path


# --------------------------------------------------------------------------- batches
def _ids(rng, lens, lo, hi) -> List[np.ndarray]:
    return [rng.integers(lo, hi, size=int(n)) for n in lens]


def batch_cfg1() -> Batch:
    """32 x 512, ids uniform [1000, 30522), 101 first / 102 last, CLS pooling."""
    ids = np.random.default_rng(10).integers(1000, 30522, size=(32, 512))
    ids[:, 0] = 101
    ids[:, 511] = 102
    return batch_from_encodings(list(ids), list(range(32)), [])


def lengths_cfg2() -> np.ndarray:
    return np.random.default_rng(1).integers(16, 512, size=256, endpoint=True)


def batch_cfg2(n_seqs: Optional[int] = None) -> Batch:
    """256 ragged sequences, lengths uniform [16, 512] (seed 1), ids uniform [1000, 30522)."""
    rng = np.random.default_rng(1)
    lens = rng.integers(16, 512, size=256, endpoint=True)
    encs = _ids(rng, lens, 1000, 30522)
    if n_seqs is not None:
        encs = encs[:n_seqs]
    return batch_from_encodings(encs, list(range(len(encs))), [])


def batch_cfg3(n_seqs: Optional[int] = None) -> Batch:
    """64 sequences, lengths uniform [512, 2048] (seed 3), NomicBERT vocab."""
    rng = np.random.default_rng(3)
    lens = rng.integers(512, 2048, size=64, endpoint=True)
    encs = _ids(rng, lens, 1000, 30528)
    if n_seqs is not None:
        encs = encs[:n_seqs]
    return batch_from_encodings(encs, list(range(len(encs))), [])


def batch_cfg4(n_pairs: Optional[int] = None) -> Batch:
    """512 query/passage pairs as <s> q </s></s> p </s>, XLM-R ids, positions offset by 2."""
    rng = np.random.default_rng(4)
    q = rng.integers(8, 32, size=512, endpoint=True)
    p = rng.integers(64, 480, size=512, endpoint=True)
    encs = []
    for qi, pi in zip(q, p):
        qi, pi = int(qi), int(pi)
        if qi + pi + 4 > 512:
            pi = 512 - 4 - qi
        body_q = rng.integers(5, 250002, size=qi)
        body_p = rng.integers(5, 250002, size=pi)
        encs.append(np.concatenate([[0], body_q, [2, 2], body_p, [2]]))
    if n_pairs is not None:
        encs = encs[:n_pairs]
    return batch_from_encodings(encs, list(range(len(encs))), [], position_offset=2)


def lengths_cfg5() -> np.ndarray:
    u = np.random.default_rng(6).random(128)
    lens = np.floor(np.exp(np.log(128.0) + u * np.log(64.0))).astype(np.int64)
    return np.clip(lens, 128, 8192)


def batch_cfg5(n_seqs: Optional[int] = None, max_len: Optional[int] = None) -> Batch:
    """128 sequences, lengths log-uniform [128, 8192] (seed 6), Qwen3 vocab."""
    lens = lengths_cfg5()
    if max_len is not None:
        lens = np.minimum(lens, max_len)
    rng = np.random.default_rng(60)
    encs = _ids(rng, lens, 1000, 151669)
    if n_seqs is not None:
        encs = encs[:n_seqs]
    return batch_from_encodings(encs, list(range(len(encs))), [])


def random_batch(seed: int, lens, vocab_lo: int, vocab_hi: int, pooled=None, raw=None,
                 type_vocab: int = 1, position_offset: int = 0) -> Batch:
    rng = np.random.default_rng(seed)
    encs = _ids(rng, lens, vocab_lo, vocab_hi)
    types = [rng.integers(0, type_vocab, size=int(n)) for n in lens] if type_vocab > 1 else None
    n = len(encs)
    if pooled is None and raw is None:
        pooled, raw = list(range(n)), []
    return batch_from_encodings(encs, pooled or [], raw or [], type_ids=types,
                                position_offset=position_offset)


# FLOP model of the hot path (dense layers + attention only; causal counts the unmasked half).
def algorithmic_flops(config: dict, lens) -> float:
    mt = config["model_type"]
    lens = np.asarray(lens, dtype=np.float64)
    T = lens.sum()
    if mt == "qwen3":
        H, I, L = config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]
        hq = config["num_attention_heads"] * config["head_dim"]
        hkv = config["num_key_value_heads"] * config["head_dim"]
        lin = 2.0 * (H * hq + 2 * H * hkv + hq * H + 3 * H * I)
        attn = 2.0 * hq * (lens * (lens + 1)).sum()
    elif mt == "nomic_bert":
        H, I, L = config["n_embd"], config["n_inner"], config["n_layer"]
        lin = 2.0 * (4 * H * H + 3 * H * I)
        attn = 4.0 * H * (lens * lens).sum()
    else:
        H, I, L = config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]
        lin = 2.0 * (4 * H * H + 2 * H * I)
        attn = 4.0 * H * (lens * lens).sum()
    return float(L * (lin * T + attn))
