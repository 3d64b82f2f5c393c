"""The oracle against an independent implementation of the same architectures: Hugging Face
`transformers` on CPU in fp32, same seeded weights.  The reference itself (Rust) cannot be built
or imported, and its snapshot tests need hub checkpoints, so this is the check that guards the
restatement against transcription mistakes.  Tolerance: 1e-4 absolute in fp32."""
import json

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from oracle import generators as G
from oracle import models as M

TOL = 1e-4


def _t(a):
    return torch.from_numpy(np.asarray(a).astype(np.int64))[None]


def _per_sequence(batch):
    cu = batch.cumulative_seq_lengths
    for s in range(len(batch)):
        yield s, int(cu[s]), int(cu[s + 1])


def test_bert_matches_hf(model_dirs):
    d = model_dirs["bert"]
    cfg = json.load(open(d / "config.json"))
    cfg["hidden_act"] = "gelu_pytorch_tanh"  # the reference's GELU is the tanh form for every spelling
    hf = transformers.BertModel(transformers.BertConfig(**cfg), add_pooling_layer=False).eval()
    _, tensors = M.load_model_dir(d)
    missing, unexpected = hf.load_state_dict(tensors, strict=False)
    assert not [m for m in missing if "position_ids" not in m] and not unexpected
    o = M.build_oracle(d, "embedding", "mean")
    b = G.random_batch(3, [5, 17, 33, 1], 0, 1000, type_vocab=2)
    hs = o.hidden_states(b)
    for s, a, e in _per_sequence(b):
        with torch.no_grad():
            ref = hf(input_ids=_t(b.input_ids[a:e]), token_type_ids=_t(b.token_type_ids[a:e]),
                     position_ids=_t(b.position_ids[a:e])).last_hidden_state[0]
        assert (ref - hs[a:e]).abs().max().item() < TOL


def test_padded_form_equals_unpadded_form(model_dirs):
    # The reference's CPU path pads and masks (bert.rs:706-812); the oracle is unpadded.
    o = M.build_oracle(model_dirs["bert"], "embedding", "mean")
    b = G.random_batch(11, [5, 17, 32, 3], 0, 1000, type_vocab=2)
    hs = o.hidden_states(b)
    hp = o.hidden_states_padded(b)
    for s, a, e in _per_sequence(b):
        assert (hp[s, : e - a] - hs[a:e]).abs().max().item() < TOL


def test_xlm_roberta_classifier_matches_hf(model_dirs):
    d = model_dirs["xlmr"]
    cfg = json.load(open(d / "config.json"))
    cfg["hidden_act"] = "gelu_pytorch_tanh"
    hf = transformers.XLMRobertaForSequenceClassification(transformers.XLMRobertaConfig(**cfg)).eval()
    _, tensors = M.load_model_dir(d)
    missing, unexpected = hf.load_state_dict(tensors, strict=False)
    assert not [m for m in missing if "position_ids" not in m] and not unexpected
    o = M.build_oracle(d, "classifier")
    b = G.random_batch(4, [9, 30, 2], 5, 1000, position_offset=2)
    sc = o.predict(b)
    for s, a, e in _per_sequence(b):
        with torch.no_grad():
            ref = hf(input_ids=_t(b.input_ids[a:e]), position_ids=_t(b.position_ids[a:e])).logits[0]
        assert (ref - sc[s]).abs().max().item() < TOL


def test_qwen3_matches_hf(model_dirs):
    d = model_dirs["qwen3"]
    cfg = json.load(open(d / "config.json"))
    hf = transformers.Qwen3Model(transformers.Qwen3Config(**cfg)).eval()
    _, tensors = M.load_model_dir(d)
    hf.load_state_dict({k[len("model."):]: v for k, v in tensors.items()}, strict=True)
    o = M.build_oracle(d, "embedding", "last_token")
    b = G.random_batch(5, [7, 40, 130], 0, 1000)
    hs = o.hidden_states(b)
    for s, a, e in _per_sequence(b):
        with torch.no_grad():
            ref = hf(input_ids=_t(b.input_ids[a:e])).last_hidden_state[0]
        assert (ref - hs[a:e]).abs().max().item() < TOL


def test_qwen2_matches_hf(model_dirs):
    d = model_dirs["qwen2"]
    cfg = json.load(open(d / "config.json"))
    hf = transformers.Qwen2Model(transformers.Qwen2Config(**cfg)).eval()
    _, tensors = M.load_model_dir(d)
    hf.load_state_dict({k[len("model."):]: v for k, v in tensors.items()}, strict=True)
    o = M.build_oracle(d, "embedding", "last_token")
    b = G.random_batch(6, [7, 40, 130], 0, 1000)
    hs = o.hidden_states(b)
    for s, a, e in _per_sequence(b):
        with torch.no_grad():
            ref = hf(input_ids=_t(b.input_ids[a:e])).last_hidden_state[0]
        assert (ref - hs[a:e]).abs().max().item() < TOL


def test_mistral_sliding_window_matches_hf(model_dirs):
    d = model_dirs["mistral"]
    cfg = json.load(open(d / "config.json"))
    # The reference hands `sliding_window` to flash-attn as window_size_left
    # (flash_mistral.rs:56,95-110): key j counts when j >= i - sliding_window, i.e. the token
    # itself plus `sliding_window` earlier ones.  Hugging Face masks `j > i - sliding_window`
    # (one key fewer), so its config gets the window + 1 to describe the same mask.
    hcfg = dict(cfg)
    hcfg["sliding_window"] = cfg["sliding_window"] + 1
    hcfg["attn_implementation"] = "eager"
    hf = transformers.MistralModel(transformers.MistralConfig(**hcfg)).eval()
    _, tensors = M.load_model_dir(d)
    hf.load_state_dict(tensors, strict=True)
    o = M.build_oracle(d, "embedding", "last_token")
    assert o.window_left == 100
    b = G.random_batch(7, [7, 101, 102, 230], 0, 1000)
    hs = o.hidden_states(b)
    for s, a, e in _per_sequence(b):
        with torch.no_grad():
            ref = hf(input_ids=_t(b.input_ids[a:e])).last_hidden_state[0]
        assert (ref - hs[a:e]).abs().max().item() < TOL
    # the window matters at these lengths: without it the long sequence comes out differently
    o.window_left = None
    assert (o.hidden_states(b)[-1] - hs[-1]).abs().max().item() > 1e-3


def test_distilbert_matches_hf(model_dirs):
    d = model_dirs["distilbert"]
    cfg = json.load(open(d / "config.json"))
    # the reference's "gelu" is the tanh approximation (layers/linear.rs:5-17)
    hf = transformers.DistilBertModel(transformers.DistilBertConfig(**dict(cfg, activation="gelu_pytorch_tanh"))).eval()
    _, tensors = M.load_model_dir(d)
    hf.load_state_dict({k[len("distilbert."):]: v for k, v in tensors.items()}, strict=True)
    o = M.build_oracle(d, "embedding", "mean")
    b = G.random_batch(9, [7, 40, 130], 0, 1000)
    hs = o.hidden_states(b)
    for s, a, e in _per_sequence(b):
        with torch.no_grad():
            ref = hf(input_ids=_t(b.input_ids[a:e])).last_hidden_state[0]
        assert (ref - hs[a:e]).abs().max().item() < TOL


def test_modernbert_matches_hf(model_dirs):
    d = model_dirs["modernbert"]
    cfg = json.load(open(d / "config.json"))
    # every GELU name means the tanh approximation on the reference's path (layers/linear.rs:5-17)
    hcfg = dict(cfg, hidden_activation="gelu_pytorch_tanh", attn_implementation="eager", reference_compile=False,
                pad_token_id=0, bos_token_id=1, eos_token_id=2, cls_token_id=1, sep_token_id=2)
    hf = transformers.ModernBertModel(transformers.ModernBertConfig(**hcfg)).eval()
    _, tensors = M.load_model_dir(d)
    hf.load_state_dict({k[len("model."):]: v for k, v in tensors.items()}, strict=True)
    o = M.build_oracle(d, "embedding", "mean")
    assert o.window == 32 and o.every == 3
    b = G.random_batch(8, [7, 33, 34, 150], 0, 1000)
    hs = o.hidden_states(b)
    for s, a, e in _per_sequence(b):
        with torch.no_grad():
            ref = hf(input_ids=_t(b.input_ids[a:e])).last_hidden_state[0]
        assert (ref - hs[a:e]).abs().max().item() < TOL
    # the local window matters at these lengths
    o.window = 10 ** 6
    assert (o.hidden_states(b)[-1] - hs[-1]).abs().max().item() > 1e-3


def test_nomic_matches_hf(model_dirs):
    mod = pytest.importorskip("transformers.models.nomic_bert.modeling_nomic_bert")
    d = model_dirs["nomic"]
    cfg = json.load(open(d / "config.json"))
    hcfg = transformers.NomicBertConfig(
        vocab_size=cfg["vocab_size"], hidden_size=cfg["n_embd"], num_hidden_layers=cfg["n_layer"],
        num_attention_heads=cfg["n_head"], intermediate_size=cfg["n_inner"], hidden_act="silu",
        max_position_embeddings=cfg["n_positions"], type_vocab_size=cfg["type_vocab_size"],
        layer_norm_eps=cfg["layer_norm_epsilon"],
        rope_parameters={"rope_theta": cfg["rotary_emb_base"], "rope_type": "default"})
    hf = mod.NomicBertModel(hcfg).eval()
    _, t = M.load_model_dir(d)
    H = cfg["n_embd"]
    sd = {"embeddings.word_embeddings.weight": t["embeddings.word_embeddings.weight"],
          "embeddings.token_type_embeddings.weight": t["embeddings.token_type_embeddings.weight"],
          "embeddings.LayerNorm.weight": t["emb_ln.weight"], "embeddings.LayerNorm.bias": t["emb_ln.bias"]}
    for i in range(cfg["n_layer"]):
        p, q = f"encoder.layers.{i}.", f"layers.{i}."
        w = t[p + "attn.Wqkv.weight"]
        sd[q + "self_attn.q_proj.weight"], sd[q + "self_attn.k_proj.weight"], sd[q + "self_attn.v_proj.weight"] = \
            w[:H], w[H:2 * H], w[2 * H:]
        sd[q + "self_attn.o_proj.weight"] = t[p + "attn.out_proj.weight"]
        # the reference: silu(fc12 x) * (fc11 x) (nomic.rs:115-121) <-> HF: act(gate) * up
        sd[q + "mlp.gate_proj.weight"] = t[p + "mlp.fc12.weight"]
        sd[q + "mlp.up_proj.weight"] = t[p + "mlp.fc11.weight"]
        sd[q + "mlp.down_proj.weight"] = t[p + "mlp.fc2.weight"]
        sd[q + "post_attention_layernorm.weight"] = t[p + "norm1.weight"]
        sd[q + "post_attention_layernorm.bias"] = t[p + "norm1.bias"]
        sd[q + "post_mlp_layernorm.weight"] = t[p + "norm2.weight"]
        sd[q + "post_mlp_layernorm.bias"] = t[p + "norm2.bias"]
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    if unexpected or [m for m in missing if "position_ids" not in m and "inv_freq" not in m]:
        pytest.skip(f"HF NomicBert parameter names differ from the assumed mapping: {missing} {unexpected}")
    o = M.build_oracle(d, "embedding", "mean")
    b = G.random_batch(6, [6, 35], 0, 1000, type_vocab=2)
    hs = o.hidden_states(b)
    for s, a, e in _per_sequence(b):
        with torch.no_grad():
            ref = hf(input_ids=_t(b.input_ids[a:e]), token_type_ids=_t(b.token_type_ids[a:e])).last_hidden_state[0]
        assert (ref - hs[a:e]).abs().max().item() < TOL


def test_post_processing():
    v = np.array([[3.0, 4.0], [1.0, 0.0]], dtype=np.float32)
    n = M.l2_normalise(v)
    assert np.allclose(n, [[0.6, 0.8], [1.0, 0.0]], atol=1e-7)
    assert np.allclose(M.sigmoid_scores(np.array([[0.0]], dtype=np.float32)), [[0.5]])
    sm = M.sigmoid_scores(np.array([[1.0, 1.0, 1.0]], dtype=np.float32))
    assert np.allclose(sm, 1.0 / 3.0)


def test_alibi_slopes_known_values():
    # 8 heads: 2^-1 ... 2^-8 (backends/candle/src/alibi.rs:18-47)
    s = M.alibi_slopes(8).numpy()
    assert np.allclose(s, [2.0 ** -(i + 1) for i in range(8)])
    s12 = M.alibi_slopes(12).numpy()
    assert np.allclose(s12[:8], [2.0 ** -(i + 1) for i in range(8)])
    assert np.allclose(s12[8:], [2.0 ** -(0.5 + i) for i in range(4)])


def test_mistral_llama3_rope_scaling_matches_hf(model_dirs):
    """The Llama3 frequency rule (layers/rotary.rs:46-85) against Hugging Face's `llama3` rope
    type on the same weights."""
    d = model_dirs["mistral_rope_l3"]
    cfg = json.load(open(d / "config.json"))
    hcfg = {k: v for k, v in cfg.items() if k not in ("rope_scaling", "rope_theta")}
    hcfg["rope_parameters"] = dict(cfg["rope_scaling"], rope_theta=cfg["rope_theta"])
    hcfg["attn_implementation"] = "eager"
    hf = transformers.MistralModel(transformers.MistralConfig(**hcfg)).eval()
    _, tensors = M.load_model_dir(d)
    hf.load_state_dict(tensors, strict=True)
    inv = M.scaled_inv_freqs(cfg["hidden_size"] // cfg["num_attention_heads"], cfg["rope_theta"], cfg["rope_scaling"])
    plain = M.scaled_inv_freqs(cfg["hidden_size"] // cfg["num_attention_heads"], cfg["rope_theta"], None)
    ratio = plain / inv
    # all three bands occur: untouched, blended, divided by the factor
    assert (ratio == 1.0).any() and (np.abs(ratio - 8.0) < 1e-4).any() and ((ratio > 1.01) & (ratio < 7.9)).any()
    o = M.build_oracle(d, "embedding", "last_token")
    b = G.random_batch(17, [7, 101, 230], 0, 1000)
    hs = o.hidden_states(b)
    for s, a, e in _per_sequence(b):
        with torch.no_grad():
            ref = hf(input_ids=_t(b.input_ids[a:e])).last_hidden_state[0]
        assert (ref - hs[a:e]).abs().max().item() < TOL
