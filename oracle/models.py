"""TEST INFRASTRUCTURE - fp32 CPU restatement of the reference's Candle CPU models.

Only tests/, `__graft_entry__.smoke()` and bench.py's cpu_baseline / reference legs may import
this package; the product path never does.

PARITY UNPINNED by the reference's own golden vectors: every snapshot under
backends/candle/tests/snapshots/ needs a hub checkpoint and tokenizer that cannot be fetched
here, and the reference (Rust, un-vendored crates) cannot be compiled or imported.  The
restatement is instead cross-checked against Hugging Face `transformers` (an independent
implementation of the same architectures) in tests/test_oracle_vs_hf.py.

What is restated (file:line in the reference):
  BERT / RoBERTa / XLM-R  backends/candle/src/models/bert.rs
      embeddings :83-101, attention (CPU arm) :246-255, layer :317-332, classification heads
      :405-465, SPLADE head :551-558, pooling :819-879; loader name fallbacks flash_bert.rs:264-356
  NomicBERT               models/nomic.rs  embeddings :84-95, gated MLP :105-153, attention
      :474-573, block (post-LN) :605-626; rotary layers/rotary.rs:29-130
  Qwen3                   models/qwen3.rs  attention :137-271, layer :360-385, pooling :639-714;
      RMSNorm layers/rms_norm.rs:30-57
  further families        JinaBERT models/jina.rs + flash_jina.rs; ModernBERT models/modernbert.rs +
      flash_modernbert.rs; DistilBERT models/distilbert.rs; GTE models/gte.rs; Qwen2 / Mistral /
      Llama flash_qwen2.rs, flash_mistral.rs; NomicBERT mixture of experts models/nomic.rs:205-421;
      Dense modules models/dense.rs - each class below cites its lines
  shared                  LayerNorm layers/layer_norm.rs:108-132; Linear + activations
      layers/linear.rs:5-29,77-101 (every GELU name means the tanh approximation)
  host post-processing    core/src/infer.rs:288-303 (L2 normalise in f64), :458-480 (sigmoid)

Shape of the restatement: dense layers run on the packed [T, H] matrix (row-wise maths, so
identical to the padded form), attention runs per sequence on its own unpadded rows.  For real
tokens this equals the reference's padded form with a -inf bias on pad keys; `forward_padded`
keeps a literal padded version for small batches so the tests can check that claim.
"""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Dict, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from .packing import Batch

Tensor = torch.Tensor


# --------------------------------------------------------------------------- building blocks
def gelu_tanh(x: Tensor) -> Tensor:
    return F.gelu(x, approximate="tanh")


def activation(name: str):
    # layers/linear.rs:5-17: gelu | gelu_new | gelu_pytorch_tanh all mean tanh-GELU.
    if name in ("gelu", "gelu_new", "gelu_pytorch_tanh"):
        return gelu_tanh
    if name == "relu":
        return torch.relu
    if name == "silu":
        return F.silu
    if name == "tanh":
        return torch.tanh
    if name == "swiglu":
        def swiglu(x):
            a, b = x.chunk(2, dim=-1)
            return F.silu(a) * b
        return swiglu
    raise ValueError(f"unsupported activation {name}")


def linear(x: Tensor, w: Tensor, b: Optional[Tensor] = None) -> Tensor:
    y = x @ w.t()
    return y if b is None else y + b


def layer_norm(x: Tensor, residual: Optional[Tensor], gamma: Tensor, beta: Tensor, eps: float) -> Tensor:
    # layers/layer_norm.rs:108-132: biased variance, eps inside the sqrt.
    if residual is not None:
        x = x + residual
    mean = x.mean(dim=-1, keepdim=True)
    xc = x - mean
    var = (xc * xc).mean(dim=-1, keepdim=True)
    return xc / torch.sqrt(var + eps) * gamma + beta


def rms_norm(x: Tensor, residual: Optional[Tensor], gamma: Tensor, eps: float) -> Tuple[Tensor, Tensor]:
    # layers/rms_norm.rs:30-57: returns (normed, x + residual).
    if residual is not None:
        x = x + residual
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * gamma, x


def scaled_inv_freqs(head_dim: int, base: float, scaling: Optional[dict]) -> np.ndarray:
    """get_inv_freqs (layers/rotary.rs:29-98) in f32.  `scaling` is the config's `rope_scaling`
    object; as in the reference's untagged enum (:11-27) its FIELDS pick the variant: with
    high_freq_factor, low_freq_factor and original_max_position_embeddings it is the Llama3 rule
    (:46-85), with `factor` alone the NTK rule (:86-93), whatever its type string says."""
    f32 = np.float32
    dim = f32(head_dim)

    def plain(b):
        return np.array([f32(1.0) / np.power(f32(b), f32(i) / dim, dtype=np.float32)
                         for i in range(0, head_dim, 2)], dtype=np.float32)

    if not scaling:
        return plain(base)
    factor = f32(scaling["factor"])
    if all(k in scaling for k in ("high_freq_factor", "low_freq_factor", "original_max_position_embeddings")):
        old = f32(scaling["original_max_position_embeddings"])
        lo_f, hi_f = f32(scaling["low_freq_factor"]), f32(scaling["high_freq_factor"])
        low_wavelen, high_wavelen = old / lo_f, old / hi_f
        out = []
        for i in range(0, head_dim, 2):
            inv_base = f32(1.0) / np.power(f32(base), f32(i) / dim, dtype=np.float32)
            wavelen = f32(2.0) * f32(np.pi) / inv_base
            if wavelen < high_wavelen:
                out.append(inv_base)
            elif wavelen > low_wavelen:
                out.append(inv_base / factor)
            else:
                smooth = (old / wavelen - lo_f) / (hi_f - lo_f)
                out.append((f32(1.0) - smooth) * (inv_base / factor) + smooth * inv_base)
        return np.array(out, dtype=np.float32)
    # NTK: base * factor in f32, then divided by factor^(2/dim) computed in f32, applied as f64
    s = float(np.power(factor, f32(2.0) / dim, dtype=np.float32))
    return (plain(f32(base) * factor).astype(np.float64) / s).astype(np.float32)


def rope_tables(head_dim: int, base: float, max_pos: int, scaling: Optional[dict] = None) -> Tuple[Tensor, Tensor]:
    # layers/rotary.rs:29-116: inv_freq_i = 1 / base^(i/dim) for even i, all in f32.
    inv = scaled_inv_freqs(head_dim, base, scaling)
    t = np.arange(max_pos, dtype=np.float32)[:, None]
    freqs = (t * inv[None, :]).astype(np.float32)
    return torch.from_numpy(np.cos(freqs).astype(np.float32)), torch.from_numpy(np.sin(freqs).astype(np.float32))


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    # layers/rotary.rs:118-130 with half-width tables: x*cos + rotate_half(x)*sin.
    # x [L, heads, D]; cos/sin [L, D/2].
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def alibi_slopes(n_heads: int) -> Tensor:
    # backends/candle/src/alibi.rs:18-47 (the usual power-of-two construction).
    def pow2_slopes(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if math.log2(n_heads).is_integer():
        s = pow2_slopes(n_heads)
    else:
        closest = 2 ** math.floor(math.log2(n_heads))
        s = pow2_slopes(closest) + pow2_slopes(2 * closest)[0::2][: n_heads - closest]
    return torch.tensor(s, dtype=torch.float32)


def attention_varlen(q: Tensor, k: Tensor, v: Tensor, cu: np.ndarray, scale: float, causal: bool,
                     slopes: Optional[Tensor] = None, window_left: Optional[int] = None,
                     window_right: Optional[int] = None) -> Tensor:
    """q [T, nh, D], k/v [T, nkv, D] -> [T, nh*D]; one softmax(QK^T)V per sequence and head.
    window_left: key j counts for query i only when j >= i - window_left (flash-attn's
    window_size_left, as passed by flash_mistral.rs:95-110 through flash_attn.rs:82-95)."""
    T, nh, D = q.shape
    nkv = k.shape[1]
    out = torch.empty(T, nh * D, dtype=q.dtype)
    for s in range(len(cu) - 1):
        a, b = int(cu[s]), int(cu[s + 1])
        L = b - a
        if L == 0:
            continue
        qs = q[a:b].transpose(0, 1)
        ks = k[a:b].transpose(0, 1)
        vs = v[a:b].transpose(0, 1)
        if nkv != nh:  # GQA: q-head i reads kv-head i // group (models/qwen3.rs:189-205)
            ks = ks.repeat_interleave(nh // nkv, dim=0)
            vs = vs.repeat_interleave(nh // nkv, dim=0)
        # Heads are independent: long sequences go through a few heads at a time so that the
        # [heads, L, L] score tensor stays below about 1 GB (same arithmetic per head).
        step = nh if nh * L * L <= (1 << 28) else max(1, (1 << 28) // (L * L))
        o_s = torch.empty(nh, L, D, dtype=q.dtype)
        for h0 in range(0, nh, step):
            h1 = min(nh, h0 + step)
            sc = (qs[h0:h1] @ ks[h0:h1].transpose(1, 2)) * scale
            if slopes is not None:
                idx = torch.arange(L)
                sc = sc - slopes[h0:h1].view(h1 - h0, 1, 1) * (idx.view(1, L, 1) - idx.view(1, 1, L)).abs()
            if causal:
                sc = sc.masked_fill(~torch.ones(L, L, dtype=torch.bool).tril(), float("-inf"))
            if window_left is not None:
                idx = torch.arange(L)
                sc = sc.masked_fill(idx.view(1, L) < idx.view(L, 1) - window_left, float("-inf"))
            if window_right is not None:  # and j <= i + window_right (flash_modernbert.rs:92-111)
                idx = torch.arange(L)
                sc = sc.masked_fill(idx.view(1, L) > idx.view(L, 1) + window_right, float("-inf"))
            o_s[h0:h1] = torch.softmax(sc, dim=-1) @ vs[h0:h1]
        out[a:b] = o_s.transpose(0, 1).reshape(L, nh * D)
    return out


# --------------------------------------------------------------------------- weights
def load_model_dir(model_dir) -> Tuple[dict, Dict[str, Tensor]]:
    """config.json + model.safetensors, every tensor as fp32 (the reference's CPU dtype)."""
    from safetensors import safe_open

    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    tensors: Dict[str, Tensor] = {}
    with safe_open(str(model_dir / "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            tensors[name] = f.get_tensor(name).to(torch.float32)
    return config, tensors


def apply_dense(pooled: Tensor, model_dir, dense_paths) -> Tensor:
    """Sentence-Transformers Dense modules on the pooled rows, in order
    (backends/candle/src/lib.rs:672-680; models/dense.rs:64-75: linear, then Tanh or Identity,
    Identity when `activation_function` is absent `:54-57`).  Paths without a weight file are
    skipped as the loader does (lib.rs:586-626)."""
    from safetensors import safe_open

    for dense_path in dense_paths or []:
        d = Path(model_dir) / dense_path
        if not (d / "model.safetensors").exists():
            continue
        cfg = json.loads((d / "config.json").read_text())
        with safe_open(str(d / "model.safetensors"), framework="pt") as f:
            w = f.get_tensor("linear.weight").to(torch.float32)
            b = f.get_tensor("linear.bias").to(torch.float32) if cfg["bias"] else None
        assert tuple(w.shape) == (cfg["out_features"], cfg["in_features"])
        pooled = linear(pooled, w, b)
        act = cfg.get("activation_function") or "torch.nn.modules.linear.Identity"
        if act == "torch.nn.modules.activation.Tanh":
            pooled = torch.tanh(pooled)
        elif act != "torch.nn.modules.linear.Identity":
            raise ValueError(f"unknown activation_function {act}")
    return pooled


class _Weights:
    def __init__(self, tensors: Dict[str, Tensor], prefixes=("",)):
        self.t = tensors
        self.prefixes = prefixes

    def has(self, name: str) -> bool:
        return any((p + name) in self.t for p in self.prefixes)

    def get(self, name: str) -> Tensor:
        for p in self.prefixes:
            if (p + name) in self.t:
                return self.t[p + name]
        raise KeyError(f"tensor {name} not found (prefixes {self.prefixes})")

    def get_any(self, *names: str) -> Tensor:
        for n in names:
            if self.has(n):
                return self.get(n)
        raise KeyError(f"none of {names} found")

    def ln(self, prefix: str) -> Tuple[Tensor, Tensor]:
        # LayerNorm::load accepts weight|gamma and bias|beta (layers/layer_norm.rs:93-98).
        return (self.get_any(prefix + ".weight", prefix + ".gamma"),
                self.get_any(prefix + ".bias", prefix + ".beta"))


# --------------------------------------------------------------------------- pooling (shared)
def pool_outputs(hidden: Tensor, batch: Batch, pool: str) -> Tuple[Optional[Tensor], Optional[Tensor]]:
    """Pooled rows (one per pooled_indices entry, in that order) and raw rows (token rows of the
    raw_indices sequences, in that order).  flash_bert.rs:396-523 / bert.rs:819-933."""
    cu = batch.cumulative_seq_lengths.astype(np.int64)
    pooled = None
    if len(batch.pooled_indices) > 0:
        rows = []
        for i in batch.pooled_indices.astype(np.int64):
            seg = hidden[int(cu[i]):int(cu[i + 1])]
            if pool == "cls":
                rows.append(seg[0])
            elif pool == "last_token":
                rows.append(seg[-1])
            elif pool == "mean":
                rows.append(seg.sum(dim=0) / float(seg.shape[0]))
            elif pool == "splade":
                rows.append(seg.max(dim=0).values)
            else:
                raise ValueError(pool)
        pooled = torch.stack(rows)
    raw = None
    if len(batch.raw_indices) > 0:
        raw = torch.cat([hidden[int(cu[i]):int(cu[i + 1])] for i in batch.raw_indices.astype(np.int64)])
    return pooled, raw


def l2_normalise(v: np.ndarray) -> np.ndarray:
    # core/src/infer.rs:288-303: scale by 1/sqrt(sum of squares), accumulated in f64.
    v64 = v.astype(np.float64)
    n = np.sqrt((v64 * v64).sum(axis=-1, keepdims=True))
    return (v64 / n).astype(np.float32)


def sigmoid_scores(x: np.ndarray) -> np.ndarray:
    # core/src/infer.rs:458-480: a single class is squashed with a sigmoid, several with softmax.
    if x.shape[-1] == 1:
        return (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32)
    z = x.astype(np.float64)
    z = np.exp(z - z.max(axis=-1, keepdims=True))
    return (z / z.sum(axis=-1, keepdims=True)).astype(np.float32)


# --------------------------------------------------------------------------- BERT family
class BertOracle:
    def __init__(self, config: dict, tensors: Dict[str, Tensor], model_type: str = "embedding",
                 pool: str = "cls"):
        self.cfg = config
        self.pool = "cls" if model_type == "classifier" else pool
        self.model_type = model_type
        mt = config["model_type"]
        self.roberta = mt in ("roberta", "xlm-roberta", "camembert")
        # flash_bert.rs:264-279 (bert) / :331-356 (roberta family): bare names first, then prefixes.
        if self.roberta:
            cand = ["", "roberta.", "xlm-roberta.", "camembert."]
        else:
            cand = ["", "bert."]
        prefix = next((p for p in cand if (p + "embeddings.word_embeddings.weight") in tensors), None)
        if prefix is None:
            raise KeyError("embeddings.word_embeddings.weight not found under any known prefix")
        self.w = _Weights(tensors, (prefix,))
        self.all = _Weights(tensors, ("",))
        self.nh = config["num_attention_heads"]
        self.hidden = config["hidden_size"]
        self.dh = self.hidden // self.nh
        self.eps = float(config["layer_norm_eps"])
        self.act = activation(config["hidden_act"])
        self.n_layers = config["num_hidden_layers"]
        if config.get("position_embedding_type", "absolute") != "absolute":
            raise ValueError("only absolute position embeddings are supported (bert.rs:51-54)")

    def hidden_states(self, batch: Batch) -> Tensor:
        w = self.w
        ids = torch.from_numpy(batch.input_ids.astype(np.int64))
        tids = torch.from_numpy(batch.token_type_ids.astype(np.int64))
        pids = torch.from_numpy(batch.position_ids.astype(np.int64))
        g, b = w.ln("embeddings.LayerNorm")
        x = w.get("embeddings.word_embeddings.weight")[ids] + w.get("embeddings.token_type_embeddings.weight")[tids]
        x = layer_norm(x, w.get("embeddings.position_embeddings.weight")[pids], g, b, self.eps)
        cu = batch.cumulative_seq_lengths
        T = x.shape[0]
        for i in range(self.n_layers):
            p = f"encoder.layer.{i}."
            q = linear(x, w.get(p + "attention.self.query.weight"), w.get(p + "attention.self.query.bias"))
            k = linear(x, w.get(p + "attention.self.key.weight"), w.get(p + "attention.self.key.bias"))
            v = linear(x, w.get(p + "attention.self.value.weight"), w.get(p + "attention.self.value.bias"))
            a = attention_varlen(q.view(T, self.nh, self.dh), k.view(T, self.nh, self.dh),
                                 v.view(T, self.nh, self.dh), cu, 1.0 / math.sqrt(self.dh), False)
            g1, b1 = w.ln(p + "attention.output.LayerNorm")
            x1 = layer_norm(linear(a, w.get(p + "attention.output.dense.weight"),
                                   w.get(p + "attention.output.dense.bias")), x, g1, b1, self.eps)
            f = self.act(linear(x1, w.get(p + "intermediate.dense.weight"), w.get(p + "intermediate.dense.bias")))
            g2, b2 = w.ln(p + "output.LayerNorm")
            x = layer_norm(linear(f, w.get(p + "output.dense.weight"), w.get(p + "output.dense.bias")),
                           x1, g2, b2, self.eps)
        return x

    def splade_head(self, x: Tensor) -> Tensor:
        a = self.all
        if self.roberta:  # bert.rs:519-541
            h = gelu_tanh(linear(x, a.get("lm_head.dense.weight"), a.get("lm_head.dense.bias")))
            g, b = a.ln("lm_head.layer_norm")
            dec_w, dec_b = a.get("lm_head.decoder.weight"), a.get("lm_head.bias")
        else:  # bert.rs:477-509
            h = self.act(linear(x, a.get("cls.predictions.transform.dense.weight"),
                                a.get("cls.predictions.transform.dense.bias")))
            g, b = a.ln("cls.predictions.transform.LayerNorm")
            dec_w = a.get_any("cls.predictions.decoder.weight", "bert.embeddings.word_embeddings.weight")
            dec_b = a.get("cls.predictions.bias")
        h = layer_norm(h, None, g, b, self.eps)
        return torch.log(1.0 + torch.relu(linear(h, dec_w, dec_b)))  # bert.rs:551-558

    def embed(self, batch: Batch) -> Tuple[Optional[Tensor], Optional[Tensor]]:
        x = self.hidden_states(batch)
        if self.pool == "splade":
            pooled, _ = pool_outputs(self.splade_head(x), batch, "splade")
            _, raw = pool_outputs(x, batch, "cls")
            return pooled, raw
        return pool_outputs(x, batch, self.pool)

    def predict(self, batch: Batch) -> Tensor:
        """Logits [n_seqs, n_classes] by batch position (flash_bert.rs:538-547)."""
        x = self.hidden_states(batch)
        cu = batch.cumulative_seq_lengths.astype(np.int64)
        cls = x[torch.from_numpy(cu[:-1])]
        a = self.all
        if self.roberta:  # RobertaClassificationHead, bert.rs:434-465
            h = torch.tanh(linear(cls, a.get("classifier.dense.weight"), a.get("classifier.dense.bias")))
            return linear(h, a.get("classifier.out_proj.weight"), a.get("classifier.out_proj.bias"))
        h = cls  # BertClassificationHead, bert.rs:374-419
        if a.has("bert.pooler.dense.weight"):
            h = torch.tanh(linear(h, a.get("bert.pooler.dense.weight"), a.get("bert.pooler.dense.bias")))
        return linear(h, a.get("classifier.weight"), a.get("classifier.bias"))

    # Literal padded form (bert.rs:706-879) for small batches: used to show that the unpadded
    # restatement above computes the same numbers.
    def hidden_states_padded(self, batch: Batch) -> Tensor:
        w = self.w
        B, L = len(batch), int(batch.max_length)
        cu = batch.cumulative_seq_lengths.astype(np.int64)
        ids = torch.zeros(B, L, dtype=torch.int64)
        tids = torch.zeros(B, L, dtype=torch.int64)
        pids = torch.zeros(B, L, dtype=torch.int64)
        bias = torch.zeros(B, 1, 1, L)
        for i in range(B):
            n = int(cu[i + 1] - cu[i])
            ids[i, :n] = torch.from_numpy(batch.input_ids[cu[i]:cu[i + 1]].astype(np.int64))
            tids[i, :n] = torch.from_numpy(batch.token_type_ids[cu[i]:cu[i + 1]].astype(np.int64))
            pids[i, :n] = torch.from_numpy(batch.position_ids[cu[i]:cu[i + 1]].astype(np.int64))
            bias[i, :, :, n:] = float("-inf")
        g, b = w.ln("embeddings.LayerNorm")
        x = w.get("embeddings.word_embeddings.weight")[ids] + w.get("embeddings.token_type_embeddings.weight")[tids]
        x = layer_norm(x, w.get("embeddings.position_embeddings.weight")[pids], g, b, self.eps)
        for i in range(self.n_layers):
            p = f"encoder.layer.{i}."

            def heads(t):
                return t.view(B, L, self.nh, self.dh).transpose(1, 2)
            q = heads(linear(x, w.get(p + "attention.self.query.weight"), w.get(p + "attention.self.query.bias")))
            k = heads(linear(x, w.get(p + "attention.self.key.weight"), w.get(p + "attention.self.key.bias")))
            v = heads(linear(x, w.get(p + "attention.self.value.weight"), w.get(p + "attention.self.value.bias")))
            sc = (q @ k.transpose(-1, -2)) * (1.0 / math.sqrt(self.dh)) + bias
            a = (torch.softmax(sc, dim=-1) @ v).transpose(1, 2).reshape(B, L, self.hidden)
            g1, b1 = w.ln(p + "attention.output.LayerNorm")
            x1 = layer_norm(linear(a, w.get(p + "attention.output.dense.weight"),
                                   w.get(p + "attention.output.dense.bias")), x, g1, b1, self.eps)
            f = self.act(linear(x1, w.get(p + "intermediate.dense.weight"), w.get(p + "intermediate.dense.bias")))
            g2, b2 = w.ln(p + "output.LayerNorm")
            x = layer_norm(linear(f, w.get(p + "output.dense.weight"), w.get(p + "output.dense.bias")),
                           x1, g2, b2, self.eps)
        return x  # [B, L, H]


# --------------------------------------------------------------------------- NomicBERT
class NomicOracle:
    def __init__(self, config: dict, tensors: Dict[str, Tensor], model_type: str = "embedding",
                 pool: str = "mean"):
        if model_type == "classifier" or pool == "splade":
            raise ValueError("NomicBERT supports neither classifier nor splade (flash_nomic.rs:222-233)")
        c = config
        # NomicConfig::valid(), models/nomic.rs:49-54
        if c["prenorm"] or c["rotary_emb_fraction"] != 1.0 or c["rotary_emb_interleaved"] or c["type_vocab_size"] <= 0:
            raise ValueError("config is not supported")
        self.cfg = c
        self.pool = pool
        self.w = _Weights(tensors, ("",))
        self.nh = c["n_head"]
        self.hidden = c["n_embd"]
        self.dh = self.hidden // self.nh
        self.eps = float(c["layer_norm_epsilon"])
        self.n_layers = c["n_layer"]
        self.act_name = c["activation_function"]
        self.cos, self.sin = rope_tables(self.dh, float(c["rotary_emb_base"]), int(c["n_positions"]))

    def hidden_states(self, batch: Batch) -> Tensor:
        w, c = self.w, self.cfg
        ids = torch.from_numpy(batch.input_ids.astype(np.int64))
        tids = torch.from_numpy(batch.token_type_ids.astype(np.int64))
        pids = torch.from_numpy(batch.position_ids.astype(np.int64))
        g, b = w.ln("emb_ln")
        x = layer_norm(w.get("embeddings.word_embeddings.weight")[ids],
                       w.get("embeddings.token_type_embeddings.weight")[tids], g, b, self.eps)
        cos, sin = self.cos[pids], self.sin[pids]
        T = x.shape[0]
        cu = batch.cumulative_seq_lengths
        for i in range(self.n_layers):
            p = f"encoder.layers.{i}."
            qkv = linear(x, w.get(p + "attn.Wqkv.weight"),
                         w.get(p + "attn.Wqkv.bias") if c["qkv_proj_bias"] else None)
            q, k, v = qkv.view(T, 3, self.nh, self.dh).unbind(dim=1)
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            a = attention_varlen(q, k, v, cu, 1.0 / math.sqrt(self.dh), False)
            a = linear(a, w.get(p + "attn.out_proj.weight"),
                       w.get(p + "attn.out_proj.bias") if c["qkv_proj_bias"] else None)
            g1, b1 = w.ln(p + "norm1")
            x1 = layer_norm(x, a, g1, b1, self.eps)
            moe_every = c.get("moe_every_n_layers") or 0
            if moe_every > 0 and i % moe_every == 1:
                m = self.moe(x1, p + "mlp.")
            elif self.act_name == "swiglu":
                # fc1 = cat[fc12; fc11]; swiglu = silu(first half) * second half (nomic.rs:115-121)
                gate = linear(x1, w.get(p + "mlp.fc12.weight"), w.get(p + "mlp.fc12.bias") if c["mlp_fc1_bias"] else None)
                up = linear(x1, w.get(p + "mlp.fc11.weight"), w.get(p + "mlp.fc11.bias") if c["mlp_fc1_bias"] else None)
                m = F.silu(gate) * up
            else:
                m = activation(self.act_name)(linear(x1, w.get(p + "mlp.fc1.weight"),
                                                     w.get(p + "mlp.fc1.bias") if c["mlp_fc1_bias"] else None))
            if not (moe_every > 0 and i % moe_every == 1):
                m = linear(m, w.get(p + "mlp.fc2.weight"), w.get(p + "mlp.fc2.bias") if c["mlp_fc2_bias"] else None)
            g2, b2 = w.ln(p + "norm2")
            x = layer_norm(x1, m, g2, b2, self.eps)
        return x

    def moe(self, x: Tensor, p: str) -> Tensor:
        """NomicMoELayer (models/nomic.rs:205-394): router logits -> fp32 softmax -> the top-k
        probabilities as they are (no renormalisation) `:229-243`; expert e computes
        act(x w1_e^T) w2_e with w1, w2 stored as [E * I, H] `:255-276`; the weighted expert outputs
        are summed per token and the shared bias is added `:325-355`."""
        w, c = self.w, self.cfg
        E, k, I = c["num_experts"], c["moe_top_k"], c["n_inner"]
        probs = torch.softmax(linear(x, w.get(p + "router.layer.weight")).float(), dim=-1)
        top_w, top_e = probs.topk(k, dim=-1)
        w1 = w.get(p + "experts.mlp.w1").view(E, I, self.hidden)
        w2 = w.get(p + "experts.mlp.w2").view(E, I, self.hidden)
        act = activation(self.act_name)
        out = torch.zeros_like(x)
        for e in range(E):
            tok, slot = (top_e == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            y = act(x[tok] @ w1[e].t()) @ w2[e]
            out.index_add_(0, tok, y * top_w[tok, slot].unsqueeze(-1))
        return out + w.get(p + "experts.bias")

    def embed(self, batch: Batch):
        return pool_outputs(self.hidden_states(batch), batch, self.pool)


# --------------------------------------------------------------------------- Qwen3
class Qwen3Oracle:
    """The decoder families: Qwen3 (models/qwen3.rs, flash_qwen3.rs), Qwen2 (flash_qwen2.rs: q/k/v
    biases, `is_causal`, no q/k norm) and Mistral / Llama (flash_mistral.rs: no biases, no q/k norm,
    optional `sliding_window` as the attention's left window; Llama configs run as Mistral,
    backends/candle/src/lib.rs:549-575)."""

    def __init__(self, config: dict, tensors: Dict[str, Tensor], model_type: str = "embedding",
                 pool: str = "last_token"):
        if model_type == "classifier" or pool == "splade":
            raise ValueError("the decoder families support neither classifier nor splade here")
        c = config
        mt = c["model_type"]
        if mt in ("qwen3", "qwen2") and c.get("use_sliding_window"):
            raise ValueError("sliding window is not supported (flash_qwen3.rs:32-34, flash_qwen2.rs:26-29)")
        if mt == "llama" and c.get("rope_scaling") is not None:
            raise ValueError("Rope scaling is not supported for FlashLlama yet")  # lib.rs:549-553
        self.qk_norm = mt == "qwen3"
        self.qkv_bias = mt == "qwen2"
        self.window_left = c.get("sliding_window") if mt == "mistral" else None
        self.cfg = c
        self.pool = pool
        prefix = "model." if "model.embed_tokens.weight" in tensors else ""
        self.w = _Weights(tensors, (prefix,))
        self.all = _Weights(tensors, ("",))
        self.nh = c["num_attention_heads"]
        self.nkv = c["num_key_value_heads"]
        self.hidden = c["hidden_size"]
        self.dh = (c.get("head_dim") if mt == "qwen3" else None) or self.hidden // self.nh
        self.eps = float(c["rms_norm_eps"])
        self.n_layers = c["num_hidden_layers"]
        theta = c.get("rope_theta")
        if theta is None:
            theta = c["rope_parameters"]["rope_theta"]
        if mt == "qwen2":
            self.causal = bool(c.get("is_causal", True))  # qwen2.rs:4-7,26-27
        else:
            self.causal = not c.get("use_bidirectional_attention", False)
        # only Mistral passes its `rope_scaling` on (flash_mistral.rs:278-283); Qwen2 / Qwen3 do not
        scaling = c.get("rope_scaling") if mt == "mistral" else None
        self.cos, self.sin = rope_tables(self.dh, float(theta), int(c["max_position_embeddings"]), scaling)

    def hidden_states(self, batch: Batch) -> Tensor:
        w = self.w
        ids = torch.from_numpy(batch.input_ids.astype(np.int64))
        pids = torch.from_numpy(batch.position_ids.astype(np.int64))
        h = w.get("embed_tokens.weight")[ids]
        cos, sin = self.cos[pids], self.sin[pids]
        T = h.shape[0]
        cu = batch.cumulative_seq_lengths
        residual = None
        for i in range(self.n_layers):
            p = f"layers.{i}."
            n, residual = rms_norm(h, residual, w.get(p + "input_layernorm.weight"), self.eps)
            bias = (lambda name: w.get(p + f"self_attn.{name}.bias")) if self.qkv_bias else (lambda name: None)
            q = linear(n, w.get(p + "self_attn.q_proj.weight"), bias("q_proj")).view(T, self.nh, self.dh)
            k = linear(n, w.get(p + "self_attn.k_proj.weight"), bias("k_proj")).view(T, self.nkv, self.dh)
            v = linear(n, w.get(p + "self_attn.v_proj.weight"), bias("v_proj")).view(T, self.nkv, self.dh)
            if self.qk_norm:
                q, _ = rms_norm(q, None, w.get(p + "self_attn.q_norm.weight"), self.eps)
                k, _ = rms_norm(k, None, w.get(p + "self_attn.k_norm.weight"), self.eps)
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            a = attention_varlen(q, k, v, cu, 1.0 / math.sqrt(self.dh), self.causal, None, self.window_left)
            o = linear(a, w.get(p + "self_attn.o_proj.weight"))
            n2, residual = rms_norm(o, residual, w.get(p + "post_attention_layernorm.weight"), self.eps)
            gate = linear(n2, w.get(p + "mlp.gate_proj.weight"))
            up = linear(n2, w.get(p + "mlp.up_proj.weight"))
            h = linear(F.silu(gate) * up, w.get(p + "mlp.down_proj.weight"))
        out, _ = rms_norm(h, residual, w.get("norm.weight"), self.eps)
        if self.all.has("linear.weight"):  # optional projection, flash_qwen3.rs:344-357,430-435
            out = linear(out, self.all.get("linear.weight"))
        return out

    def embed(self, batch: Batch):
        return pool_outputs(self.hidden_states(batch), batch, self.pool)


# --------------------------------------------------------------------------- GTE
class GTEOracle:
    """models/gte.rs (CPU arm) / flash_gte.rs: LN(word [+ token type]) (flash_gte.rs:243-268),
    post-LayerNorm blocks with biased qkv_proj / o_proj, RoPE whose inverse frequencies may be
    NTK-scaled - base * factor, divided by factor^(2 / dim) (layers/rotary.rs:86-93) - and the
    feed-forward act(second half of up_gate_proj x) * first half -> down_proj (gte.rs:216-227).
    Head: optional pooler.dense + tanh, then classifier, on the CLS row (gte.rs:282-340)."""

    def __init__(self, config: dict, tensors: Dict[str, Tensor], model_type: str = "embedding", pool: str = "cls"):
        c = config
        if pool == "splade":
            raise ValueError("`splade` is not supported for GTE")
        if c.get("logn_attention_scale") or c.get("logn_attention_clip1") or c["position_embedding_type"] != "rope":
            raise ValueError("config is not supported (flash_gte.rs:177-186)")
        self.cfg = c
        self.model_type = model_type
        self.pool = "cls" if model_type == "classifier" else pool
        prefix = "new." if "new.embeddings.word_embeddings.weight" in tensors else ""
        self.w = _Weights(tensors, (prefix,))
        self.all = _Weights(tensors, ("",))
        self.nh = c["num_attention_heads"]
        self.hidden = c["hidden_size"]
        self.dh = self.hidden // self.nh
        self.inter = c["intermediate_size"]
        self.eps = float(c["layer_norm_eps"])
        self.n_layers = c["num_hidden_layers"]
        self.act = activation(c["hidden_act"])
        theta = c.get("rope_theta")
        if theta is None:
            theta = c["rope_parameters"]["rope_theta"]
        theta = float(theta)
        scaling = c.get("rope_scaling")
        n_pos = int(c["max_position_embeddings"])
        if scaling:
            f = float(scaling["factor"])
            # inv_freq = 1 / (theta * f)^(i / dim) / f^(2 / dim), angles in f32
            i = torch.arange(0, self.dh, 2, dtype=torch.float32)
            inv = (1.0 / torch.pow(torch.tensor(theta * f, dtype=torch.float32), i / self.dh)) / (f ** (2.0 / self.dh))
            ang = torch.arange(n_pos, dtype=torch.float32)[:, None] * inv[None, :]
            cos, sin = ang.cos(), ang.sin()
        else:
            cos, sin = rope_tables(self.dh, theta, n_pos)
        self.cos, self.sin = cos, sin

    def hidden_states(self, batch: Batch) -> Tensor:
        w, c = self.w, self.cfg
        ids = torch.from_numpy(batch.input_ids.astype(np.int64))
        pids = torch.from_numpy(batch.position_ids.astype(np.int64))
        g, b = w.ln("embeddings.LayerNorm")
        typ = None
        if c["type_vocab_size"] > 0:
            typ = w.get("embeddings.token_type_embeddings.weight")[torch.from_numpy(batch.token_type_ids.astype(np.int64))]
        x = layer_norm(w.get("embeddings.word_embeddings.weight")[ids], typ, g, b, self.eps)
        cos, sin = self.cos[pids], self.sin[pids]
        T, H = x.shape
        cu = batch.cumulative_seq_lengths
        for i in range(self.n_layers):
            p = f"encoder.layer.{i}."
            qkv = linear(x, w.get(p + "attention.qkv_proj.weight"), w.get(p + "attention.qkv_proj.bias"))
            q, k, v = (qkv[:, j * H:(j + 1) * H].reshape(T, self.nh, self.dh) for j in range(3))
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            a = attention_varlen(q, k, v, cu, 1.0 / math.sqrt(self.dh), False)
            a = linear(a, w.get(p + "attention.o_proj.weight"), w.get(p + "attention.o_proj.bias"))
            g1, b1 = w.ln(p + "attn_ln")
            x1 = layer_norm(a, x, g1, b1, self.eps)
            ug = linear(x1, w.get(p + "mlp.up_gate_proj.weight"))
            m = self.act(ug[:, self.inter:]) * ug[:, :self.inter]
            m = linear(m, w.get(p + "mlp.down_proj.weight"), w.get(p + "mlp.down_proj.bias"))
            g2, b2 = w.ln(p + "mlp_ln")
            x = layer_norm(m, x1, g2, b2, self.eps)
        return x

    def embed(self, batch: Batch):
        return pool_outputs(self.hidden_states(batch), batch, self.pool)

    def predict(self, batch: Batch) -> Tensor:
        x = self.hidden_states(batch)
        cu = batch.cumulative_seq_lengths.astype(np.int64)
        h = x[torch.from_numpy(cu[:-1])]
        if self.w.has("pooler.dense.weight") and self.w.has("pooler.dense.bias"):
            h = torch.tanh(linear(h, self.w.get("pooler.dense.weight"), self.w.get("pooler.dense.bias")))
        return linear(h, self.all.get("classifier.weight"), self.all.get("classifier.bias"))


# --------------------------------------------------------------------------- DistilBERT
class DistilBertOracle:
    """models/distilbert.rs (CPU arm) / flash_distilbert.rs: BERT blocks without token types:
    LN(word + position) (distilbert.rs:58-70), q_lin / k_lin / v_lin / out_lin, sa_layer_norm on
    the attention residual, ffn.lin1 -> activation -> ffn.lin2, output_layer_norm; every
    LayerNorm with eps 1e-12 (flash_distilbert.rs:113-115)."""

    def __init__(self, config: dict, tensors: Dict[str, Tensor], model_type: str = "embedding", pool: str = "cls"):
        if model_type == "classifier" or pool == "splade":
            raise ValueError("DistilBERT: embedding models with cls / mean / last-token pooling only here")
        c = config
        self.cfg = c
        self.pool = pool
        if "embeddings.word_embeddings.weight" in tensors and "encoder.layer.0.attention.q_lin.weight" in tensors:
            self.emb, self.enc = "embeddings.", "encoder."
        elif "distilbert.embeddings.word_embeddings.weight" in tensors:
            self.emb, self.enc = "distilbert.embeddings.", "distilbert.transformer."
        else:
            self.emb, self.enc = "embeddings.", "transformer."
        self.w = _Weights(tensors, ("",))
        self.nh = c["n_heads"]
        self.hidden = c["dim"]
        self.dh = self.hidden // self.nh
        self.eps = 1e-12
        self.act = activation(c["activation"])
        self.n_layers = c["n_layers"]

    def hidden_states(self, batch: Batch) -> Tensor:
        w = self.w
        ids = torch.from_numpy(batch.input_ids.astype(np.int64))
        pids = torch.from_numpy(batch.position_ids.astype(np.int64))
        g, b = w.ln(self.emb + "LayerNorm")
        x = layer_norm(w.get(self.emb + "word_embeddings.weight")[ids],
                       w.get(self.emb + "position_embeddings.weight")[pids], g, b, self.eps)
        cu = batch.cumulative_seq_lengths
        T = x.shape[0]
        for i in range(self.n_layers):
            p = f"{self.enc}layer.{i}."
            q, k, v = (linear(x, w.get(p + f"attention.{n}.weight"), w.get(p + f"attention.{n}.bias")).view(T, self.nh, self.dh)
                       for n in ("q_lin", "k_lin", "v_lin"))
            a = attention_varlen(q, k, v, cu, 1.0 / math.sqrt(self.dh), False)
            g1, b1 = w.ln(p + "sa_layer_norm")
            x1 = layer_norm(linear(a, w.get(p + "attention.out_lin.weight"), w.get(p + "attention.out_lin.bias")),
                            x, g1, b1, self.eps)
            f = self.act(linear(x1, w.get(p + "ffn.lin1.weight"), w.get(p + "ffn.lin1.bias")))
            g2, b2 = w.ln(p + "output_layer_norm")
            x = layer_norm(linear(f, w.get(p + "ffn.lin2.weight"), w.get(p + "ffn.lin2.bias")), x1, g2, b2, self.eps)
        return x

    def embed(self, batch: Batch):
        return pool_outputs(self.hidden_states(batch), batch, self.pool)


# --------------------------------------------------------------------------- ModernBERT
class ModernBertOracle:
    """models/modernbert.rs (CPU arm) / flash_modernbert.rs: LayerNorm (weight only) after the
    token embedding; pre-norm blocks x = x + attn(attn_norm(x)), x = x + mlp(mlp_norm(x)) with no
    attn_norm in layer 0 (flash_modernbert.rs:131-139,161-191); RoPE with `global_rope_theta` on
    every `global_attn_every_n_layers`-th layer and `local_rope_theta` plus a window of
    `local_attention / 2` keys on each side elsewhere (`:53-62,92-111,299-313`); feed-forward
    act(Wi x [:I]) * Wi x [I:] -> Wo (modernbert.rs:115-131) with the tanh GELU every GELU name
    means on this backend; final LayerNorm.  Head: dense (no bias) + classifier_activation ->
    LayerNorm -> classifier on the CLS or mean row (modernbert.rs:401-456,481-489)."""

    def __init__(self, config: dict, tensors: Dict[str, Tensor], model_type: str = "embedding", pool: str = "cls"):
        c = config
        if pool == "splade":
            raise ValueError("`splade` is not supported for ModernBert")
        self.cfg = c
        self.model_type = model_type
        self.pool = (c.get("classifier_pooling") or "cls") if model_type == "classifier" else pool
        prefix = "model." if "model.embeddings.tok_embeddings.weight" in tensors else ""
        self.w = _Weights(tensors, (prefix,))
        self.all = _Weights(tensors, ("",))
        self.nh = c["num_attention_heads"]
        self.hidden = c["hidden_size"]
        self.dh = self.hidden // self.nh
        self.inter = c["intermediate_size"]
        self.eps = float(c["norm_eps"])
        self.n_layers = c["num_hidden_layers"]
        self.every = c["global_attn_every_n_layers"]
        self.window = c["local_attention"] // 2
        self.act = activation(c["hidden_activation"])
        n_pos = int(c["max_position_embeddings"])
        self.rope = {False: rope_tables(self.dh, float(c["global_rope_theta"]), n_pos),
                     True: rope_tables(self.dh, float(c["local_rope_theta"]), n_pos)}

    def hidden_states(self, batch: Batch) -> Tensor:
        w = self.w
        ids = torch.from_numpy(batch.input_ids.astype(np.int64))
        pids = torch.from_numpy(batch.position_ids.astype(np.int64))
        zero = torch.zeros(self.hidden)
        x = layer_norm(w.get("embeddings.tok_embeddings.weight")[ids], None, w.get("embeddings.norm.weight"), zero, self.eps)
        T, H = x.shape
        cu = batch.cumulative_seq_lengths
        for i in range(self.n_layers):
            p = f"layers.{i}."
            local = i % self.every != 0
            a_in = x if i == 0 else layer_norm(x, None, w.get(p + "attn_norm.weight"), zero, self.eps)
            qkv = linear(a_in, w.get(p + "attn.Wqkv.weight"), w.get(p + "attn.Wqkv.bias") if w.has(p + "attn.Wqkv.bias") else None)
            q, k, v = (qkv[:, j * H:(j + 1) * H].reshape(T, self.nh, self.dh) for j in range(3))
            cos, sin = self.rope[local]
            q, k = apply_rope(q, cos[pids], sin[pids]), apply_rope(k, cos[pids], sin[pids])
            win = self.window if local else None
            a = attention_varlen(q, k, v, cu, 1.0 / math.sqrt(self.dh), False, None, win, win)
            x = x + linear(a, w.get(p + "attn.Wo.weight"), w.get(p + "attn.Wo.bias") if w.has(p + "attn.Wo.bias") else None)
            m = layer_norm(x, None, w.get(p + "mlp_norm.weight"), zero, self.eps)
            h = linear(m, w.get(p + "mlp.Wi.weight"), w.get(p + "mlp.Wi.bias") if w.has(p + "mlp.Wi.bias") else None)
            f = self.act(h[:, :self.inter]) * h[:, self.inter:]
            x = x + linear(f, w.get(p + "mlp.Wo.weight"), w.get(p + "mlp.Wo.bias") if w.has(p + "mlp.Wo.bias") else None)
        return layer_norm(x, None, w.get("final_norm.weight"), zero, self.eps)

    def embed(self, batch: Batch):
        return pool_outputs(self.hidden_states(batch), batch, self.pool)

    def predict(self, batch: Batch) -> Tensor:
        x = self.hidden_states(batch)
        all_pooled = Batch(batch.input_ids, batch.token_type_ids, batch.position_ids, batch.cumulative_seq_lengths,
                           batch.max_length, np.arange(len(batch), dtype=np.uint32), np.zeros(0, dtype=np.uint32))
        pooled, _ = pool_outputs(x, all_pooled, self.pool)
        a = self.all
        h = activation(self.cfg["classifier_activation"])(linear(pooled, a.get("head.dense.weight")))
        h = layer_norm(h, None, a.get("head.norm.weight"), torch.zeros(self.hidden), self.eps)
        return linear(h, a.get("classifier.weight"), a.get("classifier.bias"))


# --------------------------------------------------------------------------- JinaBERT
def is_jina_bert(config: dict) -> bool:
    # BertConfigWrapper, backends/candle/src/lib.rs:83-121
    name = config.get("_name_or_path", "") or ""
    auto = (config.get("auto_map") or {}).get("AutoConfig", "") or ""
    return config.get("model_type") == "bert" and (
        name == "jinaai/jina-bert-implementation" or "jinaai/jina-bert-implementation" in auto)


class JinaBertOracle(BertOracle):
    """models/jina.rs (CPU arm) / flash_jina.rs: BERT with a gated feed-forward
    (`mlp.gated_layers` without bias -> act(first half) * second half -> `mlp.wo` -> `mlp.layernorm`
    with the residual, jina.rs:260-300, flash_jina.rs:166-189), and either ALiBi
    (bias = -slope_h * |i - j|, alibi.rs:49-80; no position table, jina.rs:54-74) or absolute
    positions.  Head: optional `bert.pooler.dense` + tanh, then `classifier` (jina.rs:342-393)."""

    def __init__(self, config: dict, tensors: Dict[str, Tensor], model_type: str = "embedding",
                 pool: str = "cls"):
        cfg = dict(config)
        pos = cfg.get("position_embedding_type", "absolute")
        if pos not in ("absolute", "alibi"):
            raise ValueError("not supported")  # flash_jina.rs:243
        cfg["position_embedding_type"] = "absolute"  # the base class only checks the field
        super().__init__(cfg, tensors, model_type, pool)
        if self.pool == "splade":
            raise ValueError("`splade` is not supported for Jina")
        self.alibi = pos == "alibi"
        self.inter = config["intermediate_size"]

    def hidden_states(self, batch: Batch) -> Tensor:
        w = self.w
        ids = torch.from_numpy(batch.input_ids.astype(np.int64))
        tids = torch.from_numpy(batch.token_type_ids.astype(np.int64))
        g, b = w.ln("embeddings.LayerNorm")
        word = w.get("embeddings.word_embeddings.weight")[ids]
        typ = w.get("embeddings.token_type_embeddings.weight")[tids]
        if self.alibi:
            x = layer_norm(word, typ, g, b, self.eps)
        else:
            pids = torch.from_numpy(batch.position_ids.astype(np.int64))
            x = layer_norm(word + typ, w.get("embeddings.position_embeddings.weight")[pids], g, b, self.eps)
        slopes = alibi_slopes(self.nh) if self.alibi else None
        cu = batch.cumulative_seq_lengths
        T = x.shape[0]
        for i in range(self.n_layers):
            p = f"encoder.layer.{i}."
            q = linear(x, w.get(p + "attention.self.query.weight"), w.get(p + "attention.self.query.bias"))
            k = linear(x, w.get(p + "attention.self.key.weight"), w.get(p + "attention.self.key.bias"))
            v = linear(x, w.get(p + "attention.self.value.weight"), w.get(p + "attention.self.value.bias"))
            a = attention_varlen(q.view(T, self.nh, self.dh), k.view(T, self.nh, self.dh),
                                 v.view(T, self.nh, self.dh), cu, 1.0 / math.sqrt(self.dh), False, slopes)
            g1, b1 = w.ln(p + "attention.output.LayerNorm")
            x1 = layer_norm(linear(a, w.get(p + "attention.output.dense.weight"),
                                   w.get(p + "attention.output.dense.bias")), x, g1, b1, self.eps)
            h = linear(x1, w.get(p + "mlp.gated_layers.weight"), None)
            f = self.act(h[:, :self.inter]) * h[:, self.inter:]
            g2, b2 = w.ln(p + "mlp.layernorm")
            x = layer_norm(linear(f, w.get(p + "mlp.wo.weight"), w.get(p + "mlp.wo.bias")), x1, g2, b2, self.eps)
        return x

    def embed(self, batch: Batch):
        return pool_outputs(self.hidden_states(batch), batch, self.pool)

    def predict(self, batch: Batch) -> Tensor:
        x = self.hidden_states(batch)
        cu = batch.cumulative_seq_lengths.astype(np.int64)
        h = x[torch.from_numpy(cu[:-1])]
        a = self.all
        if a.has("bert.pooler.dense.weight"):
            h = torch.tanh(linear(h, a.get("bert.pooler.dense.weight"), a.get("bert.pooler.dense.bias")))
        return linear(h, a.get("classifier.weight"), a.get("classifier.bias"))


def is_jina_code_bert(config: dict) -> bool:
    # BertConfigWrapper, backends/candle/src/lib.rs:83-121
    name = config.get("_name_or_path", "") or ""
    auto = (config.get("auto_map") or {}).get("AutoConfig", "") or ""
    return config.get("model_type") == "bert" and (
        name == "jinaai/jina-bert-v2-qk-post-norm" or "jinaai/jina-bert-v2-qk-post-norm" in auto)


class JinaCodeBertOracle(JinaBertOracle):
    """models/jina_code.rs / flash_jina_code.rs: JinaBERT's embeddings and ALiBi, with
      * LayerNorm over the whole q row and the whole k row before attention
        (flash_jina_code.rs:112-120),
      * a = LN_out(dense(attention) + x)  (:147-150), h = layer_norm_1(a + x)  (:226-230: the
        residual is the layer's input again),
      * up_gated_layer without bias, first half * act(second half)  (:234-240), down_layer,
        layer_norm_2(down + h)  (:243-245).
    Embedding models only (no classifier, no splade, :305-315)."""

    def __init__(self, config: dict, tensors: Dict[str, Tensor], model_type: str = "embedding",
                 pool: str = "cls"):
        if model_type == "classifier":
            raise ValueError("`classifier` model type is not supported for Jina Code")
        super().__init__(config, tensors, model_type, pool)

    def hidden_states(self, batch: Batch) -> Tensor:
        w = self.w
        ids = torch.from_numpy(batch.input_ids.astype(np.int64))
        tids = torch.from_numpy(batch.token_type_ids.astype(np.int64))
        g, b = w.ln("embeddings.LayerNorm")
        word = w.get("embeddings.word_embeddings.weight")[ids]
        typ = w.get("embeddings.token_type_embeddings.weight")[tids]
        if self.alibi:
            x = layer_norm(word, typ, g, b, self.eps)
        else:
            pids = torch.from_numpy(batch.position_ids.astype(np.int64))
            x = layer_norm(word + typ, w.get("embeddings.position_embeddings.weight")[pids], g, b, self.eps)
        slopes = alibi_slopes(self.nh) if self.alibi else None
        cu = batch.cumulative_seq_lengths
        T = x.shape[0]
        for i in range(self.n_layers):
            p = f"encoder.layer.{i}."
            q = linear(x, w.get(p + "attention.self.query.weight"), w.get(p + "attention.self.query.bias"))
            k = linear(x, w.get(p + "attention.self.key.weight"), w.get(p + "attention.self.key.bias"))
            v = linear(x, w.get(p + "attention.self.value.weight"), w.get(p + "attention.self.value.bias"))
            gq, bq = w.ln(p + "attention.self.layer_norm_q")
            gk, bk = w.ln(p + "attention.self.layer_norm_k")
            q = layer_norm(q, None, gq, bq, self.eps)
            k = layer_norm(k, None, gk, bk, self.eps)
            a = attention_varlen(q.view(T, self.nh, self.dh), k.view(T, self.nh, self.dh),
                                 v.view(T, self.nh, self.dh), cu, 1.0 / math.sqrt(self.dh), False, slopes)
            go, bo = w.ln(p + "attention.output.LayerNorm")
            a = layer_norm(linear(a, w.get(p + "attention.output.dense.weight"),
                                  w.get(p + "attention.output.dense.bias")), x, go, bo, self.eps)
            g1, b1 = w.ln(p + "layer_norm_1")
            h = layer_norm(a, x, g1, b1, self.eps)
            u = linear(h, w.get(p + "mlp.up_gated_layer.weight"), None)
            f = u[:, :self.inter] * self.act(u[:, self.inter:])
            g2, b2 = w.ln(p + "layer_norm_2")
            x = layer_norm(linear(f, w.get(p + "mlp.down_layer.weight"), w.get(p + "mlp.down_layer.bias")),
                           h, g2, b2, self.eps)
        return x


def build_oracle(model_dir, model_type: str = "embedding", pool: str = "cls"):
    """Dispatch on config.json's model_type like backends/candle/src/lib.rs:124-154,282-577."""
    config, tensors = load_model_dir(model_dir)
    mt = config["model_type"]
    if is_jina_code_bert(config):
        return JinaCodeBertOracle(config, tensors, model_type, pool)
    if is_jina_bert(config):
        return JinaBertOracle(config, tensors, model_type, pool)
    if mt in ("bert", "roberta", "xlm-roberta", "camembert"):
        return BertOracle(config, tensors, model_type, pool)
    if mt == "nomic_bert":
        return NomicOracle(config, tensors, model_type, pool)
    if mt in ("qwen3", "qwen2", "mistral", "llama"):
        return Qwen3Oracle(config, tensors, model_type, pool)
    if mt == "modernbert":
        return ModernBertOracle(config, tensors, model_type, pool)
    if mt == "distilbert":
        return DistilBertOracle(config, tensors, model_type, pool)
    if mt in ("gte", "new"):
        return GTEOracle(config, tensors, model_type, pool)
    raise ValueError(f"model_type {mt} is outside the hot path")
