"""torch-tensor wrappers of the kernel-level C ABI (include/tei_b200_ops.h).

torch is used only to hold device memory and the current stream; every call goes straight into
libtei_b200.so.  These wrappers exist for the tests and the benchmark; the serving path calls
the same kernels from C++.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib

ACT = {"none": 0, "gelu": 1, "relu": 2, "tanh": 3, "swiglu": 4, "relu_log1p": 5, "geglu": 6}
POOL = {"cls": 0, "mean": 1, "splade": 2, "max": 2, "last_token": 3}


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"unsupported dtype {t.dtype}")


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def new_status(device="cuda") -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor, what: str = "kernel"):
    code = int(status.item())
    if code != 0:
        raise RuntimeError(f"{what}: device status {code} (a bounded wait ran out)")


def linear(a, w, bias=None, residual=None, act="none", out=None, status=None):
    """out = act(a @ w.T + bias) (+ residual); for act == 'swiglu' / 'geglu' w/bias are pre-interleaved."""
    lib = _lib.load()
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if act in ("swiglu", "geglu") else N
    if out is None:
        out = torch.empty((M, n_out), dtype=a.dtype, device=a.device)
    own = status is None
    if own:
        status = new_status(a.device)
    rc = lib.tei_b200_op_linear(
        _p(a), _p(w), _p(bias), _p(residual), _p(out), M, N, K, a.stride(0), out.stride(0),
        residual.stride(0) if residual is not None else 0, ACT[act], _dt(a), _p(status), _stream())
    _check(rc, "tei_b200_op_linear")
    if own:
        check_status(status, "linear")
    return out


def linear_rope(a, w, bias, pos_ids, cos, sin, q_gamma, k_gamma, head_dim, q_cols, k_cols, eps=0.0, out=None,
                status=None):
    """The fused q/k/v projection with per-head RMSNorm (optional) + RoPE on its q and k heads."""
    lib = _lib.load()
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    own = status is None
    if own:
        status = new_status(a.device)
    rc = lib.tei_b200_op_linear_rope(
        _p(a), _p(w), _p(bias), _p(out), M, N, K, a.stride(0), out.stride(0), _p(pos_ids), _p(cos), _p(sin),
        _p(q_gamma), _p(k_gamma), int(head_dim), int(q_cols), int(k_cols), float(eps), _dt(a), _p(status), _stream())
    _check(rc, "tei_b200_op_linear_rope")
    if own:
        check_status(status, "linear_rope")
    return out


def interleave_swiglu(gate_w: torch.Tensor, up_w: torch.Tensor) -> torch.Tensor:
    """Rows [gate block 0 (128), up block 0 (128), gate block 1, ...] as the SwiGLU epilogue expects."""
    inter = gate_w.shape[0]
    assert inter % 128 == 0 and up_w.shape == gate_w.shape
    g = gate_w.reshape(inter // 128, 128, *gate_w.shape[1:])
    u = up_w.reshape(inter // 128, 128, *up_w.shape[1:])
    return torch.stack([g, u], dim=1).reshape(2 * inter, *gate_w.shape[1:]).contiguous()


def attention_plan(cu_seqlens, causal: bool, window_left: int = -1, window_right: int = -1) -> np.ndarray:
    lib = _lib.load()
    cu = np.ascontiguousarray(np.asarray(cu_seqlens, dtype=np.int32))
    n_seqs = len(cu) - 1
    cu_p = cu.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
    n = lib.tei_b200_attention_plan_windowed(cu_p, n_seqs, int(causal), window_left, window_right, None, 0)
    work = np.zeros((max(n, 1), 4), dtype=np.int32)
    n2 = lib.tei_b200_attention_plan_windowed(cu_p, n_seqs, int(causal), window_left, window_right,
                                              work.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), n)
    assert n2 == n
    return work[:n]


def attention(q, k, v, cu_seqlens, causal=False, scale=None, alibi_slopes=None, work=None,
              out=None, status=None, window_left: int = -1, window_right: int = -1):
    """q [T, nh, D], k/v [T, nkv, D] (views with unit stride in the last two dims).  Key j counts
    for query i when i - window_left <= j <= i + window_right (-1: no limit; causal: right 0)."""
    lib = _lib.load()
    T, nh, D = q.shape
    nkv = k.shape[1]
    assert q.stride(2) == 1 and q.stride(1) == D and k.stride(1) == D and v.stride(1) == D
    if scale is None:
        scale = 1.0 / float(D) ** 0.5
    if work is None:
        work = torch.from_numpy(attention_plan(cu_seqlens, causal, window_left, window_right)).to(q.device)
    if out is None:
        out = torch.empty((T, nh * D), dtype=q.dtype, device=q.device)
    own = status is None
    if own:
        status = new_status(q.device)
    rc = lib.tei_b200_op_attention_windowed(
        _p(q), _p(k), _p(v), _p(out), _p(work), work.shape[0], T, nh, nkv, D, q.stride(0),
        k.stride(0), v.stride(0), out.stride(0), int(causal), int(window_left), int(window_right),
        float(scale), _p(alibi_slopes), _dt(q), _p(status), _stream())
    _check(rc, "tei_b200_op_attention")
    if own:
        check_status(status, "attention")
    return out


def embed_layernorm(ids, type_ids, pos_ids, word, type_tab, pos_tab, gamma, beta, eps):
    lib = _lib.load()
    T = ids.shape[0]
    H = word.shape[1]
    out = torch.empty((T, H), dtype=word.dtype, device=word.device)
    rc = lib.tei_b200_op_embed_layernorm(
        _p(ids), _p(type_ids), _p(pos_ids), _p(word), _p(type_tab), _p(pos_tab), _p(gamma),
        _p(beta), _p(out), T, H, float(eps), _dt(word), _stream())
    _check(rc, "tei_b200_op_embed_layernorm")
    return out


def add_layernorm(x, residual, gamma, beta, eps):
    lib = _lib.load()
    T, H = x.shape
    out = torch.empty_like(x)
    rc = lib.tei_b200_op_add_norm(_p(x), _p(residual), _p(gamma), _p(beta), _p(out), None, T, H,
                                  float(eps), 0, _dt(x), _stream())
    _check(rc, "tei_b200_op_add_norm")
    return out


def add_rmsnorm(x, residual_f32, gamma, eps):
    """Returns (normed [T,H] model dtype, sum [T,H] fp32)."""
    lib = _lib.load()
    T, H = x.shape
    out = torch.empty_like(x)
    sum_out = torch.empty((T, H), dtype=torch.float32, device=x.device)
    rc = lib.tei_b200_op_add_norm(_p(x), _p(residual_f32), _p(gamma), None, _p(out), _p(sum_out),
                                  T, H, float(eps), 1, _dt(x), _stream())
    _check(rc, "tei_b200_op_add_norm")
    return out, sum_out


def qk_norm_rope_(q, k, pos_ids, cos, sin, q_gamma=None, k_gamma=None, eps=1e-6):
    """In place.  q [T, nh, D], k [T, nkv, D] views; cos/sin fp32 [max_pos, D/2]."""
    lib = _lib.load()
    T, nh, D = q.shape
    nkv = k.shape[1]
    rc = lib.tei_b200_op_qk_norm_rope(
        _p(q), _p(k), _p(pos_ids), _p(cos), _p(sin), _p(q_gamma), _p(k_gamma), T, nh, nkv, D,
        q.stride(0), k.stride(0), float(eps), _dt(q), _stream())
    _check(rc, "tei_b200_op_qk_norm_rope")


def pool(x, cu_seqlens_dev, seq_index_dev, mode: str, normalize: bool):
    lib = _lib.load()
    H = x.shape[1]
    n_out = seq_index_dev.shape[0]
    out = torch.empty((n_out, H), dtype=torch.float32, device=x.device)
    rc = lib.tei_b200_op_pool(_p(x), _p(cu_seqlens_dev), _p(seq_index_dev), _p(out), n_out, H,
                              POOL[mode], int(normalize), _dt(x), _stream())
    _check(rc, "tei_b200_op_pool")
    return out


def gather_rows_f32(x, row_index_dev):
    lib = _lib.load()
    n = row_index_dev.shape[0]
    H = x.shape[1]
    out = torch.empty((n, H), dtype=torch.float32, device=x.device)
    rc = lib.tei_b200_op_gather_rows_f32(_p(x), _p(row_index_dev), _p(out), n, H, _dt(x), _stream())
    _check(rc, "tei_b200_op_gather_rows_f32")
    return out


def head_linear(x_f32, w, b, act="none"):
    lib = _lib.load()
    rows, K = x_f32.shape
    N = w.shape[0]
    out = torch.empty((rows, N), dtype=torch.float32, device=x_f32.device)
    rc = lib.tei_b200_op_head_linear(_p(x_f32), _p(w), _p(b), _p(out), rows, N, K, ACT[act],
                                     _dt(w), _stream())
    _check(rc, "tei_b200_op_head_linear")
    return out


def linear_rows_dev(a, w, bias, m_rows_dev, act="none", out=None, status=None):
    """linear() on the first min(M, m_rows_dev[0]) rows of `a` (int32 device scalar)."""
    lib = _lib.load()
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if act in ("swiglu", "geglu") else N
    if out is None:
        out = torch.empty((M, n_out), dtype=a.dtype, device=a.device)
    own = status is None
    if own:
        status = new_status(a.device)
    rc = lib.tei_b200_op_linear_rows_dev(_p(a), _p(w), _p(bias), _p(out), M, N, K, a.stride(0), out.stride(0),
                                         ACT[act], _dt(a), _p(m_rows_dev), _p(status), _stream())
    _check(rc, "tei_b200_op_linear_rows_dev")
    if own:
        check_status(status, "linear_rows_dev")
    return out


def moe_route(logits, n_experts: int, top_k: int):
    """logits [T, >= n_experts] -> (expert int32 [T, k], weight fp32 [T, k], pos int32 [T, k],
    counts int32 [n_experts])."""
    lib = _lib.load()
    T = logits.shape[0]
    dev = logits.device
    te = torch.empty((T, top_k), dtype=torch.int32, device=dev)
    tw = torch.empty((T, top_k), dtype=torch.float32, device=dev)
    pos = torch.empty((T, top_k), dtype=torch.int32, device=dev)
    counts = torch.empty((n_experts,), dtype=torch.int32, device=dev)
    rc = lib.tei_b200_op_moe_route(_p(logits), logits.stride(0), T, n_experts, top_k, _p(te), _p(tw), _p(pos),
                                   _p(counts), _dt(logits), _stream())
    _check(rc, "tei_b200_op_moe_route")
    return te, tw, pos, counts


def moe_gather(x, topk_expert, pos, cap: int, n_experts: int):
    lib = _lib.load()
    T, H = x.shape
    k = topk_expert.shape[1]
    xg = torch.zeros((n_experts * cap, H), dtype=x.dtype, device=x.device)
    rc = lib.tei_b200_op_moe_gather(_p(x), _p(topk_expert), _p(pos), _p(xg), T, k, H, cap, _dt(x), _stream())
    _check(rc, "tei_b200_op_moe_gather")
    return xg


def moe_combine(yg, topk_expert, topk_weight, pos, bias, cap: int):
    lib = _lib.load()
    T, k = topk_expert.shape
    H = yg.shape[1]
    out = torch.empty((T, H), dtype=yg.dtype, device=yg.device)
    rc = lib.tei_b200_op_moe_combine(_p(yg), _p(topk_expert), _p(topk_weight), _p(pos), _p(bias), _p(out), T, k, H,
                                     cap, _dt(yg), _stream())
    _check(rc, "tei_b200_op_moe_combine")
    return out


def moe_route_noalloc(logits, n_experts: int, top_k: int, out=None):
    """moe_route through the entry point that keeps its counters inside the library and never
    allocates: the four result tensors are the caller's (`out` = (expert, weight, pos, counts),
    made here when absent - the wrapper may allocate, the library call does not)."""
    lib = _lib.load()
    T = logits.shape[0]
    dev = logits.device
    if out is None:
        out = (torch.empty((T, top_k), dtype=torch.int32, device=dev),
               torch.empty((T, top_k), dtype=torch.float32, device=dev),
               torch.empty((T, top_k), dtype=torch.int32, device=dev),
               torch.empty((n_experts,), dtype=torch.int32, device=dev))
    te, tw, pos, counts = out
    err = ctypes.create_string_buffer(256)
    rc = lib.tei_b200_op_moe_route_noalloc(_p(logits), logits.stride(0), T, n_experts, top_k, _p(te), _p(tw),
                                           _p(pos), _p(counts), _dt(logits), _stream(), err, len(err))
    if rc != 0:
        raise RuntimeError(f"tei_b200_op_moe_route_noalloc failed ({rc}): {err.value.decode(errors='replace')}")
    return te, tw, pos, counts
