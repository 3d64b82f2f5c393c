"""Kernel-level parity on the GPU, through the C ABI (include/tei_b200_ops.h).

Reference for each op is plain fp32 torch on the same device.  Tolerances (absolute, on values
of magnitude <= ~8): fp16 2e-2 for GEMM / norm outputs, 1e-2 for attention; bf16 8e-2 / 4e-2
(bf16 has 8 bits of mantissa, one rounding of a value near 8 is 3e-2).  Integer bookkeeping
(plans, gathers, CLS / last-token rows) is exact.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {"f16": torch.float16, "bf16": torch.bfloat16}


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def _close(got, ref, tol):
    got, ref = got.float(), ref.float()
    assert not torch.isnan(got).any()
    err = (got - ref).abs().max().item()
    assert err <= tol, f"max abs err {err} > {tol}"


@pytest.mark.parametrize("M,N,K,act,bias,res,dtype", [
    (128, 256, 64, "none", False, False, "f16"),      # one tile, one k-block
    (128, 256, 768, "none", True, False, "f16"),      # pipeline wraps its 4 stages
    (1, 768, 768, "none", True, False, "f16"),        # single row (health probe shape)
    (300, 768, 768, "gelu", True, False, "f16"),      # M tail
    (200, 1000, 512, "relu", True, False, "f16"),     # N tail
    (77, 1003, 128, "relu_log1p", True, False, "f16"),  # N not a multiple of 8: scalar stores
    (520, 1024, 768, "swiglu", False, False, "f16"),
    (520, 512, 256, "swiglu", True, False, "bf16"),
    (520, 1024, 768, "geglu", False, False, "f16"),
    (130, 512, 256, "geglu", True, False, "bf16"),
    (1000, 768, 3072, "none", True, True, "bf16"),
    (700, 256, 256, "tanh", True, False, "f16"),
    (20000, 2304, 768, "none", True, False, "f16"),   # many waves of the persistent loop
    (300, 512, 200, "none", True, False, "f16"),      # K tail: the last k-block is 8 of 64 wide, zero-filled by TMA
    (300, 512, 1000, "gelu", True, False, "f16"),     # K tail behind 15 full k-blocks (a Dense module of 1000 inputs)
    (100, 256, 1000, "none", False, False, "bf16"),   # the same on the single-CTA kernel
    (64, 384, 8, "none", True, False, "f16"),         # K smaller than one MMA step
    (512, 768, 3072, "none", True, False, "f16"),     # 64-column tiles, 48 k-blocks through their 6 stages
    (512, 3072, 768, "gelu", True, False, "f16"),     # 128-column tiles
    (2048, 768, 768, "none", True, False, "bf16"),    # 128-column tiles, 16 x 6 of them
    (512, 200, 768, "none", True, True, "f16"),       # narrow tiles, N tail inside a tile, fused residual (plain stores)
    (300, 1000, 256, "tanh", False, False, "bf16"),   # narrow tiles, N tail, TMA stores clipped by the tensor map
    (1000, 768, 3072, "none", True, True, "f16"),     # residual added on the TMA-store path (CTA pairs)
    (515, 768, 2048, "none", False, True, "bf16"),    # the same on 64-column tiles, no bias, M tail
    (70000, 768, 3072, "none", True, True, "f16"),    # many waves of it
])
def test_linear(lib, M, N, K, act, bias, res, dtype):
    from tei_b200 import ops
    dt = DT[dtype]
    g = _gen(M * 7 + N * 3 + K)
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(dt)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(dt)
    b = (torch.randn(N, device="cuda", generator=g) * 0.1).to(dt) if bias else None
    n_out = N // 2 if act in ("swiglu", "geglu") else N
    r = (torch.randn(M, n_out, device="cuda", generator=g) * 0.5).to(dt) if res else None
    ww, bb = w, b
    if act in ("swiglu", "geglu"):
        ww = ops.interleave_swiglu(w[: N // 2], w[N // 2:])
        bb = ops.interleave_swiglu(b[: N // 2], b[N // 2:]) if bias else None
    out = ops.linear(a, ww, bb, r, act=act)
    y = a.float() @ w.float().t()
    if bias:
        y = y + b.float()
    if act == "gelu":
        y = torch.nn.functional.gelu(y, approximate="tanh")
    elif act == "relu":
        y = torch.relu(y)
    elif act == "tanh":
        y = torch.tanh(y)
    elif act == "relu_log1p":
        y = torch.log1p(torch.relu(y))
    elif act == "swiglu":
        y = torch.nn.functional.silu(y[:, : N // 2]) * y[:, N // 2:]
    elif act == "geglu":
        y = torch.nn.functional.gelu(y[:, : N // 2], approximate="tanh") * y[:, N // 2:]
    if res:
        y = y + r.float()
    _close(out, y, 2e-2 if dtype == "f16" else 8e-2)


def test_linear_is_deterministic_and_rejects_bad_shapes(lib):
    from tei_b200 import ops
    g = _gen(5)
    a = torch.randn(1000, 768, device="cuda", generator=g).half()
    w = (torch.randn(768, 768, device="cuda", generator=g) * 0.05).half()
    o1 = ops.linear(a, w)
    o2 = ops.linear(a, w)
    assert torch.equal(o1, o2)
    with pytest.raises(RuntimeError):
        ops.linear(a[:, :100], w[:, :100])  # K not a multiple of 8
    # NaN canary: rows beyond M must stay untouched
    out = torch.full((1100, 768), float("nan"), device="cuda", dtype=torch.float16)
    ops.linear(a, w, out=out[:1000])
    assert torch.isnan(out[1000:]).all() and not torch.isnan(out[:1000]).any()


def _ref_attention(q, k, v, cu, causal, scale, slopes=None):
    T, nh, D = q.shape
    nkv = k.shape[1]
    out = torch.zeros(T, nh, D, device=q.device, dtype=torch.float32)
    for s in range(len(cu) - 1):
        a, b = cu[s], cu[s + 1]
        L = b - a
        qs = q[a:b].float().transpose(0, 1)
        ks = k[a:b].float().transpose(0, 1).repeat_interleave(nh // nkv, dim=0)
        vs = v[a:b].float().transpose(0, 1).repeat_interleave(nh // nkv, dim=0)
        sc = qs @ ks.transpose(1, 2) * scale
        if slopes is not None:
            idx = torch.arange(L, device=q.device)
            sc = sc - slopes.view(nh, 1, 1) * (idx.view(1, L, 1) - idx.view(1, 1, L)).abs()
        if causal:
            sc = sc.masked_fill(~torch.ones(L, L, device=q.device, dtype=torch.bool).tril(), float("-inf"))
        out[a:b] = (torch.softmax(sc, dim=-1) @ vs).transpose(0, 1)
    return out.reshape(T, nh * D)


@pytest.mark.parametrize("lens,nh,nkv,D,causal,alibi,dtype", [
    ([1], 1, 1, 64, False, False, "f16"),
    ([2, 15, 16, 17], 2, 2, 64, False, False, "f16"),
    ([63, 64, 65], 2, 2, 64, False, False, "f16"),
    ([127, 128, 129], 2, 2, 64, False, False, "f16"),
    ([127, 128, 129], 2, 2, 64, True, False, "f16"),
    ([5, 1, 300, 77, 128, 129, 512], 12, 12, 64, False, False, "f16"),
    ([300, 17, 129], 4, 4, 64, True, False, "bf16"),
    ([300, 40], 4, 2, 128, True, False, "bf16"),      # GQA, head_dim 128, causal
    ([200, 130], 2, 2, 128, False, False, "f16"),
    ([200, 130], 4, 4, 64, False, True, "f16"),        # ALiBi
    ([1000], 4, 1, 128, True, False, "f16"),           # MQA, 8 query tiles
    # head_dim 32 (64-byte swizzle): all-MiniLM-L6-v2, bge-small, e5-small, gte-small
    ([1], 1, 1, 32, False, False, "f16"),
    ([15, 16, 17], 2, 2, 32, False, False, "f16"),
    ([63, 64, 65], 2, 2, 32, False, False, "f16"),
    ([127, 128, 129], 2, 2, 32, False, False, "f16"),
    ([127, 128, 129], 2, 2, 32, True, False, "f16"),
    ([512, 5, 300], 12, 12, 32, False, False, "f16"),
    ([512, 77], 12, 12, 32, True, False, "bf16"),
    ([300, 40], 4, 2, 32, True, False, "bf16"),        # GQA
    ([200, 130], 4, 4, 32, False, True, "f16"),        # ALiBi
])
def test_attention(lib, lens, nh, nkv, D, causal, alibi, dtype):
    from tei_b200 import ops
    dt = DT[dtype]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    g = _gen(T + nh + D)
    width = (nh + 2 * nkv) * D
    # NaN canary rows after the batch: the kernel must never let them leak into real rows.
    buf = torch.full((T + 64, width), float("nan"), device="cuda", dtype=dt)
    buf[:T] = torch.randn(T, width, device="cuda", generator=g).to(dt)
    qkv = buf[:T]
    q = qkv[:, : nh * D].view(T, nh, D)
    k = qkv[:, nh * D: (nh + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nh + nkv) * D:].view(T, nkv, D)
    slopes = None
    if alibi:
        slopes = torch.tensor([2.0 ** (-(i + 1) * 8.0 / nh) for i in range(nh)], device="cuda")
    scale = 1.0 / D ** 0.5
    out = ops.attention(q, k, v, cu, causal=causal, scale=scale, alibi_slopes=slopes)
    ref = _ref_attention(q, k, v, cu, causal, scale, slopes)
    _close(out, ref, 1e-2 if dtype == "f16" else 4e-2)
    out2 = ops.attention(q, k, v, cu, causal=causal, scale=scale, alibi_slopes=slopes)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("lens,nh,nkv,D,causal,slope,dtype", [
    ([700, 130], 2, 2, 64, False, 0.3, "f16"),    # the maximum grows by ~28 powers of two per 64-key step
    ([700, 130], 2, 2, 64, True, 0.3, "f16"),
    ([520], 4, 2, 128, True, 0.3, "bf16"),
    ([700], 2, 2, 64, False, 0.05, "f16"),        # slow growth: raised lazily, every second or third step
    ([700], 2, 1, 128, False, 0.05, "f16"),
    ([700, 130], 2, 2, 32, False, 0.3, "f16"),
    ([700], 2, 2, 32, True, 0.05, "bf16"),
    ([4096], 2, 1, 64, False, 0.02, "f16"),       # 64 key steps: the maximum keeps growing over the whole unit
])
def test_attention_running_maximum_is_raised(lib, lens, nh, nkv, D, causal, slope, dtype):
    """Scores that keep growing along the keys for half of the rows and keep falling for the
    other half: the rows of one warp disagree on whether the maximum has to be raised, the
    partial outputs are rescaled in place, and the early keys end up with weight ~0."""
    from tei_b200 import ops
    dt = DT[dtype]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    g = _gen(7 * T + D)
    q = 0.3 * torch.randn(T, nh, D, device="cuda", generator=g)
    k = 0.3 * torch.randn(T, nkv, D, device="cuda", generator=g)
    v = torch.randn(T, nkv, D, device="cuda", generator=g)
    pos = torch.cat([torch.arange(n, device="cuda", dtype=torch.float32) for n in lens])
    sign = torch.where(torch.arange(T, device="cuda") % 2 == 0, 1.0, -1.0)
    scale = 1.0 / D ** 0.5
    # score(i, j) = sign_i * slope * j + small noise
    q[:, :, 0] = (sign / scale).view(T, 1)
    k[:, :, 0] = (slope * pos).view(T, 1)
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    out = ops.attention(q, k, v, cu, causal=causal, scale=scale)
    ref = _ref_attention(q, k, v, cu, causal, scale, None)
    _close(out, ref, 2e-2 if dtype == "f16" else 6e-2)


@pytest.mark.parametrize("lens,nh,nkv,D,causal,wl,wr,dtype", [
    ([300, 40, 129], 4, 4, 64, True, 64, -1, "f16"),      # Mistral-style: causal, left window
    ([1000, 5], 4, 2, 128, True, 100, -1, "bf16"),        # window not a multiple of the tile
    ([700], 2, 2, 64, True, 0, -1, "f16"),                # every token sees only itself
    ([513, 64, 200], 4, 4, 64, False, 64, 64, "f16"),     # ModernBERT-style local attention
    ([400], 2, 2, 128, False, 17, 130, "f16"),            # asymmetric
    ([300, 130], 4, 4, 64, True, 4096, -1, "f16"),        # window wider than the sequences
    ([300, 40, 129], 4, 4, 32, True, 64, -1, "f16"),
    ([513, 64], 4, 2, 32, False, 64, 64, "bf16"),
])
def test_attention_sliding_window(lib, lens, nh, nkv, D, causal, wl, wr, dtype):
    # flash_attn.rs:23-36,72-95: key j counts for query i when i - wl <= j <= i + wr.
    from tei_b200 import ops
    dt = DT[dtype]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    g = _gen(T + nh + D + wl)
    width = (nh + 2 * nkv) * D
    buf = torch.full((T + 64, width), float("nan"), device="cuda", dtype=dt)
    buf[:T] = torch.randn(T, width, device="cuda", generator=g).to(dt)
    qkv = buf[:T]
    q = qkv[:, : nh * D].view(T, nh, D)
    k = qkv[:, nh * D: (nh + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nh + nkv) * D:].view(T, nkv, D)
    scale = 1.0 / D ** 0.5
    out = ops.attention(q, k, v, cu, causal=causal, scale=scale, window_left=wl, window_right=wr)
    ref = torch.zeros(T, nh, D, device="cuda", dtype=torch.float32)
    for s in range(len(lens)):
        a, b = cu[s], cu[s + 1]
        L = b - a
        qs = q[a:b].float().transpose(0, 1)
        ks = k[a:b].float().transpose(0, 1).repeat_interleave(nh // nkv, dim=0)
        vs = v[a:b].float().transpose(0, 1).repeat_interleave(nh // nkv, dim=0)
        sc = qs @ ks.transpose(1, 2) * scale
        i = torch.arange(L, device="cuda").view(L, 1)
        j = torch.arange(L, device="cuda").view(1, L)
        right = 0 if causal else wr
        ok = torch.ones(L, L, device="cuda", dtype=torch.bool)
        if wl >= 0:
            ok &= j >= i - wl
        if right >= 0:
            ok &= j <= i + right
        sc = sc.masked_fill(~ok, float("-inf"))
        ref[a:b] = (torch.softmax(sc, dim=-1) @ vs).transpose(0, 1)
    _close(out, ref.reshape(T, nh * D), 1e-2 if dtype == "f16" else 4e-2)
    assert torch.equal(out, ops.attention(q, k, v, cu, causal=causal, scale=scale, window_left=wl, window_right=wr))


@pytest.mark.parametrize("lens,nh,nkv,D,causal,dtype", [
    ([8192, 100], 4, 2, 128, True, "bf16"),     # 64 query tiles, 128 key steps, the K/V rings wrap > 40 times
    ([8055], 2, 1, 128, True, "f16"),           # the longest sequence of the Qwen3-style benchmark batch
    ([2048, 2008, 513], 4, 4, 64, False, "f16"),  # the NomicBERT-style benchmark lengths
    ([4096], 2, 2, 64, False, "f16"),
    ([3000], 4, 4, 32, True, "f16"),
])
def test_attention_long_sequences(lib, lens, nh, nkv, D, causal, dtype):
    """The lengths the benchmark configurations run (up to 8,055 and 8,192 tokens) against fp32
    softmax on the same device, one head at a time so that the reference fits."""
    from tei_b200 import ops
    dt = DT[dtype]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    g = _gen(T + nh + D)
    qkv = torch.randn(T, (nh + 2 * nkv) * D, device="cuda", generator=g).to(dt)
    q = qkv[:, : nh * D].view(T, nh, D)
    k = qkv[:, nh * D: (nh + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nh + nkv) * D:].view(T, nkv, D)
    scale = 1.0 / D ** 0.5
    out = ops.attention(q, k, v, cu, causal=causal, scale=scale).view(T, nh, D)
    tol = 1e-2 if dtype == "f16" else 4e-2
    for h in range(nh):
        hk = h // (nh // nkv)
        ref = _ref_attention(q[:, h:h + 1], k[:, hk:hk + 1], v[:, hk:hk + 1], cu, causal, scale, None)
        _close(out[:, h].reshape(T, D), ref, tol)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_embedding_and_norms(lib, dtype):
    from tei_b200 import ops
    dt = DT[dtype]
    tol = 2e-2 if dtype == "f16" else 8e-2
    g = _gen(1)
    T, V = 1000, 5000
    for H in (128, 768, 1024, 2048, 4096):
        word = (torch.randn(V, H, device="cuda", generator=g) * 0.05).to(dt)
        typ = (torch.randn(2, H, device="cuda", generator=g) * 0.05).to(dt)
        pos = (torch.randn(512, H, device="cuda", generator=g) * 0.05).to(dt)
        gamma = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(dt)
        beta = (0.1 * torch.randn(H, device="cuda", generator=g)).to(dt)
        ids = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
        tids = torch.randint(0, 2, (T,), device="cuda", dtype=torch.int32)
        pids = torch.randint(0, 512, (T,), device="cuda", dtype=torch.int32)
        out = ops.embed_layernorm(ids, tids, pids, word, typ, pos, gamma, beta, 1e-12)
        x = word[ids.long()].float() + typ[tids.long()].float() + pos[pids.long()].float()
        _close(out, torch.nn.functional.layer_norm(x, (H,), gamma.float(), beta.float(), 1e-12), tol)
        out = ops.embed_layernorm(ids, None, None, word, None, None, None, None, 0.0)
        assert torch.equal(out, word[ids.long()])  # plain gather is exact

        x = torch.randn(T, H, device="cuda", generator=g).to(dt)
        r = torch.randn(T, H, device="cuda", generator=g).to(dt)
        out = ops.add_layernorm(x, r, gamma, beta, 1e-12)
        _close(out, torch.nn.functional.layer_norm(x.float() + r.float(), (H,), gamma.float(), beta.float(), 1e-12), tol)
        rf = torch.randn(T, H, device="cuda", generator=g)
        out, sm = ops.add_rmsnorm(x, rf, gamma, 1e-6)
        s = x.float() + rf
        _close(out, s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float(), tol)
        assert torch.equal(sm, s)  # the fp32 running sum is exact
        out, sm = ops.add_rmsnorm(x, None, gamma, 1e-6)
        s = x.float()
        _close(out, s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float(), tol)


@pytest.mark.parametrize("nh,nkv,D,use_norm,dtype", [(12, 12, 64, False, "f16"), (16, 8, 128, True, "bf16"),
                                                     (16, 8, 128, True, "f16"), (12, 12, 32, False, "f16"),
                                                     (4, 2, 32, True, "bf16"), (3, 3, 48, True, "f16")])
def test_qk_norm_rope(lib, nh, nkv, D, use_norm, dtype):
    from tei_b200 import ops
    dt = DT[dtype]
    g = _gen(2)
    T = 333
    qkv = torch.randn(T, (nh + 2 * nkv) * D, device="cuda", generator=g).to(dt)
    q = qkv[:, : nh * D].view(T, nh, D)
    k = qkv[:, nh * D: (nh + nkv) * D].view(T, nkv, D)
    v0 = qkv[:, (nh + nkv) * D:].clone()
    q0, k0 = q.float().clone(), k.float().clone()
    posi = torch.randint(0, 2048, (T,), device="cuda", dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(2048, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    qg = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(dt) if use_norm else None
    kg = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(dt) if use_norm else None
    ops.qk_norm_rope_(q, k, posi, cos, sin, qg, kg, 1e-6)

    def ref(x, gamma):
        if gamma is not None:
            x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float()
        c, s_ = cos[posi.long()][:, None, :], sin[posi.long()][:, None, :]
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return torch.cat([x1 * c - x2 * s_, x2 * c + x1 * s_], dim=-1)
    tol = 2e-2 if dtype == "f16" else 8e-2
    _close(q.reshape(T, -1), ref(q0, qg).reshape(T, -1), tol)
    _close(k.reshape(T, -1), ref(k0, kg).reshape(T, -1), tol)
    assert torch.equal(qkv[:, (nh + nkv) * D:], v0)  # V untouched


@pytest.mark.parametrize("M,nh,nkv,D,use_norm,bias,dtype", [
    (333, 12, 12, 64, False, False, "f16"),     # NomicBERT: 768 -> 2304, no bias
    (1000, 16, 8, 128, True, False, "bf16"),    # Qwen3: 1024 -> 4096, q/k RMSNorm, GQA
    (1000, 16, 8, 128, True, False, "f16"),
    (77, 16, 8, 128, True, False, "bf16"),      # one row tile: the single-CTA kernel
    (300, 12, 2, 128, False, True, "f16"),      # Qwen2: q/k/v biases
    (300, 3, 1, 128, True, True, "f16"),        # q and k heads share a tile; 640 columns: the last tile is partial
    (520, 12, 12, 32, False, True, "f16"),      # head_dim 32; q and k heads share a tile
    (200, 4, 2, 32, True, False, "bf16"),
    (130, 6, 6, 64, True, True, "f16"),         # q region of 384 columns: tile 1 holds q and k heads
    (100, 3, 1, 64, False, False, "bf16"),      # 320 columns: the last tile is partial
])
def test_linear_with_the_rotary_epilogue_equals_linear_then_rope(lib, M, nh, nkv, D, use_norm, bias, dtype):
    """The q/k/v projection with RMSNorm + RoPE in its epilogue against the two-kernel form
    (projection, then the in-place RoPE kernel): the same bits, and both against fp32 torch."""
    from tei_b200 import ops
    dt = DT[dtype]
    g = _gen(M + nh * D)
    K = 256 if D == 32 else 768
    Q, KV = nh * D, nkv * D
    N = Q + 2 * KV
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(dt)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(dt)
    b = (torch.randn(N, device="cuda", generator=g) * 0.1).to(dt) if bias else None
    posi = torch.randint(0, 2048, (M,), device="cuda", dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(2048, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    qg = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(dt) if use_norm else None
    kg = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(dt) if use_norm else None
    two = ops.linear(a, w, b)
    plain = two.clone()
    ops.qk_norm_rope_(two[:, :Q].view(M, nh, D), two[:, Q:Q + KV].view(M, nkv, D), posi, cos, sin, qg, kg, 1e-6)
    canary = torch.full((M + 8, N), float("nan"), device="cuda", dtype=dt)
    one = ops.linear_rope(a, w, b, posi, cos, sin, qg, kg, D, Q, KV, 1e-6, out=canary[:M])
    assert torch.isnan(canary[M:]).all()
    assert torch.equal(one, two)
    assert torch.equal(one[:, Q + KV:], plain[:, Q + KV:])  # v is the plain projection
    # and the pair against fp32
    y = a.float() @ w.float().t() + (b.float() if bias else 0.0)

    def ref(x, gamma):
        if gamma is not None:
            x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float()
        c, s_ = cos[posi.long()][:, None, :], sin[posi.long()][:, None, :]
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return torch.cat([x1 * c - x2 * s_, x2 * c + x1 * s_], dim=-1)
    tol = 3e-2 if dtype == "f16" else 1e-1
    _close(one[:, :Q], ref(y[:, :Q].view(M, nh, D), qg).reshape(M, Q), tol)
    _close(one[:, Q:Q + KV], ref(y[:, Q:Q + KV].view(M, nkv, D), kg).reshape(M, KV), tol)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_pooling_gather_and_heads(lib, dtype):
    from tei_b200 import ops
    dt = DT[dtype]
    g = _gen(3)
    lens = [5, 1, 300, 77, 128, 129]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    x = torch.randn(cu[-1], 768, device="cuda", generator=g).to(dt)
    cu_d = torch.tensor(cu, device="cuda", dtype=torch.int32)
    idx = torch.tensor([0, 2, 3, 5, 1], device="cuda", dtype=torch.int32)
    for mode in ("cls", "mean", "max", "last_token"):
        for nrm in (False, True):
            out = ops.pool(x, cu_d, idx, mode, nrm)
            rows = []
            for s in idx.tolist():
                seg = x[cu[s]:cu[s + 1]].float()
                rows.append({"cls": seg[0], "last_token": seg[-1], "mean": seg.mean(0),
                             "max": seg.max(0).values}[mode])
            ref = torch.stack(rows)
            if nrm:
                ref = ref / ref.norm(dim=-1, keepdim=True)
                _close(out, ref, 1e-5)
            elif mode in ("cls", "last_token", "max"):
                assert torch.equal(out, ref)  # row selection is exact
            else:
                _close(out, ref, 1e-5)
    ridx = torch.tensor([3, 4, 5, 100, 7], device="cuda", dtype=torch.int32)
    assert torch.equal(ops.gather_rows_f32(x, ridx), x[ridx.long()].float())
    xin = torch.randn(37, 768, device="cuda", generator=g)
    w = (torch.randn(5, 768, device="cuda", generator=g) * 0.05).to(dt)
    b = (torch.randn(5, device="cuda", generator=g) * 0.05).to(dt)
    _close(ops.head_linear(xin, w, b, "tanh"), torch.tanh(xin @ w.float().t() + b.float()), 1e-4)
    _close(ops.head_linear(xin, w, None, "none"), xin @ w.float().t(), 1e-4)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_moe_feed_forward_from_its_ops(lib, dtype):
    # NomicMoELayer::forward (backends/candle/src/models/nomic.rs:205-394) assembled from the
    # single ops, against the same computation in fp32 torch.
    from tei_b200 import ops
    dt = DT[dtype]
    g = _gen(77)
    T, H, I, E, K = 1500, 256, 512, 8, 2
    x = (torch.randn(T, H, device="cuda", generator=g) * 0.5).to(dt)
    wr = torch.zeros(8, H, device="cuda", dtype=dt)
    wr[:E] = (torch.randn(E, H, device="cuda", generator=g) * 0.2).to(dt)
    w1 = (torch.randn(E * I, H, device="cuda", generator=g) * 0.05).to(dt)
    w2 = (torch.randn(E * I, H, device="cuda", generator=g) * 0.05).to(dt)
    bias = (torch.randn(H, device="cuda", generator=g) * 0.1).to(dt)
    logits = ops.linear(x, wr)
    te, tw, pos, counts = ops.moe_route(logits, E, K)
    # routing against torch on the same logits
    probs = torch.softmax(logits[:, :E].float(), dim=-1)
    ref_w, ref_e = probs.topk(K, dim=-1)
    # the same probabilities are picked; where two logits tie exactly (they are fp16 / bf16
    # numbers) the lower expert index wins here, so indices are compared away from ties only
    assert (tw - ref_w.to(dt).float()).abs().max().item() <= 1e-6
    assert (probs.gather(1, te.long()) - ref_w).abs().max().item() <= 1e-6
    srt = probs.sort(dim=-1, descending=True).values
    no_tie = (srt[:, :K] - srt[:, 1:K + 1]).min(dim=-1).values > 0
    assert torch.equal(te.long()[no_tie], ref_e[no_tie]) and int(no_tie.sum()) > T // 2
    assert (te[:, 0] != te[:, 1]).all()
    ref_e = te.long()  # the reference below follows the picks made here
    assert int(counts.sum()) == T * K
    assert torch.equal(counts.long(), torch.bincount(ref_e.flatten(), minlength=E))
    for e in range(E):  # the rows of an expert are 0 .. count-1, each once
        p_e = pos[te == e].long().sort().values
        assert torch.equal(p_e, torch.arange(int(counts[e]), device="cuda"))
    cap = 1536
    xg = ops.moe_gather(x, te, pos, cap, E)
    yg = torch.zeros(E * cap, H, device="cuda", dtype=dt)
    w2t = w2.view(E, I, H).transpose(1, 2).contiguous()  # [E, H, I]: the [N, K] form of each expert
    for e in range(E):
        h = ops.linear_rows_dev(xg[e * cap:(e + 1) * cap], w1[e * I:(e + 1) * I], None, counts[e:e + 1], act="gelu")
        ops.linear_rows_dev(h, w2t[e], None, counts[e:e + 1], out=yg[e * cap:(e + 1) * cap])
    out = ops.moe_combine(yg, te, tw, pos, bias, cap)
    ref = torch.zeros(T, H, device="cuda")
    xf = x.float()
    for e in range(E):
        tok, slot = (ref_e == e).nonzero(as_tuple=True)
        y = torch.nn.functional.gelu(xf[tok] @ w1[e * I:(e + 1) * I].float().t(), approximate="tanh") @ w2[e * I:(e + 1) * I].float()
        ref.index_add_(0, tok, y * tw[tok, slot].unsqueeze(-1))
    ref = ref + bias.float()
    _close(out, ref, 2e-2 if dtype == "f16" else 8e-2)
    # a row count of zero leaves the output untouched
    canary = torch.full((cap, H), 7.0, device="cuda", dtype=dt)
    ops.linear_rows_dev(xg[:cap], w2t[0][:, :H].contiguous(), None, torch.zeros(1, device="cuda", dtype=torch.int32), out=canary)
    assert (canary == 7.0).all()
