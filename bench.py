"""Benchmark of the hot path: tokens/s of the packed, unpadded BERT-base forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = one forward of one packed batch.  Workload at every N: BASELINE.json configs[1] -
BERT-base (bge-base-en-v1.5 architecture, random-init seed 0), 256 ragged sequences with lengths
uniform in [16, 512] (seed 1), 68,576 tokens, mean pooling + L2 normalise, fp16 - one such batch
per GPU per step (request-level data parallelism: every GPU holds a full replica, so scaling is
weak and no collective runs on the data path; torch.distributed is used for the barrier and the
max-over-ranks of the timings only).

Printed by rank 0 as ONE JSON line:
  value        device-resident throughput: the batch is staged in HBM before the timed region,
               K forwards run back to back, timed with CUDA events on the launching stream
  e2e          the same metric through the C-ABI `embed` call with HOST buffers: host->device copy
               of the batch and device->host copy of the pooled rows inside the timed region
  roofline     dense-layer GEMM kernel: algorithmic FLOPs per launch / mean launch duration,
               measured with per-launch CUDA events inside the timed region
  cpu_baseline the fp32 CPU restatement of the reference's Candle CPU path (oracle/), timed on a
               bounded sample of the same batch on the host cores (rank 0, N = 1 only)
`--impl reference` times that CPU path alone (rank 0 only), same metric and config.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (str(ROOT), str(ROOT / "text-embeddings-inference_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

WORKLOAD = ("cfg2: BERT-base 12x768 (12 heads x 64, FFN 3072 tanh-GELU, post-LN), random-init seed 0; "
            "256 sequences, lengths uniform [16,512] seed 1, 68576 tokens packed with cu_seqlens; "
            "mean pooling + L2 normalise")
MODEL_DIR = Path(os.environ.get("TEI_B200_BENCH_DIR", "/tmp/tei_b200_bench")) / "bert_base_seed0"


def ensure_model_dir(local_rank: int) -> Path:
    """Local rank 0 writes the seeded BERT-base directory once; the others wait for it."""
    from oracle import generators as G
    marker = MODEL_DIR / ".complete"
    if marker.exists():
        return MODEL_DIR
    if local_rank == 0:
        tmp = MODEL_DIR.with_name(MODEL_DIR.name + f".tmp{os.getpid()}")
        G.write_model_dir(tmp, G.bert_config(), seed=0)
        (tmp / ".complete").write_text("ok")
        MODEL_DIR.parent.mkdir(parents=True, exist_ok=True)
        try:
            os.replace(tmp, MODEL_DIR)
        except OSError:
            pass  # somebody else finished first
    t0 = time.time()
    while not marker.exists():
        if time.time() - t0 > 600:
            raise RuntimeError("timed out waiting for the model directory")
        time.sleep(0.2)
    return MODEL_DIR


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs.
    Read-only: nothing is set or reset."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting",
        0x10: "sync_boost",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            # honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in vis.split(",") if v.strip().isdigit()]
            phys = int(ids[index]) if index < len(ids) else index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


class Ranks:
    """The only cross-rank plumbing of the benchmark: a barrier and max / sum of a scalar.  The
    data path itself has no collective (replicas share nothing).  backend "nccl" on GPUs, "gloo"
    for the CPU tests."""

    def __init__(self, world: int, local_rank: int, backend: str = "nccl"):
        self.world = world
        self.backend = backend
        self.dist = None
        self.device = "cpu"
        if world > 1:
            import torch
            import torch.distributed as dist
            if backend == "nccl":
                self.device = torch.device("cuda", local_rank)
                dist.init_process_group("nccl", device_id=self.device)
            else:
                dist.init_process_group(backend)
            self.dist = dist

    def barrier(self):
        import torch
        if self.dist is not None:
            self.dist.barrier()
        if self.backend == "nccl" and torch.cuda.is_available():
            torch.cuda.synchronize()

    def _reduce(self, x: float, op_name: str) -> float:
        if self.dist is None:
            return float(x)
        import torch
        t = torch.tensor([x], dtype=torch.float64, device=self.device)
        self.dist.all_reduce(t, op=getattr(self.dist.ReduceOp, op_name))
        return float(t.item())

    def max(self, x: float) -> float:
        return self._reduce(x, "MAX")

    def sum(self, x: float) -> float:
        return self._reduce(x, "SUM")

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


def whole_job_throughput(ranks: "Ranks", tokens_this_rank: float, steps: int, ms_this_rank: float) -> float:
    """Units all ranks processed / the slowest rank's device time."""
    ms = ranks.max(ms_this_rank)
    total = ranks.sum(float(tokens_this_rank)) * steps
    return total / (ms / 1e3)


def cpu_baseline(model_dir: Path, n_seqs: int, repeats: int = 1):
    """Times the fp32 CPU restatement of the reference's Candle CPU path on the first n_seqs
    sequences of the workload, the way that path runs them: at most 4 sequences per forward
    (backends/candle/src/lib.rs:640-646), each chunk padded to its longest sequence
    (models/bert.rs:715-757).  Returns (tokens/s, cores, seconds, tokens)."""
    import numpy as np
    import torch
    from oracle import generators as G
    from oracle import models as M
    from oracle.packing import batch_from_encodings

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    oracle = M.build_oracle(model_dir, "embedding", "mean")
    full = G.batch_cfg2(n_seqs=n_seqs)
    cu = full.cumulative_seq_lengths.astype(np.int64)
    chunks = []
    for c0 in range(0, len(full), 4):
        encs = [full.input_ids[cu[s]:cu[s + 1]] for s in range(c0, min(c0 + 4, len(full)))]
        chunks.append(batch_from_encodings(encs, list(range(len(encs))), []))
    tokens = int(cu[-1])
    best = None
    with torch.no_grad():
        for _ in range(repeats):
            t0 = time.perf_counter()
            for ch in chunks:
                hs = oracle.hidden_states_padded(ch)
                lens = ch.lengths()
                for i in range(len(ch)):
                    v = hs[i, : int(lens[i])].mean(dim=0)
                    M.l2_normalise(v.numpy()[None])
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
    return tokens / best, cores, best, tokens


def gpu_proxy(model_dir: Path, batch, steps: int, warmup: int = 3):
    """Same-box GPU yardstick, NOT the reference: the op sequence of the reference's flash BERT
    forward (backends/candle/src/models/flash_bert.rs:75-185: fused QKV linear, varlen flash
    attention, output linear, add + LayerNorm, FFN with tanh-GELU, add + LayerNorm, then mean
    pooling, flash_bert.rs:444-459) written with the libraries this image has: flash_attn 2.x
    `flash_attn_varlen_func` where the reference links candle-flash-attn, and
    torch.nn.functional.linear (cuBLASLt) where it links candle-cublaslt.  fp16, the same weights
    and the same packed batch, device-resident, timed with CUDA events on torch's stream."""
    import numpy as np
    import torch
    import torch.nn.functional as F
    try:
        from flash_attn import flash_attn_varlen_func
        from safetensors.torch import load_file
    except Exception as exc:  # the proxy is optional equipment
        return {"unavailable": f"{type(exc).__name__}: {exc}"}
    try:
        dev = torch.device("cuda", torch.cuda.current_device())
        w = {k: v.to(dev, torch.float16) for k, v in load_file(str(model_dir / "model.safetensors")).items()}
        cfg = json.loads((model_dir / "config.json").read_text())
        L, H, nh = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"]
        eps = cfg["layer_norm_eps"]
        layers = []
        for i in range(L):
            p = f"encoder.layer.{i}."
            layers.append(dict(
                wqkv=torch.cat([w[p + f"attention.self.{n}.weight"] for n in ("query", "key", "value")]),
                bqkv=torch.cat([w[p + f"attention.self.{n}.bias"] for n in ("query", "key", "value")]),
                wo=w[p + "attention.output.dense.weight"], bo=w[p + "attention.output.dense.bias"],
                g1=w[p + "attention.output.LayerNorm.weight"], b1=w[p + "attention.output.LayerNorm.bias"],
                wi=w[p + "intermediate.dense.weight"], bi=w[p + "intermediate.dense.bias"],
                wd=w[p + "output.dense.weight"], bd=w[p + "output.dense.bias"],
                g2=w[p + "output.LayerNorm.weight"], b2=w[p + "output.LayerNorm.bias"]))
        ids = torch.from_numpy(batch.input_ids.astype(np.int64)).to(dev)
        tids = torch.from_numpy(batch.token_type_ids.astype(np.int64)).to(dev)
        pids = torch.from_numpy(batch.position_ids.astype(np.int64)).to(dev)
        cu = torch.from_numpy(batch.cumulative_seq_lengths.astype(np.int32)).to(dev)
        lens = (cu[1:] - cu[:-1]).to(torch.int64)
        seq_of_token = torch.repeat_interleave(torch.arange(len(lens), device=dev), lens)
        max_s = int(batch.max_length)
        T = ids.numel()
        scale = 1.0 / (H // nh) ** 0.5

        def forward():
            x = w["embeddings.word_embeddings.weight"][ids] + w["embeddings.token_type_embeddings.weight"][tids] + \
                w["embeddings.position_embeddings.weight"][pids]
            x = F.layer_norm(x, (H,), w["embeddings.LayerNorm.weight"], w["embeddings.LayerNorm.bias"], eps)
            for ly in layers:
                qkv = F.linear(x, ly["wqkv"], ly["bqkv"]).view(T, 3, nh, H // nh)
                a = flash_attn_varlen_func(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, cu, max_s, max_s, softmax_scale=scale,
                                           causal=False).reshape(T, H)
                x1 = F.layer_norm(F.linear(a, ly["wo"], ly["bo"]) + x, (H,), ly["g1"], ly["b1"], eps)
                f = F.gelu(F.linear(x1, ly["wi"], ly["bi"]), approximate="tanh")
                x = F.layer_norm(F.linear(f, ly["wd"], ly["bd"]) + x1, (H,), ly["g2"], ly["b2"], eps)
            pooled = torch.zeros(len(lens), H, device=dev, dtype=torch.float32).index_add_(0, seq_of_token, x.float())
            return F.normalize(pooled / lens[:, None].float(), dim=-1)

        with torch.no_grad():
            for _ in range(warmup):
                out = forward()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                out = forward()
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        import flash_attn
        return {"value": T / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms, "rows": out,
                "what": f"PROXY, not the reference: flash_attn {flash_attn.__version__} varlen + torch F.linear (cuBLASLt) + "
                        "torch LayerNorm / GELU, op for op after flash_bert.rs:75-185, fp16, same weights and batch, "
                        "device-resident, CUDA events"}
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"}


def run_reference(args, rank: int):
    """`--impl reference`: the reference's own implementation cannot be built here (Rust, crates
    not vendored), so this arm times its CPU restatement (oracle/, kind "port") on a bounded
    sample of the workload with all host threads."""
    if rank != 0:
        return
    model_dir = ensure_model_dir(0)
    n_seqs = 32
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_baseline(model_dir, 8)
    times, tokens, cores = [], 0, 1
    for _ in range(max(args.steps, 1)):
        tps, cores, dt, tokens = cpu_baseline(model_dir, n_seqs)
        times.append(dt)
    total = sum(times)
    value = tokens * len(times) / total
    sample = f"first {n_seqs} of the 256 sequences ({tokens} tokens) per step, forwards of <=4 sequences padded to the chunk max"
    line = {
        "impl": "reference", "metric": "tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_kernel(args):
    """`--kernel NAME`: one kernel of the forward alone at the workload's shapes (68,576 tokens),
    timed with CUDA events on torch's current stream, which is the stream it is launched on.
    Used for the burst roofline figures and as the small, single-kernel command for ncu."""
    import numpy as np
    import torch
    from tei_b200 import ops
    from oracle import generators as G

    torch.cuda.set_device(0)
    lens = [int(x) for x in G.lengths_cfg2()]
    T, H, I, nh, D = int(sum(lens)), 768, 3072, 12, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    dt = torch.float16

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device="cuda", generator=g) * scale).to(dt)

    name = args.kernel
    flops = bytes_ = 0.0
    extra = []
    st = ops.new_status()
    if name.startswith("gemm_"):
        N, K, act = {"gemm_qkv": (3 * H, H, "none"), "gemm_out": (H, H, "none"),
                     "gemm_ffn1": (I, H, "gelu"), "gemm_ffn2": (H, I, "none")}[name]
        a, w, b = rnd(T, K, scale=0.5), rnd(N, K, scale=0.05), rnd(N, scale=0.1)
        out = torch.empty(T, N, device="cuda", dtype=dt)
        fn = lambda: ops.linear(a, w, b, act=act, out=out, status=st)  # noqa: E731
        flops = 2.0 * T * N * K
        bytes_ = 2.0 * (T * K + N * K + T * N)
    elif name == "attention":
        qkv = rnd(T, 3 * H)
        q, k, v = (qkv[:, i * H:(i + 1) * H].view(T, nh, D) for i in range(3))
        cu = np.concatenate([[0], np.cumsum(lens)])
        work = torch.from_numpy(ops.attention_plan(cu, False)).cuda()
        out = torch.empty(T, H, device="cuda", dtype=dt)
        fn = lambda: ops.attention(q, k, v, cu, work=work, out=out, status=st)  # noqa: E731
        flops = 4.0 * H * float(sum(n * n for n in lens))
        bytes_ = 2.0 * 4 * T * H
    elif name in ("attention_long", "attention_causal128", "attention_d32", "rope_qwen3"):
        # 16 x 2048 tokens, 12 heads x 64, bidirectional / 4 x 4096 tokens, 16 query and 8 key-value
        # heads x 128, causal, bf16 (the Qwen3 shape) / RoPE + q/k RMSNorm on the latter / the ragged
        # batch with 12 heads x 32 (the all-MiniLM-L6-v2 shape)
        if name == "attention_long":
            lens, nh, nkv, D, causal = [2048] * 16, 12, 12, 64, False
        elif name == "attention_d32":
            nh, nkv, D, causal = 12, 12, 32, False
        else:
            lens, nh, nkv, D, causal, dt = [4096] * 4, 16, 8, 128, True, torch.bfloat16
        T = int(sum(lens))
        qkv = rnd(T, (nh + 2 * nkv) * D).to(dt)
        q = qkv[:, : nh * D].view(T, nh, D)
        k = qkv[:, nh * D: (nh + nkv) * D].view(T, nkv, D)
        v = qkv[:, (nh + nkv) * D:].view(T, nkv, D)
        cu = np.concatenate([[0], np.cumsum(lens)])
        if name == "rope_qwen3":
            pos = torch.cat([torch.arange(n, device="cuda", dtype=torch.int32) for n in lens])
            inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D))
            ang = torch.arange(max(lens), device="cuda", dtype=torch.float32)[:, None] * inv[None, :]
            cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
            qg, kg = torch.ones(D, device="cuda", dtype=dt), torch.ones(D, device="cuda", dtype=dt)
            fn = lambda: ops.qk_norm_rope_(q, k, pos, cos, sin, qg, kg, 1e-6)  # noqa: E731
            bytes_ = 2.0 * 2 * T * (nh + nkv) * D
        else:
            work = torch.from_numpy(ops.attention_plan(cu, causal)).cuda()
            out = torch.empty(T, nh * D, device="cuda", dtype=dt)
            fn = lambda: ops.attention(q, k, v, cu, causal=causal, work=work, out=out, status=st)  # noqa: E731
            flops = (2.0 if causal else 4.0) * nh * D * float(sum(n * (n + 1) if causal else n * n for n in lens))
            bytes_ = 2.0 * T * (2 * nh + 2 * nkv) * D
    elif name in ("qkv_rope_nomic", "qkv_rope_qwen3"):
        # The fused q/k/v projection with RoPE (and Qwen3's q/k RMSNorm) in its epilogue against the
        # projection followed by the in-place RoPE kernel: NomicBERT (78,106 tokens, 768 -> 2304,
        # 12 heads x 64, fp16) / Qwen3-0.6B (131,072 tokens, 1024 -> 4096, 16 + 8 heads x 128, bf16).
        if name == "qkv_rope_nomic":
            T, K, nh, nkv, D, norm = 78106, 768, 12, 12, 64, False
        else:
            T, K, nh, nkv, D, norm, dt = 131072, 1024, 16, 8, 128, True, torch.bfloat16
        Q, KV = nh * D, nkv * D
        N = Q + 2 * KV
        a, w = rnd(T, K, scale=0.5).to(dt), rnd(N, K, scale=0.05).to(dt)
        pos = (torch.arange(T, device="cuda", dtype=torch.int32) % 2048).contiguous()
        inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D))
        ang = torch.arange(2048, device="cuda", dtype=torch.float32)[:, None] * inv[None, :]
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        qg = torch.ones(D, device="cuda", dtype=dt) if norm else None
        kg = torch.ones(D, device="cuda", dtype=dt) if norm else None
        out = torch.empty(T, N, device="cuda", dtype=dt)

        def split():
            ops.linear(a, w, None, out=out, status=st)
            ops.qk_norm_rope_(out[:, :Q].view(T, nh, D), out[:, Q:Q + KV].view(T, nkv, D), pos, cos, sin, qg, kg, 1e-6)
        fn = lambda: ops.linear_rope(a, w, None, pos, cos, sin, qg, kg, D, Q, KV, 1e-6, out=out, status=st)  # noqa: E731
        flops = 2.0 * T * N * K
        bytes_ = 2.0 * (T * K + N * K + T * N)
        for f in (split, lambda: ops.linear(a, w, None, out=out, status=st)):
            for _ in range(3):
                f()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                f()
            e1.record()
            torch.cuda.synchronize()
            extra.append(e0.elapsed_time(e1) / args.steps)
    elif name in ("add_layernorm", "add_layernorm_h1024"):
        if name.endswith("h1024"):  # the XLM-RoBERTa-large / Qwen3 width at the cfg4 token count
            T, H = 153855, 1024
        x, r, gm, bt = rnd(T, H), rnd(T, H), rnd(H), rnd(H)
        fn = lambda: ops.add_layernorm(x, r, gm, bt, 1e-12)  # noqa: E731
        bytes_ = 3.0 * T * H * 2
    elif name == "pool_mean":
        x = rnd(T, H)
        cu_d = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), device="cuda", dtype=torch.int32)
        idx = torch.arange(len(lens), device="cuda", dtype=torch.int32)
        fn = lambda: ops.pool(x, cu_d, idx, "mean", True)  # noqa: E731
        bytes_ = T * H * 2.0 + len(lens) * H * 4.0
    else:
        raise SystemExit(f"unknown kernel {name}")
    for _ in range(max(args.warmup, 1)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    ops.check_status(st, name)
    line = {"kernel": name, "ms_per_launch": ms, "tokens": T,
            "tflops": flops / ms / 1e9 if flops else None, "algorithmic_gbs": bytes_ / ms / 1e6}
    if extra:
        line["ms_projection_then_rope_kernel"], line["ms_projection_alone"] = extra
    print(json.dumps(line), flush=True)


def run_config(args):
    """One of the other benchmark configurations (BASELINE.json configs[0], [2], [3], [4]) through
    the same harness on one GPU: device-resident and end-to-end tokens/s, per-class kernel time and
    the algorithmic TFLOP/s of the dense layers + attention.  The headline line stays cfg2."""
    import numpy as np
    import torch
    import tei_b200
    from oracle import generators as G

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    name = args.config
    base = Path(os.environ.get("TEI_B200_BENCH_DIR", "/tmp/tei_b200_bench"))
    if name == "cfg2":  # only reached with --in-flight: the headline line comes from main()
        cfg, seed, kw = G.bert_config(), 0, {}
        batch, mtype, pool, dtype = G.batch_cfg2(), "embedding", "mean", "float16"
        what = WORKLOAD
    elif name == "cfg1":
        cfg, seed, kw = G.bert_config(), 0, {}
        batch, mtype, pool, dtype = G.batch_cfg1(), "embedding", "cls", "float16"
        what = "cfg1: BERT-base, 32 sequences x 512 tokens, CLS pooling"
    elif name == "cfg3":
        cfg, seed, kw = G.nomic_config(), 2, {}
        batch, mtype, pool, dtype = G.batch_cfg3(), "embedding", "mean", "float16"
        what = "cfg3: NomicBERT 12x768 (RoPE theta 1000, SwiGLU), 64 sequences of 512..2048 tokens, mean pooling"
    elif name == "cfg4":
        cfg = G.bert_config(hidden=1024, layers=24, heads=16, inter=4096, vocab=250002, max_pos=514, type_vocab=1,
                            model_type="xlm-roberta", pad_token_id=1, id2label={"0": "LABEL_0"})
        seed, kw = 4, {"classifier": "roberta"}
        batch, mtype, pool, dtype = G.batch_cfg4(), "classifier", "cls", "float16"
        what = "cfg4: XLM-RoBERTa-large reranker (24x1024), 512 query/passage pairs, one logit per pair"
    elif name == "cfg5":
        cfg, seed, kw = G.qwen3_config(), 5, {}
        batch, mtype, pool, dtype = G.batch_cfg5(), "embedding", "last_token", args.dtype or "bfloat16"
        what = "cfg5: Qwen3-0.6B-style (28x1024, 16/8 heads x 128, causal), 128 sequences of 128..8192 tokens, last-token pooling"
    else:
        raise SystemExit(f"unknown config {name}")
    dtype = args.dtype or dtype
    model_dir = base / f"{name}_seed{seed}"
    if not (model_dir / ".complete").exists():
        G.write_model_dir(model_dir, cfg, seed=seed, store_dtype="float16", **kw)
        (model_dir / ".complete").write_text("ok")
    be = tei_b200.B200Backend(model_dir, dtype, mtype, pool, devices=[0])
    if args.fused_residual:
        be.set_fused_residual(True)
    predict = mtype == "classifier"
    tokens = int(batch.cumulative_seq_lengths[-1])
    flops = G.algorithmic_flops(cfg, batch.lengths())
    be.stage(batch, normalize=not predict, predict=predict)
    for _ in range(max(args.warmup, 3)):
        be.run_staged()
    be.sync()
    be.set_profiling(True)
    sampler = ClockSampler(0)
    sampler.start()
    ms = be.run_staged_timed(args.steps)
    clocks = sampler.stop()
    kt = be.kernel_times()
    be.set_profiling(False)
    launches = be.stats()["launches"]
    call = (lambda: be.predict(batch)) if predict else (lambda: be.embed(batch, normalize=True))
    for _ in range(3):
        call()
    # a short forward is timed over at least 20 calls: one host hiccup among 5 calls of 4 ms would
    # otherwise be the result
    e2e_steps = args.steps if ms / args.steps > 50.0 else max(args.steps, 20)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        call()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    st = be.stats()
    in_flight = None
    if args.in_flight > 1:
        # Several batches in flight on ONE GPU: a handle with K replicas of device 0 and K caller
        # threads, each running whole batches on its own replica (`tei_b200_embed_on`), so one
        # batch's copies and host work overlap the other's kernels.  Same host buffers in and out.
        import threading
        k = args.in_flight
        be.close()
        be = tei_b200.B200Backend(model_dir, dtype, mtype, pool, devices=[0] * k)
        call_on = ((lambda r: be.predict(batch, replica=r)) if predict
                   else (lambda r: be.embed(batch, normalize=True, replica=r)))
        for r in range(k):
            for _ in range(3):
                call_on(r)
        threads = [threading.Thread(target=lambda r=r: [call_on(r) for _ in range(args.steps)]) for r in range(k)]
        t0 = time.perf_counter()
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        in_flight = {"batches_in_flight": k, "value": tokens * args.steps * k / dt, "unit": "tokens/s",
                     "ms_per_batch": 1e3 * dt / (args.steps * k)}
    line = {
        "metric": "tokens_per_sec", "value": tokens * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {"float16": "f16", "bfloat16": "bf16"}[dtype], "data": "synthetic",
        "config": {"workload": what, "per_gpu_batch_tokens": tokens, "sequences": len(batch),
                   "l2": "no flush: activations and weights of a step are far above the 126 MB L2"},
        "e2e": {"value": tokens * e2e_steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": st["h2d_bytes"],
                "d2h_bytes_per_step": st["d2h_bytes"], "ms_per_step": 1e3 * e2e_s / e2e_steps, "calls": e2e_steps},
        "gpu_launches": int(launches * args.steps),
        "algorithmic_tflop_per_step": flops / 1e12,
        "step_tflops": flops / (ms / args.steps / 1e3) / 1e12,
        "per_class_ms_per_step": {k: v["ms"] / args.steps for k, v in kt.items()},
        "clocks": clocks,
    }
    if in_flight:
        line["e2e_in_flight"] = in_flight
    print(json.dumps(line), flush=True)
    be.close()


def run_latency(args):
    """`--latency bs1|bs32`: the two cases the reference publishes latencies for (its README's
    benchmark table: bge-base-en-v1.5, sequence length 512, batch 1 and batch 32): p50 / p90 of the
    end-to-end time of one `embed` call through the C ABI with host buffers (tokens in, CLS-pooled
    normalised rows out), one call at a time as the router's single backend thread makes them."""
    import numpy as np
    import torch
    import tei_b200
    from oracle import generators as G

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    n_seqs = {"bs1": 1, "bs32": 32}[args.latency]
    model_dir = ensure_model_dir(0)
    be = tei_b200.B200Backend(model_dir, "float16", "embedding", "cls", devices=[0])
    rng = np.random.default_rng(10)
    encs = [np.concatenate([[101], rng.integers(1000, 30522, size=510), [102]]) for _ in range(n_seqs)]
    batch = G.batch_from_encodings(encs, list(range(n_seqs)), [])
    tokens = n_seqs * 512
    for _ in range(max(args.warmup, 10)):
        be.embed(batch, normalize=True)
    n = max(args.steps, 100)
    times, dev_ms = [], []
    for _ in range(n):
        t0 = time.perf_counter()
        be.embed(batch, normalize=True)
        times.append(1e3 * (time.perf_counter() - t0))
        dev_ms.append(be.stats()["gpu_ms"])
    st = be.stats()
    times.sort()
    px = gpu_proxy(model_dir, batch, n, 10)
    px.pop("rows", None)
    print(json.dumps({
        "metric": "latency_ms_p50", "value": times[n // 2], "unit": "ms", "n_gpus": 1, "steps": n,
        "warmup": max(args.warmup, 10), "higher_is_better": False, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"{args.latency}: BERT-base (bge-base-en-v1.5 architecture), {n_seqs} x 512 tokens, CLS pooling + "
                               "L2 normalise, one embed() call at a time with host buffers"},
        "p90_ms": times[(9 * n) // 10], "mean_ms": sum(times) / n, "device_ms_median": statistics.median(dev_ms),
        "tokens_per_sec_at_p50": tokens / (times[n // 2] / 1e3), "launches_per_call": st["launches"],
        "h2d_bytes_per_call": st["h2d_bytes"], "d2h_bytes_per_call": st["d2h_bytes"],
        "gpu_proxy_device_resident": px,
    }), flush=True)
    be.close()


def run_in_handle(args):
    """`--handle-devices N`: the drop-in mode behind an unchanged router, which keeps one batch in
    flight: ONE process, ONE handle with a replica on each of N GPUs; every `embed` call splits the
    packed cfg2 batch at sequence boundaries, runs the shards concurrently and scatters the rows
    back.  Wall-clock end to end (host buffers in and out), since the call spans several devices."""
    import torch
    import tei_b200
    from oracle import generators as G

    n = args.handle_devices
    if torch.cuda.device_count() < n:
        raise SystemExit(f"--handle-devices {n} needs {n} visible GPUs")
    model_dir = ensure_model_dir(0)
    be = tei_b200.B200Backend(model_dir, "float16", "embedding", "mean", devices=list(range(n)))
    batch = G.batch_cfg2()
    tokens = int(batch.cumulative_seq_lengths[-1])
    for _ in range(max(args.warmup, 3)):
        be.embed(batch, normalize=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        be.embed(batch, normalize=True)
    dt = time.perf_counter() - t0
    print(json.dumps({
        "metric": "tokens_per_sec", "value": tokens * args.steps / dt, "unit": "tokens/s", "n_gpus": n,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": f"one handle, batch split over {n} replicas inside each call",
                   "timing": "wall clock around embed() with host buffers"},
    }), flush=True)
    be.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fused-residual", action="store_true",
                    help="add the feed-forward residual in the output projection's epilogue instead of the "
                         "LayerNorm kernel behind it (the default, the reference's form)")
    ap.add_argument("--no-gpu-proxy", action="store_true",
                    help="skip the flash_attn + cuBLASLt proxy forward that follows the main arm at N = 1")
    ap.add_argument("--kernel", default=None,
                    help="time one kernel alone: gemm_qkv | gemm_out | gemm_ffn1 | gemm_ffn2 | attention | "
                         "attention_long | attention_causal128 | attention_d32 | rope_qwen3 | qkv_rope_nomic | qkv_rope_qwen3 | add_layernorm | "
                         "add_layernorm_h1024 | pool_mean")
    ap.add_argument("--config", default="cfg2", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5"],
                    help="cfg2 is the headline workload (default, any --gpus); the others run on one GPU")
    ap.add_argument("--dtype", default=None, choices=["float16", "bfloat16"],
                    help="only with --config cfg1/3/4/5 (cfg5 defaults to bfloat16)")
    ap.add_argument("--in-flight", type=int, default=1,
                    help="one GPU, any --config: also measure end to end with this many batches in flight "
                         "(one caller thread per replica of device 0); prints the single-config line")
    ap.add_argument("--latency", default=None, choices=["bs1", "bs32"],
                    help="p50 end-to-end latency of one embed() call: BERT-base, 1 x 512 or 32 x 512 tokens")
    ap.add_argument("--handle-devices", type=int, default=0,
                    help="one process, one handle with this many replicas: each embed() call splits the batch")
    args = ap.parse_args()
    if args.kernel:
        run_kernel(args)
        return
    if args.latency:
        run_latency(args)
        return
    if args.handle_devices > 0:
        run_in_handle(args)
        return
    if (args.config != "cfg2" or args.in_flight > 1) and args.impl == "b200":
        run_config(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import numpy as np
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    ranks = Ranks(world, local_rank, backend="nccl")
    barrier, max_over_ranks, sum_over_ranks = ranks.barrier, ranks.max, ranks.sum

    import tei_b200
    from oracle import generators as G

    model_dir = ensure_model_dir(local_rank)
    be = tei_b200.B200Backend(model_dir, "float16", "embedding", "mean", devices=[local_rank])
    if args.fused_residual:
        be.set_fused_residual(True)
    batch = G.batch_cfg2()
    tokens = int(batch.cumulative_seq_lengths[-1])
    lens = batch.lengths()
    cfg = G.bert_config()

    # ---------------------------------------------------------------- device-resident value
    be.stage(batch, normalize=True)
    for _ in range(args.warmup):
        be.run_staged()
    be.sync()
    be.set_profiling(True)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    ms = be.run_staged_timed(args.steps)
    clocks = sampler.stop()
    barrier()
    kt = be.kernel_times()
    be.set_profiling(False)
    launches_per_step = be.stats()["launches"] / args.steps
    ms = max_over_ranks(ms)
    total_tokens = sum_over_ranks(float(tokens)) * args.steps
    value = total_tokens / (ms / 1e3)

    # ---------------------------------------------------------------- end-to-end through embed
    for _ in range(args.warmup):
        be.embed(batch, normalize=True)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        be.embed(batch, normalize=True)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    st = be.stats()
    e2e_s = max_over_ranks(e2e_s)
    e2e_value = total_tokens / e2e_s

    # ---------------------------------------------------------------- roofline of the GEMM kernel
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    gemm_flops_per_step = L * 2.0 * tokens * (4 * H * H + 2 * H * I)
    attn_flops_per_step = L * 4.0 * H * float((lens.astype(np.float64) ** 2).sum())
    peaks = {}
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peaks = json.loads(peaks_file.read_text())
    peak_tf = float(peaks.get("bf16_tflops_sustained", 1400.0))
    peak_burst = float(peaks.get("bf16_tflops", 1590.0))
    peak_src = ("measured (MEASURED_PEAKS.json: bf16_tflops_sustained for `peak`, bf16_tflops for `peak_burst`)" if peaks
                else "fallback 1.4 PFLOP/s sustained, 1.59 PFLOP/s burst")
    gemm_ms_per_step = kt["gemm"]["ms"] / args.steps
    gemm_launches = kt["gemm"]["launches"] / args.steps
    achieved = gemm_flops_per_step / (gemm_ms_per_step / 1e3) / 1e12 if gemm_ms_per_step > 0 else 0.0
    attn_ms_per_step = kt["attention"]["ms"] / args.steps
    roofline = {
        "kernel": "gemm_tcgen05_pair_kernel (dense layers: QKV, attention output, FFN up + GELU, FFN down)",
        "bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
        "frac": achieved / peak_tf if peak_tf else None, "peak_source": peak_src,
        "peak_burst": peak_burst, "frac_burst": achieved / peak_burst if peak_burst else None,
        # dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures of the four
        # GEMM shapes (profiles/gemm_tcgen05_bert_base_shapes.md), mean over the shapes.
        "traffic": 382e6, "traffic_unit": "bytes per launch (mean of the 4 shapes, ncu)",
        # inputs + weights + outputs of QKV, attention-output, FFN-up and FFN-down, mean per launch
        "algorithmic_bytes_per_launch": 2.0 * (tokens * (4 * H + 2 * H + 2 * (H + I)) + 4 * H * H + 2 * H * I) / 4.0,
        "flops_per_launch": gemm_flops_per_step / gemm_launches if gemm_launches else None,
        "ms_per_launch": gemm_ms_per_step / gemm_launches if gemm_launches else None,
        "launches_per_step": gemm_launches,
        "per_class_ms_per_step": {k: v["ms"] / args.steps for k, v in kt.items()},
        "attention_tflops": attn_flops_per_step / (attn_ms_per_step / 1e3) / 1e12 if attn_ms_per_step > 0 else None,
        "step_tflops": (gemm_flops_per_step + attn_flops_per_step) / (ms / args.steps / 1e3) / 1e12,
    }
    # attention + GEMM kernels together against the tensor peak
    ag_ms = gemm_ms_per_step + attn_ms_per_step
    if ag_ms > 0:
        ag = (gemm_flops_per_step + attn_flops_per_step) / (ag_ms / 1e3) / 1e12
        roofline["attention_plus_gemm"] = {"tflops": ag, "frac": ag / peak_tf, "frac_burst": ag / peak_burst}
    # Attention at head_dim 64 is bounded by the exp2 unit before the tensor pipe: one ex2 per
    # score, 16 per clock and SM (4 per scheduler), against 4 x head_dim FLOP per score.
    if attn_ms_per_step > 0 and clocks.get("sm_mhz"):
        n_sms = torch.cuda.get_device_properties(local_rank).multi_processor_count
        head_dim = H // cfg["num_attention_heads"]
        exp_peak = 16.0 * n_sms * clocks["sm_mhz"] * 1e6 * 4.0 * head_dim / 1e12
        roofline["attention_exp2_bound"] = {
            "tflops": roofline["attention_tflops"], "peak_tflops_at_sampled_clock": exp_peak,
            "frac": roofline["attention_tflops"] / exp_peak,
            "what": "16 ex2 per clock and SM x 4*head_dim FLOP per score, at the sampled median SM clock"}
    # The step runs under the power cap at whatever clock the box settles at; time x clock compares
    # runs at different clocks (time at the maximum clock = time x sampled median / maximum).
    if clocks.get("sm_mhz") and clocks.get("sm_max_mhz"):
        ratio = clocks["sm_mhz"] / clocks["sm_max_mhz"]
        roofline["clock_normalised"] = {
            "sm_mhz_median": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"],
            "gemm_ms_x_ghz": gemm_ms_per_step * clocks["sm_mhz"] / 1e3,
            "gemm_ms_per_step_at_max_clock": gemm_ms_per_step * ratio,
            "gemm_tflops_at_max_clock": achieved / ratio if ratio > 0 else None,
        }

    line = {
        "metric": "tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu_batch_tokens": tokens, "parallelism": f"replicas x{world}",
                   "l2": "no flush: every step streams >1 GB of activations and 218 MB of weights, far above the 126 MB L2"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": st["h2d_bytes"],
                "d2h_bytes_per_step": st["d2h_bytes"], "ms_per_step": 1e3 * e2e_s / args.steps},
        "gpu_launches": int(round(launches_per_step * args.steps)),
        "roofline": roofline, "clocks": clocks,
    }

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tps, cores, dt, sample_tokens = cpu_baseline(model_dir, 48)
        line["cpu_baseline"] = {
            "value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first 48 of the 256 sequences ({sample_tokens} tokens, {dt:.1f} s), forwards of <=4 sequences "
                      "padded to the chunk max, fp32 torch CPU restatement of the reference's Candle CPU path",
        }
    else:
        line["cpu_baseline"] = None
    if rank == 0 and world == 1 and not args.no_gpu_proxy:
        rows_ours = be.embed(batch, normalize=True)
        be.close()  # the proxy gets the GPU to itself
        px = gpu_proxy(model_dir, batch, args.steps, args.warmup)
        rows = px.pop("rows", None)
        if rows is not None:  # the proxy computes the same thing: its rows agree with this backend's
            ours = np.stack([rows_ours[i].values for i in range(len(batch))])
            px["min_cosine_vs_this_backend"] = float((ours * rows.float().cpu().numpy()).sum(-1).min())
            px["this_backend_over_proxy"] = value / px["value"]
        line["gpu_proxy"] = px
    if rank == 0:
        print(json.dumps(line), flush=True)
    be.close()
    ranks.close()


if __name__ == "__main__":
    main()
