"""CUDA-event microbenchmarks of the hot kernels against their rooflines.

Counterpart of the reference's roofline probes and kernel benches
(crates/onnx-genai-bench/src/bin/roofline_gemv.rs, marlin_bench.rs).  Every timing follows the
same hygiene: >= 3 warm-up launches, an L2 flush (a write larger than the 126 MB L2) before each
timed launch, CUDA events on the launching stream.  Peaks come from MEASURED_PEAKS.json when it
is present next to the repository root, otherwise from the documented fallback figures.

    python -m onnx_genai_b200.bench.kernel_bench --what gemm,attn --json out.json
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch

from .. import ops
from ..ops import reference as ref


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Timer:
    def __init__(self, flush_mb=256):
        self.flush = torch.empty(flush_mb * 1024 * 1024, dtype=torch.uint8, device="cuda")

    def time(self, fn, iters=10, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            self.flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        return ts[len(ts) // 2], ts[0]


def bench_gemm(timer, pk, shapes=None):
    rows = []
    shapes = shapes or [
        # (M, N, K, epilogue) -- Qwen2.5-7B projections at decode / mixed / prefill step sizes
        (256, 4608, 3584, "none"), (256, 3584, 3584, "residual"), (256, 37888, 3584, "swiglu"), (256, 3584, 18944, "residual"),
        (1280, 4608, 3584, "none"), (1280, 3584, 3584, "residual"), (1280, 37888, 3584, "swiglu"), (1280, 3584, 18944, "residual"),
        (2048, 4608, 3584, "none"), (2048, 37888, 3584, "swiglu"), (2048, 3584, 18944, "residual"),
        (256, 152064, 3584, "none"), (8192, 8192, 8192, "none"),
    ]
    for m, n, k, epi in shapes:
        a = (torch.randn(m, k, device="cuda") * 0.1).bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
        res = torch.randn(m, n, device="cuda").bfloat16() if epi == "residual" else None
        n_out = n // 2 if epi == "swiglu" else n
        out = torch.empty(m, n_out, device="cuda", dtype=torch.bfloat16)
        best = None
        for bn in ((256, 128) if epi == "swiglu" else (256, 128, 64)):
            if epi == "swiglu":
                fn = lambda: ops.gemm(a, w, epilogue="swiglu", swiglu_half=bn // 2, out=out)
            elif epi == "residual":
                fn = lambda: ops.gemm(a, w, residual=res, epilogue="residual", out=out, bn=bn)
            else:
                fn = lambda: ops.gemm(a, w, out=out, bn=bn)
            med, mn = timer.time(fn)
            if best is None or med < best[0]:
                best = (med, mn, bn)
        full = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        lib_med, _ = timer.time(lambda: torch.matmul(a, w.t(), out=full))
        flops = 2.0 * m * n * k
        byts = 2.0 * (m * k + n * k + m * n_out)
        tf = flops / best[0] / 1e9
        rows.append({
            "kernel": "gemm_bf16_tcgen05", "M": m, "N": n, "K": k, "epilogue": epi, "bn": best[2],
            "ms": round(best[0], 4), "tflops": round(tf, 1), "frac_of_%s_bf16_peak" % pk["source"]: round(tf / pk["bf16_tflops"], 3),
            "gbs": round(byts / best[0] / 1e6, 1), "frac_of_%s_hbm" % pk["source"]: round(byts / best[0] / 1e6 / pk["hbm_gbs"], 3),
            "cublas_ms": round(lib_med, 4), "vs_cublas": round(lib_med / best[0], 3),
        })
        print(json.dumps(rows[-1]), flush=True)
    ops.check_status()
    return rows


def bench_attention(timer, pk):
    rows = []
    hq, hkv, d = 28, 4, 128
    for n, ctx in [(256, 1200), (256, 2304), (64, 8192), (8, 32768)]:
        pages_per = (ctx + 15) // 16
        total = n * pages_per
        pool = (torch.randn(total, hkv, 2, 16, d, device="cuda") * 0.5).bfloat16()
        table = torch.randperm(total, device="cuda").to(torch.int32).view(n, pages_per)
        ctx_t = torch.full((n,), ctx, dtype=torch.int32, device="cuda")
        q = torch.randn(n, (hq + 2 * hkv) * d, device="cuda").bfloat16()
        out = torch.empty(n, hq * d, device="cuda", dtype=torch.bfloat16)
        for splits in (1, 2, 4, 8, 16):
            if n * hkv * splits > 148 * 16 and splits > 1:
                continue
            po = torch.empty(n * hq * splits * d, dtype=torch.float32, device="cuda")
            pm = torch.empty(n * hq * splits * 2, dtype=torch.float32, device="cuda")
            med, _ = timer.time(lambda: ops.paged_decode(q, out, pool, table, ctx_t, hq, hkv, d, num_splits=splits,
                                                         part_o=po, part_ml=pm))
            byts = float(n) * ctx * hkv * 2 * d * 2
            rows.append({"kernel": "paged_decode", "seqs": n, "ctx": ctx, "splits": splits, "ms": round(med, 4),
                         "gbs": round(byts / med / 1e6, 1),
                         "frac_of_%s_hbm" % pk["source"]: round(byts / med / 1e6 / pk["hbm_gbs"], 3)})
            print(json.dumps(rows[-1]), flush=True)
        del pool
    # (q_len, past, sequences, query heads, kv heads): the last rows are one rank's share at TP=4 / TP=8, where tiles x heads
    # no longer fill the machine and the kernel switches to 32- / 16-row CTAs
    for q_len, past, nseq, hq, hkv in [(1024, 0, 4, 28, 4), (2048, 0, 4, 28, 4), (512, 1536, 4, 28, 4), (1024, 0, 1, 7, 1),
                                       (1024, 0, 1, 4, 1), (256, 0, 4, 4, 1)]:
        ctx = q_len + past
        pages_per = (ctx + 15) // 16
        total = nseq * pages_per
        pool = (torch.randn(total, hkv, 2, 16, d, device="cuda") * 0.5).bfloat16()
        table = torch.randperm(total, device="cuda").to(torch.int32).view(nseq, pages_per)
        ctx_t = torch.full((nseq,), ctx, dtype=torch.int32, device="cuda")
        t = nseq * q_len
        q = torch.randn(t, (hq + 2 * hkv) * d, device="cuda").bfloat16()
        out = torch.empty(t, hq * d, device="cuda", dtype=torch.bfloat16)
        cu = torch.arange(0, t + 1, q_len, dtype=torch.int32, device="cuda")
        ts, tq = ops.prefill_tiles([q_len] * nseq)
        tsd = torch.tensor(ts, dtype=torch.int32, device="cuda")
        tqd = torch.tensor(tq, dtype=torch.int32, device="cuda")
        med, _ = timer.time(lambda: ops.paged_prefill(q, out, pool, table, ctx_t, cu, tsd, tqd, len(ts), hq, hkv, d))
        flops = 4.0 * nseq * hq * d * (q_len * past + q_len * (q_len + 1) / 2)
        rows.append({"kernel": "paged_prefill", "seqs": nseq, "q_len": q_len, "past": past, "hq": hq, "hkv": hkv, "ms": round(med, 4),
                     "tflops": round(flops / med / 1e9, 1)})
        print(json.dumps(rows[-1]), flush=True)
    ops.check_status()
    return rows


def bench_attention_tp_shapes(timer, pk):
    """Decode attention as one rank of a tensor-parallel group sees it: one KV head and 7 (TP=4) or 4 (TP=8) query heads, 255
    sequences with contexts drawn from U[128, 2304] as in the serving bench.  Launch trains over distinct pools (together
    larger than L2) so that a launch's host path does not count."""
    rows = []
    d, n = 128, 255
    g = torch.Generator(device="cpu").manual_seed(5)
    ctx = torch.randint(128, 2305, (n,), generator=g)
    pages_per = int((int(ctx.max()) + 15) // 16)
    total = int(((ctx + 15) // 16).sum()) + 1
    copies = 3
    for hq, hkv in ((7, 1), (4, 1)):
        pools = [(torch.randn(total, hkv, 2, 16, d, device="cuda") * 0.5).bfloat16() for _ in range(copies)]
        perm = torch.randperm(total)
        table = torch.zeros(n, pages_per, dtype=torch.int32)
        o = 0
        for s in range(n):
            k = int((ctx[s] + 15) // 16)
            table[s, :k] = perm[o:o + k].to(torch.int32)
            o += k
        table, ctx_t = table.cuda(), ctx.to(torch.int32).cuda()
        q = torch.randn(n, (hq + 2 * hkv) * d, device="cuda").bfloat16()
        out = torch.empty(n, hq * d, device="cuda", dtype=torch.bfloat16)
        byts = float(ctx.sum()) * hkv * 2 * d * 2
        for splits in (1, 2, 4):
            po = torch.empty(n * hq * splits * d, dtype=torch.float32, device="cuda")
            pm = torch.empty(n * hq * splits * 2, dtype=torch.float32, device="cuda")

            def fn():
                for i in range(2 * copies):
                    ops.paged_decode(q, out, pools[i % copies], table, ctx_t, hq, hkv, d, num_splits=splits, part_o=po, part_ml=pm)

            med, _ = timer.time(fn)
            per = med / (2 * copies)
            rows.append({"kernel": "paged_decode_tp_rank", "hq": hq, "hkv": hkv, "seqs": n, "ctx": "U[128,2304]", "splits": splits, "ms": round(per, 4),
                         "gbs": round(byts / per / 1e6, 1), "frac_of_%s_hbm" % pk["source"]: round(byts / per / 1e6 / pk["hbm_gbs"], 3)})
            print(json.dumps(rows[-1]), flush=True)
        del pools
    ops.check_status()
    return rows


def bench_attention_one_byte(timer, pk):
    """Decode attention over one-byte KV pages (e4m3 and int8): same contexts as the bf16 rows, half the bytes."""
    rows = []
    hq, hkv, d = 28, 4, 128
    for fmt, dtype in (("fp8", torch.uint8), ("int8", torch.int8)):
        for n, ctx, splits in [(256, 1200, 1), (256, 2304, 2), (64, 8192, 8), (8, 32768, 16)]:
            pages_per = (ctx + 15) // 16
            total = n * pages_per
            if fmt == "fp8":
                pool = (torch.randn(total, hkv, 2, 16, d, device="cuda") * 0.5).to(torch.float8_e4m3fn).view(torch.uint8)
            else:
                pool = torch.randint(-127, 128, (total, hkv, 2, 16, d), device="cuda", dtype=torch.int8)
            scales = torch.rand(total, hkv, 2, device="cuda") * 0.02 + 0.005
            table = torch.randperm(total, device="cuda").to(torch.int32).view(n, pages_per)
            ctx_t = torch.full((n,), ctx, dtype=torch.int32, device="cuda")
            q = torch.randn(n, (hq + 2 * hkv) * d, device="cuda").bfloat16()
            out = torch.empty(n, hq * d, device="cuda", dtype=torch.bfloat16)
            po = torch.empty(n * hq * splits * d, dtype=torch.float32, device="cuda")
            pm = torch.empty(n * hq * splits * 2, dtype=torch.float32, device="cuda")
            med, _ = timer.time(lambda: ops.paged_decode(q, out, pool, table, ctx_t, hq, hkv, d, num_splits=splits, part_o=po, part_ml=pm,
                                                         kv_scales=scales))
            byts = float(n) * ctx * hkv * 2 * d
            rows.append({"kernel": "paged_decode_" + fmt, "seqs": n, "ctx": ctx, "splits": splits, "ms": round(med, 4),
                         "gbs": round(byts / med / 1e6, 1), "frac_of_%s_hbm" % pk["source"]: round(byts / med / 1e6 / pk["hbm_gbs"], 3)})
            print(json.dumps(rows[-1]), flush=True)
            del pool
    ops.check_status()
    return rows


def bench_misc(timer, pk):
    rows = []
    x = torch.randn(1280, 3584, device="cuda").bfloat16()
    w = torch.randn(3584, device="cuda").bfloat16()
    out = torch.empty_like(x)
    med, _ = timer.time(lambda: ops.rmsnorm(x, w, 1e-6, out=out))
    rows.append({"kernel": "rmsnorm", "rows": 1280, "hidden": 3584, "ms": round(med, 4),
                 "gbs": round(2 * x.numel() * 2 / med / 1e6, 1)})
    logits = torch.randn(256, 152064, device="cuda").bfloat16()
    temp = torch.full((256,), 0.7, device="cuda")
    tk = torch.zeros(256, dtype=torch.int32, device="cuda")
    tp = torch.full((256,), 0.9, device="cuda")
    mp = torch.zeros(256, device="cuda")
    u = torch.rand(256, device="cuda")
    work = torch.empty(256 * 152064, dtype=torch.int32, device="cuda")
    med, _ = timer.time(lambda: ops.sample(logits, temp, tk, tp, mp, u, work=work))
    rows.append({"kernel": "sample_topp", "rows": 256, "vocab": 152064, "ms": round(med, 4)})
    med, _ = timer.time(lambda: ops.argmax(logits))
    rows.append({"kernel": "argmax", "rows": 256, "vocab": 152064, "ms": round(med, 4)})
    for r in rows:
        print(json.dumps(r), flush=True)
    return rows


def bench_w4a16(timer, pk):
    """Decode-size int4 projections (block 32, bf16 scales) of the 7B and 0.5B shapes: bytes streamed per launch
    (nibbles + scales) over the measured copy bandwidth.  A launch lasts 10-40 us, the same order as the host's launch
    path, so each sample times a train of launches over distinct copies of the weights (together larger than L2, so
    every launch streams from HBM) and divides."""
    from onnx_genai_b200.ops.quant import QuantLinear

    rows = []
    cases = [("7b_gate_up", 37888, 3584, "rmsnorm"), ("7b_down", 3584, 18944, "silu_mul"), ("7b_qkv", 4608, 3584, "rmsnorm"),
             ("0.5b_gate_up", 9728, 896, "rmsnorm"), ("0.5b_down", 896, 4864, "silu_mul")]
    for name, n_, k_, pro in cases:
        nbytes = n_ * k_ // 2 + n_ * (k_ // 32) * 2
        copies = max(2, min(64, (192 << 20) // nbytes + 1))
        q = torch.randint(0, 256, (n_, k_ // 32, 16), dtype=torch.uint8)
        sc = (torch.rand(n_, k_ // 32) * 0.02 + 0.005).bfloat16()
        lins = [QuantLinear(q, sc, None, None, k=k_, device="cuda") for _ in range(copies)]
        train = 2 * copies
        for m in (1, 4):
            out = torch.empty(m, n_, device="cuda", dtype=torch.bfloat16)
            if pro == "rmsnorm":
                x = torch.randn(m, k_, device="cuda").bfloat16()
                g = torch.ones(k_, device="cuda", dtype=torch.bfloat16)
                one = lambda lin: lin.fused(x, out, norm_weight=g, eps=1e-6)
            else:
                x = torch.randn(m, 2 * k_, device="cuda").bfloat16()
                one = lambda lin: lin.fused(x, out, silu_mul=True)

            def fn():
                for i in range(train):
                    one(lins[i % copies])

            med, _ = timer.time(fn)
            per = med / train
            rows.append({"kernel": "w4a16_gemv_fused", "case": name, "m": m, "n": n_, "k": k_, "ms": round(per, 4), "launches_per_sample": train,
                         "gbs": round(nbytes / per / 1e6, 1), "frac_of_measured_hbm": round(nbytes / per / 1e6 / pk["hbm_gbs"], 3)})
            print(json.dumps(rows[-1]), flush=True)
    return rows


def bench_w4a16_gemm(timer, pk):
    """The int4 tensor-core GEMM (B tiles dequantised in shared memory) at batch sizes above the GEMV range, beside the bf16
    GEMM over a dequantised copy of the same weights: time, FLOP rate against the measured cuBLAS bf16 rate, int4 bytes
    streamed against the measured copy bandwidth, and the device bytes each arm keeps per projection."""
    from onnx_genai_b200.ops.quant import QuantLinear

    rows = []
    for name, n_, k_ in (("7b_gate_up", 37888, 3584), ("7b_down", 3584, 18944), ("7b_qkv", 4608, 3584)):
        q = torch.randint(0, 256, (n_, k_ // 32, 16), dtype=torch.uint8)
        sc = (torch.rand(n_, k_ // 32) * 0.02 + 0.005).bfloat16()
        lin = QuantLinear(q, sc, None, None, k=k_, device="cuda")
        dense = QuantLinear(q, sc, None, None, k=k_, device="cuda")
        dense.large_m = "dense"
        nbytes = n_ * k_ // 2 + n_ * (k_ // 32) * 2
        for m in (16, 64, 128, 256, 1024, 2048):
            x = (torch.randn(m, k_, device="cuda") * 0.3).bfloat16()
            out = torch.empty(m, n_, device="cuda", dtype=torch.bfloat16)
            dense(x, out=out)                               # builds the copy outside the timed region
            t_int4, _ = timer.time(lambda: lin(x, out=out))
            t_dense, _ = timer.time(lambda: dense(x, out=out))
            fl = 2.0 * m * n_ * k_
            rows.append({"kernel": "gemm_w4a16_tcgen05", "case": name, "m": m, "n": n_, "k": k_, "ms": round(t_int4, 4),
                         "tflops": round(fl / t_int4 / 1e9, 1), "frac_of_measured_bf16": round(fl / t_int4 / 1e9 / pk["bf16_tflops"], 3),
                         "int4_gbs": round(nbytes / t_int4 / 1e6, 1), "frac_of_measured_hbm": round(nbytes / t_int4 / 1e6 / pk["hbm_gbs"], 3),
                         "bf16_copy_gemm_ms": round(t_dense, 4), "int4_over_bf16_time": round(t_int4 / t_dense, 2),
                         "device_bytes_int4": lin.device_weight_bytes(), "device_bytes_bf16_copy": dense.device_weight_bytes()})
            print(json.dumps(rows[-1]), flush=True)
    return rows


def ncu_case(name: str, iters: int = 3):
    """Small single-kernel workloads for `ncu` captures: inputs larger than L2 where DRAM figures matter,
    a few hundred MB on the device at most, `iters` launches of the one kernel of interest."""
    hq, hkv, d = 28, 4, 128
    if name in ("gemm_swiglu", "gemm_down", "gemm_qkv"):
        m = 1280
        n, k, epi = {"gemm_swiglu": (37888, 3584, "swiglu"), "gemm_down": (3584, 18944, "residual"), "gemm_qkv": (4608, 3584, "none")}[name]
        a = (torch.randn(m, k, device="cuda") * 0.1).bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
        out = torch.empty(m, n // 2 if epi == "swiglu" else n, device="cuda", dtype=torch.bfloat16)
        res = torch.randn(m, n, device="cuda").bfloat16() if epi == "residual" else None
        for _ in range(iters):
            if epi == "swiglu":
                ops.gemm(a, w, epilogue="swiglu", swiglu_half=128, out=out)
            elif epi == "residual":
                ops.gemm(a, w, residual=res, epilogue="residual", out=out)
            else:
                ops.gemm(a, w, out=out)
    elif name in ("w4a16_gemm_m1024", "w4a16_gemm_m64"):
        from onnx_genai_b200.ops.quant import QuantLinear

        m, n, k = (1024 if name.endswith("1024") else 64), 37888, 3584
        lin = QuantLinear(torch.randint(0, 256, (n, k // 32, 16), dtype=torch.uint8), (torch.rand(n, k // 32) * 0.02 + 0.005).bfloat16(),
                          None, None, k=k, device="cuda")
        x = (torch.randn(m, k, device="cuda") * 0.3).bfloat16()
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        for _ in range(iters):
            lin(x, out=out)
    elif name == "decode_step_0p5b_int4":
        # whole decode steps of the Qwen2.5-0.5B-shape int4 model at batch 1 (512-token prompt), launched one kernel
        # at a time so a launch list shows the device time of every kernel of a step
        import tempfile

        import numpy as np

        from onnx_genai_b200.bench.config_bench import _export
        from onnx_genai_b200.engine.api import Engine, GenerateOptions

        with tempfile.TemporaryDirectory() as tmp:
            cfg = _export("qwen2.5-0.5b", tmp, "bf16")
            eng = Engine.from_dir(tmp, device="cuda", max_seqs=1, max_seq_len=640, cuda_graphs=False)
            prompt = np.random.default_rng(0).integers(0, cfg.vocab, size=512).tolist()
            eng.generate_batch([prompt], GenerateOptions(max_new_tokens=1 + iters, greedy=True, ignore_eos=True))
    elif name == "w4a16_gemv":
        # decode-size int4 projection of the 7B shape: gate_up (N = 37888, K = 3584) with the RMSNorm prologue, one row
        from onnx_genai_b200.ops import reference as ref
        from onnx_genai_b200.ops.quant import QuantLinear

        n_, k_ = 37888, 3584
        q = torch.randint(0, 256, (n_, k_ // 32, 16), dtype=torch.uint8)
        sc = (torch.rand(n_, k_ // 32) * 0.02 + 0.005).bfloat16()
        lin = QuantLinear(q, sc, None, None, k=k_, device="cuda")
        x = torch.randn(1, k_, device="cuda").bfloat16()
        g = torch.ones(k_, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(1, n_, device="cuda", dtype=torch.bfloat16)
        for _ in range(iters):
            lin.fused(x, out, norm_weight=g, eps=1e-6)
    elif name == "decode":
        n, ctx = 256, 1200
        pages_per = (ctx + 15) // 16
        pool = (torch.randn(n * pages_per, hkv, 2, 16, d, device="cuda") * 0.5).bfloat16()
        table = torch.randperm(n * pages_per, device="cuda").to(torch.int32).view(n, pages_per)
        ctx_t = torch.full((n,), ctx, dtype=torch.int32, device="cuda")
        q = torch.randn(n, (hq + 2 * hkv) * d, device="cuda").bfloat16()
        out = torch.empty(n, hq * d, device="cuda", dtype=torch.bfloat16)
        for _ in range(iters):
            ops.paged_decode(q, out, pool, table, ctx_t, hq, hkv, d)
    elif name == "decode_fp8":
        n, ctx = 256, 1200
        pages_per = (ctx + 15) // 16
        pool = (torch.randn(n * pages_per, hkv, 2, 16, d, device="cuda") * 0.5).to(torch.float8_e4m3fn).view(torch.uint8)
        scales = torch.rand(n * pages_per, hkv, 2, device="cuda") * 0.02 + 0.005
        table = torch.randperm(n * pages_per, device="cuda").to(torch.int32).view(n, pages_per)
        ctx_t = torch.full((n,), ctx, dtype=torch.int32, device="cuda")
        q = torch.randn(n, (hq + 2 * hkv) * d, device="cuda").bfloat16()
        out = torch.empty(n, hq * d, device="cuda", dtype=torch.bfloat16)
        for _ in range(iters):
            ops.paged_decode(q, out, pool, table, ctx_t, hq, hkv, d, kv_scales=scales)
    elif name == "prefill":
        nseq, q_len = 4, 1024
        pages_per = q_len // 16
        pool = (torch.randn(nseq * pages_per, hkv, 2, 16, d, device="cuda") * 0.5).bfloat16()
        table = torch.randperm(nseq * pages_per, device="cuda").to(torch.int32).view(nseq, pages_per)
        ctx_t = torch.full((nseq,), q_len, dtype=torch.int32, device="cuda")
        q = torch.randn(nseq * q_len, (hq + 2 * hkv) * d, device="cuda").bfloat16()
        out = torch.empty(nseq * q_len, hq * d, device="cuda", dtype=torch.bfloat16)
        cu = torch.arange(0, nseq * q_len + 1, q_len, dtype=torch.int32, device="cuda")
        ts, tq = ops.prefill_tiles([q_len] * nseq)
        tsd, tqd = torch.tensor(ts, dtype=torch.int32, device="cuda"), torch.tensor(tq, dtype=torch.int32, device="cuda")
        for _ in range(iters):
            ops.paged_prefill(q, out, pool, table, ctx_t, cu, tsd, tqd, len(ts), hq, hkv, d)
    elif name == "sample":
        logits = torch.randn(256, 152064, device="cuda").bfloat16()
        f = lambda v: torch.full((256,), v, device="cuda")
        work = torch.empty(256 * 152064, dtype=torch.int32, device="cuda")
        for _ in range(iters):
            ops.sample(logits, f(0.7), torch.zeros(256, dtype=torch.int32, device="cuda"), f(0.9), f(0.0), torch.rand(256, device="cuda"), work=work)
    else:
        raise SystemExit(f"unknown ncu case {name!r}")
    torch.cuda.synchronize()
    ops.check_status()
    print("ncu case", name, "ok")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ncu-case", default="", help="run one small single-kernel workload (for ncu) and exit")
    ap.add_argument("--what", default="gemm,attn,misc", help="comma list of gemm, attn, attn_tp (one rank's decode share at TP=4 / 8), attn8 (one-byte KV pages), misc, w4 (int4 decode projections), w4gemm (int4 tensor-core GEMM against the bf16 GEMM over a dequantised copy)")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    if args.ncu_case:
        return ncu_case(args.ncu_case)
    pk = peaks()
    timer = Timer()
    res = {"peaks": pk}
    what = args.what.split(",")
    if "gemm" in what:
        res["gemm"] = bench_gemm(timer, pk)
    if "attn" in what:
        res["attn"] = bench_attention(timer, pk)
    if "attn_tp" in what:
        res["attn_tp"] = bench_attention_tp_shapes(timer, pk)
    if "attn8" in what:
        res["attn8"] = bench_attention_one_byte(timer, pk)
    if "misc" in what:
        res["misc"] = bench_misc(timer, pk)
    if "w4" in what:
        res["w4a16"] = bench_w4a16(timer, pk)
    if "w4gemm" in what:
        res["w4a16_gemm"] = bench_w4a16_gemm(timer, pk)
    if args.json:
        Path(args.json).write_text(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
