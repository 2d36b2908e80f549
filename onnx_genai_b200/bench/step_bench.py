"""One representative engine step, replayed: the optimisation target behind bench.py.

Builds a synthetic steady-state step directly in the packed plan (no ramp): ``--decode`` rows
whose contexts are uniform in [min_ctx, max_ctx] plus ``--prefill`` chunks of ``--chunk`` new
tokens, on the full model shape, then replays it in three ways:

  native   one call into the C++ step executor per step        (what the engine runs)
  python   the same kernels launched one by one from Python    (no events inside)
  per-op   python path with a CUDA-event pair around every op  (breakdown; perturbs clocks)

    python -m onnx_genai_b200.bench.step_bench --model qwen2.5-7b --decode 255 --prefill 1 --chunk 1025
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np
import torch

from .. import ops
from ..engine.core import HDR
from ..engine.llm_engine import EngineConfig, LLMEngine
from ..models.config import preset


def build_plan(eng: LLMEngine, n_decode, n_prefill, chunk, min_ctx, max_ctx, past, seed=0):
    L, pn = eng.L, eng.plan_np
    rng = np.random.default_rng(seed)
    mp = eng.core.cfg.max_pages_per_seq
    pn[:] = 0
    t = 0
    free_pages = rng.permutation(eng.num_pages)
    pp = 0
    rows = 0
    ctxs = []
    for i in range(n_decode):
        ctx = int(rng.integers(min_ctx, max_ctx + 1))
        npg = (ctx + 15) // 16
        pages = free_pages[pp:pp + npg]
        pp += npg
        pn[L.page_table + rows * mp: L.page_table + rows * mp + npg] = pages
        pn[L.ctx_len + rows] = ctx
        pn[L.token_ids + t] = rng.integers(0, eng.cfg.model.vocab)
        pn[L.positions + t] = ctx - 1
        pn[L.slots + t] = pages[(ctx - 1) // 16] * 16 + (ctx - 1) % 16
        pn[L.logit_rows + rows] = t
        ctxs.append(ctx)
        t += 1
        rows += 1
    base = t
    tiles = 0
    for j in range(n_prefill):
        ctx = past + chunk
        npg = (ctx + 15) // 16
        pages = free_pages[pp:pp + npg]
        pp += npg
        pn[L.page_table + rows * mp: L.page_table + rows * mp + npg] = pages
        pn[L.ctx_len + rows] = ctx
        pos = np.arange(past, ctx)
        pn[L.token_ids + t: L.token_ids + t + chunk] = rng.integers(0, eng.cfg.model.vocab, size=chunk)
        pn[L.positions + t: L.positions + t + chunk] = pos
        pn[L.slots + t: L.slots + t + chunk] = pages[pos // 16] * 16 + pos % 16
        pn[L.cu_q + j] = t - base
        pn[L.cu_q + j + 1] = t - base + chunk
        for q0 in range(((chunk - 1) // 64) * 64, -1, -64):
            pn[L.tile_seq + tiles] = j
            pn[L.tile_q0 + tiles] = q0
            tiles += 1
        pn[L.logit_rows + rows] = t + chunk - 1
        t += chunk
        rows += 1
    assert pp <= eng.num_pages, "not enough KV pages for the synthetic step"
    r = rows
    pn[L.temperature: L.temperature + r] = np.full(r, 0.7, np.float32).view(np.int32)
    pn[L.top_p: L.top_p + r] = np.full(r, 0.9, np.float32).view(np.int32)
    pn[L.uniform: L.uniform + r] = rng.random(r, dtype=np.float32).view(np.int32)
    si = eng.si
    si.num_tokens, si.num_decode, si.num_prefill_seqs, si.num_tiles, si.num_logit_rows = t, n_decode, n_prefill, tiles, r
    si.max_ctx = max(ctxs + [past + chunk])
    eng.plan_dev.copy_(eng.plan_host[: eng.dev_words])
    torch.cuda.synchronize()
    return t, sum(ctxs)


def run(eng, iters):
    si = eng.si
    r = si.num_logit_rows
    for _ in range(iters):
        logits = eng.model.forward(si, eng.kv)
        ops.sample(logits, eng.temperature[:r], eng.top_k[:r], eng.top_p[:r], eng.min_p[:r], eng.uniform[:r],
                   work=eng.sample_work, out=eng.sampled_dev[:r])


def timed(eng, iters, warmup=3):
    run(eng, warmup)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(eng, iters)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--decode", type=int, default=255)
    ap.add_argument("--prefill", type=int, default=1)
    ap.add_argument("--chunk", type=int, default=1025)
    ap.add_argument("--past", type=int, default=0)
    ap.add_argument("--min-ctx", type=int, default=129)
    ap.add_argument("--max-ctx", type=int, default=2304)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--modes", default="native,python,per-op")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    model = preset(args.model)
    if args.layers:
        model = model.replace(num_layers=args.layers)
    max_len = max(args.max_ctx, args.past + args.chunk) + 16
    cfg = EngineConfig(model=model, max_seqs=args.decode + args.prefill,
                       max_tokens_per_step=args.decode + args.prefill * args.chunk, max_seq_len=max_len,
                       prefill_chunk=args.chunk, enable_prefix_cache=False)
    eng = LLMEngine(cfg, device="cuda")
    t, kv_tokens = build_plan(eng, args.decode, args.prefill, args.chunk, args.min_ctx, args.max_ctx, args.past)
    res = {"tokens": t, "decode_rows": args.decode, "decode_kv_tokens": kv_tokens, "layers": model.num_layers}
    modes = args.modes.split(",")
    native = eng.model.native
    if "native" in modes and native:
        res["native_ms"] = round(timed(eng, args.iters), 4)
    eng.model.native = None
    if "python" in modes:
        res["python_ms"] = round(timed(eng, args.iters), 4)
    if "per-op" in modes:
        run(eng, 2)
        ops.profile_start()
        run(eng, 4)
        agg = ops.profile_stop()
        tot = sum(v[0] for v in agg.values())
        res["per_op_sum_ms"] = round(tot / 4, 4)
        res["per_op"] = {k: [round(v[0] / 4, 4), v[1] // 4] for k, v in sorted(agg.items(), key=lambda kv: -kv[1][0])}
    eng.model.native = native
    eng.check_device_status()
    print(json.dumps(res, indent=1))
    if args.json:
        open(args.json, "w").write(json.dumps(res, indent=1))


if __name__ == "__main__":
    sys.exit(main())
