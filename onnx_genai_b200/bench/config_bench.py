"""End-to-end runs of the secondary benchmark configurations through the public ``Engine`` API.

``--config 1``  tiny Llama-style decoder on CPU (4 layers, hidden 256, 8/2 heads of 32, intermediate 688, vocab
                32000, tied embeddings), every linear layer MatMulNBits int4 block 32 with fp32 scales, exported
                as an ONNX package, loaded back, batch of 4 prompts x 32 random tokens, 64 greedy tokens each,
                fp32 activations.  Also checks that the C++ kernels and the PyTorch statements produce the same
                tokens.
``--config 2``  Qwen2.5-0.5B-shape int4 (bf16 scales) on one GPU: prompts of 512 random tokens, 256 greedy output
                tokens, batch sizes 1..64.

Each prints one JSON line.  Weights are seeded N(0, 0.02); prompts are uniform-random token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

import numpy as np
import torch


def _export(preset_name: str, out_dir: str, scale_dtype: str, layers: int = 0):
    from onnx_genai_b200.models.config import preset
    from onnx_genai_b200.models.decoder import random_weights
    from onnx_genai_b200.package.export import export_package

    cfg = preset(preset_name)
    if layers:
        cfg = cfg.replace(num_layers=layers)
    w = random_weights(cfg, "cpu", seed=0, dtype=torch.float32)
    export_package(cfg, w, out_dir, dtype="fp32", int4=True, scale_dtype=scale_dtype)
    return cfg


def config1(args) -> dict:
    from onnx_genai_b200.engine.api import Engine, GenerateOptions
    from onnx_genai_b200.ops import cpu

    with tempfile.TemporaryDirectory() as tmp:
        cfg = _export("tiny-llama", tmp, "fp32")
        rng = np.random.default_rng(0)
        prompts = [rng.integers(0, cfg.vocab, size=32).tolist() for _ in range(4)]
        opt = GenerateOptions(max_new_tokens=64, greedy=True, ignore_eos=True)
        runs = {}
        for mode in ("int4-kernels", "dense"):
            eng = Engine.from_dir(tmp, device="cpu", max_seqs=4, max_seq_len=128, keep_int4=(mode == "int4-kernels"))
            eng.generate_batch(prompts, GenerateOptions(max_new_tokens=4, greedy=True, ignore_eos=True))   # warm-up
            best = None
            for _ in range(args.repeats):
                t0 = time.perf_counter()
                res = eng.generate_batch(prompts, opt)
                dt = time.perf_counter() - t0
                best = dt if best is None else min(best, dt)
            runs[mode] = {"tokens": [r.token_ids for r in res], "s": best}
        same = sum(a == b for a, b in zip(runs["int4-kernels"]["tokens"], runs["dense"]["tokens"]))
        out_tokens = 4 * 64
        return {"config": 1, "metric": "output tok/s (tiny Llama int4 on CPU, batch 4 x 32 prompt x 64 new, greedy, fp32)",
                "value": round(out_tokens / runs["int4-kernels"]["s"], 1), "unit": "tok/s",
                "dense_weights_tok_s": round(out_tokens / runs["dense"]["s"], 1),
                "cpp_kernels": cpu.available(), "cpp_kernel_calls": dict(cpu.calls),
                "sequences_identical_between_int4_kernels_and_dense": f"{same}/4",
                "threads": torch.get_num_threads(), "data": "synthetic"}


def config2(args) -> dict:
    from onnx_genai_b200 import ops
    from onnx_genai_b200.engine.api import Engine, GenerateOptions

    with tempfile.TemporaryDirectory() as tmp:
        cfg = _export("qwen2.5-0.5b", tmp, "bf16", layers=args.layers)
        rng = np.random.default_rng(0)
        rows = []
        for batch in args.batches:
            eng = Engine.from_dir(tmp, device="cuda", max_seqs=batch, max_seq_len=512 + 256 + 16,
                                  max_tokens_per_step=max(2048, batch + 512))
            prompts = [rng.integers(0, cfg.vocab, size=512).tolist() for _ in range(batch)]
            eng.generate_batch(prompts[:1], GenerateOptions(max_new_tokens=4, greedy=True, ignore_eos=True))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = eng.generate_batch(prompts, GenerateOptions(max_new_tokens=256, greedy=True, ignore_eos=True))
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            ttft = float(np.median([r.ttft_s for r in res]))
            decode = sum(r.completion_tokens - 1 for r in res) / max(dt - ttft, 1e-9)
            rows.append({"batch": batch, "output_tok_s": round(sum(r.completion_tokens for r in res) / dt, 1),
                         "decode_tok_s": round(decode, 1), "ttft_ms_p50": round(ttft * 1e3, 2)})
            del eng
            torch.cuda.empty_cache()
        ops.check_status()
        return {"config": 2, "metric": "output tok/s (Qwen2.5-0.5B-shape int4, 512-token prompts, 256 greedy tokens)",
                "rows": rows, "layers": args.layers or cfg.num_layers, "launches": dict(ops.launch_counts), "data": "synthetic"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=1, choices=[1, 2])
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--batches", type=int, nargs="+", default=[1, 8, 64])
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (the result is then not a config-2 number)")
    args = ap.parse_args(argv)
    res = config1(args) if args.config == 1 else config2(args)
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
