"""End-to-end runs of the secondary benchmark configurations through the public ``Engine`` API.

``--config 1``  tiny Llama-style decoder on CPU (4 layers, hidden 256, 8/2 heads of 32, intermediate 688, vocab
                32000, tied embeddings), every linear layer MatMulNBits int4 block 32 with fp32 scales, exported
                as an ONNX package, loaded back, batch of 4 prompts x 32 random tokens, 64 greedy tokens each,
                fp32 activations.  Also checks that the C++ kernels and the PyTorch statements produce the same
                tokens.
``--config 2``  Qwen2.5-0.5B-shape int4 (bf16 scales) on one GPU: prompts of 512 random tokens, 256 greedy output
                tokens, batch sizes 1..64.

``--config 5``  long-context speculative decoding (see :func:`config5`); run under torchrun for TP > 1.

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
            wbytes = 0                                   # device bytes of the int4 projections (a bf16 copy would show here)
            for lw in eng.llm.weights.layers:
                for lin in (lw.quant or {}).values():
                    for one in (lin if isinstance(lin, (list, tuple)) else [lin]):
                        if hasattr(one, "device_weight_bytes"):
                            wbytes += one.device_weight_bytes()
            rows.append({"batch": batch, "output_tok_s": round(sum(r.completion_tokens for r in res) / dt, 1),
                         "decode_tok_s": round(decode, 1), "ttft_ms_p50": round(ttft * 1e3, 2),
                         "int4_projection_device_bytes": int(wbytes)})
            del eng
            torch.cuda.empty_cache()
        ops.check_status()
        return {"config": 2, "metric": "output tok/s (Qwen2.5-0.5B-shape int4, 512-token prompts, 256 greedy tokens)",
                "rows": rows, "layers": args.layers or cfg.num_layers, "launches": dict(ops.launch_counts), "data": "synthetic"}


def config5(args) -> dict:
    """Long-context speculative decoding: Qwen2.5-7B-shape target (TP = world size), Qwen2.5-0.5B-shape draft
    replicated on every rank, 4 draft tokens per step with greedy verification and KV rewind, fp8 e4m3 KV pages
    with per-(page, head) scales, `--prompt-len` random prompt tokens and `--output-tokens` new tokens per
    sequence, batch `--batch`.  Run under torchrun for TP > 1.  With random weights the draft and the target
    agree only by chance, so accepted tokens per step stays near its floor of 1 (the bonus token)."""
    from onnx_genai_b200 import ops
    from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
    from onnx_genai_b200.models.config import preset
    from onnx_genai_b200.parallel import comm as comm_mod
    from onnx_genai_b200.speculative import DraftModelProposer, NgramProposer

    on_gpu = args.device != "cpu"
    rank, world, local_rank = comm_mod.init_distributed() if on_gpu else (0, 1, 0)
    dev = torch.device("cuda", local_rank) if on_gpu else torch.device("cpu")
    if on_gpu:
        torch.cuda.set_device(dev)
    comm = None
    if world > 1:
        comm = comm_mod.NcclComm()
        try:
            from onnx_genai_b200.parallel.fused import FusedComm

            comm = FusedComm(comm, dev)
        except Exception as exc:
            print(f"fused communicator unavailable ({exc}); using NCCL", file=sys.stderr)
    target_cfg = preset("qwen2.5-7b")
    # the draft takes the target's vocabulary (the target's tokens are its inputs)
    draft_cfg = preset("qwen2.5-0.5b").replace(weight_format="bf16", vocab=target_cfg.vocab)
    if args.layers:
        target_cfg, draft_cfg = target_cfg.replace(num_layers=args.layers), draft_cfg.replace(num_layers=max(1, args.layers // 2))
    k = args.draft_tokens
    max_len = args.prompt_len + args.output_tokens + 32
    target = LLMEngine(EngineConfig(model=target_cfg.replace(max_position=max(target_cfg.max_position, max_len)), max_seqs=args.batch,
                                    max_tokens_per_step=2048 + args.batch * (k + 1), max_seq_len=max_len, prefill_chunk=2048,
                                    kv_dtype="fp8" if on_gpu else "bf16", max_draft_tokens=k, enable_prefix_cache=False, seed=0),
                       device=dev, tp=world, rank=rank, comm=comm)
    draft = None
    if args.proposer == "draft":
        draft = LLMEngine(EngineConfig(model=draft_cfg.replace(max_position=max(draft_cfg.max_position, max_len)), max_seqs=args.batch,
                                       max_tokens_per_step=2048 + args.batch, max_seq_len=max_len, prefill_chunk=2048,
                                       enable_prefix_cache=True, seed=1), device=dev)
    rng = np.random.default_rng(0)
    sids = []
    for _ in range(args.batch):
        ids = rng.integers(0, target_cfg.vocab, size=args.prompt_len, dtype=np.int64).astype(np.int32)
        sid = target.add_request(ids, args.output_tokens, temperature=0.0, ignore_eos=True)
        target.proposers[sid] = DraftModelProposer(draft) if draft is not None else NgramProposer()
        sids.append(sid)
    if on_gpu:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    first = {}
    produced = 0
    steps = decode_steps = 0
    t_prefill_done = None
    while target.has_work:
        out = target.step()
        steps += 1
        for sid, tok, fin in out.events:
            produced += 1
            first.setdefault(sid, time.perf_counter() - t0)
        if t_prefill_done is None and len(first) == args.batch:
            t_prefill_done = time.perf_counter()
        elif t_prefill_done is not None:
            decode_steps += 1
    if on_gpu:
        torch.cuda.synchronize()
    t1 = time.perf_counter()
    target.check_device_status()
    core = target.core
    decode_s = t1 - (t_prefill_done or t0)
    decode_tokens = produced - args.batch
    res = {"config": 5, "metric": "output tok/s (long-context speculative decode, Qwen2.5-7B-shape target + 0.5B-shape draft, fp8 KV)",
           "value": round(decode_tokens / max(decode_s, 1e-9), 1), "unit": "tok/s (decode phase, all sequences)",
           "n_gpus": world, "batch": args.batch, "prompt_len": args.prompt_len, "output_tokens": args.output_tokens,
           "draft_tokens": k, "proposer": args.proposer, "kv": "fp8 e4m3 pages, per-(page, head) scales" if on_gpu else "bf16 pages (CPU smoke run)",
           "accepted_tokens_per_step": round(decode_tokens / max(1, decode_steps) / args.batch, 3),
           "spec_steps": int(core.spec_steps), "spec_proposed": int(core.spec_proposed), "spec_accepted": int(core.spec_accepted),
           "ttft_s_p50": round(float(np.median(list(first.values()))), 2), "prefill_tok_s": round(args.batch * args.prompt_len / max((t_prefill_done or t1) - t0, 1e-9), 1),
           "total_s": round(t1 - t0, 2), "engine_steps": steps, "layers": args.layers or target_cfg.num_layers,
           "launches": {k2: v for k2, v in ops.launch_counts.items() if "fp8" in k2 or "spec" in k2 or "scatter" in k2}, "data": "synthetic"}
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return res if rank == 0 else None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=1, choices=[1, 2, 5])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=32768)
    ap.add_argument("--output-tokens", type=int, default=512)
    ap.add_argument("--draft-tokens", type=int, default=4)
    ap.add_argument("--proposer", default="draft", choices=["draft", "ngram"])
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"], help="config 5 only: cpu runs a smoke check with bf16 KV")
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--batches", type=int, nargs="+", default=[1, 8, 64])
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (the result is then not a config-2 number)")
    args = ap.parse_args(argv)
    res = {1: config1, 2: config2, 5: config5}[args.config](args)
    if res is not None:
        print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
