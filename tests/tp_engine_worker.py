"""Worker of tests/test_tp_engine_cpu.py: loads one exported package as a tensor-parallel group through the public API
(rank 0 generates, the other ranks follow) or on a single rank, and writes rank 0's tokens."""
import os
import sys
import tempfile

import numpy as np
import torch

from onnx_genai_b200.engine.api import Engine, GenerateOptions
from onnx_genai_b200.engine.tp_driver import bootstrap
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import random_weights
from onnx_genai_b200.package.export import export_package


def _launches():
    from onnx_genai_b200 import ops

    return {k: v for k, v in ops.launch_counts.items() if v}


def main():
    out_path = sys.argv[1]
    dev_kind = "cpu" if os.environ.get("OGB_TEST_DEVICE") == "cpu" or not torch.cuda.is_available() else "cuda"
    rank, world, dev, comm = bootstrap(dev_kind)
    if dev.type == "cuda":          # shapes the CUDA kernels take (head dim 64, tile-sized widths); bf16 shards
        cfg = DecoderConfig(name="tpe", num_layers=3, hidden=512, num_heads=8, num_kv_heads=2, head_dim=64, intermediate=1024, vocab=2048,
                            rope_theta=1e6, tie_embeddings=False, qkv_bias=True, max_position=1024)
        std = 0.05
    else:
        cfg = DecoderConfig(name="tpe", num_layers=2, hidden=256, num_heads=8, num_kv_heads=2, head_dim=32, intermediate=512, vocab=512,
                            rope_theta=1e4, tie_embeddings=False, qkv_bias=True, max_position=256)
        std = 0.3
    with tempfile.TemporaryDirectory() as tmp:                  # every rank writes the same seeded package for itself
        export_package(cfg, random_weights(cfg, "cpu", seed=3, std=std, dtype=torch.float32), tmp, dtype="fp32", int4=False)
        eng = Engine.from_dir(tmp, device=str(dev), max_seqs=4, max_seq_len=128, num_pages=64, tp=world, tp_rank=rank, comm=comm)
    if rank != 0:
        steps = eng.follow()
        assert steps > 0
    else:
        rng = np.random.default_rng(5)
        prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (5, 33, 18)]
        greedy = eng.generate_batch(prompts, GenerateOptions(max_new_tokens=10, greedy=True, ignore_eos=True))
        sampled = eng.generate(prompts[0], GenerateOptions(max_new_tokens=8, temperature=0.8, top_p=0.9, seed=7, ignore_eos=True))
        streamed = [t for t, _d, _f in eng.generate_stream(prompts[1], GenerateOptions(max_new_tokens=6, greedy=True, ignore_eos=True))]
        refused = ""
        if world > 1:
            try:
                eng.generate(prompts[0], GenerateOptions(max_new_tokens=4, greedy=True, logprobs=2))
            except ValueError as exc:
                refused = str(exc)
        eng.shutdown()
        torch.save({"greedy": [r.token_ids for r in greedy], "sampled": sampled.token_ids, "streamed": streamed, "refused": refused,
                    "world": world, "steps": eng.llm.steps, "device": str(dev),
                    "comm": type(comm).__name__ if comm is not None else "", "launches": dict(_launches())}, out_path)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
