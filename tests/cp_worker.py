"""Worker of tests/test_context_parallel_cpu.py: ring attention over gloo ranks; rank 0 gathers every rank's rows."""
import sys

import torch
import torch.distributed as dist

from onnx_genai_b200.parallel import comm as comm_mod
from onnx_genai_b200.parallel import context_parallel as cp


def model_case(out_path, rank, world, comm):
    """The whole decoder: a prompt's prefill split over the ranks against the same schedule on one rank."""
    from onnx_genai_b200.models.config import DecoderConfig
    from onnx_genai_b200.models.decoder import random_weights

    cfg = DecoderConfig(name="cp", num_layers=2, hidden=128, num_heads=4, num_kv_heads=2, head_dim=32, intermediate=256, vocab=300,
                        rope_theta=1e4, tie_embeddings=False, qkv_bias=True, max_position=256)
    w = random_weights(cfg, "cpu", seed=9, std=0.2, dtype=torch.float32)
    ids = torch.randint(0, cfg.vocab, (45,), generator=torch.Generator().manual_seed(2)).tolist()
    pos, hidden, kv = cp.context_parallel_prefill(cfg, w, ids, comm, rank, world)
    gathered = [None] * world
    dist.all_gather_object(gathered, (pos, hidden, kv))
    if rank == 0:
        _, want_hidden, want_kv = cp.context_parallel_prefill(cfg, w, ids, comm_mod.LocalComm(), 0, 1)
        got_hidden = torch.zeros_like(want_hidden)
        got_k = [torch.zeros_like(k) for k, _ in want_kv]
        got_v = [torch.zeros_like(v) for _, v in want_kv]
        for p, h, layers in gathered:
            got_hidden[p] = h
            for i, (k, v) in enumerate(layers):
                got_k[i][p], got_v[i][p] = k, v
        from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine

        eng = LLMEngine(EngineConfig(model=cfg, num_pages=32, max_seqs=2, max_tokens_per_step=64, max_seq_len=128), weights=w, device="cpu")
        first = eng.generate([ids], max_new_tokens=1)[0][0]
        torch.save({"hidden": got_hidden, "want_hidden": want_hidden, "k": got_k, "v": got_v, "want_k": [k for k, _ in want_kv],
                    "want_v": [v for _, v in want_kv], "first_cp": int((got_hidden[-1].float() @ w.lm_head.float().t()).argmax()),
                    "first_engine": first, "world": world}, out_path)
    dist.barrier()
    dist.destroy_process_group()


def main():
    out_path, mode = sys.argv[1], sys.argv[2]
    rank, world, _ = comm_mod.init_distributed("gloo")
    comm = comm_mod.NcclComm()
    if mode == "model":
        return model_case(out_path, rank, world, comm)
    torch.manual_seed(11)                                   # every rank draws the same full tensors and keeps its slice
    b, hq, hkv, t, d = 2, 6, 2, 53, 32
    q, k, v = torch.randn(b, hq, t, d), torch.randn(b, hkv, t, d), torch.randn(b, hkv, t, d)
    slices = cp.zigzag_slices(t, world) if mode.startswith("zigzag") else cp.contiguous_slices(t, world)
    window = 17 if mode.endswith("window") else 0
    mine = slices[rank]
    out, lse = cp.ring_attention(q[:, :, mine], k[:, :, mine], v[:, :, mine], mine, comm, rank, world, [len(s) for s in slices],
                                 all_positions=slices, causal=True, window=window)
    gathered = [None] * world
    dist.all_gather_object(gathered, (mine, out, lse))
    if rank == 0:
        full = torch.zeros(b, hq, t, d)
        full_lse = torch.zeros(b, hq, t)
        for pos, o, l in gathered:
            full[:, :, pos], full_lse[:, :, pos] = o, l
        torch.save({"out": full, "lse": full_lse, "q": q, "k": k, "v": v, "window": window, "world": world}, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
