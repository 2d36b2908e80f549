"""Worker for the tensor-parallel GPU tests (launched by torch.distributed.run, one rank per GPU)."""
import json
import os
import sys

import numpy as np
import torch

from onnx_genai_b200 import ops
from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.parallel import comm as comm_mod


def comm_api(comm, rank, world, dev, out_path):
    """Variable-size exchange, point-to-point ring and token-sharded expert dispatch over the process group."""
    from onnx_genai_b200.parallel.ep_dispatch import EpDispatcher

    counts = [rank + d + 1 for d in range(world)]
    rows = torch.tensor([[rank, d] for d in range(world) for _ in range(counts[d])], dtype=torch.int64, device=dev)
    recv = comm.exchange_counts(counts)
    got = comm.all_to_all_v(rows, counts, recv)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    token = torch.tensor([float(rank)], device=dev)
    inbox = torch.zeros(1, device=dev)
    if rank % 2 == 0:
        comm.send(token, nxt)
        comm.recv(inbox, prv)
    else:
        comm.recv(inbox, prv)
        comm.send(token, nxt)
    torch.manual_seed(0)
    experts, hid, k, t_per = 3 * world, 16, 2, 9
    w_exp = (torch.randn(experts, hid, hid) * 0.2).to(dev)
    hidden = torch.randn(world, t_per, hid).to(dev)
    ids = torch.stack([torch.stack([torch.randperm(experts)[:k] for _ in range(t_per)]) for _ in range(world)]).to(dev)
    wts = torch.rand(world, t_per, k).to(dev)
    d = EpDispatcher(comm, experts)
    base = rank * d.per_rank
    mine = d.run(hidden[rank], ids[rank], wts[rank], lambda x, e: torch.tanh(x @ w_exp[base + e]))
    dense = torch.zeros(t_per, hid, device=dev)
    for i in range(t_per):
        for j in range(k):
            dense[i] += wts[rank, i, j] * torch.tanh(hidden[rank, i] @ w_exp[ids[rank, i, j]])
    ok = torch.tensor([float(torch.allclose(mine, dense, atol=1e-5))], device=dev)
    comm.all_reduce(ok)
    if rank == 0:
        torch.save({"backend": comm.backend_name, "recv": recv, "rows": got.cpu().tolist(), "ring": float(inbox.item()),
                    "ep_ok": int(ok.item()), "world": world}, out_path)


def main():
    mode, out_path = sys.argv[1], sys.argv[2]
    on_cpu = os.environ.get("OGB_TEST_DEVICE") == "cpu" or not torch.cuda.is_available()
    rank, world, local_rank = comm_mod.init_distributed("gloo" if on_cpu else None)
    dev = torch.device("cpu") if on_cpu else torch.device("cuda", local_rank)
    if not on_cpu:
        torch.cuda.set_device(dev)
    cfg = DecoderConfig(name="tp", num_layers=3, hidden=512, num_heads=8, num_kv_heads=2, head_dim=64, intermediate=1024,
                        vocab=2048, rope_theta=1e6, tie_embeddings=False, qkv_bias=True, max_position=1024)
    if mode.endswith("-moe"):
        from onnx_genai_b200.models.config import MoEConfig

        mode = mode[: -len("-moe")]
        cfg = cfg.replace(name="tp-moe", intermediate=0, moe=MoEConfig(num_experts=8, top_k=2, expert_intermediate=256, renormalize=True))
    comm = comm_mod.NcclComm() if world > 1 else None
    if mode == "comm-api":
        return comm_api(comm, rank, world, dev, out_path)
    if mode.startswith("fused") and world > 1:
        from onnx_genai_b200.parallel.fused import FusedComm

        comm = FusedComm(comm, dev)
    pipeline = mode == "pp" and world > 1
    eng = LLMEngine(EngineConfig(model=cfg, num_pages=256, max_seqs=16, max_tokens_per_step=512, max_seq_len=512,
                                 seed=21, native_executor=(mode != "fused-py")), device=dev, tp=1 if pipeline else world, rank=rank,
                    comm=comm, pp=world if pipeline else 1)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab, size=n).astype(np.int32) for n in (3, 64, 97, 200)]
    for p in prompts:
        eng.add_request(p, 12)
    eng.step()
    n = len(prompts)
    if pipeline:
        # only the last stage has logits; every stage must hold its own layers' weights and KV pools and nothing else
        import torch.distributed as dist

        lo, hi = eng.stage_plan.ranges[rank]
        assert [i for i, l in enumerate(eng.weights.layers) if l is not None] == list(range(lo, hi))
        assert [i for i, p in enumerate(eng.kv.pools) if p is not None] == list(range(lo, hi))
        shares = [None] * world
        dist.all_gather_object(shares, eng.model.logits[:n].float().cpu().clone() if rank == world - 1 else None)
        logits = shares[world - 1]
    elif world > 1 and eng._shard_rows(n):
        # each rank ran lm_head for its share of the rows only: collect the shares in rank order
        import torch.distributed as dist

        chunk = (n + world - 1) // world
        n_loc = max(0, min(n, (rank + 1) * chunk) - rank * chunk)
        shares = [None] * world
        dist.all_gather_object(shares, eng.model.logits[:n_loc].float().cpu().clone())
        logits = torch.cat(shares)[:n]
    else:
        logits = eng.model.logits[:n].float().cpu().clone()      # on CPU .float().cpu() aliases the static buffer
    toks = []
    while eng.has_work:
        toks += [(sid, tok) for sid, tok, _ in eng.step().events]
    if not on_cpu:
        torch.cuda.synchronize()
        ops.check_status()
    gathered = [None] * world
    if world > 1:
        import torch.distributed as dist

        dist.all_gather_object(gathered, toks)
        assert all(g == gathered[0] for g in gathered), "ranks diverged"
    if rank == 0:
        torch.save({"logits": logits, "tokens": toks, "launches": dict(ops.launch_counts),
                    "backend": getattr(comm, "backend_name", "none")}, out_path)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
