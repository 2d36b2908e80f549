"""Row-parallel projection micro-benchmark: fused GEMM + exchange kernels against GEMM + NCCL all-reduce.

Launch with one rank per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m onnx_genai_b200.bench.tp_bench --rows 1472 --hidden 3584 --k 18944 3584

For every K (the full, unsharded reduction dimension; each rank multiplies K/TP of it) it times, with CUDA
events after warm-up and as the max over ranks:

* ``nccl``   our tcgen05 GEMM writing a partial product, ``ncclAllReduce`` over it, residual add (the baseline);
* ``fused``  ``ogb_gemm_bf16_scatter`` + ``ogb_tp_reduce_bcast`` (peer loads, or NVSwitch multicast when bound).

With ``OGB_TP_STAMPS=1`` device timestamps of the exchange kernel's first CTA (microseconds after its start: row
group complete on all ranks, own stores issued, CTA's stores issued, fence done, rows signalled, all rows
received) are printed per rank, which separates waiting for the slowest
peer from moving bytes.  The roofline printed beside each result is
``max(GEMM FLOPs / measured bf16 peak, bytes that must cross NVLink / link bandwidth)``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=1472)
    ap.add_argument("--hidden", type=int, default=3584)
    ap.add_argument("--k", type=int, nargs="+", default=[18944, 3584])
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--gemm-tflops", type=float, default=1376.4, help="measured bf16 GEMM peak used for the roofline")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="measured NVLink bandwidth per direction per GPU")
    args = ap.parse_args(argv)

    from onnx_genai_b200 import ops
    from onnx_genai_b200.parallel import comm as comm_mod
    from onnx_genai_b200.parallel.fused import FusedComm

    rank, world, local_rank = comm_mod.init_distributed()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world < 2:
        print("tp_bench needs at least 2 ranks", file=sys.stderr)
        return 2
    base = comm_mod.NcclComm()
    fc = FusedComm(base, dev, hidden=args.hidden, max_tokens=args.rows)
    rows, n = args.rows, args.hidden
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)       # larger than L2: written between iterations
    torch.manual_seed(7 + rank)
    results = []

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        base.barrier()
        torch.cuda.synchronize()
        tot = 0.0
        samples = []
        for _ in range(args.iters):
            flush.zero_()
            base.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
            samples.append(e0.elapsed_time(e1) * 1e3)
        samples.sort()
        timed.median_us = base.max_float(samples[len(samples) // 2])
        timed.max_us = base.max_float(samples[-1])
        return base.max_float(tot / args.iters * 1e3)   # microseconds, slowest rank

    for k_full in args.k:
        k = k_full // world // 64 * 64
        a = (torch.randn(rows, k, device=dev) * 0.05).bfloat16()
        w = (torch.randn(n, k, device=dev) * 0.05).bfloat16()
        part = torch.empty(rows, n, dtype=torch.bfloat16, device=dev)
        x_ref = torch.zeros(rows, n, dtype=torch.bfloat16, device=dev)

        norm_w = torch.ones(n, dtype=torch.bfloat16, device=dev)
        h_ref = torch.empty(rows, n, dtype=torch.bfloat16, device=dev)
        x_own = torch.zeros(rows, n, dtype=torch.bfloat16, device=dev)
        fc.bind_residual(x_own)

        # all three paths end with the normed activation of the next GEMM in place on every rank
        def nccl_path():
            ops.gemm(a, w, out=part)
            base.all_reduce(part)
            ops.rmsnorm(x_ref, norm_w, 1e-6, delta=part, out=h_ref)

        turn = [0]

        def fused_bcast_path():
            # replicated residual: reduce + broadcast of x by the exchange kernel, then a stand-alone norm
            turn[0] ^= 1                     # consecutive exchanges alternate between the two slots, as in a decoder layer
            fc.row_parallel(a, w, rows, slot=turn[0])
            ops.rmsnorm(fc.x[:rows], norm_w, 1e-6, out=h_ref)

        def fused_path():
            # row-sharded residual: reduce-scatter + residual + norm + all-gather in one kernel; the wait stands in for
            # the next GEMM's per-tile waits
            turn[0] ^= 1
            fc.row_parallel_norm(a, w, rows, turn[0], norm_w, 1e-6)
            fc.wait_ready(turn[0], rows)

        def gemm_only():
            ops.gemm(a, w, out=part)

        t_gemm = timed(gemm_only)
        t_nccl = timed(nccl_path)
        fc.x.zero_()
        t_bcast = timed(fused_bcast_path)
        fc.barrier()
        t_fused = timed(fused_path)
        fused_median, fused_max = timed.median_us, timed.max_us
        ops.check_status()
        flops = 2.0 * rows * n * k
        # reduce-scatter + all-gather of a [rows, n] bf16 tensor: (tp-1)/tp of it in and out, twice, per GPU
        # (the multicast path halves that: the switch adds and replicates)
        wire = rows * n * 2 * (world - 1) / world * (1 if fc.nvls else 2)
        roof_us = max(flops / (args.gemm_tflops * 1e12), wire / (args.link_gbs * 1e9)) * 1e6
        rec = {"k_per_rank": k, "rows": rows, "n": n, "tp": world, "backend": fc.backend_name, "gemm_us": round(t_gemm, 1),
               "gemm_nccl_norm_us": round(t_nccl, 1), "fused_bcast_norm_us": round(t_bcast, 1), "fused_us": round(t_fused, 1),
               "fused_median_us": round(fused_median, 1), "fused_max_us": round(fused_max, 1), "roofline_us": round(roof_us, 1),
               "fused_frac_of_roofline": round(roof_us / t_fused, 3), "nccl_frac_of_roofline": round(roof_us / t_nccl, 3)}
        if fc.dbg is not None:
            torch.cuda.synchronize()
            s = fc.dbg.cpu().tolist()
            rec["stamps_us_rank%d" % rank] = [round((s[i] - s[0]) / 1e3, 1) for i in (1, 4, 5, 6, 2, 3)]
        results.append(rec)
        if fc.dbg is not None:
            import torch.distributed as dist

            allst = [None] * world
            dist.all_gather_object(allst, rec.get("stamps_us_rank%d" % rank))
            rec["stamps_us_all_ranks"] = allst
    if rank == 0:
        for r in results:
            print(json.dumps(r))
    import torch.distributed as dist

    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
