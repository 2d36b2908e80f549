"""Headline benchmark: continuous-batching output tokens/s on the Qwen2.5-7B shape, TP = --gpus.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload: a closed loop of 256 concurrent requests; prompts of uniform-random token ids with
lengths uniform in 128..2048; 256 output tokens each (EOS ignored); temperature 0.7, top-p 0.9;
paged KV with 16-token bf16 pages; bf16 weights drawn N(0, 0.02).  Requests enter at the
steady-state rate (one per engine step) until 256 are in flight; from then on a finished request
is replaced at once, so every step mixes ~250 decode rows with the prefill chunk of a new
prompt.  A "step" is one engine step (schedule + forward + sample + commit).

Two timed regions, both after the ramp and W warm-up steps:
  e2e     K steps through the public API (LLMEngine.step): each step builds the plan in pinned
          host memory, copies it to the device, runs the kernels, and reads the sampled tokens
          back.  Wall clock bracketed by barrier + synchronize.
  device  the same K steps replayed from their recorded device-resident plans (forward +
          sampler only; no host scheduling, no copies), timed with CUDA events.  `value` and
          `ms_per_step` come from here.  Inputs per step (15 GB of weights / TP + KV pages) are far
          larger than the 126 MB L2, so no explicit L2 flush is issued between steps.
Multi-GPU numbers take the max over ranks of the elapsed time.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

BASELINE_CONTEXT = {"qwen2.5-7b int4 batch-1 decode tok/s on 1xH200 (reference native CUDA EP)": 308.34}


def reference_arm(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference is a Rust workspace (cargo/rustc/maturin absent offline; `pip install` of the reference tree "
                       "reports 'neither setup.py nor pyproject.toml', its Python crate needs maturin) and it has no "
                       "multi-GPU or NCCL path at all",
    }))
    return 0


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self, t0, t1):
        rows = [r for ts, r in self.rows if t0 <= ts <= t1 and len(r) >= 9] or [r for _, r in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in rows if r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in rows:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(rows)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--output-tokens", type=int, default=256)
    ap.add_argument("--greedy", action="store_true", help="greedy decoding instead of temperature 0.7 / top-p 0.9 (the MoE config)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--comm", default="auto", choices=["auto", "nccl", "fused"])
    ap.add_argument("--tp", type=int, default=0,
                    help="tensor-parallel degree (0 = all GPUs, the headline layout); with a smaller value the GPUs form --gpus / --tp "
                         "replicas that share the concurrent requests, each with its own engine (a deployment layout, labelled in the output)")
    ap.add_argument("--token-multiple", type=int, default=128,
                    help="the scheduler trims the last prefill chunk so a step's token count is a multiple of this (GEMM M tile)")
    ap.add_argument("--deadline", type=int, default=900, help="seconds after which a stuck run dumps stacks and exits")
    ap.add_argument("--no-native-executor", action="store_true", help="drive the layer stack from Python (for op profiling)")
    ap.add_argument("--profile-gpu", default="", help="after the timed regions and the latency sample, replay the recorded steps once more under "
                    "the CUPTI activity collector and write the per-kernel device-time table (JSON) here; the bench line is not affected")
    ap.add_argument("--profile-ops", action="store_true", help="after the timed regions, replay 4 steps with per-op CUDA-event timing (stderr)")
    ap.add_argument("--no-anchor", action="store_true",
                    help="skip the labelled library arm (cuBLAS GEMMs + ncclAllReduce) that is replayed on the same steps for vs_baseline")
    ap.add_argument("--latency-requests", type=int, default=256,
                    help="after the timed regions keep the closed loop running until this many requests have finished (TTFT / TPOT sample)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)
    # stdout carries exactly one JSON line: anything libraries print (NCCL's version banner, torchrun
    # notices) is sent to stderr by pointing fd 1 at fd 2 and keeping a private handle on the real stdout
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    # a rank that stops making progress (a peer died, a collective never completes) must not hold the
    # GPUs forever: dump the stacks and exit after the deadline
    import faulthandler

    faulthandler.dump_traceback_later(args.deadline, exit=True)

    import numpy as np
    import torch

    from onnx_genai_b200 import ops
    from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
    from onnx_genai_b200.models.config import preset
    from onnx_genai_b200.parallel import comm as comm_mod

    rank, world, local_rank = comm_mod.init_distributed()
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run", file=sys.stderr)
        if world == 1 and args.gpus > 1:
            return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.impl == "baseline":
        os.environ["OGB_BASELINE"] = "1"
        ops.set_baseline(True)
    model = preset(args.model)
    # Replicas x tensor parallelism: rank r is rank r % tp of replica r // tp.  Every replica runs its own engine over its
    # own share of the concurrent requests; the timed regions are bracketed by barriers over all ranks.
    tp = args.tp if args.tp > 0 else world      # the headline metric is tensor parallelism over all GPUs; --tp asks for replicas
    if world % tp or args.concurrency % (world // tp):
        if rank == 0:
            print(f"bench.py: --tp {tp} does not divide {world} GPUs, or {world // tp} replicas do not divide {args.concurrency} requests", file=sys.stderr)
        return 2
    dp, replica, tp_rank = world // tp, rank // tp, rank % tp
    wcomm = comm_mod.NcclComm() if world > 1 else None          # all ranks: barriers and the reductions of the report
    args.concurrency //= dp
    args.latency_requests = (args.latency_requests + dp - 1) // dp
    comm = None
    if tp > 1:
        comm = wcomm
        if dp > 1:
            import torch.distributed as dist

            groups = [dist.new_group(ranks=list(range(g * tp, (g + 1) * tp))) for g in range(dp)]   # every rank creates every group
            comm = comm_mod.NcclComm(groups[replica])
        if args.comm in ("auto", "fused") and args.impl == "ours":
            try:
                from onnx_genai_b200.parallel.fused import FusedComm

                comm = FusedComm(comm, dev)
            except Exception as exc:  # stays on the NCCL path and says so
                if rank == 0:
                    print(f"bench.py: fused communicator unavailable ({exc}); using NCCL", file=sys.stderr)

    invalid = None
    if args.layers:
        model = model.replace(num_layers=args.layers)
        invalid = "reduced layer count (debug)"
    max_len = args.max_prompt + args.output_tokens
    cfg = EngineConfig(model=model, max_seqs=args.concurrency, max_tokens_per_step=args.concurrency + args.max_prompt,
                       max_seq_len=max_len, prefill_chunk=args.max_prompt, enable_prefix_cache=False, seed=0,
                       token_multiple=args.token_multiple,
                       native_executor=not (args.no_native_executor or args.profile_ops),
                       sync_sampled_tokens=True)
    eng = LLMEngine(cfg, device=dev, tp=tp, rank=tp_rank, comm=comm)
    rng = np.random.default_rng(1234 + replica)  # same stream on every rank of a replica: they schedule identically

    def new_request():
        n = int(rng.integers(args.min_prompt, args.max_prompt + 1))
        ids = rng.integers(0, model.vocab, size=n, dtype=np.int64).astype(np.int32)
        return eng.add_request(ids, args.output_tokens, temperature=0.0 if args.greedy else 0.7, top_p=1.0 if args.greedy else 0.9,
                               seed=int(rng.integers(1, 2**31)),
                               ignore_eos=True)

    active = 0
    finished_ids = []

    def one_step():
        nonlocal active
        out = eng.step()
        for sid, tok, fin in out.events:
            if fin is not None:
                active -= 1
                finished_ids.append(sid)
        return out

    # ---- ramp: one admission per step until the batch is full and requests have started to turn over ----
    t_ramp = time.perf_counter()
    ramp_steps = 0
    admitted = 0
    while not finished_ids:
        if admitted < args.concurrency:
            new_request()
            admitted += 1
            active += 1
        one_step()
        ramp_steps += 1
        if ramp_steps > 4 * (args.concurrency + args.output_tokens):
            break

    def closed_loop_step():
        nonlocal active
        while active < args.concurrency:
            new_request()
            active += 1
        return one_step()

    for _ in range(args.warmup):
        closed_loop_step()
    eng.check_device_status()
    ramp_s = time.perf_counter() - t_ramp

    # ---- region 1: end to end through the public API ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    plans = torch.empty(args.steps, eng.dev_words, dtype=torch.int32, device=dev)
    shapes = []
    launches0 = sum(ops.launch_counts.values())
    h2d0, d2h0 = eng.h2d_bytes, eng.d2h_bytes
    if wcomm is not None:
        wcomm.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_tokens = 0
    for i in range(args.steps):
        out = closed_loop_step()
        e2e_tokens += len(out.events)
        plans[i].copy_(eng.plan_dev)   # device-to-device record for region 2 (tiny; part of neither claim)
        si = eng.si
        shapes.append((si.num_tokens, si.num_decode, si.num_prefill_seqs, si.num_tiles, si.num_logit_rows, si.max_ctx,
                       eng.model.decode_splits))
    if wcomm is not None:
        wcomm.barrier()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    e2e_s = t1 - t0
    launches_e2e = sum(ops.launch_counts.values()) - launches0
    h2d = (eng.h2d_bytes - h2d0) / args.steps
    d2h = (eng.d2h_bytes - d2h0) / args.steps

    # ---- region 2: the same K steps, kernels only, from device-resident plans ----
    def replay(i):
        eng.plan_dev.copy_(plans[i])
        si = eng.si
        (si.num_tokens, si.num_decode, si.num_prefill_seqs, si.num_tiles, si.num_logit_rows, si.max_ctx, splits) = shapes[i]
        if splits != eng.model.decode_splits:
            eng.model.set_decode_splits(splits)
        si.verify_table = si.verify_ctx = None      # per-step state of the live engine does not apply to a replayed plan
        si.force_python = False
        r = si.num_logit_rows
        if r and eng._shard_rows(r):       # TP: the engine's own split of the lm_head + sampler rows, tokens all-gathered
            eng.forward_and_sample_sharded(si, r, args.greedy)
            return
        logits = eng.model.forward(si, eng.kv)
        if r:
            if args.greedy:
                ops.argmax(logits, out=eng.sampled_dev[:r])
            else:
                ops.sample(logits, eng.temperature[:r], eng.top_k[:r], eng.top_p[:r], eng.min_p[:r], eng.uniform[:r],
                           work=eng.sample_work, out=eng.sampled_dev[:r])

    for i in range(min(3, args.steps)):
        replay(i)
    if wcomm is not None:
        wcomm.barrier()
    torch.cuda.synchronize()
    launches1 = sum(ops.launch_counts.values())
    tp_counts0 = (eng.model.native_counter(1), eng.model.native_counter(2), ops.launch_counts["gemm_bf16_scatter"],
                  ops.launch_counts["tp_exchange_norm"])
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    td0 = time.perf_counter()
    ev0.record()
    for i in range(args.steps):
        replay(i)
    ev1.record()
    if wcomm is not None:
        wcomm.barrier()
    torch.cuda.synchronize()
    td1 = time.perf_counter()
    dev_ms = ev0.elapsed_time(ev1)
    launches_dev = sum(ops.launch_counts.values()) - launches1
    tp_counts1 = (eng.model.native_counter(1), eng.model.native_counter(2), ops.launch_counts["gemm_bf16_scatter"],
                  ops.launch_counts["tp_exchange_norm"])
    sampler.stop()
    eng.check_device_status()

    # ---- labelled baseline arm on the same recorded steps: library GEMMs (torch.matmul -> cuBLAS, unfused epilogues),
    # ncclAllReduce for the row-parallel projections, stand-alone RMSNorm; attention and sampler stay this repo's kernels
    # (no library kernel reads this page layout).  Driven op by op from Python, timed on the device like region 2. ----
    base_ms = None
    if args.impl == "ours" and not args.no_anchor:
        m = eng.model
        saved = (m.fused_comm, m.comm, m.native)
        try:
            ops.set_baseline(True)
            m.fused_comm, m.native = None, None
            if tp > 1:
                m.comm = getattr(comm, "base", comm)
            for i in range(min(3, args.steps)):
                replay(i)
            if wcomm is not None:
                wcomm.barrier()
            torch.cuda.synchronize()
            b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b0.record()
            for i in range(args.steps):
                replay(i)
            b1.record()
            if wcomm is not None:
                wcomm.barrier()
            torch.cuda.synchronize()
            base_ms = b0.elapsed_time(b1)
        finally:
            ops.set_baseline(False)
            m.fused_comm, m.comm, m.native = saved
        if wcomm is not None:
            base_ms = wcomm.max_float(base_ms)
        eng.check_device_status()

    # ---- latency sample: requests that arrive after the timed regions (the replays above stretch the wall-clock gaps of
    # the requests that were in flight), run until enough of them have finished ----
    extra_steps = 0
    t_lat0 = time.perf_counter()
    lat_done = 0
    seen = len(finished_ids)
    while lat_done < args.latency_requests and extra_steps < 3 * (args.output_tokens + args.latency_requests):
        closed_loop_step()
        extra_steps += 1
        for sid in finished_ids[seen:]:
            if eng.stats[sid].arrival >= t_lat0:
                lat_done += 1
        seen = len(finished_ids)
    eng.check_device_status()
    if args.profile_ops:
        # every rank replays (the steps contain collectives); rank 0 reports
        n_prof = min(4, args.steps)
        ops.profile_start()
        for i in range(n_prof):
            replay(i)
        agg = ops.profile_stop()
        tot = sum(t for t, _ in agg.values())
    if args.profile_ops and rank == 0:
        print("per-op device time over %d replayed steps (ms per step, calls per step, share):" % n_prof, file=sys.stderr)
        for name, (t, c) in sorted(agg.items(), key=lambda kv: -kv[1][0]):
            print("  %-44s %8.3f ms %6.1f calls %5.1f%%" % (name, t / n_prof, c / n_prof, 100 * t / tot), file=sys.stderr)
        print("  %-44s %8.3f ms" % ("sum", tot / n_prof), file=sys.stderr)
        try:      # findings (what / why / how) over the same table, with the cost model's FLOPs and bytes per part
            from onnx_genai_b200.utils import diagnose as _dg
            from onnx_genai_b200.utils.cost_model import StepShape

            sh = shapes[0]
            shape_ = StepShape(decode_rows=int(sh[1]), prefill_tokens=int(sh[0]) - int(sh[1]), mean_context=(args.min_prompt + args.max_prompt) // 2 + args.output_tokens // 2,
                               prefill_context=(args.min_prompt + args.max_prompt) // 4)
            print(_dg.diagnose_samples(_dg.samples_from_profile(agg, model, shape_, tp=tp, steps=n_prof), steps=n_prof).report(), file=sys.stderr)
        except Exception as exc:   # the diagnosis is a convenience: never let it break the bench line
            print(f"diagnosis skipped: {exc}", file=sys.stderr)

    if args.profile_gpu:
        # every rank replays (the steps contain collectives); rank 0 collects.  Through the same executor as the timed
        # region, so the table is the kernel-level breakdown of `ms_per_step` (plus CUPTI's own cost per launch).
        from onnx_genai_b200.utils.gpu_activity import GpuActivityCollector, short_name

        gpu = None
        if rank == 0:
            try:
                gpu = GpuActivityCollector(copies=True).start()
            except Exception as exc:
                print(f"--profile-gpu: device activity is not collected: {exc}", file=sys.stderr)
        torch.cuda.synchronize()
        for i in range(args.steps):
            replay(i)
        torch.cuda.synchronize()
        if gpu is not None:
            gpu.stop()
            rows = [{**r, "name": short_name(r["name"]), "ms_per_step": r["total_us"] / 1e3 / args.steps, "calls_per_step": r["count"] / args.steps}
                    for r in gpu.summary()]
            busy_ms = gpu.busy_fraction() * (gpu.records[-1].end_s - gpu.records[0].start_s) * 1e3 / args.steps if gpu.records else 0.0
            with open(args.profile_gpu, "w", encoding="utf-8") as f:
                json.dump({"steps": args.steps, "device_busy_ms_per_step": busy_ms, "sum_ms_per_step": sum(r["ms_per_step"] for r in rows),
                           "dropped": gpu.dropped, "kernels": rows}, f, indent=1)
            print(gpu.table(30), file=sys.stderr)

    dev_tokens = sum(s[4] for s in shapes)
    if wcomm is not None:
        dev_ms = wcomm.max_float(dev_ms)
        e2e_s = wcomm.max_float(e2e_s)
        if dp > 1:      # tokens of all replicas: every rank of a replica holds the same count, so the sum over ranks counts it tp times
            tot = torch.tensor([float(dev_tokens), float(e2e_tokens)], dtype=torch.float64, device=dev)
            wcomm.all_reduce(tot)
            dev_tokens, e2e_tokens = float(tot[0]) / tp, float(tot[1]) / tp
    value = dev_tokens / (dev_ms / 1e3)
    e2e_value = e2e_tokens / e2e_s

    ttft, tpot = [], []
    for sid in finished_ids:
        st = eng.stats.get(sid)
        if st and st.finished and st.output_tokens > 1 and st.arrival >= t_lat0:
            ttft.append((st.first_token - st.arrival) * 1e3)
            tpot.append((st.finished - st.first_token) * 1e3 / (st.output_tokens - 1))
    clocks = sampler.summary(t0, td1)
    pct = lambda xs, q: round(float(np.percentile(xs, q)), 3) if xs else None
    base_value = dev_tokens / (base_ms / 1e3) if base_ms else None
    if rank == 0:
        result = {
            "metric": "output tok/s (%s-shape, continuous batching, %d concurrent, %s=%d)" % (
                {"qwen2.5-7b": "Qwen2.5-7B", "qwen3-30b-a3b": "Qwen3-30B-A3B"}.get(model.name, model.name), args.concurrency * dp,
                "TP=EP" if model.moe.num_experts > 0 else "TP", tp) + (" x %d replicas" % dp if dp > 1 else ""),
            "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / base_value, 4) if base_value else None, "dtype": "bf16", "data": "synthetic (uniform-random token ids, N(0,0.02) weights)",
            "impl": args.impl,
            "config": {"model": model.name + "-shape", "global_batch": args.concurrency * dp, "seq_len": f"prompt U[{args.min_prompt},{args.max_prompt}] + {args.output_tokens} out",
                       "parallelism": f"tp{tp}" + (f" x dp{dp} (each replica serves {args.concurrency} of the requests)" if dp > 1 else ""), "kv": "paged, 16-token bf16 pages", "sampling": "greedy" if args.greedy else "temperature 0.7, top-p 0.9",
                       "l2": "per-step inputs (weights + KV) exceed L2; no explicit flush",
                       "comm": getattr(comm, "backend_name", "none"),
                       "tokens_per_step_mean": round(sum(s[0] for s in shapes) / len(shapes), 1),
                       "decode_rows_mean": round(sum(s[1] for s in shapes) / len(shapes), 1),
                       "kv_pages": eng.num_pages, "ramp_steps": ramp_steps, "ramp_s": round(ramp_s, 2)},
            "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "ms_per_step": round(e2e_s * 1e3 / args.steps, 4)},
            "baseline": None if not base_value else {
                "what": "same %d recorded steps replayed on this repo's labelled library arm: torch.matmul (cuBLAS) GEMMs with unfused "
                        "epilogues, ncclAllReduce for the row-parallel projections, stand-alone RMSNorm; attention and sampler kernels "
                        "as in the product arm; device-timed, max over ranks" % args.steps,
                "value": round(base_value, 1), "unit": "tok/s", "ms_per_step": round(base_ms / args.steps, 4)},
            "latency_scope": "replica 0" if dp > 1 else "all requests",
            "tp_launches_per_step": {
                "gemm_bf16_scatter": ((tp_counts1[0] - tp_counts0[0]) + (tp_counts1[2] - tp_counts0[2])) / args.steps,
                "tp_exchange_norm": ((tp_counts1[1] - tp_counts0[1]) + (tp_counts1[3] - tp_counts0[3])) / args.steps},
            "gpu_launches": int(launches_dev),
            "gpu_launches_e2e": int(launches_e2e),
            "clocks": clocks,
            "latency": {"ttft_ms_p50": pct(ttft, 50), "ttft_ms_p99": pct(ttft, 99), "tpot_ms_p50": pct(tpot, 50),
                        "tpot_ms_p99": pct(tpot, 99), "finished_requests": len(ttft), "extra_steps": extra_steps},
            "baseline_context": BASELINE_CONTEXT,
        }
        if invalid:
            result["invalid"] = invalid
        real_stdout.write(json.dumps(result) + "\n")
        real_stdout.flush()
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
