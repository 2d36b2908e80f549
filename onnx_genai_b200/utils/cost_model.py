"""Roofline cost model of one engine step: what should a step take on this hardware, and where does it go.

Every operator of a decoder step is either a matrix product (bounded by tensor-core rate or by reading its weights),
attention over the paged cache (bounded by KV bytes for decode rows, by FLOPs for prefill chunks), or a row-wise
pass (bounded by activation bytes).  Given the measured rates of the device -- copy bandwidth, sustained bf16 GEMM
rate, NVLink bandwidth, the fixed cost of a launch and of a tensor-parallel exchange -- the model predicts the time of
each part and of the step, for any architecture, batch mix and tensor-parallel degree.  Per-part efficiency factors
fitted from one measured breakdown (:meth:`CostModel.calibrate`) turn the ideal into an estimate; the model and its
calibration persist as JSON.  It answers planning questions without a GPU: which tensor-parallel degree serves a
latency target, how many concurrent sequences fit a token budget, how to cost pipeline stages.

Structure follows the reference's rate-based placement cost model with JSON persistence and calibration
(crates/onnx-runtime-cost-model/src/model.rs, calibration.rs, transfer.rs).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field

PARTS = ("qkv", "o_proj", "mlp", "lm_head", "decode_attention", "prefill_attention", "rowwise", "sampler", "exchange")


@dataclass
class HardwareRates:
    hbm_gbs: float = 6446.6                # measured copy bandwidth (read + write bytes per second)
    bf16_tflops: float = 1376.4            # sustained dense GEMM rate
    nvlink_gbs: float = 770.0              # per direction per GPU
    launch_us: float = 2.5                 # fixed cost of a kernel launch in a stream of launches
    exchange_us: float = 20.0              # fence-and-signal latency of one fused reduce + broadcast
    prefill_attention_tflops: float = 200.0   # mma.sync flash attention rate of the prefill kernel
    name: str = "NVIDIA B200"

    @classmethod
    def from_measured(cls, path: str) -> "HardwareRates":
        """Rates from a measured-peaks file (keys hbm_gbs, bf16_tflops_sustained); missing keys keep the defaults."""
        with open(path, encoding="utf-8") as f:
            m = json.load(f)
        r = cls()
        r.hbm_gbs = float(m.get("hbm_gbs", r.hbm_gbs))
        r.bf16_tflops = float(m.get("bf16_tflops_sustained", m.get("bf16_tflops", r.bf16_tflops)))
        r.name = str(m.get("gpu_name", r.name))
        return r


@dataclass
class StepShape:
    decode_rows: int = 0
    prefill_tokens: int = 0
    mean_context: int = 0                  # mean KV length read by a decode row
    prefill_context: int = 0               # mean KV length a prefill token attends to (past + half its chunk)
    logit_rows: int | None = None          # default: decode rows + one per prefill sequence (approximated as decode rows + 1)
    kv_bytes: int = 2                      # bytes per stored K/V element (1 for fp8 / int8 pages)


@dataclass
class CostModel:
    rates: HardwareRates = field(default_factory=HardwareRates)
    efficiency: dict = field(default_factory=dict)    # part -> measured / ideal (>= 1 means slower than the roofline)

    # ---------------------------------------------------------------- ideal times (milliseconds)
    def _gemm_ms(self, m: int, n: int, k: int, weight_bytes_per_elem: float) -> float:
        flops = 2.0 * m * n * k
        bytes_ = n * k * weight_bytes_per_elem + 2.0 * m * (n + k)
        return max(flops / (self.rates.bf16_tflops * 1e12), bytes_ / (self.rates.hbm_gbs * 1e9)) * 1e3

    def ideal(self, cfg, shape: StepShape, tp: int = 1) -> dict:
        """Roofline time of each part of one step, in milliseconds, for one rank of a ``tp``-way group."""
        r = self.rates
        t = shape.decode_rows + shape.prefill_tokens
        wb = 2.0 if cfg.weight_format == "bf16" else 0.5 + 2.0 / cfg.int4_block
        hq, hkv = max(1, cfg.num_heads // tp), max(1, -(-cfg.num_kv_heads // tp))
        d, hid, layers = cfg.head_dim, cfg.hidden, cfg.num_layers
        out = dict.fromkeys(PARTS, 0.0)
        out["qkv"] = layers * self._gemm_ms(t, (hq + 2 * hkv) * d, hid, wb)
        out["o_proj"] = layers * self._gemm_ms(t, hid, hq * d, wb)
        if cfg.moe.num_experts:
            ei, k = cfg.moe.expert_intermediate, cfg.moe.top_k
            local = max(1, cfg.moe.num_experts // tp)
            touched = min(local, max(1, t * k // tp))                       # experts that see at least one token on this rank
            flops = 2.0 * (t * k / tp) * 3 * ei * hid
            bytes_ = touched * 3 * ei * hid * wb
            out["mlp"] = layers * max(flops / (r.bf16_tflops * 1e12), bytes_ / (r.hbm_gbs * 1e9)) * 1e3
        else:
            inter = cfg.intermediate // tp
            out["mlp"] = layers * (self._gemm_ms(t, 2 * inter, hid, wb) + self._gemm_ms(t, hid, inter, wb))
        rows = shape.logit_rows if shape.logit_rows is not None else shape.decode_rows + (1 if shape.prefill_tokens else 0)
        out["lm_head"] = self._gemm_ms(max(1, -(-rows // tp)), cfg.vocab, hid, 2.0)
        kv_token = 2 * hkv * d * shape.kv_bytes
        out["decode_attention"] = layers * shape.decode_rows * shape.mean_context * kv_token / (r.hbm_gbs * 1e9) * 1e3
        out["prefill_attention"] = layers * 4.0 * shape.prefill_tokens * shape.prefill_context * hq * d / (r.prefill_attention_tflops * 1e12) * 1e3
        # two norms, rotary + append, residual traffic: about 8 reads or writes of the [t, hidden] activations per layer
        out["rowwise"] = layers * 8.0 * t * hid * 2 / (r.hbm_gbs * 1e9) * 1e3
        out["sampler"] = 3.0 * max(1, -(-rows // tp)) * cfg.vocab * 2 / (r.hbm_gbs * 1e9) * 1e3
        if tp > 1:
            wire = 2.0 * t * hid * 2 * (tp - 1) / tp                         # reduce + broadcast of the residual rows
            out["exchange"] = layers * 2 * max(r.exchange_us * 1e-3, wire / (r.nvlink_gbs * 1e9) * 1e3)
        return out

    def estimate(self, cfg, shape: StepShape, tp: int = 1) -> dict:
        """Calibrated estimate: ideal x efficiency per part, the total, and derived rates."""
        parts = {k: v * self.efficiency.get(k, 1.0) for k, v in self.ideal(cfg, shape, tp).items()}
        total = sum(parts.values())
        floor = (cfg.num_layers * 12 + 6) * self.rates.launch_us * 1e-3       # a step cannot beat its own launch train
        total = max(total, floor)
        return {"parts_ms": parts, "total_ms": total, "output_tok_s": shape.decode_rows / total * 1e3 if total else 0.0,
                "tokens_per_s": (shape.decode_rows + shape.prefill_tokens) / total * 1e3 if total else 0.0, "tp": tp}

    # ---------------------------------------------------------------- calibration and persistence
    def calibrate(self, cfg, shape: StepShape, measured_ms: dict, tp: int = 1) -> dict:
        """Fit per-part efficiencies from one measured breakdown (part -> ms).  Parts not measured keep their factor."""
        ideal = self.ideal(cfg, shape, tp)
        for part, ms in measured_ms.items():
            if part not in ideal:
                raise KeyError(f"unknown part {part!r}; parts are {', '.join(PARTS)}")
            if ideal[part] > 0:
                self.efficiency[part] = float(ms) / ideal[part]
        return dict(self.efficiency)

    def save(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            json.dump({"version": 1, "rates": asdict(self.rates), "efficiency": self.efficiency}, f, indent=1)

    @classmethod
    def load(cls, path: str) -> "CostModel":
        with open(path, encoding="utf-8") as f:
            d = json.load(f)
        if d.get("version") != 1:
            raise ValueError(f"{path}: cost-model file version {d.get('version')!r} is not supported (expected 1)")
        return cls(rates=HardwareRates(**d["rates"]), efficiency=dict(d.get("efficiency") or {}))

    # ---------------------------------------------------------------- planning helpers
    def pick_tp(self, cfg, shape: StepShape, degrees=(1, 2, 4, 8), max_step_ms: float | None = None) -> dict:
        """Smallest tensor-parallel degree whose step meets ``max_step_ms`` (or the fastest one when none does / no target)."""
        table = {tp: self.estimate(cfg, shape, tp)["total_ms"] for tp in degrees if cfg.num_heads % tp == 0 or tp <= cfg.num_heads}
        if max_step_ms is not None:
            for tp in sorted(table):
                if table[tp] <= max_step_ms:
                    return {"tp": tp, "step_ms": table[tp], "table": table}
        best = min(table, key=table.get)
        return {"tp": best, "step_ms": table[best], "table": table}

    def layer_costs(self, cfg, shape: StepShape, tp: int = 1) -> dict:
        """Costs for a pipeline planner: per layer, plus the extras of the first and last stage."""
        est = self.estimate(cfg, shape, tp)["parts_ms"]
        per_layer = sum(est[k] for k in ("qkv", "o_proj", "mlp", "decode_attention", "prefill_attention", "rowwise", "exchange")) / cfg.num_layers
        return {"layer": per_layer, "embed": 0.0, "head": est["lm_head"] + est["sampler"]}


def main(argv=None) -> int:
    import argparse

    from ..models.config import PRESETS

    ap = argparse.ArgumentParser(description="Estimate one engine step from measured hardware rates")
    ap.add_argument("--model", default="qwen2.5-7b", choices=sorted(PRESETS))
    ap.add_argument("--decode", type=int, default=255)
    ap.add_argument("--prefill", type=int, default=1025)
    ap.add_argument("--ctx", type=int, default=1200)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json")
    ap.add_argument("--load", help="a saved cost model (rates + calibration)")
    args = ap.parse_args(argv)
    if args.load:
        cm = CostModel.load(args.load)
    else:
        cm = CostModel(HardwareRates.from_measured(args.peaks) if os.path.exists(args.peaks) else HardwareRates())
    shape = StepShape(args.decode, args.prefill, args.ctx, args.ctx // 2)
    print(json.dumps(cm.estimate(PRESETS[args.model], shape, args.tp), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
