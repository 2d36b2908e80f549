"""Decoder architecture description and the named shapes used by the benchmarks.

The reference never keys behaviour on a model name: every choice is structural (heads, sizes,
operators found in the graph; crates/onnx-runtime-ep-cuda/src/kernels/matmul_nbits.rs:5900-6035).
The same rule holds here: ``DecoderConfig`` is filled either from an ONNX model package
(:mod:`onnx_genai_b200.package`) or from one of the presets below, which only exist so
benchmarks and tests can name a shape.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field


@dataclass
class MoEConfig:
    num_experts: int = 0
    top_k: int = 0
    expert_intermediate: int = 0
    renormalize: bool = True
    score_function: str = "softmax"


@dataclass
class DecoderConfig:
    name: str = "decoder"
    num_layers: int = 2
    hidden: int = 256
    num_heads: int = 8
    num_kv_heads: int = 2
    head_dim: int = 32
    intermediate: int = 688
    vocab: int = 32000
    rope_theta: float = 1e4
    rms_eps: float = 1e-6
    tie_embeddings: bool = True
    qkv_bias: bool = False
    max_position: int = 8192
    rotary_interleaved: bool = False
    rotary_dim: int = 0           # 0 = head_dim
    sliding_window: int = 0
    attention_sinks: int = 0      # with a sliding window: leading tokens every query keeps seeing (rounded up to whole KV pages)
    weight_format: str = "bf16"   # "bf16" | "int4" (MatMulNBits block 32)
    int4_block: int = 32
    int4_scale_dtype: str = "bf16"
    moe: MoEConfig = field(default_factory=MoEConfig)
    eos_token: int = -1

    @property
    def sink_len(self) -> int:
        """Attention-sink keys as the kernels see them: whole 16-token pages, and only under a sliding window."""
        return ((self.attention_sinks + 15) // 16) * 16 if self.sliding_window > 0 and self.attention_sinks > 0 else 0

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def replace(self, **kw) -> "DecoderConfig":
        return dataclasses.replace(self, **kw)

    def weight_bytes(self) -> int:
        per = 2 if self.weight_format == "bf16" else 0.5 + 2.0 / self.int4_block
        qkv = (self.q_size + 2 * self.kv_size) * self.hidden
        o = self.hidden * self.q_size
        if self.moe.num_experts:
            mlp = self.moe.num_experts * 3 * self.moe.expert_intermediate * self.hidden + self.moe.num_experts * self.hidden
        else:
            mlp = 3 * self.intermediate * self.hidden
        layer = (qkv + o + mlp) * per
        emb = self.vocab * self.hidden * 2 * (1 if self.tie_embeddings else 2)
        return int(self.num_layers * layer + emb)

    def kv_bytes_per_token(self, kv_dtype_bytes: int = 2) -> int:
        return self.num_layers * 2 * self.num_kv_heads * self.head_dim * kv_dtype_bytes


PRESETS = {
    # config 1: tiny Llama-style decoder, CPU plumbing / parity
    "tiny-llama": DecoderConfig(name="tiny-llama", num_layers=4, hidden=256, num_heads=8, num_kv_heads=2, head_dim=32,
                                intermediate=688, vocab=32000, rope_theta=1e4, rms_eps=1e-6, tie_embeddings=True,
                                weight_format="int4", int4_scale_dtype="fp32", max_position=2048),
    # config 2
    "qwen2.5-0.5b": DecoderConfig(name="qwen2.5-0.5b", num_layers=24, hidden=896, num_heads=14, num_kv_heads=2,
                                  head_dim=64, intermediate=4864, vocab=151936, rope_theta=1e6, tie_embeddings=True,
                                  qkv_bias=True, weight_format="int4", int4_scale_dtype="bf16", max_position=8192),
    # config 3 / 5 target
    "qwen2.5-7b": DecoderConfig(name="qwen2.5-7b", num_layers=28, hidden=3584, num_heads=28, num_kv_heads=4,
                                head_dim=128, intermediate=18944, vocab=152064, rope_theta=1e6, tie_embeddings=False,
                                qkv_bias=True, weight_format="bf16", max_position=40960),
    # config 4
    "qwen3-30b-a3b": DecoderConfig(name="qwen3-30b-a3b", num_layers=48, hidden=2048, num_heads=32, num_kv_heads=4,
                                   head_dim=128, intermediate=0, vocab=151936, rope_theta=1e6, tie_embeddings=False,
                                   qkv_bias=False, weight_format="bf16", max_position=40960,
                                   moe=MoEConfig(num_experts=128, top_k=8, expert_intermediate=768, renormalize=True)),
}


def preset(name: str, **overrides) -> DecoderConfig:
    cfg = PRESETS[name]
    return cfg.replace(**overrides) if overrides else dataclasses.replace(cfg)
