"""Write decoder packages: random-init benchmark shapes or any DecoderWeights, with tokenizer and metadata.

    python -m onnx_genai_b200.package.export --preset tiny-llama --out /tmp/tiny --int4
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import yaml

from .. import metadata as md
from ..models.config import DecoderConfig, preset
from ..models.decoder import random_weights
from ..ops import reference as ref
from .decoder_graph import export_decoder


def unpack_gate_up(packed: torch.Tensor, half: int):
    """Inverse of ops.pack_gate_up: returns (gate_w, up_w) in natural [intermediate, hidden] layout."""
    n2, k = packed.shape
    v = packed.view(n2 // (2 * half), 2, half, k)
    return v[:, 0].reshape(n2 // 2, k).contiguous(), v[:, 1].reshape(n2 // 2, k).contiguous()


def byte_tokenizer_json(vocab_size: int) -> dict:
    """A self-contained byte-level tokenizer (tokenizers JSON): ids 0..255 are bytes, the rest are filler
    tokens so any id below ``vocab_size`` decodes; <|endoftext|> takes the last id and, for vocabularies of 272
    entries or more, the three Qwen-style fill-in-the-middle sentinels the ids before it."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers

    alphabet = pre_tokenizers.ByteLevel.alphabet()
    vocab = {ch: i for i, ch in enumerate(sorted(alphabet))}
    fim = ["<|fim_prefix|>", "<|fim_middle|>", "<|fim_suffix|>"] if vocab_size >= 272 else []
    for i in range(len(vocab), vocab_size - 1 - len(fim)):
        vocab[f"<|extra_{i}|>"] = i
    for name in fim:                                   # fill-in-the-middle sentinels just below <|endoftext|>
        vocab[name] = len(vocab)
    tok = Tokenizer(models.BPE(vocab=vocab, merges=[]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)
    tok.decoder = decoders.ByteLevel()
    tok.add_special_tokens(fim + ["<|endoftext|>"])
    return json.loads(tok.to_str())


DEFAULT_CHAT_TEMPLATE = (
    "{% for message in messages %}<|im_start|>{{ message['role'] }}\n{{ message['content'] }}<|im_end|>\n{% endfor %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")


def export_package(cfg: DecoderConfig, weights, out_dir: str, dtype: str = "fp32", int4: bool = False,
                   scale_dtype: str = "fp32", generation_defaults=None, tokenizer: bool = True) -> str:
    os.makedirs(out_dir, exist_ok=True)
    half = weights.swiglu_half
    import copy

    def natural(li):  # strip the zero padding the executor may have added to the intermediate dimension
        g, u = unpack_gate_up(weights.layers[li].gate_up_w.float().cpu(), half)
        return g[: cfg.intermediate], u[: cfg.intermediate]

    if weights.layers[0].down_w.shape[1] != cfg.intermediate:
        weights = copy.copy(weights)
        weights.layers = [copy.copy(l) for l in weights.layers]
        for l in weights.layers:
            l.down_w = l.down_w[:, : cfg.intermediate].contiguous()
    export_decoder(cfg, natural, weights,
                   os.path.join(out_dir, "decoder.onnx"), dtype=dtype, int4=int4, scale_dtype=scale_dtype)
    doc = md.emit(cfg, generation_defaults=generation_defaults)
    if int4:
        doc["quantization"] = {"weights": {"format": "MatMulNBits", "bits": 4, "block_size": cfg.int4_block,
                                          "symmetric": True}}
    with open(os.path.join(out_dir, "inference_metadata.yaml"), "w", encoding="utf-8") as f:
        yaml.safe_dump(doc, f, sort_keys=False)
    if tokenizer:
        with open(os.path.join(out_dir, "tokenizer.json"), "w", encoding="utf-8") as f:
            json.dump(byte_tokenizer_json(cfg.vocab), f)
        with open(os.path.join(out_dir, "chat_template.jinja"), "w", encoding="utf-8") as f:
            f.write(DEFAULT_CHAT_TEMPLATE)
    return out_dir


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="tiny-llama")
    ap.add_argument("--out", required=True)
    ap.add_argument("--int4", action="store_true")
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16", "fp16"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0)
    args = ap.parse_args()
    cfg = preset(args.preset)
    if args.layers:
        cfg = cfg.replace(num_layers=args.layers)
    w = random_weights(cfg, "cpu", seed=args.seed, dtype=torch.float32)
    export_package(cfg, w, args.out, dtype=args.dtype, int4=args.int4,
                   scale_dtype="fp32" if cfg.int4_scale_dtype == "fp32" else "bf16")
    print(args.out)


if __name__ == "__main__":
    main()
