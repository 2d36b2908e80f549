"""Load-time cache of a lowered decoder: the recognised configuration and the device-ready weight layout.

Lowering a decoder package means parsing the ONNX graph, matching its layers, transposing or concatenating projections
and packing gate / up rows for the SwiGLU epilogue; for a multi-gigabyte model that dominates the time to the first token
of a fresh process.  This module writes the *result* of that work next to the model (``ogb_context/index.json`` +
``weights.bin``) and reads it back with one memory map, keyed by a fingerprint of the source files, the runtime version and
the lowering options, so a stale cache is never used.  It plays the role of the reference's EPContext caching
(crates/onnx-runtime-ep-cuda: a compiled-context blob embedded beside the graph so that the provider skips its
compilation step on the next load); there is no compiled code to cache here, the expensive artefact is the weight layout.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os

import numpy as np
import torch

FORMAT = 1
_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16, "uint8": torch.uint8, "int8": torch.int8,
           "int32": torch.int32, "int64": torch.int64}


def fingerprint(model_path: str, dtype, keep_int4: bool) -> str:
    """Identity of a lowering: every file of the model's directory that the graph can draw from (name, size, mtime), the
    runtime version, this format and the options that change the result."""
    from .. import __version__

    h = hashlib.sha256()
    base = os.path.dirname(os.path.abspath(model_path))
    stem = os.path.basename(model_path)
    for name in sorted(os.listdir(base)):
        if name == stem or name.startswith(stem) or name.endswith((".data", ".bin", ".onnx_data")):
            st = os.stat(os.path.join(base, name))
            h.update(f"{name}:{st.st_size}:{st.st_mtime_ns};".encode())
    h.update(f"v={__version__};f={FORMAT};dtype={dtype};int4={int(bool(keep_int4))}".encode())
    return h.hexdigest()[:32]


def _flatten(weights) -> tuple:
    """(tensors by name, structure) of a DecoderWeights object; ``_Lin`` projections of int4 layers are stored field by field."""
    tensors: dict = {}
    layers = []
    for i, lw in enumerate(weights.layers):
        entry = {"fields": [], "quant": {}}
        for f in dataclasses.fields(lw):
            v = getattr(lw, f.name)
            if isinstance(v, torch.Tensor):
                tensors[f"layers.{i}.{f.name}"] = v
                entry["fields"].append(f.name)
        for name, lin in (lw.quant or {}).items():
            many = isinstance(lin, (list, tuple))
            metas = []
            for j, one in enumerate(lin if many else [lin]):
                meta = {"block": int(one.block), "k": None if one.k is None else int(one.k), "parts": []}
                for part in ("w", "q", "scales", "zp", "bias"):
                    t = getattr(one, part, None)
                    if isinstance(t, torch.Tensor):
                        tensors[f"layers.{i}.quant.{name}.{j}.{part}"] = t
                        meta["parts"].append(part)
                metas.append(meta)
            entry["quant"][name] = {"many": many, "items": metas}
        layers.append(entry)
    top = {}
    for name in ("embed", "final_norm", "lm_head", "cos_sin"):
        v = getattr(weights, name, None)
        if isinstance(v, torch.Tensor):
            if name == "lm_head" and v is weights.embed:
                top[name] = "embed"                     # tied: one copy
                continue
            tensors[name] = v
            top[name] = name
    return tensors, {"layers": layers, "top": top, "swiglu_half": int(weights.swiglu_half)}


def save(cache_dir: str, key: str, cfg, weights) -> str:
    """Write the cache; returns the directory.  Written to a temporary name first, so a reader never sees half a cache."""
    tensors, structure = _flatten(weights)
    os.makedirs(cache_dir, exist_ok=True)
    index = {"format": FORMAT, "key": key, "config": dataclasses.asdict(cfg), "structure": structure, "tensors": {}}
    tmp_bin = os.path.join(cache_dir, f"weights.bin.{os.getpid()}.tmp")
    off = 0
    with open(tmp_bin, "wb") as f:
        for name, t in tensors.items():
            c = t.detach().contiguous().cpu()
            dt = str(c.dtype).replace("torch.", "")
            if dt not in _DTYPES:
                raise ValueError(f"context cache: tensor {name} has dtype {dt}, which the cache does not store")
            raw = c.view(torch.uint8).reshape(-1).numpy() if c.numel() else np.zeros(0, dtype=np.uint8)
            pad = (-off) % 256
            f.write(b"\0" * pad)
            off += pad
            f.write(raw.tobytes())
            index["tensors"][name] = {"dtype": dt, "shape": list(c.shape), "offset": off, "nbytes": int(raw.nbytes)}
            off += int(raw.nbytes)
    os.replace(tmp_bin, os.path.join(cache_dir, "weights.bin"))
    tmp_idx = os.path.join(cache_dir, f"index.json.{os.getpid()}.tmp")
    with open(tmp_idx, "w", encoding="utf-8") as f:
        json.dump(index, f)
    os.replace(tmp_idx, os.path.join(cache_dir, "index.json"))
    return cache_dir


def load(cache_dir: str, key: str, device="cpu"):
    """(DecoderConfig, DecoderWeights) from a cache written for ``key``, or None when there is none or it is stale."""
    from ..models.config import DecoderConfig, MoEConfig
    from ..models.decoder import DecoderWeights, LayerWeights
    from .decoder_graph import _Lin

    idx_path = os.path.join(cache_dir, "index.json")
    bin_path = os.path.join(cache_dir, "weights.bin")
    if not (os.path.exists(idx_path) and os.path.exists(bin_path)):
        return None
    try:
        with open(idx_path, encoding="utf-8") as f:
            index = json.load(f)
    except (OSError, ValueError):
        return None
    if index.get("format") != FORMAT or index.get("key") != key:
        return None
    blob = np.memmap(bin_path, dtype=np.uint8, mode="r")
    size = blob.shape[0]
    dev = torch.device(device)

    def tensor(name):
        m = index["tensors"][name]
        if m["offset"] + m["nbytes"] > size:
            raise ValueError(f"context cache {cache_dir} is truncated at tensor {name}")
        raw = torch.from_numpy(np.array(blob[m["offset"]:m["offset"] + m["nbytes"]], copy=True))
        return raw.view(_DTYPES[m["dtype"]]).reshape(m["shape"]).to(dev)

    try:
        c = dict(index["config"])
        moe = c.pop("moe", None)
        cfg = DecoderConfig(**c, **({"moe": MoEConfig(**moe)} if moe is not None else {}))
        st = index["structure"]
        layers = []
        for i, entry in enumerate(st["layers"]):
            kw = {name: tensor(f"layers.{i}.{name}") for name in entry["fields"]}
            for req in ("ln1", "qkv_w", "o_w", "ln2"):
                kw.setdefault(req, None)
            kw.setdefault("qkv_b", None)
            lw = LayerWeights(**kw)
            for name, q in entry["quant"].items():
                items = []
                for j, meta in enumerate(q["items"]):
                    lin = _Lin()
                    lin.block, lin.k = meta["block"], meta["k"]
                    for part in meta["parts"]:
                        setattr(lin, part, tensor(f"layers.{i}.quant.{name}.{j}.{part}").cpu())   # int4 parts are placed by QuantLinear
                    items.append(lin)
                lw.quant[name] = items if q["many"] else items[0]
            layers.append(lw)
        top = {name: tensor(src) for name, src in st["top"].items() if src == name}
        embed = top["embed"]
        weights = DecoderWeights(embed=embed, layers=layers, final_norm=top["final_norm"],
                                 lm_head=embed if st["top"].get("lm_head") == "embed" else top["lm_head"], swiglu_half=st["swiglu_half"])
        if "cos_sin" in top:
            weights.cos_sin = top["cos_sin"]
    except (KeyError, TypeError, ValueError):
        return None
    return cfg, weights


def lower_with_cache(model_path: str, loader, dtype, device, keep_int4: bool, cache_dir: str | None = None):
    """``lower_decoder`` behind the cache: ``loader()`` parses the model only on a miss.  Returns (cfg, weights, hit)."""
    from .decoder_graph import lower_decoder

    cache_dir = cache_dir or os.path.join(os.path.dirname(os.path.abspath(model_path)), "ogb_context")
    key = fingerprint(model_path, dtype, keep_int4)
    got = load(cache_dir, key, device)
    if got is not None:
        return got[0], got[1], True
    cfg, weights, _ = lower_decoder(loader(), dtype=dtype, device=device, keep_int4=keep_int4)
    try:
        save(cache_dir, key, cfg, weights)
    except OSError:
        pass                                           # a read-only model directory just stays uncached
    return cfg, weights, False
