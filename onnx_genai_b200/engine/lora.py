"""Low-rank parameter overlays (LoRA) selected per request row: the ``onnx-genai.parameter-overlay`` adapter.

A package may ship several adapters for the same projection.  Each request row names the adapters it wants (up to
``max_adapters``), with a scale for each; rows of one batch can name different sets.  The overlay computes, for every
row, the base projection plus the selected low-rank updates::

    y[row] = x[row] @ W  +  sum_j  scales[row, j] * (alpha_j / rank_j) * (x[row] @ A_j^T) @ B_j      (j < counts[row], if active[row])

Selection is positional: ``segments[row, j]`` is the ``index`` of an adapter in the package's ``adapters.artifacts`` table,
nothing carries over between submissions.  Adapter weights load on first use and sit in a small least-recently-used
cache (``adapters.cache.max_entries``), so a package can list more adapters than are ever resident.  Same contract and
numbers as the reference's adapter workflow (crates/onnx-genai-engine/src/pipeline/adapters.rs;
tests/adapter_workflow_e2e.rs: identity base, red a=[1,0] b=[1,2] on x=[1,2] gives [2,4]).

Weight files: ``format: json`` -- ``{"targets": {weight_key: {"a": [rank x in, row-major], "b": [rank x out, row-major]}}}``;
``format: hf_peft`` -- safetensors with ``...<module>.lora_A.weight`` [rank, in] and ``...lora_B.weight`` [out, rank].
"""
from __future__ import annotations

import json
import os
from collections import OrderedDict

import numpy as np
import torch


class AdapterError(RuntimeError):
    pass


class AdapterStore:
    """The ``adapters.artifacts`` table of a package, loaded lazily with an LRU cache."""

    def __init__(self, package_dir: str, adapters_doc: dict):
        self.dir = package_dir
        self.targets = {t["id"]: t for t in ((adapters_doc.get("target_manifest") or {}).get("targets") or [])}
        self.by_index = {}
        for name, art in (adapters_doc.get("artifacts") or {}).items():
            self.by_index[int(art["index"])] = {**art, "name": name}
        self.max_entries = int((adapters_doc.get("cache") or {}).get("max_entries", 8))
        self.cache: OrderedDict = OrderedDict()
        self.loads = self.cache_hits = self.evictions = 0

    def get(self, index: int) -> dict:
        """``{target id: (A [rank, in], B [rank, out], alpha / rank)}`` of adapter ``index``."""
        if index in self.cache:
            self.cache.move_to_end(index)
            self.cache_hits += 1
            return self.cache[index]
        art = self.by_index.get(index)
        if art is None:
            raise AdapterError(f"adapter index {index} is not in the package (known: {sorted(self.by_index)})")
        weights = self._load(art)
        self.loads += 1
        self.cache[index] = weights
        while len(self.cache) > self.max_entries:
            self.cache.popitem(last=False)
            self.evictions += 1
        return weights

    def _load(self, art: dict) -> dict:
        rank, alpha = int(art.get("rank", 1)), float(art.get("alpha", 1.0))
        sources = art.get("weights") or []
        errors = []
        for src in sources:
            path = os.path.join(self.dir, src["location"])
            if not os.path.exists(path):
                errors.append(f"{src['location']} does not exist")
                continue
            scale = alpha / rank if src.get("scale_encoding", "alpha_over_rank") == "alpha_over_rank" else 1.0
            raw = self._read_json(path) if src.get("format", "json") == "json" else self._read_peft(path)
            out = {}
            for bind in art.get("bindings") or []:
                target = self.targets.get(bind["target"])
                if target is None:
                    raise AdapterError(f"adapter '{art['name']}' binds target '{bind['target']}', which the target manifest does not list")
                key = bind.get("weight_key", bind["target"])
                if key not in raw:
                    raise AdapterError(f"adapter '{art['name']}': {src['location']} has no weights for '{key}' (it has {sorted(raw)})")
                a, b = raw[key]
                n_in, n_out = int(target["input_features"]), int(target["output_features"])
                a = torch.as_tensor(np.asarray(a, dtype=np.float32)).reshape(-1)
                b = torch.as_tensor(np.asarray(b, dtype=np.float32))
                if a.numel() != rank * n_in or b.numel() != rank * n_out:
                    raise AdapterError(f"adapter '{art['name']}' target '{bind['target']}': A has {a.numel()} and B {b.numel()} values; rank "
                                       f"{rank} with {n_in} inputs and {n_out} outputs needs {rank * n_in} and {rank * n_out}")
                out[bind["target"]] = (a.reshape(rank, n_in), b.reshape(rank, n_out), scale)
            return out
        raise AdapterError(f"adapter '{art['name']}' has no readable weights: " + ("; ".join(errors) or "none listed"))

    @staticmethod
    def _read_json(path):
        with open(path, encoding="utf-8") as f:
            doc = json.load(f)
        return {k: (v["a"], v["b"]) for k, v in (doc.get("targets") or {}).items()}

    @staticmethod
    def _read_peft(path):
        from safetensors.torch import load_file

        tensors, out = load_file(path), {}
        for name, t in tensors.items():
            if ".lora_A" in name:
                module = name.split(".lora_A")[0].split(".")[-1]
                b_name = name.replace(".lora_A", ".lora_B")
                if b_name in tensors:
                    out[module] = (t.float().numpy(), tensors[b_name].float().T.contiguous().numpy())   # A [rank, in]; B [out, rank] -> [rank, out]
        return out


def parameter_overlay_adapter(base_weight: torch.Tensor, store: AdapterStore, target: str, selection: dict, input_port="input", output_port="output"):
    """Workflow component.  ``selection`` names the workflow values that carry segments / adapter_counts / scales / active;
    the runtime hands them over next to the bound ports (``extra_inputs``)."""
    base = base_weight.float()
    max_adapters = int(selection.get("max_adapters", 0)) or None

    def component(ports: dict) -> dict:
        x = torch.as_tensor(np.asarray(ports[input_port]) if not isinstance(ports[input_port], torch.Tensor) else ports[input_port]).float()
        y = x @ base
        seg = ports.get("__segments")
        if seg is None:
            return {output_port: y}
        seg = torch.as_tensor(np.asarray(seg)).long().reshape(x.shape[0], -1)
        counts = torch.as_tensor(np.asarray(ports["__adapter_counts"])).long().reshape(-1) if ports.get("__adapter_counts") is not None \
            else (seg >= 0).sum(dim=1)
        scales = torch.as_tensor(np.asarray(ports["__scales"])).float().reshape(x.shape[0], -1) if ports.get("__scales") is not None \
            else torch.ones_like(seg, dtype=torch.float32)
        active = torch.as_tensor(np.asarray(ports["__active"])).bool().reshape(-1) if ports.get("__active") is not None \
            else torch.ones(x.shape[0], dtype=torch.bool)
        y = y.clone()
        # rows that chose the same adapter are updated together: one pair of small products per distinct adapter
        jobs: dict = {}
        for row in range(x.shape[0]):
            if not bool(active[row]):
                continue
            n = int(counts[row])
            if max_adapters is not None and n > max_adapters:
                raise AdapterError(f"row {row} selects {n} adapters; this package allows {max_adapters}")
            for j in range(n):
                idx = int(seg[row, j])
                if idx < 0:
                    raise AdapterError(f"row {row} counts {n} adapters but slot {j} is empty")
                jobs.setdefault(idx, []).append((row, float(scales[row, j])))
        for idx, rows in jobs.items():
            weights = store.get(idx).get(target)
            if weights is None:
                continue
            a, b, scale = weights
            r = torch.tensor([row for row, _ in rows])
            s = torch.tensor([sc for _, sc in rows])[:, None] * scale
            y[r] += s * ((x[r] @ a.T) @ b)
        return {output_port: y}

    component.extra_inputs = {"__segments": selection.get("segments"), "__adapter_counts": selection.get("adapter_counts"),
                              "__scales": selection.get("scales"), "__active": selection.get("active")}
    component.store = store
    return component
