"""Python half of the C interface (``csrc/capi/capi.cpp`` calls these two functions).

``load`` opens a model directory with :class:`onnx_genai_b200.engine.api.Engine`; ``generate`` runs one
request, optionally with a sampler that lives in the C caller: the callback's address arrives as an
integer and is called through ``ctypes`` with the processed fp32 logits row, the tokens generated so far
and the step index, as the C header documents.
"""
from __future__ import annotations

import ctypes

import numpy as np

from .engine.api import Engine, GenerateOptions
from .engine.processors import Sampler

_SAMPLE_FN = ctypes.CFUNCTYPE(ctypes.c_uint32, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float), ctypes.c_size_t,
                              ctypes.POINTER(ctypes.c_uint32), ctypes.c_size_t, ctypes.c_size_t)


class ForeignSampler(Sampler):
    """Adapter from the engine's ``Sampler`` seam to a C ``OgeSampleFn``."""

    def __init__(self, fn_addr: int, user_data: int, name: str = "foreign"):
        self.fn = _SAMPLE_FN(fn_addr)
        self.user_data = ctypes.c_void_p(user_data or None)
        self.name = name or "foreign"
        self.generated: list[int] = []

    def sample(self, logits: np.ndarray, u: float = 0.0) -> int:
        row = np.ascontiguousarray(logits, dtype=np.float32)
        gen = np.asarray(self.generated, dtype=np.uint32)
        tok = int(self.fn(self.user_data, row.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), row.size,
                          gen.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), gen.size, len(self.generated)))
        if not 0 <= tok < row.size:
            raise ValueError(f"sampler '{self.name}' returned token {tok}, outside the vocabulary of {row.size}; "
                             "return an index below logits_len")
        self.generated.append(tok)
        return tok


def load(model_dir: str) -> Engine:
    return Engine.from_dir(model_dir)


def generate(engine: Engine, prompt: str, max_new_tokens: int, sample_fn: int = 0, user_data: int = 0, name: str = "") -> str:
    defaults = engine.metadata.generation_defaults or {}
    opt = GenerateOptions()
    if max_new_tokens:
        opt.max_new_tokens = int(max_new_tokens)
    elif defaults.get("max_new_tokens"):
        opt.max_new_tokens = int(defaults["max_new_tokens"])
    if defaults.get("do_sample"):
        opt.greedy = False
        opt.temperature = float(defaults.get("temperature", 1.0))
        opt.top_k = int(defaults.get("top_k", 0))
        opt.top_p = float(defaults.get("top_p", 1.0))
    sampler = ForeignSampler(sample_fn, user_data, name) if sample_fn else None
    return engine.generate(prompt, opt, sampler=sampler).text
