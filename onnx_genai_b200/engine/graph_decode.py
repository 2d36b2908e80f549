"""Decode loop over the generic graph executor: any decoder ONNX graph with past / present KV tensors, no lowering.

The engine's fast path recognises Llama-style decoder graphs and runs them on its own kernels.  A graph it does not
recognise -- another architecture, or an exporter's idiom the pattern matcher has not met -- can still be served
through this session: the graph runs node by node (:class:`GraphExecutor`), and the session threads the KV tensors
from each call's ``present.*`` outputs into the next call's ``past_key_values.*`` inputs, as the reference's dynamic
past / present decode session does on its ONNX Runtime backend
(crates/onnx-genai-ort/src/decode/mod.rs; the `model.io` block of the inference metadata names the ports).
It is also the independent oracle for the fast path: same package, different executor, same greedy tokens.

Throughput is whatever library tensor operations give; nothing here is tuned, and batch size is one sequence.
"""
from __future__ import annotations

import numpy as np
import torch

from ..package.graph_executor import _TORCH_DTYPE, GraphExecutor


def _rows(logits):
    """[1, n, vocab] or batch-less [n, vocab] logits -> [n, vocab] float32."""
    return (logits[0] if logits.dim() == 3 else logits.reshape(-1, logits.shape[-1])).float()


class GraphDecodeSession:
    def __init__(self, model, device="cpu", io: dict | None = None, dtype=None, extra_outputs=(), extra_feeds: dict | None = None):
        """``model``: path or parsed model.  ``io`` (optional) names the ports: token_input, attention_mask_input,
        position_ids_input, logits_output, kv_inputs, kv_outputs, state_pairs -- the ``model.io`` block; by default they
        are found by the usual names (``input_ids``, ``attention_mask``, ``position_ids``, ``logits``, ``past*`` /
        ``present*``, and ``X.in`` / ``X.out`` for loop-carried recurrent state).

        ``state_pairs`` (``[{input, output}, ...]``) are fixed-size tensors a hybrid decoder carries from call to call
        (convolution or linear-attention state); they start at zero.  Such state cannot be cut back to an earlier length,
        so :meth:`rewind` on a session that has any re-feeds the kept tokens from the start -- the same full recompute
        the reference forces for recurrent models (crates/onnx-genai-engine/src/kv_bridge.rs:1189-1212).
        ``extra_feeds`` maps any other graph input to a tensor, or to ``fn(past_len, n_new) -> tensor``.  Position ids
        declared with three axes ``[axes, batch, tokens]`` get the same text position on every axis."""
        self.ex = model if isinstance(model, GraphExecutor) else GraphExecutor(model, device, dtype)
        g = self.ex.model.graph
        io = dict(io or {})
        names = self.ex.input_names
        self.token_in = io.get("token_input") or next((n for n in names if n in ("input_ids", "tokens")), None)
        if self.token_in is None:
            raise ValueError(f"cannot tell which of the inputs {names} takes token ids; pass io={{'token_input': ...}}")
        self.mask_in = io.get("attention_mask_input") or ("attention_mask" if "attention_mask" in names else None)
        self.pos_in = io.get("position_ids_input") or ("position_ids" if "position_ids" in names else None)
        self.logits_out = io.get("logits_output") or ("logits" if "logits" in self.ex.output_names else self.ex.output_names[0])
        self.kv_in = list(io.get("kv_inputs") or [n for n in names if n.startswith(("past", "key_cache", "value_cache"))])
        self.kv_out = list(io.get("kv_outputs") or [n for n in self.ex.output_names if n.startswith("present")])
        if len(self.kv_in) != len(self.kv_out):
            raise ValueError(f"{len(self.kv_in)} KV inputs but {len(self.kv_out)} KV outputs; name them in io")
        pairs = io.get("state_pairs")
        if pairs is None:
            pairs = [{"input": n, "output": n[:-3] + ".out"} for n in names if n.endswith(".in") and n[:-3] + ".out" in self.ex.output_names]
        self.state_in = [p["input"] for p in pairs]
        self.state_out = [p["output"] for p in pairs]
        self.kv_in = [n for n in self.kv_in if n not in self.state_in]
        self.extra_feeds = dict(extra_feeds or {})
        extra = [n for n in names if n not in {self.token_in, self.mask_in, self.pos_in, *self.kv_in, *self.state_in, *self.extra_feeds}]
        if extra:
            raise ValueError(f"the graph has inputs this session does not know how to feed: {extra}")
        self.info = {vi.name: vi for vi in g.inputs}
        self.extra_outputs = [n for n in extra_outputs]     # e.g. a hidden-state output that a draft head consumes
        self.last_extra: dict = {}
        self.reset()

    def reset(self) -> None:
        self.tokens: list = []
        self.past = {}
        for name in self.kv_in:
            vi = self.info[name]
            shape, seq_axis = [], None
            for axis, dim in enumerate(vi.shape):
                if isinstance(dim, int):
                    shape.append(dim)
                elif axis == 0:
                    shape.append(1)                                  # batch
                else:
                    shape.append(0)                                  # the past length
                    seq_axis = axis
            self.past[name] = torch.zeros(shape, dtype=_TORCH_DTYPE.get(vi.elem_type, torch.float32), device=self.ex.device)
            self.seq_axis = seq_axis if seq_axis is not None else 2
        self.state = {}
        for name in self.state_in:
            vi = self.info[name]
            self.state[name] = torch.zeros([d if isinstance(d, int) else 1 for d in vi.shape],
                                           dtype=_TORCH_DTYPE.get(vi.elem_type, torch.float32), device=self.ex.device)

    @property
    def length(self) -> int:
        return len(self.tokens)

    def feed(self, token_ids) -> torch.Tensor:
        """Append tokens; returns the logits of every fed position [n, vocab]."""
        ids = [int(t) for t in token_ids]
        if not ids:
            raise ValueError("feed needs at least one token")
        past_len = self.length
        feeds = {self.token_in: torch.tensor([ids], dtype=torch.int64)}
        if self.mask_in:
            feeds[self.mask_in] = torch.ones(1, past_len + len(ids), dtype=torch.int64)
        if self.pos_in:
            pos = torch.arange(past_len, past_len + len(ids), dtype=torch.int64)[None]
            declared = self.info[self.pos_in].shape
            feeds[self.pos_in] = pos[None].expand(int(declared[0]), 1, len(ids)).contiguous() if len(declared) == 3 and isinstance(declared[0], int) else pos
        for name, value in self.extra_feeds.items():
            feeds[name] = value(past_len, len(ids)) if callable(value) else value
        feeds.update(self.past)
        feeds.update(self.state)
        out = self.ex.run(feeds, [self.logits_out, *self.kv_out, *self.state_out, *self.extra_outputs])
        for src, dst in zip(self.kv_out, self.kv_in):
            self.past[dst] = out[src]
        for src, dst in zip(self.state_out, self.state_in):
            self.state[dst] = out[src]
        self.last_extra = {n: out[n][0] for n in self.extra_outputs}
        self.tokens += ids
        return _rows(out[self.logits_out])

    def rewind(self, new_len: int) -> None:
        if not 0 <= new_len <= self.length:
            raise ValueError(f"cannot rewind to {new_len}: the session holds {self.length} tokens")
        if self.state_in and new_len < self.length:
            keep = self.tokens[:new_len]
            self.reset()
            if keep:
                self.feed(keep)
            return
        self.tokens = self.tokens[:new_len]
        for name, t in self.past.items():
            self.past[name] = t.narrow(self.seq_axis, 0, new_len).contiguous()

    def generate(self, prompt, max_new_tokens: int, eos_token_ids=(), sampler=None) -> list:
        """Greedy by default; ``sampler(logits [vocab] numpy) -> token`` replaces the argmax."""
        logits = self.feed(prompt)[-1]
        out = []
        for _ in range(max_new_tokens):
            tok = int(sampler(logits.cpu().numpy())) if sampler is not None else int(torch.argmax(logits))
            out.append(tok)
            if tok in eos_token_ids:
                break
            logits = self.feed([tok])[-1]
        return out

    @classmethod
    def from_dir(cls, model_dir: str, device="cpu") -> "GraphDecodeSession":
        """A model directory or package (binary or text-format ONNX); ports come from its ``model.io`` block when it has one."""
        import os

        from .. import package as pkg
        from ..package.onnx_text import load_any

        text = os.path.join(model_dir, "model.onnx.textproto")
        if os.path.exists(text):
            path, meta_path = text, os.path.join(model_dir, "inference_metadata.yaml")
        else:
            d = pkg.open_model_directory(model_dir)
            path, meta_path = d.model_path, d.metadata_path
        io = None
        if meta_path and os.path.exists(meta_path):
            import yaml

            with open(meta_path, encoding="utf-8") as f:
                io = ((yaml.safe_load(f) or {}).get("model") or {}).get("io")
        return cls(load_any(path), device, io)


class StaticCacheDecodeSession:
    """Decode over a graph with fixed-size KV caches updated in place by indexed scatter: inputs ``key_cache.*`` /
    ``value_cache.*`` of full length, ``write_indices`` (where this call's tokens go) and ``nonpad_kv_seqlen`` (valid length
    after the write); outputs ``updated_*`` caches that feed the next call.  The reference's static-cache decode session
    for graphs exported with ``TensorScatter`` (crates/onnx-genai-ort/src/decode, `StaticCacheDecodeSession`; metadata
    ``kv_update: indexed_scatter``).  Shapes never change between calls, which is what capture-friendly backends want."""

    def __init__(self, model, device="cpu"):
        self.ex = model if isinstance(model, GraphExecutor) else GraphExecutor(model, device)
        names = self.ex.input_names
        self.token_in = next((n for n in names if n in ("input_ids", "tokens")), None)
        self.cache_in = [n for n in names if n.startswith(("key_cache", "value_cache"))]
        self.cache_out = [n for n in self.ex.output_names if n.startswith("updated_")]
        if self.token_in is None or not self.cache_in or len(self.cache_in) != len(self.cache_out):
            raise ValueError(f"not a static-cache decoder: inputs {names}, outputs {self.ex.output_names}")
        for need in ("write_indices", "nonpad_kv_seqlen"):
            if need not in names:
                raise ValueError(f"a static-cache decoder takes '{need}'; this graph takes {names}")
        self.logits_out = "logits" if "logits" in self.ex.output_names else self.ex.output_names[0]
        self.info = {vi.name: vi for vi in self.ex.model.graph.inputs}
        self.reset()

    def reset(self) -> None:
        self.tokens: list = []
        self.cache = {}
        for name in self.cache_in:
            vi = self.info[name]
            shape = [d if isinstance(d, int) else 1 for d in vi.shape]
            self.cache[name] = torch.zeros(shape, dtype=_TORCH_DTYPE.get(vi.elem_type, torch.float32), device=self.ex.device)
        first = self.info[self.cache_in[0]].shape
        self.capacity = int(next(d for d in first[1:] if isinstance(d, int)))

    def feed(self, token_ids) -> torch.Tensor:
        ids = [int(t) for t in token_ids]
        past = len(self.tokens)
        if past + len(ids) > self.capacity:
            raise ValueError(f"{past} cached + {len(ids)} new tokens exceed the cache length {self.capacity}")
        feeds = {self.token_in: torch.tensor([ids], dtype=torch.int64), "write_indices": torch.tensor([past], dtype=torch.int64),
                 "nonpad_kv_seqlen": torch.tensor([past + len(ids)], dtype=torch.int64), **self.cache}
        out = self.ex.run(feeds, [self.logits_out, *self.cache_out])
        for src, dst in zip(self.cache_out, self.cache_in):
            self.cache[dst] = out[src]
        self.tokens += ids
        return _rows(out[self.logits_out])

    def generate(self, prompt, max_new_tokens: int) -> list:
        logits = self.feed(prompt)[-1]
        out = []
        for _ in range(max_new_tokens):
            out.append(int(torch.argmax(logits)))
            if len(out) < max_new_tokens:
                logits = self.feed([out[-1]])[-1]
        return out


class GraphMtpSpeculator:
    """Greedy speculative decoding with an ONNX multi-token-prediction head, both graphs on the generic executor.

    The target graph also outputs its last hidden states; the head graph takes the embedding of the token just chosen and
    the hidden state behind it (``inputs_embeds``, ``hidden_states``, mask, positions, its own small KV) and returns the
    hidden state one position ahead, which the target's shared LM head turns into a draft token; the head's output is
    threaded back in for the following drafts (hidden-threaded: each head call sees one position and an empty cache).
    The target then scores ``[chosen token, drafts...]`` in one pass, keeps the drafts it agrees with and rewinds its cache
    past the first disagreement.  Tokens are exactly those of plain greedy decoding.  Same contract as the reference's MTP
    decode session over a Mobius-exported head (crates/onnx-genai-engine/src/speculative/mod.rs:999-1170; fixture
    tests/fixtures/tiny-mtp-full: ``embedding.f32`` and ``lm_head.f32`` are the shared tables)."""

    def __init__(self, target: GraphDecodeSession, head, embedding: torch.Tensor, lm_head: torch.Tensor, hidden_output: str, draft_tokens: int = 3):
        self.target, self.k = target, int(draft_tokens)
        self.head = head if isinstance(head, GraphExecutor) else GraphExecutor(head, target.ex.device)
        self.embed, self.lm_head, self.hidden_output = embedding.float(), lm_head.float(), hidden_output
        if hidden_output not in target.extra_outputs:
            raise ValueError(f"the target session must be built with extra_outputs=['{hidden_output}']")
        self.head_kv_in = [n for n in self.head.input_names if n.startswith("past")]
        self.head_kv_out = [n for n in self.head.output_names if n.startswith("present")]
        self.head_info = {vi.name: vi for vi in self.head.model.graph.inputs}
        self.stats = {"target_passes": 0, "proposed": 0, "accepted": 0}

    @classmethod
    def from_dir(cls, d: str, draft_tokens: int = 3, device="cpu") -> "GraphMtpSpeculator":
        """A directory laid out like the upstream fixture: target graph + ``mtp/`` head graph + ``embedding.f32`` / ``lm_head.f32``."""
        import os

        import numpy as np
        import yaml

        from ..package.onnx_text import load_any

        with open(os.path.join(d, "inference_metadata.yaml"), encoding="utf-8") as f:
            io = ((yaml.safe_load(f) or {}).get("model") or {}).get("io") or {}
        hidden_out = io.get("hidden_output", "hidden_states.0")
        find = lambda base: next(os.path.join(base, n) for n in ("model.onnx", "model.onnx.textproto") if os.path.exists(os.path.join(base, n)))
        session_io = {k: v for k, v in io.items() if k != "hidden_output"}
        target = GraphDecodeSession(load_any(find(d)), device, session_io, extra_outputs=[hidden_out])
        hidden = next(vi.shape[-1] for vi in target.ex.model.graph.outputs if vi.name == hidden_out)
        table = lambda name: torch.from_numpy(np.fromfile(os.path.join(d, name), dtype="<f4").reshape(-1, int(hidden)).copy())
        return cls(target, load_any(find(os.path.join(d, "mtp"))), table("embedding.f32"), table("lm_head.f32"), hidden_out, draft_tokens)

    def _draft(self, hidden: torch.Tensor, token: int, position: int) -> list:
        """Hidden-threaded drafting: every head call sees one position with an empty cache; what links the calls is the hidden
        state handed from one to the next (the mode the reference uses for heads whose graphs take no history)."""
        empty = {}
        for name in self.head_kv_in:
            shape = [d if isinstance(d, int) else (1 if axis == 0 else 0) for axis, d in enumerate(self.head_info[name].shape)]
            empty[name] = torch.zeros(shape, device=self.head.device)
        drafts, h, tok = [], hidden.reshape(1, 1, -1).float(), int(token)
        for j in range(self.k):
            feeds = {"inputs_embeds": self.embed[tok].reshape(1, 1, -1), "hidden_states": h, "attention_mask": torch.ones(1, 1, dtype=torch.int64),
                     "position_ids": torch.tensor([[position + j]], dtype=torch.int64), **empty}
            out = self.head.run({k: v for k, v in feeds.items() if k in self.head.input_names})
            h = out["mtp_hidden"] if "mtp_hidden" in out else out[self.head.output_names[0]]
            tok = int(torch.argmax(h.reshape(-1).float() @ self.lm_head.T))
            drafts.append(tok)
        return drafts

    def generate(self, prompt, max_new_tokens: int) -> list:
        t = self.target
        logits = t.feed(prompt)
        self.stats["target_passes"] += 1
        hidden = t.last_extra[self.hidden_output][-1]
        out = []
        while len(out) < max_new_tokens:
            chosen = int(torch.argmax(logits[-1]))
            out.append(chosen)
            if len(out) >= max_new_tokens:
                break
            drafts = self._draft(hidden, chosen, t.length)[: max_new_tokens - len(out)]
            base = t.length
            rows = t.feed([chosen] + drafts)                       # row i predicts the token after fed position i
            self.stats["target_passes"] += 1
            self.stats["proposed"] += len(drafts)
            accepted = 0
            while accepted < len(drafts) and int(torch.argmax(rows[accepted])) == drafts[accepted]:
                accepted += 1
            self.stats["accepted"] += accepted
            out += drafts[:accepted]
            hidden = t.last_extra[self.hidden_output][accepted]
            logits = rows[accepted:accepted + 1]
            t.rewind(base + 1 + accepted)                          # drop the cache entries of the rejected drafts
        return out[:max_new_tokens]


def open_decode_session(model_dir: str, device="cpu"):
    """The decode session that fits the directory's graph: fixed-size scatter-updated caches get a
    :class:`StaticCacheDecodeSession`, past / present graphs a :class:`GraphDecodeSession`."""
    import os

    from ..package.onnx_text import load_any

    text = os.path.join(model_dir, "model.onnx.textproto")
    if os.path.exists(text):
        path = text
    else:
        from .. import package as pkg

        path = pkg.open_model_directory(model_dir).model_path
    model = load_any(path)
    names = [vi.name for vi in model.graph.inputs]
    if "write_indices" in names and any(n.startswith(("key_cache", "value_cache")) for n in names):
        return StaticCacheDecodeSession(model, device)
    return GraphDecodeSession.from_dir(model_dir, device)
