"""Public engine API: load a model directory, generate, stream, sessions, extension seams.

Surface of the reference's `Engine` (crates/onnx-genai-engine/src/engine/runtime.rs:340-1524) and
its Python binding (`onnx_genai.Engine.from_dir / generate / generate_stream / tokenize`,
crates/onnx-genai-python/src/lib.rs:186-343): `GenerateOptions` carries the same request fields as
the reference's 26-field struct (src/config.rs:1176-1274); `Sampler`, `LogitProcessor` and
`SpeculativeProposer` are the user-pluggable seams; sessions offer create / close / reset /
checkpoint / restore / rewind / fork (runtime.rs:1240-1330, config.rs:472-484).
"""
from __future__ import annotations

import os

import time
from dataclasses import dataclass, field

import numpy as np
import torch

from .. import metadata as md
from .. import package as pkg
from ..package import onnx_pb
from ..package.decoder_graph import lower_decoder
from ..package.onnx_text import load_any
from ..speculative import SpeculativeStats
from . import processors as procs
from .llm_engine import EngineConfig, LLMEngine


@dataclass
class GenerateOptions:
    max_new_tokens: int = 256
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    top_a: float = 0.0
    typical_p: float = 1.0
    greedy: bool = True
    repetition_penalty: float = 1.0
    repetition_window: int = 0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_sequence_breakers: tuple = ()
    mirostat: bool = False
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    xtc_probability: float = 0.0
    xtc_threshold: float = 0.1
    banned_tokens: tuple = ()
    seed: int = 0
    stop: tuple = ()                 # stop strings
    stop_token_ids: tuple = ()
    ignore_eos: bool = False
    logprobs: int = 0                # top-N log-probabilities per generated token (0 = off)
    priority: int = 0
    tenant: int = 0
    speculative: bool = False
    # None, a constraints.Constraint, or (kind, argument) with kind json | json_object | json_schema | regex | choice
    constraint: object = None

    def validate(self):
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0; pass a non-negative token budget")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0; use greedy=True (or temperature=0) for deterministic decoding")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]; 1 disables nucleus filtering")
        if self.logprobs < 0 or self.logprobs > 20:
            raise ValueError("logprobs must be between 0 and 20")


@dataclass
class GenerateResult:
    text: str
    token_ids: list
    finish_reason: str | None
    prompt_tokens: int
    completion_tokens: int
    ttft_s: float = 0.0
    total_s: float = 0.0
    logprobs: list = field(default_factory=list)   # per token: (token logprob, [(id, logprob) top-N])
    speculative: SpeculativeStats | None = None

    @property
    def decode_tokens_per_s(self) -> float:
        dt = self.total_s - self.ttft_s
        return (self.completion_tokens - 1) / dt if dt > 0 and self.completion_tokens > 1 else 0.0


@dataclass
class SessionCheckpoint:
    session_id: int
    position: int


class _Session:
    def __init__(self, sid):
        self.id = sid
        self.tokens: list = []


class Engine:
    """One model, one device (or one tensor-parallel group), one owner thread."""

    def __init__(self, llm: LLMEngine, tokenizer=None, chat_template: str | None = None, metadata=None,
                 eos_token_ids=(), draft: "Engine | None" = None):
        self.llm = llm
        self.tokenizer = tokenizer
        self.chat_template = chat_template
        self.metadata = metadata or md.InferenceMetadata()
        self.eos_token_ids = tuple(eos_token_ids)
        self.draft = draft
        self.sessions: dict[int, _Session] = {}
        self._next_session = 1
        self.proposer_factory = None      # () -> SpeculativeProposer; default prompt lookup

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dir(cls, model_dir: str, device=None, page_size: int | None = None, max_seqs: int = 32,
                 max_seq_len: int | None = None, num_pages: int = 0, max_tokens_per_step: int = 2048,
                 kv_dtype: str = "bf16", max_draft_tokens: int = 0, draft_model_dir: str | None = None,
                 keep_int4: bool | None = None, context_cache=None, tp: int = 1, tp_rank: int = 0, comm=None, **engine_kw):
        """Load a flat model directory or a model package.  ``page_size`` is accepted for API
        compatibility; pages hold 16 tokens (the attention kernels' tile).  ``context_cache``: True (or a directory) keeps the
        lowered weight layout beside the model (``ogb_context/``) and reads it back on the next load instead of parsing and
        packing the graph again; ``ONNX_GENAI_CONTEXT_CACHE=1`` turns it on for every load.  ``tp`` > 1: this process is
        rank ``tp_rank`` of a tensor-parallel group that talks over ``comm`` (engine/tp_driver.py ``bootstrap`` gives all
        three from the launcher's environment); it loads its shard of the weights, rank 0 serves and the others call
        :meth:`follow`."""
        if page_size not in (None, 16):
            raise ValueError(f"page_size={page_size} is not supported: KV pages hold 16 tokens")
        # precedence: the caller's arguments > ONNX_GENAI_* environment (utils/runtime_config.py) > metadata > built-in
        from ..utils.runtime_config import runtime_config

        rt = runtime_config()
        device = device or rt.default_device(torch.cuda.is_available())
        if rt.require_cuda and not str(device).startswith("cuda"):
            raise RuntimeError(f"ONNX_GENAI_REQUIRE_CUDA is set but the engine was asked to load on {device!r}")
        if rt.baseline_gemm and str(device).startswith("cuda"):
            from .. import ops as _ops

            _ops.set_baseline(True)          # ONNX_GENAI_BASELINE_GEMM: library GEMMs, for comparisons
        d = pkg.open_model_directory(model_dir, ep="cuda" if str(device).startswith("cuda") else "cpu",
                                     device="gpu" if str(device).startswith("cuda") else "cpu")
        meta = d.load_metadata()
        dtype = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
        if tp > 1:
            if comm is None:
                raise ValueError("tensor parallelism needs a communicator: use engine.tp_driver.bootstrap() under a launcher")
            keep_int4, context_cache = False, False       # shards are cut from dense weights; the cache holds whole models
        if keep_int4 is None:   # MatMulNBits weights stay packed wherever a kernel reads them directly
            from ..ops import cpu as _cpu_ops

            keep_int4 = str(device).startswith("cuda") or _cpu_ops.available()
        if context_cache is None:
            context_cache = os.environ.get("ONNX_GENAI_CONTEXT_CACHE", "0") not in ("", "0")
        cache_hit = None
        if context_cache:
            from ..package.context_cache import lower_with_cache

            cfg, weights, cache_hit = lower_with_cache(d.model_path, lambda: load_any(d.model_path), dtype, device, keep_int4,
                                                       cache_dir=context_cache if isinstance(context_cache, str) else None)
        else:
            cfg, weights, _ = lower_decoder(load_any(d.model_path), dtype=dtype, device=device, keep_int4=keep_int4, tp=tp, rank=tp_rank)
        if meta.vocab_size and meta.vocab_size != cfg.vocab:
            raise md.MetadataError(f"{d.metadata_path}: model.vocab_size={meta.vocab_size} but the graph's embedding has "
                                   f"{cfg.vocab} rows; fix the metadata or re-export the model")
        if meta.sliding_window and cfg.sliding_window <= 0:
            cfg.sliding_window = int(meta.sliding_window)         # graphs exported without local_window_size
        if cfg.sliding_window > 0 and meta.sink_tokens:
            cfg.attention_sinks = int(meta.sink_tokens)
        limit = meta.max_sequence_length or cfg.max_position
        max_seq_len = min(max_seq_len or limit, limit, cfg.max_position)
        tok = None
        eos = []
        if d.tokenizer_path:
            from tokenizers import Tokenizer

            tok = Tokenizer.from_file(d.tokenizer_path)
            for name in ("<|endoftext|>", "<|im_end|>", "</s>", "<|eot_id|>"):
                tid = tok.token_to_id(name)
                if tid is not None:
                    eos.append(tid)
        if d.genai_config:
            from ..package.genai_config import eos_token_ids

            eos = eos_token_ids(d.genai_config) or eos
        cfg = cfg.replace(eos_token=eos[0] if eos else -1)
        rt.apply_engine_defaults(engine_kw, str(device).startswith("cuda"))
        ecfg = EngineConfig(model=cfg, num_pages=num_pages, max_seqs=max_seqs, max_seq_len=max_seq_len,
                            max_tokens_per_step=max_tokens_per_step, prefill_chunk=meta.chunked_prefill_size or 2048,
                            kv_dtype=kv_dtype, max_draft_tokens=max_draft_tokens, **engine_kw)
        llm = LLMEngine(ecfg, weights=weights, device=device, tp=tp, rank=tp_rank, comm=comm)
        draft = cls.from_dir(draft_model_dir, device=device, max_seqs=max_seqs, max_seq_len=max_seq_len) if (draft_model_dir and tp == 1) else None
        eng = cls(llm, tok, d.chat_template, meta, eos, draft)
        if tp > 1:
            from .tp_driver import TpControl

            eng.tp_control = TpControl(llm, tp_rank, tp, getattr(getattr(comm, "base", comm), "group", None))
            if tp_rank == 0:
                eng.tp_control.install()
        eng.context_cache_hit = cache_hit            # None: cache off, False: written by this load, True: read back
        mtp_path = os.path.join(os.path.dirname(d.model_path), "mtp_head.safetensors")
        if max_draft_tokens > 0 and draft is None and os.path.exists(mtp_path):
            # a package that ships an MTP head drafts with it (speculative requests only)
            from ..speculative.mtp import MtpHead, attach_mtp

            attach_mtp(eng, MtpHead.load(mtp_path, weights.embed, weights.lm_head))
        return eng

    # ------------------------------------------------------------------ text helpers
    def tokenize(self, text: str) -> list:
        if self.tokenizer is None:
            raise RuntimeError("this engine was built without a tokenizer; pass token ids or load a directory with tokenizer.json")
        return self.tokenizer.encode(text, add_special_tokens=False).ids

    def detokenize(self, ids) -> str:
        if self.tokenizer is None:
            return " ".join(str(int(i)) for i in ids)
        return self.tokenizer.decode([int(i) for i in ids], skip_special_tokens=False)

    def apply_chat_template(self, messages, add_generation_prompt=True, tools=None, **extra) -> str:
        import jinja2

        tmpl = self.chat_template or ("{% for m in messages %}{{ m['role'] }}: {{ m['content'] }}\n{% endfor %}"
                                      "{% if add_generation_prompt %}assistant: {% endif %}")
        env = jinja2.Environment(trim_blocks=False, lstrip_blocks=False)
        env.globals["raise_exception"] = lambda msg: (_ for _ in ()).throw(ValueError(msg))
        return env.from_string(tmpl).render(messages=messages, add_generation_prompt=add_generation_prompt, tools=tools,
                                            **extra)

    # ------------------------------------------------------------------ generation
    def _submit(self, ids, opt: GenerateOptions, sampler=None, processors=()):
        opt.validate()
        defaults = self.metadata.generation_defaults or {}
        greedy = opt.greedy or opt.temperature == 0
        temperature = 0.0 if greedy else (opt.temperature if opt.temperature is not None else defaults.get("temperature", 1.0))
        stop_ids = tuple(opt.stop_token_ids) + (() if opt.ignore_eos else self.eos_token_ids)
        tpc = getattr(self, "tp_control", None)
        if tpc is not None:
            # what the followers cannot mirror is refused before the request reaches any scheduler
            if opt.constraint is not None or sampler is not None or processors or opt.logprobs:
                tpc.refuse("constrained decoding / a custom sampler or processor / log-probabilities")
            eff0 = GenerateOptions(**{**opt.__dict__, "greedy": greedy})
            if procs.device_sampling_plan(procs.build_processor_chain(eff0, len(ids), np.random.default_rng(0)), eff0, False) == "host":
                tpc.refuse("this combination of sampling options (it runs on the host)")
            if opt.speculative:
                tpc.refuse("speculative decoding")
        if getattr(self, "kv_offload", None) is not None:
            self.kv_offload.restore(ids)
        sid = self.llm.add_request(np.asarray(ids, dtype=np.int32), opt.max_new_tokens, temperature=temperature,
                                   top_k=opt.top_k, top_p=opt.top_p, min_p=opt.min_p, seed=opt.seed, priority=opt.priority,
                                   tenant=opt.tenant, ignore_eos=opt.ignore_eos, stop_ids=stop_ids)
        rng = np.random.default_rng(opt.seed or None)
        eff = GenerateOptions(**{**opt.__dict__, "greedy": greedy})
        cproc = None
        if opt.constraint is not None:
            from . import constraints as cons

            cproc = cons.ConstraintProcessor(cons.make_constraint(opt.constraint), self.token_texts(), stop_ids)
        chain = procs.build_processor_chain(eff, len(ids), rng, extra=processors, constraint=cproc)
        plan = procs.device_sampling_plan(chain, eff, sampler is not None)
        state = {"ids": list(int(i) for i in ids), "chain": chain, "logprobs": [], "plan": plan, "constraint": cproc}
        if plan == "host":
            smp = sampler or (procs.GreedySampler() if greedy else procs.CategoricalSampler())

            def host_fn(row_logits, u, st=state, smp=smp, n_lp=opt.logprobs):
                logits = st["chain"].process(st["ids"], row_logits.astype(np.float32, copy=True))
                tok = int(smp.sample(logits, u))
                if n_lp:
                    lp = procs.log_softmax(row_logits)
                    top = np.argsort(-lp)[:n_lp]
                    st["logprobs"].append((float(lp[tok]), [(int(i), float(lp[i])) for i in top]))
                for p in st["chain"].processors:
                    if hasattr(p, "observe"):
                        p.observe(tok)
                return tok

            self.llm.host_samplers[sid & 0x7FFFFFFF] = host_fn
        if opt.speculative and self.llm.cfg.max_draft_tokens > 0 and greedy:
            from ..speculative import DraftModelProposer, NgramProposer

            if self.proposer_factory is not None:
                self.llm.proposers[sid] = self.proposer_factory()
            elif self.draft is not None:
                self.llm.proposers[sid] = DraftModelProposer(self.draft.llm)
            else:
                self.llm.proposers[sid] = NgramProposer()
        return sid, state

    def token_texts(self) -> list:
        """Decoded text of every vocabulary entry ('' for special tokens and incomplete byte sequences);
        computed once, used by constrained decoding."""
        if getattr(self, "_token_texts", None) is None:
            if self.tokenizer is None:
                raise ValueError("constrained decoding needs the model's tokenizer (tokenizer.json is missing)")
            vocab = self.llm.cfg.model.vocab
            n_tok = self.tokenizer.get_vocab_size()
            texts = []
            for i in range(vocab):
                t = self.tokenizer.decode([i], skip_special_tokens=True) if i < n_tok else ""
                texts.append("" if "\ufffd" in t else t)
            self._token_texts = texts
        return self._token_texts

    @staticmethod
    def constraint_finished(state) -> bool:
        c = state.get("constraint")
        return c is not None and c.constraint.terminal(c.token_texts)

    def attach_kv_connector(self, connector) -> None:
        """Offload the K/V of finished requests to ``connector`` and restore it on later prefix hits
        (see :mod:`onnx_genai_b200.engine.kv_connector`).  Needs the device prefix cache."""
        from .kv_connector import KvOffload

        if not self.llm.cfg.enable_prefix_cache:
            raise ValueError("a KV connector extends the device prefix cache; build the engine with enable_prefix_cache=True")
        self.kv_offload = KvOffload(self.llm, connector)
        # the connector's host tier is a reclaimable consumer of host memory: its bytes show in the ledger, and when some
        # other consumer is short the pressure queue asks it to spill to disk before anyone has to wait
        if hasattr(connector, "shrink_host"):
            from .memory import PressureQueue

            ledger = self.llm.memory
            lease = ledger.lease("kv_offload", "host", 0, "offloaded KV chunks held in host memory")

            def account(nbytes, lease=lease, ledger=ledger):
                try:
                    lease.resize(int(nbytes))
                except Exception:            # over the host limit: give back the excess, keep the rest on disk
                    connector.max_host_bytes = max(0, (ledger.available("host") or 0) + lease.nbytes)
                    connector.shrink_host(max(0, int(nbytes) - connector.max_host_bytes))

            connector.on_host_bytes = account
            self.host_pressure = PressureQueue(ledger, "host", reclaim=connector.shrink_host)

    def _finish(self, sid, tokens=None):
        if tokens is not None and getattr(self, "kv_offload", None) is not None:
            try:
                self.kv_offload.save(tokens)
            except Exception:          # offload is an optimisation: a full disk must not fail the request
                pass
        self.llm.host_samplers.pop(sid & 0x7FFFFFFF, None)
        prop = self.llm.proposers.pop(sid, None)
        if prop is not None and hasattr(prop, "close"):
            prop.close()
        self.llm.core.release(sid)
        self.llm.stats.pop(sid, None)

    def generate_stream(self, prompt, options: GenerateOptions | None = None, sampler=None, processors=()):
        """Yields (token_id, text_delta, finish_reason | None) as tokens are produced."""
        opt = options or GenerateOptions()
        ids = self.tokenize(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
        sid, state = self._submit(ids, opt, sampler, processors)
        out_ids, emitted = [], ""
        try:
            done = False
            while not done and self.llm.has_work:
                for esid, tok, fin in self.llm.step().events:
                    if esid != sid:
                        continue
                    out_ids.append(tok)
                    state["ids"].append(tok)
                    text = self.detokenize(out_ids) if self.tokenizer is not None else ""
                    delta = text[len(emitted):]
                    if opt.stop and self.tokenizer is not None:
                        hit = min((text.find(s) for s in opt.stop if s and text.find(s) >= 0), default=-1)
                        if hit >= 0:
                            delta = text[len(emitted):hit] if hit > len(emitted) else ""
                            self.llm.core.cancel(sid)
                            fin = "stop"
                    if fin is None and self.constraint_finished(state):
                        self.llm.core.cancel(sid)
                        fin = "stop"
                    emitted += delta
                    yield tok, delta, fin
                    if fin is not None:
                        done = True
                        break
        finally:
            self._last_state = state
            self._finish(sid, state["ids"])

    def generate(self, prompt, options: GenerateOptions | None = None, sampler=None, processors=(), on_token=None) -> GenerateResult:
        opt = options or GenerateOptions()
        ids = self.tokenize(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
        t0 = time.perf_counter()
        c0 = (self.llm.core.spec_steps, self.llm.core.spec_proposed, self.llm.core.spec_accepted)
        toks, text, fin, ttft = [], "", None, 0.0
        for tok, delta, f in self.generate_stream(ids, opt, sampler, processors):
            if not toks:
                ttft = time.perf_counter() - t0
            toks.append(tok)
            text += delta
            fin = f
            if on_token is not None:
                on_token(tok, delta)
        spec = None
        if opt.speculative:
            c1 = (self.llm.core.spec_steps, self.llm.core.spec_proposed, self.llm.core.spec_accepted)
            spec = SpeculativeStats(c1[0] - c0[0], c1[1] - c0[1], c1[2] - c0[2])
        if self.tokenizer is None:
            text = ""
        return GenerateResult(text=text, token_ids=toks, finish_reason=fin, prompt_tokens=len(ids), completion_tokens=len(toks),
                              ttft_s=ttft, total_s=time.perf_counter() - t0, logprobs=list(self._last_state["logprobs"]),
                              speculative=spec)

    def generate_batch(self, prompts, options: GenerateOptions | None = None):
        """Continuous batching over many prompts; returns results in prompt order."""
        opt = options or GenerateOptions()
        t0 = time.perf_counter()
        entries = []
        for p in prompts:
            ids = self.tokenize(p) if isinstance(p, str) else [int(t) for t in p]
            sid, state = self._submit(ids, opt)
            entries.append({"sid": sid, "ids": ids, "state": state, "out": [], "fin": None, "ttft": 0.0})
        by_sid = {e["sid"]: e for e in entries}
        pending = len(entries)
        while pending and self.llm.has_work:
            for sid, tok, fin in self.llm.step().events:
                e = by_sid.get(sid)
                if e is None or e["fin"] is not None:
                    continue
                if not e["out"]:
                    e["ttft"] = time.perf_counter() - t0
                e["out"].append(tok)
                e["state"]["ids"].append(tok)
                if fin is None and self.constraint_finished(e["state"]):
                    self.llm.core.cancel(sid)
                    fin = "stop"
                if fin is not None:
                    e["fin"] = fin
                    pending -= 1
        results = []
        for e in entries:
            self._finish(e["sid"], e["state"]["ids"])
            text = self.detokenize(e["out"]) if self.tokenizer is not None else ""
            results.append(GenerateResult(text, e["out"], e["fin"], len(e["ids"]), len(e["out"]), e["ttft"],
                                          time.perf_counter() - t0, list(e["state"]["logprobs"])))
        return results

    # ------------------------------------------------------------------ fill in the middle
    FIM_FORMATS = (("<|fim_prefix|>", "<|fim_suffix|>", "<|fim_middle|>"),          # Qwen2.5-Coder, StarCoder2
                   ("<fim_prefix>", "<fim_suffix>", "<fim_middle>"),                # StarCoder
                   ("<PRE>", "<SUF>", "<MID>"),                                     # Code Llama (with spaces, handled below)
                   ("<｜fim▁begin｜>", "<｜fim▁hole｜>", "<｜fim▁end｜>"))           # DeepSeek-Coder (prefix, hole, end)

    def fim_prompt(self, prefix: str, suffix: str) -> str:
        """The model's fill-in-the-middle prompt for (prefix, suffix): the first known sentinel triple whose tokens
        all exist in the tokenizer (the reference resolves the same sentinels, crates/onnx-genai-engine/src/fim.rs)."""
        if self.tokenizer is None:
            raise ValueError("fill-in-the-middle needs the model's tokenizer")
        for a, b, c in self.FIM_FORMATS:
            if all(self.tokenizer.token_to_id(t) is not None for t in (a, b, c)):
                if a == "<｜fim▁begin｜>":
                    return f"{a}{prefix}{b}{suffix}{c}"
                if a == "<PRE>":
                    return f"{a} {prefix} {b}{suffix} {c}"
                return f"{a}{prefix}{b}{suffix}{c}"
        raise ValueError("this model's tokenizer has no fill-in-the-middle sentinel tokens (looked for "
                         + ", ".join(f[0] for f in self.FIM_FORMATS) + ")")

    def generate_fim(self, prefix: str, suffix: str, options: GenerateOptions | None = None, **kw) -> GenerateResult:
        return self.generate(self.fim_prompt(prefix, suffix), options, **kw)

    # ------------------------------------------------------------------ embeddings
    def embed(self, inputs, normalize: bool = True) -> np.ndarray:
        """[n, hidden] fp32: the final-normed hidden state of each input's last token (last-token pooling, the
        usual choice for decoder-only models), L2-normalised unless ``normalize`` is False.  Inputs are strings
        or token-id lists; they run as one continuous batch of prefill-only requests."""
        if getattr(self, "tp_control", None) is not None:
            self.tp_control.refuse("embeddings (hidden-state taps)")
        if isinstance(inputs, str) or (inputs and isinstance(inputs[0], int)):
            inputs = [inputs]
        sids = []
        for item in inputs:
            ids = self.tokenize(item) if isinstance(item, str) else [int(t) for t in item]
            if not ids:
                raise ValueError("cannot embed an empty input")
            sid = self.llm.add_request(np.asarray(ids, dtype=np.int32), 1, temperature=0.0, ignore_eos=True)
            self.llm.hidden_taps[sid & 0x7FFFFFFF] = None
            sids.append(sid)
        pending = set(sids)
        while pending and self.llm.has_work:
            for sid, _tok, fin in self.llm.step().events:
                if fin is not None:
                    pending.discard(sid)
        out = []
        for sid in sids:
            vec = self.llm.hidden_taps.pop(sid & 0x7FFFFFFF, None)
            self.llm.core.release(sid)
            self.llm.stats.pop(sid, None)
            if vec is None:
                raise RuntimeError("the engine finished an embedding request without producing its hidden state")
            if normalize:
                vec = vec / max(float(np.linalg.norm(vec)), 1e-12)
            out.append(vec.astype(np.float32))
        return np.stack(out)

    # ------------------------------------------------------------------ sessions
    def create_session(self) -> int:
        sid = self._next_session
        self._next_session += 1
        self.sessions[sid] = _Session(sid)
        return sid

    def follow(self) -> int:
        """Ranks other than 0 of a tensor-parallel group: mirror the leader's requests and steps until it shuts down."""
        if getattr(self, "tp_control", None) is None or self.tp_control.rank == 0:
            raise RuntimeError("follow() is for ranks 1..n-1 of an engine loaded with tp > 1")
        return self.tp_control.follow()

    def shutdown(self) -> None:
        """Rank 0 of a tensor-parallel group: release the followers.  A no-op for a single-GPU engine."""
        if getattr(self, "tp_control", None) is not None:
            self.tp_control.shutdown()

    def close_session(self, session_id: int) -> None:
        self.sessions.pop(session_id, None)

    def reset_session(self, session_id: int) -> None:
        self._session(session_id).tokens = []

    def _session(self, session_id) -> _Session:
        s = self.sessions.get(session_id)
        if s is None:
            raise KeyError(f"session {session_id} does not exist; create it with create_session()")
        return s

    def generate_in_session(self, session_id: int, prompt, options: GenerateOptions | None = None, **kw) -> GenerateResult:
        """Continue a conversation: the session's token history is the prefix; its KV pages are found again
        through the prefix cache, so only the new tokens are prefilled."""
        s = self._session(session_id)
        new_ids = self.tokenize(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
        res = self.generate(s.tokens + new_ids, options, **kw)
        s.tokens = s.tokens + new_ids + list(res.token_ids)
        return res

    def checkpoint_session(self, session_id: int) -> SessionCheckpoint:
        return SessionCheckpoint(session_id, len(self._session(session_id).tokens))

    def restore_session(self, cp: SessionCheckpoint) -> None:
        self.rewind_session(cp.session_id, cp.position)

    def rewind_session(self, session_id: int, position: int) -> None:
        s = self._session(session_id)
        if not 0 <= position <= len(s.tokens):
            raise ValueError(f"cannot rewind session {session_id} to {position}: it holds {len(s.tokens)} tokens")
        s.tokens = s.tokens[:position]

    def fork_session(self, session_id: int) -> int:
        """Copy-on-write clone: the child shares every full KV page of the parent through the prefix cache."""
        child = self.create_session()
        self.sessions[child].tokens = list(self._session(session_id).tokens)
        return child

    def session_len(self, session_id: int) -> int:
        return len(self._session(session_id).tokens)

    # ------------------------------------------------------------------ introspection
    def resource_snapshot(self) -> dict:
        core = self.llm.core
        total = self.llm.num_pages
        return {"kv_pages_total": total, "kv_pages_free": core.num_free_pages, "kv_usage": 1.0 - core.num_free_pages / max(1, total),
                "waiting": core.num_waiting, "running": core.num_running, "swapped": core.num_swapped,
                "prefix_cache_hits": core.prefix_hits, "prefix_cache_lookups": core.prefix_lookups,
                "preemptions": core.num_preemptions, "steps": self.llm.steps, "sessions": len(self.sessions),
                "memory": self.llm.memory.snapshot(),
                "allocator": self.llm.allocator.stats() if self.llm.allocator is not None else {"kind": "torch"},
                "deferred_releases": self.llm.release_queue.stats()}
