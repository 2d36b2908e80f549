"""Command line: ``python -m onnx_genai_b200 {serve,generate,run,show,list,version,export,bench}``.

Mirrors the reference CLI (crates/onnx-genai-cli/src/lib.rs:92-330): sampling flags
(``--max-new-tokens --temperature --top-p --top-k --greedy/--no-greedy --stop --raw``), engine flags
(``--device auto|cpu|cuda[:N]``), global ``--profile / --profile-json / --profile-trace``, the
``run`` REPL with slash commands (``/help /system /raw /stats /profile /reset /quit``) and the
compact per-turn stats line (TTFT, decode tok/s, finish reason).
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import sys
import time

from . import __version__


def _add_sampling(p):
    p.add_argument("--max-new-tokens", type=int, default=256)
    p.add_argument("--max-context", type=int, default=0)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--min-p", type=float, default=0.0)
    p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--greedy", dest="greedy", action="store_true", default=False)
    p.add_argument("--no-greedy", dest="greedy", action="store_false")
    p.add_argument("--stop", action="append", default=[])
    p.add_argument("--raw", action="store_true", help="do not apply the chat template")
    p.add_argument("--speculative", action="store_true", help="prompt-lookup speculative decoding (greedy only)")
    p.add_argument("--json", dest="json_output", action="store_true", help="constrain the output to one JSON object")
    p.add_argument("--json-schema", default="", help="file with a JSON Schema the output must satisfy")
    p.add_argument("--regex", default="", help="regular expression the whole output must match")


def _add_engine(p):
    p.add_argument("--device", default="auto", help="auto | cpu | cuda[:N]")
    p.add_argument("--backend", default="native", choices=["native", "graph"],
                   help="native: this package's kernels and scheduler; graph: interpret the ONNX graph node by node "
                        "(any decoder architecture, `generate` only, one sequence)")
    p.add_argument("--kv-cache-dtype", default="bf16", choices=["bf16", "fp8_e4m3fn", "fp8_e5m2", "int8"])
    p.add_argument("--max-batch", type=int, default=32)
    p.add_argument("--vram-limit", default="0.85", help="0.85 (fraction of the device the engine may fill), auto, or a size such as 8GiB for weights + activations + KV")
    p.add_argument("--context-cache", action="store_true", help="keep the lowered weight layout beside the model (ogb_context/) and reuse it on the next load")
    p.add_argument("--weight-offload-layers", type=int, default=0, help="keep the matrices of the last N layers in pinned host memory and stream them every step (CUDA)")
    p.add_argument("--kv-max-pages", type=int, default=0, help="reserve address space for this many KV pages and back them on demand (CUDA, one GPU)")
    p.add_argument("--host-ram-limit", default="auto", help="cap on pinned host memory for KV swap and the KV offload host tier: auto, a size such as 32GiB, or a fraction of RAM")
    p.add_argument("--cpu-cores", type=int, default=0, help="threads for CPU kernels and host-side work (0: leave as is)")
    p.add_argument("--draft-model", default="", help="directory of a smaller model that drafts for speculative requests")
    p.add_argument("--draft-tokens", type=int, default=0,
                   help="draft tokens per verification step when speculation is on (default: ONNX_GENAI_SPEC_TOKENS, else 4)")
    p.add_argument("--proposer", default="auto", choices=["auto", "ngram", "draft", "mtp", "eagle3", "shared-kv"],
                   help="who drafts for speculative requests (auto: the draft model if given, a packaged MTP head, else prompt lookup)")
    p.add_argument("--kv-offload-dir", default="", help="keep the K/V of finished prompts in host memory and this directory; restored on prefix hits")
    p.add_argument("--kv-offload-host-gib", type=float, default=4.0)
    p.add_argument("--kv-offload-disk-gib", type=float, default=64.0)


def _options(args):
    from .engine.api import GenerateOptions

    constraint = None
    if getattr(args, "json_schema", ""):
        import json

        with open(args.json_schema, encoding="utf-8") as f:
            constraint = ("json_schema", json.load(f))
    elif getattr(args, "regex", ""):
        constraint = ("regex", args.regex)
    elif getattr(args, "json_output", False):
        constraint = ("json_object",)
    return GenerateOptions(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                           min_p=args.min_p, repetition_penalty=args.repetition_penalty, seed=args.seed,
                           greedy=args.greedy or args.temperature == 0, stop=tuple(args.stop),
                           speculative=args.speculative or getattr(args, "proposer", "auto") != "auto" or bool(getattr(args, "draft_model", "")),
                           constraint=constraint)


def _load(args):
    import torch

    from .engine.api import Engine

    from .utils.runtime_config import runtime_config

    rt = runtime_config()
    dev = args.device
    if dev == "auto":       # no --device: ONNX_GENAI_CUDA_DEVICE / ONNX_GENAI_REQUIRE_CUDA decide
        dev = rt.default_device(torch.cuda.is_available())
    for name, why in rt.ignored.items():
        print(f"note: {name} is set but has no effect here: {why}", file=sys.stderr)
    # --vram-limit: a fraction keeps its old meaning (share of the device the engine may fill); a size such as 8GiB
    # caps weights + activations + KV pool through the memory ledger
    try:
        util = float(args.vram_limit)
        limit = None
    except ValueError:
        util, limit = 0.85, (None if args.vram_limit == "auto" else args.vram_limit)
    if getattr(args, "cpu_cores", 0) > 0:
        torch.set_num_threads(args.cpu_cores)
        os.environ["OMP_NUM_THREADS"] = str(args.cpu_cores)
    proposer = getattr(args, "proposer", "auto")
    speculative = getattr(args, "speculative", False) or proposer != "auto" or bool(getattr(args, "draft_model", ""))
    if proposer == "draft" and not getattr(args, "draft_model", ""):
        raise SystemExit("--proposer draft needs --draft-model DIR")
    extra = {"kv_max_pages": args.kv_max_pages} if getattr(args, "kv_max_pages", 0) > 0 else {}
    # Launched by torchrun (WORLD_SIZE > 1): the processes form one tensor-parallel group; this function returns on rank 0
    # only -- the other ranks follow the leader's requests inside it and exit when the leader does.
    tp_world = int(os.environ.get("WORLD_SIZE", "1"))
    if tp_world > 1:
        from .engine.tp_driver import bootstrap

        tp_rank, tp_world, tp_dev, tp_comm = bootstrap(None if dev == "auto" else dev)
        dev = str(tp_dev)
        if speculative:
            raise SystemExit("speculative decoding is not available under tensor parallelism (launch one process for it)")
        extra.update(tp=tp_world, tp_rank=tp_rank, comm=tp_comm)
    if getattr(args, "context_cache", False):
        extra["context_cache"] = True
    if getattr(args, "weight_offload_layers", 0) > 0:
        extra["weight_offload_layers"] = args.weight_offload_layers
    eng = Engine.from_dir(args.model, device=dev, max_seqs=args.max_batch, kv_dtype={"fp8_e4m3fn": "fp8", "int8": "int8", "fp8_e5m2": "fp8_e5m2"}.get(args.kv_cache_dtype, "bf16"),
                          gpu_memory_utilization=util if 0 < util <= 1 else 0.85, vram_limit=limit,
                          max_draft_tokens=(getattr(args, "draft_tokens", 0) or rt.spec_tokens) if speculative else 0,
                          draft_model_dir=(getattr(args, "draft_model", "") or None) if proposer in ("auto", "draft") else None,
                          max_seq_len=args.max_context or None, **extra)
    if tp_world > 1:
        if tp_rank != 0:
            steps = eng.follow()
            print(f"rank {tp_rank}: followed {steps} steps", file=sys.stderr)
            import torch.distributed as dist

            dist.barrier()
            raise SystemExit(0)
        import atexit

        def _release_followers():
            import torch.distributed as dist

            eng.shutdown()
            dist.barrier()

        atexit.register(_release_followers)
    if proposer == "ngram":
        from .speculative import NgramProposer

        eng.proposer_factory = NgramProposer
    elif proposer in ("mtp", "eagle3", "shared-kv"):
        from .speculative import mtp as heads

        {"mtp": heads.attach_mtp, "eagle3": heads.attach_eagle3, "shared-kv": heads.attach_shared_kv}[proposer](eng)
    host_limit = None
    if getattr(args, "host_ram_limit", "auto") not in ("", "auto"):
        from .engine.memory import parse_limit

        total = os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
        host_limit = parse_limit(args.host_ram_limit, total)
        eng.llm.memory.limits["host"] = host_limit
    if getattr(args, "kv_offload_dir", ""):
        from .engine.kv_connector import LocalTieredConnector

        host_bytes = int(args.kv_offload_host_gib * (1 << 30))
        if host_limit is not None:       # the offload tier lives inside what the host limit leaves
            host_bytes = min(host_bytes, max(0, host_limit - eng.llm.memory.used("host")))
        eng.attach_kv_connector(LocalTieredConnector(args.kv_offload_dir, max_host_bytes=host_bytes,
                                                     max_disk_bytes=int(args.kv_offload_disk_gib * (1 << 30))))
    return eng


def _prompt_text(engine, text, raw, system=None):
    if raw or engine.tokenizer is None:
        return text
    msgs = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": text}]
    return engine.apply_chat_template(msgs, add_generation_prompt=True)


def _stats_line(res):
    return (f"[{res.completion_tokens} tok | TTFT {res.ttft_s * 1e3:.1f} ms | decode {res.decode_tokens_per_s:.1f} tok/s | "
            f"finish {res.finish_reason}]")


def _generate_on_graph_backend(args) -> int:
    """``--backend graph``: run the model's ONNX graph node by node (any decoder architecture, one sequence, library
    tensor operations) with the host processor chain and samplers."""
    import numpy as np

    from . import package as pkg
    from .engine import processors as procs
    from .engine.graph_decode import GraphDecodeSession

    sess = GraphDecodeSession.from_dir(args.model, "cuda" if args.device.startswith("cuda") else "cpu")
    tok_path = os.path.join(args.model, "tokenizer.json")
    if not os.path.exists(tok_path):
        tok_path = pkg.open_model_directory(args.model).tokenizer_path
    if not tok_path:
        print("generate --backend graph: the model directory has no tokenizer.json", file=sys.stderr)
        return 2
    from tokenizers import Tokenizer

    tok = Tokenizer.from_file(tok_path)
    prompt = args.prompt if args.prompt is not None else sys.stdin.read()
    ids = tok.encode(prompt, add_special_tokens=False).ids
    opt = _options(args)
    chain = procs.build_processor_chain(opt, len(ids))
    sampler = procs.GreedySampler() if opt.greedy else procs.CategoricalSampler()
    rng = np.random.default_rng(opt.seed or None)
    t0 = time.perf_counter()
    logits = sess.feed(ids)[-1]
    ttft, out = time.perf_counter() - t0, []
    for _ in range(opt.max_new_tokens):
        row = chain.process(np.asarray(sess.tokens), logits.cpu().numpy().astype(np.float32))
        out.append(sampler.sample(row, float(rng.random())))
        sys.stdout.write(tok.decode(out)[len(tok.decode(out[:-1])):])
        sys.stdout.flush()
        if len(out) == opt.max_new_tokens:
            break
        logits = sess.feed([out[-1]])[-1]
    sys.stdout.write("\n")
    total = time.perf_counter() - t0
    print(f"[{len(out)} tok | TTFT {ttft * 1e3:.1f} ms | decode {max(len(out) - 1, 0) / max(total - ttft, 1e-9):.1f} tok/s | backend graph]",
          file=sys.stderr)
    return 0


def cmd_generate(args, profiler):
    if getattr(args, "backend", "native") == "graph":
        return _generate_on_graph_backend(args)
    from .package.decoder_graph import GraphPatternError

    try:
        eng = _load(args)
    except GraphPatternError as e:
        print(f"generate: {e}\nThe fast path does not recognise this decoder graph; it can still run node by node: add --backend graph",
              file=sys.stderr)
        return 2
    prompt = args.prompt if args.prompt is not None else sys.stdin.read()
    t_lat = []
    last = [time.perf_counter()]

    def on_token(tok, delta):
        now = time.perf_counter()
        t_lat.append(now - last[0])
        last[0] = now
        sys.stdout.write(delta)
        sys.stdout.flush()

    with profiler.span("generate"):
        res = eng.generate(_prompt_text(eng, prompt, args.raw), _options(args), on_token=on_token)
    sys.stdout.write("\n")
    print(_stats_line(res), file=sys.stderr)
    profiler.report(res, t_lat[1:], eng)
    return 0


class Repl:
    """State and command handling of the interactive session (``run``).  Slash commands, as in the reference's REPL
    (crates/onnx-genai-cli/src/lib.rs:1254-1383): /system /raw /stats /profile /reset /model, plus /image and /audio
    (attachments for the next prompt, answered by the media chat of ``--multimodal-package``), /ep (show or switch the
    device the engine runs on) and /backend (show or switch between the fused executor and the node-by-node graph
    backend)."""

    HELP = ("/system TEXT  /raw  /stats  /profile  /reset  /model  /image PATH|clear  /audio PATH|clear  /ep [cpu|cuda]  "
            "/backend [native|graph]  /quit")

    def __init__(self, args, profiler, loader=None, media_chat=None, out=None):
        self.args, self.profiler = args, profiler
        self.loader = loader or _load
        self.out = out or (lambda text: print(text))
        self.eng = self.loader(args)
        self.session = self.eng.create_session()
        self.system, self.raw, self.stats = None, getattr(args, "raw", False), True
        self.media_chat = media_chat
        self.images, self.audio = [], None
        self.done = False

    def _reload(self):
        self.eng = self.loader(self.args)
        self.session = self.eng.create_session()

    def command(self, line: str) -> None:
        cmd, _, rest = line.partition(" ")
        rest = rest.strip()
        if cmd in ("/quit", "/exit"):
            self.done = True
        elif cmd == "/help":
            self.out(self.HELP)
        elif cmd == "/system":
            self.system = rest or None
        elif cmd == "/raw":
            self.raw = not self.raw
            self.out(f"raw = {self.raw}")
        elif cmd == "/stats":
            self.stats = not self.stats
        elif cmd == "/reset":
            self.eng.reset_session(self.session)
            self.images, self.audio = [], None
        elif cmd == "/model":
            self.out(json.dumps(self.eng.resource_snapshot(), indent=1))
        elif cmd == "/profile":
            self.profiler.enabled = not self.profiler.enabled
            self.out(f"profile = {self.profiler.enabled}")
        elif cmd in ("/image", "/audio"):
            kind = cmd[1:]
            if not rest:
                held = [f"{len(b)} bytes" for b in self.images] if kind == "image" else ([f"{len(self.audio)} bytes"] if self.audio else [])
                self.out(f"{kind}: " + (", ".join(held) if held else "nothing attached") + f"; {cmd} PATH attaches a file to the next prompt")
            elif rest == "clear":
                if kind == "image":
                    self.images = []
                else:
                    self.audio = None
            elif self.media_chat is None or not self.media_chat.accepts.get(kind):
                self.out(f"{cmd}: this session has no {kind} pipeline; start it with --multimodal-package DIR (a workflow package with "
                         f"a typed {kind} input)")
            else:
                try:
                    with open(os.path.expanduser(rest), "rb") as f:
                        data = f.read()
                except OSError as exc:
                    self.out(f"{cmd}: {exc}")
                    return
                if kind == "image":
                    self.images.append(data)
                else:
                    self.audio = data
                self.out(f"{kind} attached ({len(data)} bytes); it goes with the next prompt")
        elif cmd == "/ep":
            cur = str(getattr(self.eng.llm, "device", getattr(self.args, "device", "cpu")))
            if not rest:
                self.out(f"execution device: {cur} (/ep cpu or /ep cuda reloads the model there)")
            elif rest not in ("cpu", "cuda"):
                self.out("/ep: expected cpu or cuda")
            else:
                if rest == "cuda":
                    import torch

                    if not torch.cuda.is_available():
                        self.out("/ep: no CUDA device is visible to this process")
                        return
                self.args.device = rest
                self._reload()
                self.out(f"model reloaded on {rest}; the session starts over")
        elif cmd == "/backend":
            cur = getattr(self.args, "backend", "native")
            if not rest:
                self.out(f"decode backend: {cur} (native = fused executor over paged KV, graph = the ONNX graph node by node)")
            elif rest not in ("native", "graph"):
                self.out("/backend: expected native or graph")
            else:
                self.args.backend = rest
                self.out(f"decode backend = {rest}" + ("; prompts now run one at a time through the graph executor, without the session's history"
                                                       if rest == "graph" else ""))
        else:
            self.out(f"unknown command {cmd}; /help lists commands")

    def prompt(self, line: str, on_text=None) -> object:
        on_text = on_text or (lambda d: (sys.stdout.write(d), sys.stdout.flush()))
        if self.images or self.audio is not None:
            ids = self.eng.tokenizer.encode(_prompt_text(self.eng, line, self.raw, self.system))
            image, audio = (self.images[0] if self.images else None), self.audio
            self.images, self.audio = [], None
            out_ids = self.media_chat.generate(ids, image=image, audio=audio, max_new_tokens=getattr(self.args, "max_tokens", 64) or 64)
            text = self.eng.tokenizer.decode(list(out_ids))
            on_text(text)
            return None
        if getattr(self.args, "backend", "native") == "graph":
            a = copy.copy(self.args)
            a.prompt = line
            _generate_on_graph_backend(a)
            return None
        text = _prompt_text(self.eng, line, self.raw, self.system if self.eng.session_len(self.session) == 0 else None)
        return self.eng.generate_in_session(self.session, text, _options(self.args), on_token=lambda t, d: on_text(d))


def cmd_run(args, profiler):
    media = None
    if getattr(args, "multimodal_package", ""):
        from .server.multimodal import WorkflowMediaChat

        media = WorkflowMediaChat(args.multimodal_package, "cuda" if str(args.device).startswith("cuda") else "cpu")
    repl = Repl(args, profiler, media_chat=media)
    print("interactive session; /help lists commands", file=sys.stderr)
    while not repl.done:
        try:
            line = input(">>> ")
        except (EOFError, KeyboardInterrupt):
            print()
            return 0
        if not line.strip():
            continue
        if line.startswith("/"):
            repl.command(line)
            continue
        res = repl.prompt(line)
        print()
        if repl.stats and res is not None:
            print(_stats_line(res), file=sys.stderr)
    return 0


def cmd_serve(args, profiler):
    import uvicorn

    from .server import create_app

    host, _, port = args.addr.rpartition(":")
    app_kw = dict(max_output_tokens=args.max_output_tokens, max_queue_depth=args.max_queue_depth,
                  enable_debug_endpoints=args.enable_debug_endpoints, node_id=args.node_id,
                  admission_window_ms=args.admission_window_ms, default_reasoning_effort=args.default_reasoning_effort or None)
    if args.models_dir or args.models_config:
        import copy

        from .server.registry import ModelRegistry, RegistryApp

        per_model: dict = {}

        def loader(path):
            a = copy.copy(args)
            a.model = path
            for key, value in per_model.get(path, {}).items():       # per-model overrides of the engine flags
                setattr(a, key.replace("-", "_"), value)
            return _load(a)

        if args.models_config:
            import yaml

            with open(args.models_config, encoding="utf-8") as f:
                doc = yaml.safe_load(f) or {}
            entries = doc.get("models") or {}
            if not entries:
                print(f"serve: {args.models_config} lists no models (expected `models: {{name: {{path: DIR}}}}`)", file=sys.stderr)
                return 2
            base = os.path.dirname(os.path.abspath(args.models_config))
            found = {}
            for name, spec in entries.items():
                spec = {"path": spec} if isinstance(spec, str) else dict(spec or {})
                if "path" not in spec:
                    print(f"serve: model {name!r} in {args.models_config} has no path", file=sys.stderr)
                    return 2
                path = os.path.normpath(os.path.join(base, spec.pop("path")))
                found[name] = path
                per_model[path] = spec
            reg = ModelRegistry(found, max_loaded=args.max_loaded_models, loader=loader, **app_kw)
        else:
            reg = ModelRegistry.from_dir(args.models_dir, max_loaded=args.max_loaded_models, loader=loader, **app_kw)
        if args.model:
            reg.warmup([os.path.basename(os.path.abspath(args.model))])
        app = RegistryApp(reg, enable_admin_endpoints=args.enable_admin_endpoints)
    else:
        media_device = "cuda" if args.device.startswith("cuda") else "cpu"
        if not args.model and (args.image_package or args.speech_package):
            from fastapi import FastAPI

            app = FastAPI(title="onnx-genai-b200 media")
            if args.image_package:
                from .server.images import ImagePipeline, add_image_routes

                add_image_routes(app, ImagePipeline(args.image_package, media_device), os.path.basename(os.path.abspath(args.image_package)))
            if args.speech_package:
                from .server.audio import SpeechPipeline, add_speech_routes

                add_speech_routes(app, SpeechPipeline(args.speech_package, media_device))
            app.get("/health")(lambda: {"status": "ok"})
            uvicorn.run(app, host=host or "127.0.0.1", port=int(port), log_level="info")
            return 0
        if not args.model:
            print("serve: give a model directory, --models-dir, --models-config, --image-package or --speech-package", file=sys.stderr)
            return 2
        eng = _load(args)
        if args.image_package:
            from .server.images import ImagePipeline

            app_kw["image_pipeline"] = ImagePipeline(args.image_package, media_device)
        if args.speech_package:
            from .server.audio import SpeechPipeline

            app_kw["speech_pipeline"] = SpeechPipeline(args.speech_package, media_device)
        if getattr(args, "multimodal_package", ""):
            from .server.multimodal import WorkflowMediaChat

            app_kw["media_chat"] = WorkflowMediaChat(args.multimodal_package, media_device)
        if getattr(args, "transcribe_package", ""):
            from .server.transcribe import WorkflowTranscriber

            app_kw["transcriber"] = WorkflowTranscriber(args.transcribe_package, media_device)
        app = create_app(eng, model_name=os.path.basename(os.path.abspath(args.model)), **app_kw)
    uvicorn.run(app, host=host or "127.0.0.1", port=int(port), log_level="info")
    return 0


def cmd_run_workflow(args) -> int:
    """Run a multi-model package outside the token engine: diffusion, codec, video and policy-only workflows whose
    components are ONNX graphs.  Prints one JSON line with the shape of every output."""
    import numpy as np

    from .engine.workflow_runtime import WorkflowRuntimeError, WorkflowSession

    feeds = {}
    for item in args.input:
        name, sep, value = item.partition("=")
        if not sep:
            print(f"run-workflow: --input wants NAME=VALUE, got {item!r}", file=sys.stderr)
            return 2
        if value.endswith(".npy"):
            feeds[name] = np.load(value)
        elif value.startswith("ids:"):
            feeds[name] = np.asarray([[int(t) for t in value[4:].split(",") if t]], dtype=np.int64)
        else:
            try:
                feeds[name] = np.asarray(json.loads(value))
            except ValueError:
                print(f"run-workflow: cannot read the value of {name!r}: {value!r} is neither a .npy file, ids:..., nor JSON", file=sys.stderr)
                return 2
            if feeds[name].ndim == 0:
                feeds[name] = feeds[name].reshape(1)
    try:
        sess = WorkflowSession.from_package(args.package, device=args.device)
        out = sess.run(feeds)
    except WorkflowRuntimeError as e:
        print(f"run-workflow: {e}", file=sys.stderr)
        return 1
    summary = {}
    if args.out:
        os.makedirs(args.out, exist_ok=True)
    for name, value in out.items():
        vals = value if isinstance(value, list) else [value]
        arrs = [np.asarray(v.detach().cpu() if hasattr(v, "detach") else v) for v in vals]
        summary[name] = [list(a.shape) for a in arrs] if isinstance(value, list) else list(arrs[0].shape)
        if args.out:
            arr = np.stack(arrs) if isinstance(value, list) and len({a.shape for a in arrs}) == 1 else arrs[-1]
            np.save(os.path.join(args.out, name + ".npy"), arr)
            last = arrs[-1]
            if last.ndim == 4 and last.shape[1] in (1, 3) and name in ("image", "images"):      # NCHW in [-1, 1] or [0, 1]
                _save_png(os.path.join(args.out, name + ".png"), last[0])
    print(json.dumps({"outputs": summary, "invocations": sess.stats["invocations"], "iterations": sess.stats["iterations"]}))
    return 0


def _save_png(path: str, chw) -> None:
    from .utils.png import encode_png

    with open(path, "wb") as f:
        f.write(encode_png(chw))


def cmd_show(args, profiler):
    from . import package as pkg
    from .package.onnx_text import load_any
    from .package.decoder_graph import lower_decoder

    d = pkg.open_model_directory(args.model)
    meta = d.load_metadata()
    model = load_any(d.model_path)
    ops_count: dict = {}
    for n in model.graph.nodes:
        key = (n.domain + "::" if n.domain else "") + n.op_type
        ops_count[key] = ops_count.get(key, 0) + 1
    from .package.decoder_graph import GraphPatternError

    try:
        cfg, _, _ = lower_decoder(model)
        arch = {k: getattr(cfg, k) for k in ("num_layers", "hidden", "num_heads", "num_kv_heads", "head_dim",
                                             "intermediate", "vocab", "weight_format", "tie_embeddings", "qkv_bias")}
        weight_bytes = cfg.weight_bytes()
    except GraphPatternError as e:      # not a decoder the fast path lowers: still describable, and runnable with --backend graph
        arch = {"recognised_by_fast_path": False, "reason": str(e), "runs_with": "--backend graph"}
        weight_bytes = sum(int(t.array.nbytes) for t in model.graph.initializers.values() if t.array is not None)
    out = {"model_path": d.model_path, "variant": d.variant, "tokenizer": d.tokenizer_path, "metadata": d.metadata_path,
           "architecture": arch,
           "max_sequence_length": meta.max_sequence_length, "required_capabilities": meta.required_capabilities,
           "operators": dict(sorted(ops_count.items())), "weight_bytes": weight_bytes}
    print(json.dumps(out, indent=1))
    return 0


def cmd_validate(args, profiler):
    """Checks a model directory the way the loader will read it and prints every problem found (exit 1 if any):
    the graph is a recognised decoder, metadata parses and agrees with the graph, tokenizer and template are present,
    int4 tensors have consistent shapes.  The counterpart of the reference's `validate_metadata` tool and checker."""
    from . import metadata as md
    from . import package as pkg
    from .package.onnx_text import load_any
    from .package.decoder_graph import lower_decoder

    problems, notes = [], []
    try:
        d = pkg.open_model_directory(args.model)
    except Exception as exc:
        print(json.dumps({"ok": False, "problems": [f"{exc}"]}, indent=1))
        return 1
    meta = None
    try:
        meta = d.load_metadata()
    except Exception as exc:
        problems.append(f"metadata: {exc}")
    cfg = None
    try:
        cfg, weights, _ = lower_decoder(load_any(d.model_path), keep_int4=True)
        notes.append(f"decoder graph recognised: {cfg.num_layers} layers, hidden {cfg.hidden}, {cfg.num_heads}/{cfg.num_kv_heads} heads "
                     f"of {cfg.head_dim}, vocab {cfg.vocab}, weights {cfg.weight_format}")
        for li, lw in enumerate(weights.layers):
            for name, lin in (lw.quant or {}).items():
                for one in (lin if isinstance(lin, list) else [lin]):
                    kb = (one.k + one.block - 1) // one.block
                    if tuple(one.q.shape) != (one.q.shape[0], kb, one.block // 2):
                        problems.append(f"layer {li} {name}: MatMulNBits weight has shape {tuple(one.q.shape)}, expected [N, {kb}, {one.block // 2}]")
                    if tuple(one.scales.shape)[:2] != (one.q.shape[0], kb) and one.scales.numel() != one.q.shape[0] * kb:
                        problems.append(f"layer {li} {name}: scales have {one.scales.numel()} entries, expected {one.q.shape[0] * kb}")
    except Exception as exc:
        problems.append(f"graph: {exc}")
    try:   # well-formedness: single assignment, defined inputs, no cycle, operator arity and attribute kinds
        from .package import onnx_checker as ck

        found = ck.check_model(load_any(d.model_path))
        problems.extend(f"checker: {p}" for p in ck.errors(found))
        warn = [p for p in found if p.severity == "warning"]
        notes.append(f"checker: {len(found) - len(warn)} errors, {len(warn)} warnings" + (f" (first: {warn[0]})" if warn else ""))
    except Exception as exc:
        notes.append(f"checker skipped: {exc}")
    try:   # static shapes: what resolves without running the graph, and what the graph's declared outputs disagree with
        from .package import shape_inference as si

        rep = si.infer(load_any(d.model_path), policy="strict")
        notes.append(f"shape inference: {len(rep.types) - len(rep.unresolved)} of {len(rep.types)} values resolved"
                     + (f", {rep.fresh_symbols} data-dependent extents" if rep.fresh_symbols else "")
                     + (f"; no rule for {sorted(rep.unregistered)}" if rep.unregistered else ""))
    except si.ShapeInferenceError as exc:
        problems.append(f"shape inference: {exc}")
    except Exception as exc:
        notes.append(f"shape inference skipped: {exc}")
    if meta is not None and cfg is not None:
        if meta.vocab_size and meta.vocab_size != cfg.vocab:
            problems.append(f"metadata model.vocab_size={meta.vocab_size} but the embedding has {cfg.vocab} rows")
        if meta.max_sequence_length and meta.max_sequence_length > cfg.max_position:
            notes.append(f"metadata max_sequence_length {meta.max_sequence_length} exceeds the rotary table ({cfg.max_position}); the smaller wins")
    if d.tokenizer_path is None:
        notes.append("no tokenizer.json: text prompts are unavailable, token-id prompts still work")
    else:
        try:
            from tokenizers import Tokenizer

            tok = Tokenizer.from_file(d.tokenizer_path)
            if cfg is not None and tok.get_vocab_size() > cfg.vocab:
                problems.append(f"tokenizer has {tok.get_vocab_size()} entries but the model's vocabulary is {cfg.vocab}")
        except Exception as exc:
            problems.append(f"tokenizer: {exc}")
    if d.chat_template is None:
        notes.append("no chat template: `run` and /v1/chat/completions fall back to a plain role-prefixed format")
    print(json.dumps({"ok": not problems, "model": d.model_path, "problems": problems, "notes": notes}, indent=1))
    return 0 if not problems else 1


def cmd_list(args, profiler):
    root = args.models_dir
    for name in sorted(os.listdir(root)):
        p = os.path.join(root, name)
        if os.path.isdir(p) and (os.path.exists(os.path.join(p, "manifest.json")) or any(f.endswith(".onnx") for f in os.listdir(p))):
            print(name)
    return 0


def cmd_export(args, profiler):
    from .package import export

    sys.argv = ["export", "--preset", args.preset, "--out", args.out] + (["--int4"] if args.int4 else []) + \
        (["--layers", str(args.layers)] if args.layers else [])
    export.main()
    return 0


class Profiler:
    """--profile: per-stage wall clock table + latency percentiles; --profile-json / --profile-trace write files."""

    def __init__(self, enabled, json_path=None, trace_path=None, gpu=False):
        self.enabled, self.json_path, self.trace_path = enabled or bool(json_path) or bool(trace_path) or gpu, json_path, trace_path
        self.spans = []
        # --profile-gpu: device activity (kernels, copies) through CUPTI for the whole command; its per-kernel table goes
        # to stderr and, with --profile-trace, one track per GPU stream joins the timeline
        self.gpu = None
        if gpu:
            from .utils.gpu_activity import GpuActivityCollector

            try:
                self.gpu = GpuActivityCollector().start()
            except Exception as exc:
                print(f"--profile-gpu: device activity is not collected: {exc}", file=sys.stderr)

    def span(self, name):
        prof = self

        class _S:
            def __enter__(self):
                self.t0 = time.perf_counter()

            def __exit__(self, *a):
                prof.spans.append((name, self.t0, time.perf_counter()))

        return _S()

    def report(self, res, itl, eng):
        if not self.enabled:
            return
        itl_ms = sorted(x * 1e3 for x in itl)
        pct = lambda p: itl_ms[min(len(itl_ms) - 1, int(p * len(itl_ms)))] if itl_ms else 0.0
        rep = {"ttft_ms": res.ttft_s * 1e3, "decode_tok_per_s": res.decode_tokens_per_s,
               "e2e_tok_per_s": res.completion_tokens / res.total_s if res.total_s else 0.0,
               "itl_ms": {"mean": sum(itl_ms) / len(itl_ms) if itl_ms else 0.0, "p50": pct(0.5), "p90": pct(0.9), "p99": pct(0.99),
                          "max": itl_ms[-1] if itl_ms else 0.0},
               "finish_reason": res.finish_reason, "prompt_tokens": res.prompt_tokens, "completion_tokens": res.completion_tokens,
               "kv": eng.resource_snapshot(), "stages": [{"name": n, "ms": (b - a) * 1e3} for n, a, b in self.spans]}
        print("profile: TTFT %.1f ms | decode %.2f tok/s | ITL p50 %.1f / p99 %.1f ms | %s" %
              (rep["ttft_ms"], rep["decode_tok_per_s"], rep["itl_ms"]["p50"], rep["itl_ms"]["p99"], rep["finish_reason"]), file=sys.stderr)
        gpu_spans = []
        if self.gpu is not None:
            self.gpu.stop()
            rep["gpu_activity"] = {"busy_fraction": self.gpu.busy_fraction(), "dropped": self.gpu.dropped, "top": self.gpu.summary()[:40]}
            gpu_spans = self.gpu.spans()
            print(self.gpu.table(), file=sys.stderr)
        if self.json_path:
            json.dump(rep, open(self.json_path, "w"), indent=1)
        if self.trace_path:
            from .utils.trace import write_chrome_trace

            write_chrome_trace(self.trace_path, [(n, a, b, "cli") for n, a, b in self.spans] + gpu_spans)


# ------------------------------------------------------------------------------------------
# transcribe: WAV files or a live PCM stream on standard input -> text / JSON lines / SubRip
# (the reference's `transcribe` subcommand, crates/onnx-genai-cli/src/transcribe.rs)
# ------------------------------------------------------------------------------------------
def srt_timestamp(seconds: float) -> str:
    ms = int(round(max(0.0, seconds) * 1000.0))
    return "%02d:%02d:%02d,%03d" % (ms // 3600000, (ms // 60000) % 60, (ms // 1000) % 60, ms % 1000)


def format_transcript(fmt: str, index: int, start: float, end: float, text: str) -> str:
    if fmt == "json":
        return json.dumps({"index": index, "start": round(start, 3), "end": round(end, 3), "text": text}, ensure_ascii=False)
    if fmt == "srt":
        return "%d\n%s --> %s\n%s\n" % (index + 1, srt_timestamp(start), srt_timestamp(end), text)
    return text


class PcmStreamReader:
    """Mono float samples from a byte stream of 16-bit PCM.  A stream that begins with a RIFF/WAVE header declares its own
    rate and channel count (its data chunk may claim any length: a pipe has no end until it closes); otherwise the
    caller's rate and channel count describe the raw samples.  Channels are averaged."""

    def __init__(self, stream, sample_rate: int, channels: int, chunk_seconds: float = 0.25):
        import struct

        self.stream = stream
        self.sample_rate, self.channels = int(sample_rate), max(1, int(channels))
        self.left = b""
        head = self._read_exact(12)
        if len(head) == 12 and head[:4] == b"RIFF" and head[8:12] == b"WAVE":
            while True:
                hdr = self._read_exact(8)
                if len(hdr) < 8:
                    raise ValueError("the WAV stream ended before its data chunk")
                tag, size = hdr[:4], struct.unpack("<I", hdr[4:])[0]
                if tag == b"fmt ":
                    fmt = self._read_exact(size + (size & 1))
                    code, ch, rate, _, _, bits = struct.unpack("<HHIIHH", fmt[:16])
                    if code not in (1, 0xFFFE) or bits != 16:
                        raise ValueError(f"standard input carries WAV format {code} with {bits} bits; 16-bit PCM is read")
                    self.sample_rate, self.channels = int(rate), max(1, int(ch))
                elif tag == b"data":
                    break
                else:
                    self._read_exact(size + (size & 1))
        else:
            self.left = head
        if self.sample_rate <= 0:
            raise ValueError("the sample rate must be positive")
        self.frame_bytes = 2 * self.channels
        self.chunk_bytes = max(1, int(self.sample_rate * chunk_seconds)) * self.frame_bytes

    def _read_exact(self, n: int) -> bytes:
        out = b""
        while len(out) < n:
            got = self.stream.read(n - len(out))
            if not got:
                break
            out += got
        return out

    def read_chunk(self):
        """The next block of samples (empty at end of stream).  A trailing partial frame is dropped."""
        import numpy as np

        data = self.left + self._read_exact(max(0, self.chunk_bytes - len(self.left)))
        usable = len(data) // self.frame_bytes * self.frame_bytes
        self.left = data[usable:] if usable and len(data) >= self.chunk_bytes else b""
        if usable == 0:
            return np.zeros(0, np.float32)
        x = np.frombuffer(data[:usable], dtype="<i2").astype(np.float32) / 32768.0
        return x.reshape(-1, self.channels).mean(axis=1).astype(np.float32)


def cmd_transcribe(args, profiler, transcriber=None, stdin=None, out=None):
    import numpy as np

    from .preprocess import StreamSegmenter, resample
    from .server.transcribe import read_wav

    out = out or sys.stdout
    t_load = time.perf_counter()
    if transcriber is None:
        from .server.transcribe import WorkflowTranscriber

        try:
            transcriber = WorkflowTranscriber(args.model, getattr(args, "device", "cpu"))
        except Exception as exc:
            print(f"What: {args.model} could not be loaded as a speech package.\nWhy: {exc}\n"
                  "How: point `transcribe` at a speech-to-text workflow package (a waveform input, a token output, tokenizer.json).",
                  file=sys.stderr)
            return 2
    profiler.spans.append(("model load", t_load, time.perf_counter()))
    window = float(getattr(transcriber, "window_seconds", 30.0) or 30.0)
    seg_seconds = args.segment_seconds if args.segment_seconds else window
    if seg_seconds > window + 1e-6:
        print(f"What: --segment-seconds {seg_seconds:g} was rejected.\nWhy: this model's declared audio input holds at most {window:.2f}s, "
              f"so a longer segment could not be encoded.\nHow: request at most {window:.2f}s per segment.", file=sys.stderr)
        return 2
    want_rate = int(getattr(transcriber, "sample_rate", 16000) or 16000)
    totals = {"audio_s": 0.0, "compute_s": 0.0, "segments": 0, "slowest_ms": 0.0}
    index = [0]

    def drain(segments, rate):
        for samples, start_sample in segments:
            start, dur = start_sample / rate, len(samples) / rate
            t0 = time.perf_counter()
            x = resample(samples, rate, want_rate) if rate != want_rate else samples
            text = str(transcriber.transcribe(np.asarray(x, dtype=np.float32), args.language or None)).strip()
            dt = time.perf_counter() - t0
            totals["audio_s"] += dur
            totals["compute_s"] += dt
            totals["segments"] += 1
            totals["slowest_ms"] = max(totals["slowest_ms"], dt * 1e3)
            if not text:
                continue
            print(format_transcript(args.format, index[0], start, start + dur, text), file=out, flush=True)   # per segment: a live stream is read while it runs
            index[0] += 1

    def segmenter(rate):
        return StreamSegmenter(rate, seg_seconds, args.silence_seconds, args.silence_threshold, args.min_segment_seconds)

    t_run = time.perf_counter()
    for source in (args.audio or ["-"]):
        if source == "-":
            try:
                reader = PcmStreamReader(stdin or sys.stdin.buffer, args.sample_rate, args.channels)
            except ValueError as exc:
                print(f"What: standard input could not be read as audio.\nWhy: {exc}\nHow: pipe raw 16-bit PCM (with --sample-rate / "
                      "--channels) or a 16-bit PCM WAV stream.", file=sys.stderr)
                return 2
            print(f"listening on stdin: {reader.sample_rate} Hz, {reader.channels} channel{'s' if reader.channels != 1 else ''}, "
                  f"up to {seg_seconds:.2f}s per segment (Ctrl-C to stop)", file=sys.stderr)
            seg = segmenter(reader.sample_rate)
            try:
                while True:
                    chunk = reader.read_chunk()
                    if len(chunk) == 0:
                        break
                    drain(seg.push(chunk), reader.sample_rate)
            except KeyboardInterrupt:
                pass
            last = seg.flush()
            drain([last] if last is not None else [], reader.sample_rate)
        else:
            try:
                with open(source, "rb") as f:
                    samples, rate = read_wav(f.read())
            except OSError as exc:
                print(f"What: the audio file {source} could not be read.\nWhy: {exc}\nHow: check the path and that the file is readable.",
                      file=sys.stderr)
                return 2
            except ValueError as exc:
                print(f"What: the audio file {source} could not be decoded.\nWhy: {exc}\nHow: provide a PCM WAV file "
                      "(convert with `ffmpeg -i in.mp3 -ar 16000 -ac 1 out.wav`).", file=sys.stderr)
                return 2
            seg = segmenter(rate)
            drain(seg.push(samples), rate)
            last = seg.flush()
            drain([last] if last is not None else [], rate)
    profiler.spans.append(("transcription", t_run, time.perf_counter()))
    if totals["segments"] and totals["audio_s"] > 0:
        rtf = totals["compute_s"] / totals["audio_s"]
        print("transcribed %.2fs of audio in %d segment%s, real-time factor %.3fx (below 1.0 keeps up with a live stream), slowest segment %.0f ms"
              % (totals["audio_s"], totals["segments"], "" if totals["segments"] == 1 else "s", rtf, totals["slowest_ms"]), file=sys.stderr)
    if profiler.enabled and profiler.json_path:
        rep = {"stages": [{"name": n, "ms": (b - a) * 1e3} for n, a, b in profiler.spans], "audio_seconds": totals["audio_s"],
               "segments": totals["segments"], "slowest_segment_ms": totals["slowest_ms"],
               "real_time_factor": totals["compute_s"] / totals["audio_s"] if totals["audio_s"] else None}
        json.dump(rep, open(profiler.json_path, "w"), indent=1)
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser(prog="onnx-genai-b200")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--profile-json", default=None)
    ap.add_argument("--profile-trace", default=None)
    ap.add_argument("--profile-gpu", action="store_true",
                    help="collect kernels and copies with their device timestamps (CUPTI): table on stderr, tracks in --profile-trace")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate")
    g.add_argument("model")
    g.add_argument("--prompt", default=None)
    _add_sampling(g)
    _add_engine(g)
    r = sub.add_parser("run")
    r.add_argument("model")
    _add_sampling(r)
    _add_engine(r)
    r.add_argument("--multimodal-package", default="",
                   help="workflow package with a typed image or audio input: /image and /audio attachments are answered by it")
    s = sub.add_parser("serve")
    s.add_argument("model", nargs="?", default="", help="model directory (or use --models-dir)")
    s.add_argument("--models-dir", default="", help="serve every model directory below this one; requests pick one by name")
    s.add_argument("--max-loaded-models", type=int, default=1, help="models kept resident; the least recently used idle one is evicted")
    s.add_argument("--admission-window-ms", type=float, default=2.0, help="an idle server waits this long for companion requests before its first step")
    s.add_argument("--addr", default="127.0.0.1:8080")
    s.add_argument("--max-output-tokens", type=int, default=4096)
    s.add_argument("--max-sessions", type=int, default=256)
    s.add_argument("--max-queue-depth", type=int, default=256)
    s.add_argument("--enable-debug-endpoints", action="store_true")
    s.add_argument("--enable-admin-endpoints", action="store_true", help="with --models-dir: /v1/admin/models load / warmup / unload")
    s.add_argument("--node-id", default="node-0")
    s.add_argument("--default-reasoning-effort", default="", choices=["", "low", "medium", "high"],
                   help="reasoning effort handed to chat templates that take one, when a request names none")
    s.add_argument("--image-package", default="", help="text-to-image workflow package to serve at /v1/images/generations and /sdapi/v1/txt2img")
    s.add_argument("--speech-package", default="", help="text-to-speech workflow package to serve at /v1/audio/speech")
    s.add_argument("--transcribe-package", default="", help="speech-to-text workflow package to serve at /v1/audio/transcriptions")
    s.add_argument("--multimodal-package", default="",
                   help="workflow package with a typed image or audio input: chat requests that carry an image_url / input_audio part run on it")
    s.add_argument("--models-config", default="", help="YAML or JSON file: models: {name: {path: DIR, ...engine flags}}")
    s.add_argument("--max-context", type=int, default=0)
    _add_engine(s)
    sh = sub.add_parser("show")
    sh.add_argument("model")
    va = sub.add_parser("validate", help="check a model directory and report every problem")
    va.add_argument("model")
    pm = sub.add_parser("plan-memory", help="lifetimes, arena size and lower bound of a graph's intermediates (JSON)")
    pm.add_argument("graph", help=".onnx or .onnx.textproto file")
    pm.add_argument("--bind", action="append", default=[], metavar="SYMBOL=N", help="value of a symbolic dimension (repeatable)")
    pm.add_argument("--values", action="store_true", help="also list every value with its lifetime and offset")
    ls = sub.add_parser("list")
    ls.add_argument("--models-dir", default=".")
    sub.add_parser("version")
    ex = sub.add_parser("export")
    ex.add_argument("--preset", default="tiny-llama")
    ex.add_argument("--out", required=True)
    ex.add_argument("--int4", action="store_true")
    ex.add_argument("--layers", type=int, default=0)
    ic = sub.add_parser("import-comfyui", help="convert a ComfyUI API-format graph into a workflow metadata document")
    ic.add_argument("graph")
    ic.add_argument("-o", "--out", default="-")
    tr = sub.add_parser("transcribe", help="speech to text: WAV files, or a live 16-bit PCM stream on standard input")
    tr.add_argument("model", help="speech-to-text workflow package directory")
    tr.add_argument("audio", nargs="*", help="PCM WAV files; `-` (the default) reads a stream from standard input and prints each "
                                             "segment as soon as it is recognised")
    tr.add_argument("--language", default="", help="spoken language token, e.g. en or zh (default: the model's own choice)")
    tr.add_argument("--format", default="text", choices=["text", "json", "srt"])
    tr.add_argument("--segment-seconds", type=float, default=0.0, help="longest segment transcribed at once (default and maximum: the model's window)")
    tr.add_argument("--silence-seconds", type=float, default=0.5, help="silence that ends a segment early; 0 cuts on the window alone")
    tr.add_argument("--silence-threshold", type=float, default=0.01, help="amplitude at or below which audio counts as silence")
    tr.add_argument("--min-segment-seconds", type=float, default=0.1, help="shortest segment worth transcribing (ignores brief clicks)")
    tr.add_argument("--sample-rate", type=int, default=16000, help="rate of raw PCM16 on standard input (a WAV header overrides it)")
    tr.add_argument("--channels", type=int, default=1, help="channels of raw PCM16 on standard input; they are mixed to mono")
    tr.add_argument("--device", default="cpu")
    rw = sub.add_parser("run-workflow", help="run a workflow package (every ONNX component on the generic graph executor)")
    rw.add_argument("package", help="directory with inference_metadata.yaml and the component graphs")
    rw.add_argument("--input", action="append", default=[], metavar="NAME=VALUE",
                    help="a workflow input: a .npy file, a JSON literal (3, [1,2], 0.5) or ids:1,2,3 for a row of token ids")
    rw.add_argument("--out", default="", help="directory for the outputs (one .npy per output, .png for image outputs)")
    rw.add_argument("--device", default="cpu")
    dgp = sub.add_parser("diagnose", help="findings (what / why / how) and rooflines from a Chrome-trace JSON")
    dgp.add_argument("trace", help="trace written by ONNX_GENAI_TRACE, --profile-trace or /v1/debug/trace/perfetto")
    dgp.add_argument("--category", default=None, help="only events of this category")
    dgp.add_argument("--peaks", default=None, help="measured-peaks JSON (hbm_gbs, bf16_tflops_sustained)")
    args = ap.parse_args(argv)
    if args.cmd == "diagnose":
        from .utils.diagnose import main as diagnose_main
        return diagnose_main([args.trace] + (["--category", args.category] if args.category else []) + (["--peaks", args.peaks] if args.peaks else []))
    if args.cmd == "run-workflow":
        return cmd_run_workflow(args)
    if args.cmd == "plan-memory":
        from .package.memory_plan import plan_memory
        from .package.onnx_text import load_any

        try:
            symbols = {k: int(v) for k, v in (b.split("=", 1) for b in args.bind)}
        except ValueError:
            print("plan-memory: --bind takes SYMBOL=N with N an integer", file=sys.stderr)
            return 2
        plan = plan_memory(load_any(args.graph), symbols=symbols)
        plan.check()
        doc = plan.summary()
        if plan.unsized:
            doc["unsized_values"] = plan.unsized[:20]
        if args.values:
            doc["lifetimes"] = [{"name": v.name, "born": v.born, "dies": v.dies, "bytes": v.bytes, "offset": v.offset, "alias_of": v.alias_of}
                                for v in sorted(plan.values.values(), key=lambda v: v.born)]
        print(json.dumps(doc, indent=1))
        return 0
    if args.cmd == "import-comfyui":
        from .package.comfyui import main as comfy_main
        return comfy_main([args.graph, "-o", args.out])
    if args.cmd == "version":
        print(f"onnx-genai-b200 {__version__}")
        return 0
    profiler = Profiler(args.profile, args.profile_json, args.profile_trace, gpu=getattr(args, "profile_gpu", False))
    return {"generate": cmd_generate, "run": cmd_run, "serve": cmd_serve, "show": cmd_show, "validate": cmd_validate, "list": cmd_list,
            "export": cmd_export, "transcribe": cmd_transcribe}[args.cmd](args, profiler)


if __name__ == "__main__":
    sys.exit(main())
