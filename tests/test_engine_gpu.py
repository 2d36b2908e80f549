"""Engine on the GPU: the CUDA kernel path against the CPU fp32 engine on the same weights."""
import numpy as np
import pytest
import torch

from onnx_genai_b200 import ops
from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import DecoderModel, KVCache, StepInputs, random_weights

pytestmark = pytest.mark.gpu

CFG = DecoderConfig(name="g", num_layers=3, hidden=256, num_heads=8, num_kv_heads=2, head_dim=64, intermediate=512,
                    vocab=1024, rope_theta=1e6, tie_embeddings=False, qkv_bias=True, max_position=1024)


def test_first_token_logits_match_cpu_engine():
    """Teacher-forced comparison: same prompts, logits of the first sampled position, GPU bf16 vs CPU fp32."""
    wg = random_weights(CFG, "cuda", seed=11, std=0.05)
    wc = random_weights(CFG, "cpu", seed=11, std=0.05, dtype=torch.float32)
    # the CPU copy must hold exactly the bf16-rounded GPU weights
    for lg, lc in zip(wg.layers, wc.layers):
        for name in ("qkv_w", "qkv_b", "o_w", "gate_up_w", "down_w"):
            getattr(lc, name).copy_(getattr(lg, name).float().cpu())
    wc.embed.copy_(wg.embed.float().cpu())
    wc.lm_head.copy_(wg.lm_head.float().cpu())
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, CFG.vocab, size=n).astype(np.int32) for n in (3, 64, 65, 200)]
    res = {}
    for dev, w in (("cuda", wg), ("cpu", wc)):
        eng = LLMEngine(EngineConfig(model=CFG, num_pages=128, max_seqs=8, max_tokens_per_step=512, max_seq_len=512),
                        weights=w, device=dev)
        for p in prompts:
            eng.add_request(p, 4)
        eng.step()
        res[dev] = eng.model.logits[: len(prompts)].float().cpu().clone()
    if torch.cuda.is_available():
        ops.check_status()
    err = float((res["cuda"] - res["cpu"]).norm() / res["cpu"].norm())
    assert err < 3e-2, err


def test_generate_mixed_batch_runs_and_counts_kernels():
    cfg = CFG
    eng = LLMEngine(EngineConfig(model=cfg, num_pages=256, max_seqs=16, max_tokens_per_step=256, max_seq_len=512,
                                 prefill_chunk=128), device="cuda")
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, cfg.vocab, size=n).astype(np.int32) for n in (5, 300, 77, 129, 16, 250)]
    before = dict(ops.launch_counts)
    outs = eng.generate(prompts, max_new_tokens=24, temperature=0.8, top_p=0.9, top_k=50, seed=3)
    ops.check_status()
    assert all(len(o) == 24 for o in outs)
    assert all(0 <= t < cfg.vocab for o in outs for t in o)
    assert eng.native_executor
    for k in ("native_step_kernels", "sample"):
        assert ops.launch_counts[k] > before.get(k, 0), k
    # the Python-driven path launches the same kernels one by one and must agree token for token
    eng_py = LLMEngine(EngineConfig(model=cfg, num_pages=256, max_seqs=16, max_tokens_per_step=256, max_seq_len=512,
                                    prefill_chunk=128, native_executor=False), weights=eng.weights, device="cuda")
    outs_py = eng_py.generate(prompts, max_new_tokens=24, temperature=0.8, top_p=0.9, top_k=50, seed=3)
    for k in ("gemm_bf16_tcgen05", "paged_decode", "paged_prefill", "rope_kv_append", "rmsnorm"):
        assert ops.launch_counts[k] > before.get(k, 0), k
    assert outs_py == outs
    # same seeds -> same tokens on a second engine (device sampler is deterministic)
    eng2 = LLMEngine(EngineConfig(model=cfg, num_pages=256, max_seqs=16, max_tokens_per_step=256, max_seq_len=512,
                                  prefill_chunk=128), weights=eng.weights, device="cuda")
    outs2 = eng2.generate(prompts, max_new_tokens=24, temperature=0.8, top_p=0.9, top_k=50, seed=3)
    assert outs == outs2


def test_greedy_gpu_matches_baseline_library_path():
    """Hand-written kernels vs the library (cuBLAS) GEMM path: greedy streams agree on a well-separated model."""
    w = random_weights(CFG, "cuda", seed=5, std=0.08)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, CFG.vocab, size=n).astype(np.int32) for n in (40, 90)]
    outs = {}
    for base in (False, True):
        ops.set_baseline(base)
        try:
            eng = LLMEngine(EngineConfig(model=CFG, num_pages=128, max_seqs=8, max_tokens_per_step=256, max_seq_len=512),
                            weights=w, device="cuda")
            eng.add_request(prompts[0], 1)
            eng.add_request(prompts[1], 1)
            eng.step()
            outs[base] = eng.model.logits[:2].float().cpu().clone()
        finally:
            ops.set_baseline(False)
    err = float((outs[False] - outs[True]).norm() / outs[True].norm())
    assert err < 3e-2, err        # two bf16 pipelines that round at different points (the bound of GPU-vs-CPU logits above)


def test_int4_package_runs_in_kernel_dequant_on_gpu(tmp_path):
    """A MatMulNBits package loaded on the GPU keeps its weights int4 (GEMV / dequant kernels) and agrees with the CPU path."""
    from onnx_genai_b200.engine.api import Engine, GenerateOptions
    from onnx_genai_b200.package.export import export_package

    cfg = DecoderConfig(name="q", num_layers=2, hidden=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate=688,
                        vocab=512, rope_theta=1e4, tie_embeddings=False, qkv_bias=True, max_position=256)
    w = random_weights(cfg, "cpu", seed=2, std=0.08, dtype=torch.float32)
    d = export_package(cfg, w, str(tmp_path / "q4"), int4=True)
    outs = {}
    for dev in ("cuda", "cpu"):
        eng = Engine.from_dir(d, device=dev, num_pages=64, max_seqs=4, max_tokens_per_step=64)
        before = ops.launch_counts["w4a16_gemv_fused"]
        eng.llm.add_request(np.arange(3, 40, dtype=np.int32), 3)
        eng.llm.step()
        first = eng.llm.model.logits[:1].float().cpu().clone()
        eng.llm.step()
        outs[dev] = (first, eng.llm.model.logits[:1].float().cpu().clone())
        if dev == "cuda":
            assert not eng.llm.native_executor and ops.launch_counts["w4a16_gemv_fused"] > before
    ops.check_status()
    for a, b in zip(outs["cuda"], outs["cpu"]):
        assert float((a - b).norm() / b.norm()) < 4e-2


def test_cuda_graph_replay_of_decode_steps_matches_eager():
    """Decode-only steps replayed from captured graphs (padded to a row bucket) give the eager tokens."""
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, CFG.vocab, size=n).astype(np.int32) for n in (9, 40, 3, 120, 17)]   # 5 rows -> bucket 8
    outs = {}
    for graphs in (False, True):
        eng = LLMEngine(EngineConfig(model=CFG, num_pages=256, max_seqs=16, max_tokens_per_step=256, max_seq_len=512,
                                     cuda_graphs=graphs), device="cuda")
        for sampling in (dict(temperature=0.0), dict(temperature=0.9, top_p=0.8, seed=5)):
            outs[(graphs, sampling["temperature"])] = eng.generate(prompts, max_new_tokens=20, **sampling)
        ops.check_status()
        if graphs:
            assert not eng.graph_declines, eng.graph_declines
            assert eng.graph_replays >= 30 and len(eng.graphs) == 2      # one graph per sampler kind, many replays
    assert outs[(True, 0.0)] == outs[(False, 0.0)]
    assert outs[(True, 0.9)] == outs[(False, 0.9)]


CFG128 = DecoderConfig(name="g128", num_layers=2, hidden=256, num_heads=4, num_kv_heads=2, head_dim=128, intermediate=512,
                       vocab=1024, rope_theta=1e6, tie_embeddings=False, qkv_bias=True, max_position=4096)


def test_fp8_kv_engine_stays_close_to_bf16_kv():
    w = random_weights(CFG128, "cuda", seed=5, std=0.05)
    prompt = np.random.default_rng(2).integers(0, CFG128.vocab, size=300).astype(np.int32)
    logits = {}
    for kv in ("bf16", "fp8", "int8", "fp8_e5m2"):
        eng = LLMEngine(EngineConfig(model=CFG128, num_pages=64, max_seqs=2, max_tokens_per_step=512, max_seq_len=512,
                                     kv_dtype=kv), weights=w, device="cuda")
        eng.add_request(prompt, 2)
        eng.step()
        eng.step()                                            # second step: a decode row that reads the stored pages
        logits[kv] = eng.model.logits[:1].float().cpu().clone()
    ops.check_status()
    for kv in ("fp8", "int8", "fp8_e5m2"):
        err = float((logits[kv] - logits["bf16"]).norm() / logits["bf16"].norm())
        assert err < (0.12 if kv == "fp8_e5m2" else 6e-2), (kv, err)
    assert ops.launch_counts["paged_decode_fp8"] > 0 and ops.launch_counts["paged_prefill_fp8"] > 0


@pytest.mark.parametrize("kv", ["fp8", "bf16"])
def test_long_context_draft_rows_run_on_the_split_kv_decode_kernel(kv):
    """Speculative verification over a 2.2k-token context with fp8 pages: the draft rows go to the decode kernel
    (one page-table row and context length per query row); tokens equal the non-speculative run."""
    from onnx_genai_b200.speculative import SpeculativeProposer

    w = random_weights(CFG128, "cuda", seed=6, std=0.08)
    prompt = np.random.default_rng(3).integers(0, CFG128.vocab, size=2200).astype(np.int32)
    mk = lambda k: LLMEngine(EngineConfig(model=CFG128, num_pages=400, max_seqs=2, max_tokens_per_step=2304, max_seq_len=2400,
                                          kv_dtype=kv, max_draft_tokens=k, enable_prefix_cache=False), weights=w, device="cuda")
    want = mk(0).generate([prompt], max_new_tokens=16)[0]

    class Mixed(SpeculativeProposer):                     # true continuation, every third proposal corrupted
        calls = 0

        def propose(self, token_ids, k):
            done = len(token_ids) - len(prompt)
            out = np.asarray(want[done:done + k], dtype=np.int32).copy()
            Mixed.calls += 1
            if Mixed.calls % 3 == 0 and len(out):
                out[-1] = (int(out[-1]) + 7) % CFG128.vocab
            return out

    eng = mk(3)
    sid = eng.add_request(prompt, 16)
    eng.proposers[sid] = Mixed()
    got = []
    while eng.has_work:
        got += [tok for s, tok, fin in eng.step().events if s == sid]
    ops.check_status()
    assert eng.verify_on_decode_kernel > 0 and eng.core.spec_accepted > 0
    agree = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), len(want))
    assert agree >= 12, (agree, got, want)                # identical unless an fp8 near-tie flips late in the run


def test_mtp_proposer_drafts_from_device_hidden_states():
    """The MTP head runs on the device from the hidden rows the engine hands over.  A random head is almost never right,
    so its run must equal that of a proposer that is always wrong (same verification shapes, every draft rewound), and
    stay with plain greedy decoding up to bf16 near-ties between the 4-row verification pass and the 1-row decode pass."""
    from onnx_genai_b200.speculative import SpeculativeProposer
    from onnx_genai_b200.speculative.mtp import MtpHead, MtpProposer

    w = random_weights(CFG128, "cuda", seed=7, std=0.08)
    prompt = np.random.default_rng(4).integers(0, CFG128.vocab, size=90).astype(np.int32)
    mk = lambda k: LLMEngine(EngineConfig(model=CFG128, num_pages=64, max_seqs=2, max_tokens_per_step=512, max_seq_len=512,
                                          max_draft_tokens=k, enable_prefix_cache=False), weights=w, device="cuda")
    plain = mk(0).generate([prompt], max_new_tokens=12)[0]

    class Wrong(SpeculativeProposer):
        def propose(self, token_ids, k):
            return np.full(k, (int(token_ids[-1]) + 1) % 7, dtype=np.int32)

    def run(proposer):
        eng = mk(3)
        sid = eng.add_request(prompt, 12)
        eng.proposers[sid] = proposer
        got = []
        while eng.has_work:
            got += [tok for s, tok, fin in eng.step().events if s == sid]
        ops.check_status()
        return got, eng

    want, _ = run(Wrong())
    prop = MtpProposer(MtpHead.random(w.embed, w.lm_head, inter=256, seed=1))
    got, eng = run(prop)
    assert prop.hidden is not None and prop.hidden.is_cuda and prop.hidden.shape == (CFG128.hidden,)
    assert eng.core.spec_proposed >= 3
    if eng.core.spec_accepted == 0:
        assert got == want                                # same shapes, same rewinds: bit-identical runs
    agree = next((i for i, (a, b) in enumerate(zip(got, plain)) if a != b), len(plain))
    assert agree >= 4, (agree, got, plain)      # a near-tie ends the common prefix; the kernels of the two passes round differently


def test_kv_pool_grows_in_place_and_results_do_not_change():
    """A pool that starts with 8 backed pages inside a 256-page address range: the engine backs more as the scheduler
    runs low; page ids, tensor addresses and results are those of a pool that was large from the start."""
    w = random_weights(CFG128, "cuda", seed=8, std=0.05)
    prompts = [np.random.default_rng(s).integers(0, CFG128.vocab, size=n).astype(np.int32) for s, n in ((5, 300), (6, 170))]
    mk = lambda pages, mx: LLMEngine(EngineConfig(model=CFG128, num_pages=pages, kv_max_pages=mx, max_seqs=2, max_tokens_per_step=64,
                                                  max_seq_len=512, enable_prefix_cache=False), weights=w, device="cuda")
    want = mk(256, 0).generate(prompts, max_new_tokens=8)
    eng = mk(8, 256)
    base = [p.data_ptr() for p in eng.kv.pools]
    assert eng.kv.growable and eng.kv.num_pages == 8 and eng.kv.pools[0].shape[0] == 256
    got = eng.generate(prompts, max_new_tokens=8)
    ops.check_status()
    assert got == want
    assert eng.kv_grows >= 2 and eng.kv_grow_error is None and 8 < eng.kv.num_pages <= 256 and eng.core.num_pages == eng.kv.num_pages
    assert [p.data_ptr() for p in eng.kv.pools] == base
    snap = eng.memory.snapshot()["vram"]["by_role"]["kv"]
    assert snap == eng.kv.mapped_bytes() >= eng.kv.num_pages * eng.kv.page_nbytes * CFG128.num_layers


def test_shared_kv_proposer_reads_target_pages_on_the_device():
    """The shared-KV head's attention runs on the paged decode kernel over the target's own pages; a dense restatement
    over the gathered pages gives the same attention output."""
    from onnx_genai_b200.ops import reference as ref
    from onnx_genai_b200.speculative.mtp import SharedKvHead, SharedKvProposer

    w = random_weights(CFG128, "cuda", seed=9, std=0.08)
    prompt = np.random.default_rng(7).integers(0, CFG128.vocab, size=150).astype(np.int32)
    eng = LLMEngine(EngineConfig(model=CFG128, num_pages=64, max_seqs=2, max_tokens_per_step=512, max_seq_len=512,
                                 max_draft_tokens=2, enable_prefix_cache=False), weights=w, device="cuda")
    head = SharedKvHead.random(w.embed, w.lm_head, eng.model.hq, eng.model.d, seed=3, std=0.05)
    sid = eng.add_request(prompt, 6)
    prop = eng.proposers[sid] = SharedKvProposer(head)
    got = []
    while eng.has_work:
        got += [tok for s, tok, fin in eng.step().events if s == sid]
    ops.check_status()
    assert len(got) == 6 and eng.core.spec_proposed >= 2 and prop.llm is eng
    # one attention read against a dense computation
    sid = eng.add_request(prompt, 2)
    eng.step()
    ctx = len(prompt)
    pages = eng.core.seq_pages(sid)[: -(-ctx // 16)]
    m = eng.model
    q = torch.randn(1, (m.hq + 2 * m.hkv) * m.d, device="cuda").bfloat16()
    out = torch.zeros(1, m.hq * m.d, device="cuda", dtype=torch.bfloat16)
    ops.paged_decode(q, out, eng.kv.pools[-1], torch.from_numpy(pages[None].copy()).cuda(), torch.tensor([ctx], dtype=torch.int32, device="cuda"),
                     m.hq, m.hkv, m.d, m.scale)
    torch.cuda.synchronize()
    k_all, v_all = ref._gather_kv(eng.kv.pools[-1], torch.from_numpy(pages).cuda(), ctx)
    g = m.hq // m.hkv
    qh = q[0, : m.hq * m.d].float().view(m.hq, m.d)
    want = torch.cat([torch.softmax((qh[h] @ k_all[h // g].T) * m.scale, -1) @ v_all[h // g] for h in range(m.hq)])
    assert float((out[0].float() - want).norm() / want.norm()) < 2e-2


@pytest.mark.parametrize("kv", ["bf16", "fp8"])
def test_swap_preemption_and_cow_fork_on_the_device_keep_tokens(kv):
    """A pool too small for the batch forces swap preemption; a fork forces a copy-on-write page copy.  Pages (and, for
    one-byte pages, their scale rows) travel through pinned host memory by the swap kernels on the side stream;
    tokens must equal those of an unpressured engine."""
    w = random_weights(CFG128, "cuda", seed=9, std=0.05)
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, CFG128.vocab, size=30).astype(np.int32) for _ in range(6)]
    mk = lambda **kw: LLMEngine(EngineConfig(model=CFG128, max_seqs=8, max_tokens_per_step=64, max_seq_len=256,
                                             enable_prefix_cache=False, kv_dtype=kv, **kw), weights=w, device="cuda")
    roomy = mk(num_pages=128)
    want = roomy.generate(prompts, 20)
    tight = mk(num_pages=14, num_host_pages=64, preempt="swap")
    moves0 = ops.launch_counts["kv_move_pages"]
    got = tight.generate(prompts, 20)
    ops.check_status()
    assert tight.core.num_preemptions > 0 and tight.direct_swap
    assert ops.launch_counts["kv_move_pages"] > moves0
    assert got == want
    # fork: parent and child share pages until the first divergent token, then the written page is copied
    eng = mk(num_pages=64)
    sid = eng.add_request(prompts[0], 12)
    eng.step()                                  # prefill: 30 tokens, the second page is half full
    child = eng.core.fork(sid)
    eng.stats[child] = type(eng.stats[sid])()
    outs = {sid: [], child: []}
    copies0 = eng.swap_moves
    while eng.core.has_work:
        for s, tok, fin in eng.step().events:
            outs[s].append(tok)
    ops.check_status()
    assert eng.swap_moves > copies0             # the copy-on-write copy ran on the device
    n = min(len(outs[sid]), len(outs[child]))
    assert n >= 8 and outs[sid][:n] == outs[child][:n] == want[0][1:n + 1]      # both continue the unforked run


def test_weight_paging_streams_layers_from_pinned_memory_and_changes_no_token():
    """The last layers' matrices live in pinned host memory and pass through two device slots per step; greedy tokens
    equal the resident run, the ledger shows the bytes on the host tier, and every step copies each paged layer once."""
    cfg = CFG128.replace(num_layers=5) if hasattr(CFG128, "replace") else CFG128
    w = random_weights(cfg, "cuda", seed=9, std=0.05)
    prompts = [np.random.default_rng(4).integers(0, cfg.vocab, size=n).astype(np.int32) for n in (40, 300)]
    outs = {}
    import copy

    for paged in (0, 3):
        eng = LLMEngine(EngineConfig(model=cfg, num_pages=128, max_seqs=4, max_tokens_per_step=512, max_seq_len=512,
                                     weight_offload_layers=paged), weights=copy.deepcopy(w), device="cuda")
        sids = [eng.add_request(p, 12, ignore_eos=True) for p in prompts]
        steps = 0
        while eng.core.has_work:
            eng.step()
            steps += 1
        outs[paged] = [list(eng.core.seq_tokens(s)) for s in sids]
        if paged:
            assert eng.model.weight_copies() == steps * paged
            snap = eng.memory.snapshot()
            assert snap["host"]["by_role"]["weights"] == eng.model.paged_weight_bytes > 0
            assert all(getattr(lw, "qkv_w") is None for lw in eng.model.w.layers[-paged:])
    ops.check_status()
    assert outs[0] == outs[3]
    with pytest.raises(ValueError, match="weight_offload_layers needs the C\\+\\+ step executor"):
        LLMEngine(EngineConfig(model=cfg, num_pages=64, max_seqs=2, max_tokens_per_step=256, max_seq_len=256, kv_dtype="fp8",
                               weight_offload_layers=2), weights=copy.deepcopy(w), device="cuda")
